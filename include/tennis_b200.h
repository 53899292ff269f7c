/*
 * tennis_b200 -- C ABI of the B200 (sm_100a) int8 quantized-convolution path for TenniS.
 *
 * Plain C: pointers, sizes and an opaque plan handle; no C++ or framework types.  All tensor pointers are
 * DEVICE pointers unless a parameter name ends in `_host`.  `stream` is a cudaStream_t passed as void*.
 * Every function returns a status: 0 = ok, < 0 = invalid argument (nothing was launched),
 * > 0 = a CUDA runtime/driver error code.  tsb_last_error() gives the text of the last failure on the
 * calling thread.  Nothing here falls back to the CPU.
 *
 * The TenniS operator classes in tennis_b200/plugin/ (TS_REGISTER_OPERATOR on device "gpu") are thin C++
 * shells over exactly these entry points; each entry point names the reference interface it stands in for
 * (paths relative to the TenniS source tree).
 */
#ifndef TENNIS_B200_H
#define TENNIS_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* exported from libtennis_b200.so */
#if defined(__GNUC__)
#define TSB_API __attribute__((visibility("default")))
#else
#define TSB_API
#endif

#define TSB_OK 0
#define TSB_ERR_INVALID_ARGUMENT (-1)
#define TSB_ERR_UNSUPPORTED (-2)
#define TSB_ERR_WORKSPACE_TOO_SMALL (-3)
#define TSB_ERR_DEVICE_TIMEOUT (-4)

/* activation that follows add_bias in a quantized graph */
#define TSB_ACT_NONE 0
#define TSB_ACT_RELU 1       /* src/kernels/cpu/relu.cpp:30-52 */
#define TSB_ACT_LEAKY_RELU 2 /* src/kernels/cpu/leaky_relu.cpp:39-67, attribute "scale" */

/* memory layouts of activations */
#define TSB_LAYOUT_NCHW 0     /* the operator-visible layout of TenniS tensors */
#define TSB_LAYOUT_NHWC_PAD 1 /* internal: [N][H][W][Cp], Cp = tsb_padded_channels(C), padding channels zero */
#define TSB_LAYOUT_STAGED 2   /* input only: already in the plan's workspace, written by tsb_conv2d_i8_quantize_input */

/* which convolution kernel a plan uses */
#define TSB_KERNEL_AUTO 0
#define TSB_KERNEL_DIRECT 1  /* CUDA-core direct convolution (any shape, any padding_value) */
#define TSB_KERNEL_TCGEN05 2 /* TMA + tcgen05 kind::i8 implicit GEMM (padding_value 0) */

TSB_API const char *tsb_last_error(void);
TSB_API const char *tsb_status_string(int status);
TSB_API int tsb_version(void);

/* Channel count of the internal NHWC layout for C real channels. */
TSB_API int tsb_padded_channels(int channels);

/*
 * quantize: fp32 -> int8.  Stands in for ts::cpu::Quantize::quantize
 * (src/kernels/cpu/quantize.cpp:69-141; shell src/backend/base/base_quantize.cpp:12-49).
 *   y[i] = clamp_int8(round(x[i] * scales[g(i)])), one fp32 multiply, contiguous tensors of `count` elements.
 *   nscales == 1 : elements i < (count/8)*8 round half-to-even, the tail rounds half-away-from-zero;
 *   nscales  > 1 : group g covers ceil(count/nscales) consecutive elements (fp32 ceil as in the reference),
 *                  all elements round half-away-from-zero.
 * Values whose product is NaN or beyond the int32 range give -128, as the x86 conversion does.
 */
TSB_API int tsb_quantize_f32_i8(const float *x, int8_t *y, int64_t count, const float *scales_host, int nscales,
                        void *stream);

/*
 * quantize without any allocation (this entry point has no counterpart in the reference).
 *
 * For callers that are not allowed to obtain device memory at call time: a serving process that handed the whole
 * GPU to its own arena at start-up and treats any later cudaMalloc as a bug, a latency-critical loop that cannot
 * afford the device-wide synchronisation an allocation or free may imply, or a host that forbids plugins to
 * allocate after initialisation.  tsb_quantize_f32_i8 needs a device-side scale table when it is given more than
 * 64 scales and takes it from a stream-ordered temporary; this variant keeps the table in storage built into the
 * library instead.  Results are bit-identical to tsb_quantize_f32_i8.
 *
 *   - Limit: nscales <= 4096.  More is rejected with TSB_ERR_UNSUPPORTED before anything is launched.
 *   - Cost: the table is a fixed 16 KiB of device memory on every GPU that loads the library, held until exit.
 *   - The first call on each GPU looks up the table's device address (once, then remembered).  Make that first
 *     call ahead of any CUDA stream capture on that GPU.
 *   - All calls on one GPU share the table, and each call overwrites the entries it uses.  Calls whose work may
 *     overlap on the GPU (different streams) therefore race: keep them on one stream or order them with events.
 *   - It calls no cudaMalloc/cudaFree (nor their async forms) and no allocating library routine; x, y and the
 *     host scale list are the caller's.  The host list may be reused as soon as the call returns.
 */
TSB_API int tsb_quantize_f32_i8_static(const float *x, int8_t *y, int64_t count, const float *scales_host,
                                       int nscales, void *stream);

/*
 * The same arithmetic on an NCHW fp32 tensor (rounding positions and scale groups follow the NCHW element
 * index), written in the internal NHWC_PAD layout that the tcgen05 convolution consumes directly.
 */
TSB_API int tsb_quantize_f32_nchw_to_nhwc(const float *x, int8_t *y, int n, int c, int h, int w,
                                  const float *scales_host, int nscales, void *stream);

/* int8 NCHW -> internal NHWC_PAD (used when conv2d_quantized receives an operator-visible int8 tensor). */
TSB_API int tsb_repack_i8_nchw_to_nhwc(const int8_t *x, int8_t *y, int n, int c, int h, int w, void *stream);
/* internal NHWC_PAD -> int8 NCHW (inverse of the above; tests and debugging). */
TSB_API int tsb_repack_i8_nhwc_to_nchw(const int8_t *x, int8_t *y, int n, int c, int h, int w, void *stream);

/*
 * conv2d_quantized.  Stands in for ts::cpu::Conv2DQuantizedCore::conv2d
 * (src/kernels/cpu/quantized/conv2d_quantized_core.cpp:18-147) with the attribute meaning of
 * ts::base::Conv2DQuantized (src/backend/base/base_conv2d_quantized.cpp:13-219): NCHW int8 input,
 * OIHW int8 weights, padding {top,bottom,left,right}, int8(padding_value) in the halo, stride, dilation,
 * output size floor((X + pad - (d*(K-1)+1)) / s + 1) (include/backend/common_function.h:30-40).
 */
typedef struct tsb_conv_desc {
    int n, c, h, w;                                 /* input  [N,C,H,W] */
    int o, kh, kw;                                  /* weight [O,C,KH,KW] */
    int pad_top, pad_bottom, pad_left, pad_right;
    int stride_h, stride_w;
    int dilation_h, dilation_w;
    float padding_value;
    int kernel;                                     /* TSB_KERNEL_* */
} tsb_conv_desc;

/*
 * What happens to the int32 accumulators.  In operator order:
 *   v = float(acc) * dequantize_scales[o]           (conv2d_quantized_core.cpp:80-107)
 *   v = v + bias[o]                 if bias         (add_bias,   src/kernels/cpu/add_bias.cpp:47-85)
 *   v = v + residual[...]           if residual     (add,        fp32, same layout as out_f32)
 *   v = relu(v) | leaky_relu(v)     per activation
 *   out_f32[...] = v                if out_f32
 *   out_i8[...]  = quantize(v)      if out_i8       (the next layer's quantize, rules of tsb_quantize_f32_i8
 *                                                    applied on the NCHW element index)
 * Each step is a separately rounded fp32 operation (no fused multiply-add), so the result has the bits the
 * reference produces by running the operators one after another.
 */
typedef struct tsb_conv_epilogue {
    const float *dequantize_scales; /* [O] device, required */
    const float *bias;              /* [O] device or NULL */
    const float *residual;          /* device or NULL; layout = out_f32_layout */
    int activation;                 /* TSB_ACT_* */
    float leaky_scale;
    float *out_f32;                 /* device or NULL */
    int out_f32_layout;             /* TSB_LAYOUT_NCHW, or TSB_LAYOUT_NHWC_PAD meaning [N][OH][OW][O] (unpadded) */
    int8_t *out_i8;                 /* device or NULL */
    int out_i8_layout;              /* TSB_LAYOUT_NCHW or TSB_LAYOUT_NHWC_PAD */
    const float *requant_scales_host; /* [n_requant_scales] host; 1 scale, or one per sample */
    int n_requant_scales;
    int32_t *out_acc;               /* device or NULL: raw int32 accumulators, NCHW (parity checks) */
    int residual_after_activation;  /* 0: act(conv + bias + residual), a ResNet block's tail;
                                       1: act(conv + bias) + residual, a Darknet shortcut (operators
                                          conv2d_quantized -> add_bias -> leaky_relu -> add) */
} tsb_conv_epilogue;

typedef struct tsb_conv_plan tsb_conv_plan;

TSB_API int tsb_conv2d_i8_plan_create(const tsb_conv_desc *desc, tsb_conv_plan **plan);
TSB_API int tsb_conv2d_i8_plan_destroy(tsb_conv_plan *plan);
/* output extent {N,O,OH,OW} */
TSB_API int tsb_conv2d_i8_output_shape(const tsb_conv_plan *plan, int shape[4]);
/* TSB_KERNEL_DIRECT or TSB_KERNEL_TCGEN05: what the plan resolved to */
TSB_API int tsb_conv2d_i8_kernel(const tsb_conv_plan *plan);
/*
 * One line of text saying how the plan will run (kernel, load mode, MMA orientation, tile shape, tile counts,
 * pipeline stages, shared memory) for its primary configuration and, after " | alt: ", for the configuration of the
 * other orientation when the plan keeps one.  For logs and tests (no counterpart in the reference, whose operators
 * have one code path); returns the length written (without the
 * terminating zero) or a negative status.
 */
TSB_API int tsb_conv2d_i8_plan_describe(const tsb_conv_plan *plan, char *text, size_t text_bytes);
/*
 * Scratch the caller provides to tsb_conv2d_i8_run (256-byte aligned device memory, >= this many bytes):
 * the repacked weights and, for NCHW input, the NHWC_PAD staging of the activations.  The library
 * allocates no device memory itself.
 */
TSB_API size_t tsb_conv2d_i8_workspace_bytes(const tsb_conv_plan *plan);
/*
 * Repack OIHW weights into the plan's workspace.  Weights are constant across runs
 * (src/runtime/program.cpp:91-107), so this runs once per weight tensor; tsb_conv2d_i8_run then only reads.
 */
TSB_API int tsb_conv2d_i8_set_weights(tsb_conv_plan *plan, const int8_t *w_oihw, void *workspace, size_t workspace_bytes,
                              void *stream);
/*
 * quantize (rules of tsb_quantize_f32_i8 on the NCHW element index) an fp32 NCHW input straight into the layout
 * this plan's kernel reads, inside the plan's workspace.  Follow with tsb_conv2d_i8_run(plan, NULL,
 * TSB_LAYOUT_STAGED, ...).  This is the shortest route from an fp32 tensor to the convolution: no int8 NCHW
 * tensor is materialised and no separate repack runs.
 */
TSB_API int tsb_conv2d_i8_quantize_input(tsb_conv_plan *plan, const float *x_f32_nchw, const float *scales_host,
                                         int nscales, void *workspace, size_t workspace_bytes, void *stream);

/*
 * Run one convolution.  x_layout says whether x is operator-visible NCHW int8 or the internal NHWC_PAD
 * tensor written by tsb_quantize_f32_nchw_to_nhwc / a previous run's out_i8.
 */
TSB_API int tsb_conv2d_i8_run(tsb_conv_plan *plan, const int8_t *x, int x_layout, const tsb_conv_epilogue *epilogue,
                      void *workspace, size_t workspace_bytes, void *stream);

/*
 * Reads back the status word the tensor-core kernel keeps in the workspace and synchronises the stream:
 * TSB_OK, or TSB_ERR_DEVICE_TIMEOUT when one of the kernel's bounded waits ran out (the run's outputs are
 * then invalid; the CUDA context stays usable).
 */
TSB_API int tsb_conv2d_i8_status(tsb_conv_plan *plan, void *workspace, void *stream);

/*
 * Host-buffer convenience over the three calls above (what a CPU-resident TenniS tensor goes through):
 * copies x / w / scales / bias from host memory, runs quantize -> conv2d_quantized -> add_bias -> activation,
 * copies the fp32 NCHW result back and synchronises the stream.  `device_scratch` must hold
 * tsb_conv2d_host_scratch_bytes(plan) bytes.
 */
TSB_API size_t tsb_conv2d_host_scratch_bytes(const tsb_conv_plan *plan);
TSB_API int tsb_conv2d_quantized_host(tsb_conv_plan *plan, const float *x_f32_host, const float *quantize_scales_host,
                              int n_quantize_scales, const int8_t *w_host, const float *dequantize_scales_host,
                              const float *bias_host, int activation, float leaky_scale, float *out_f32_host,
                              void *device_scratch, size_t device_scratch_bytes, int weights_resident,
                              void *stream);
/*
 * The same without the final wait: every copy and kernel is enqueued on `stream` and the call returns; the result in
 * `out_f32_host` is valid once the caller has synchronised that stream.  Host buffers should be pinned, otherwise the
 * copies are not asynchronous.  Calls on different streams (each plan with its own scratch) overlap: one layer's
 * upload runs under another's kernels and a third's download.  No counterpart in the reference, whose tensors
 * synchronise on every host view (src/memory/memory_gpu.cpp:106-108).
 */
TSB_API int tsb_conv2d_quantized_host_async(tsb_conv_plan *plan, const float *x_f32_host, const float *quantize_scales_host,
                              int n_quantize_scales, const int8_t *w_host, const float *dequantize_scales_host,
                              const float *bias_host, int activation, float leaky_scale, float *out_f32_host,
                              void *device_scratch, size_t device_scratch_bytes, int weights_resident,
                              void *stream);

/* Standalone fp32 epilogue operators on NCHW tensors (what follows conv2d_quantized when nothing is fused). */
TSB_API int tsb_add_bias_f32_nchw(const float *x, float *y, int n, int c, int hw, const float *bias, void *stream);
TSB_API int tsb_relu_f32(const float *x, float *y, int64_t count, void *stream);
TSB_API int tsb_leaky_relu_f32(const float *x, float *y, int64_t count, float scale, void *stream);

/*
 * The operators around the convolutions of a quantized ResNet-style network, on the convolution path's layouts.
 *  - max pooling (operator "pooling2d", type max; src/kernels/gpu/pooling2d_core.cu) on int8 NHWC_PAD: because
 *    quantize is monotonic, pooling the int8 tensor equals quantizing the pooled fp32 tensor with the same scale;
 *    taps outside the image are ignored (identical to zero padding for post-ReLU inputs);
 *  - global average pooling ("global_pooling2d", type avg) on fp32 [N][pixels][C] -> [N][C];
 *  - inner product ("inner_prod"; the reference calls cuBLAS SGEMM) y[n][o] = sum_k x[n][k] * w[o][k] + bias[o].
 * The two fp32 reductions sum in a fixed order that differs from the CPU reference's, so they agree to rounding
 * (1e-5 relative), not bit for bit.
 */
TSB_API int tsb_maxpool_i8_nhwc(const int8_t *x, int8_t *y, int n, int h, int w, int channels, int k, int stride, int pad,
                                void *stream);
TSB_API int tsb_global_avgpool_f32_nhwc(const float *x, float *y, int n, int pixels, int channels, void *stream);
TSB_API int tsb_inner_prod_f32(const float *x, const float *w, const float *bias, float *y, int n, int k, int o,
                               void *stream);
/*
 * Channel concatenation (operator "concat" on dim 1, src/kernels/gpu/concat.cu) of two int8 NHWC_PAD tensors with the
 * same pixels: y[pixel] = [a's channels_a | b's channels_b | zero padding].  Both inputs must have been quantized with
 * the scale of the consumer, which makes this equal to quantizing the concatenated fp32 tensors.
 */
TSB_API int tsb_concat_i8_nhwc(const int8_t *a, int channels_a, const int8_t *b, int channels_b, int8_t *y, int64_t pixels,
                               void *stream);

/* Debugging aid: while a device buffer of 2048 bytes is set, CTA 0 of each tensor-core convolution launch records a
 * timeline (eight nanosecond stamps per tile for its first 32 tiles) into it.  NULL (the default) switches it off. */
TSB_API int tsb_debug_set_trace_buffer(void *device_buffer);

/* Number of kernels this library has launched on the calling process since load (bench bookkeeping). */
TSB_API int64_t tsb_kernel_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* TENNIS_B200_H */
