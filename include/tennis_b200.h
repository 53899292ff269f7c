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
 * quantize of an fp64 tensor: the FLOAT64 branch of ts::cpu::Quantize::quantize (src/kernels/cpu/quantize.cpp:134 ->
 * the generic cpu_quantize_compute_run<double>, :38-67, with to_int8<double>, :30-36).  The product x[i] * scale is
 * formed in double, rounded half away from zero for EVERY element (this path has no half-to-even vector body), then
 * converted and clamped as above; scale groups as for fp32.
 */
TSB_API int tsb_quantize_f64_i8(const double *x, int8_t *y, int64_t count, const float *scales_host, int nscales,
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
 *     host scale list are the caller's.
 *   - The scale list reaches the table by a copy enqueued on `stream`.  A list in ordinary (pageable) host memory
 *     has been read when the call returns and may be reused at once; a list in pinned or registered host memory
 *     is read later, when the stream gets to the copy, and must stay unchanged until then.
 *   - The remembered table address belongs to the device's current CUDA context: it does not survive a
 *     cudaDeviceReset.
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
    /*
     * Overrides of the plan heuristics, each TSB_TUNE_AUTO (0: the library chooses -- what every caller outside the
     * test-suite passes), TSB_TUNE_OFF or TSB_TUNE_ON.  They change speed only, never results; a mode that the
     * geometry does not admit stays off.  Zero-initialise the descriptor and leave them alone.
     */
    int mma_orientation;                            /* OFF: pixels on the MMA's M side; ON: channels on M (O <= 128) */
    int raw_row_mode;                               /* few-channel layers: one bulk copy of the staged rows per tile */
    int patch_mode;                                 /* stride-1 multi-tap filters: one input patch per tile */
} tsb_conv_desc;

#define TSB_TUNE_AUTO 0
#define TSB_TUNE_OFF 1
#define TSB_TUNE_ON 2

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
    int n_requant_scales;           /* at most TSB_MAX_REQUANT_SCALES: the scales travel as kernel arguments, so a
                                       fused requantize serves batches up to that size; beyond it the call is
                                       rejected with TSB_ERR_UNSUPPORTED and the caller runs tsb_quantize_f32_i8 on
                                       the fp32 output instead */
    int32_t *out_acc;               /* device or NULL: raw int32 accumulators, NCHW (parity checks) */
    int residual_after_activation;  /* 0: act(conv + bias + residual), a ResNet block's tail;
                                       1: act(conv + bias) + residual, a Darknet shortcut (operators
                                          conv2d_quantized -> add_bias -> leaky_relu -> add) */
} tsb_conv_epilogue;

#define TSB_MAX_REQUANT_SCALES 128

typedef struct tsb_conv_plan tsb_conv_plan;

TSB_API int tsb_conv2d_i8_plan_create(const tsb_conv_desc *desc, tsb_conv_plan **plan);
TSB_API int tsb_conv2d_i8_plan_destroy(tsb_conv_plan *plan);
/* output extent {N,O,OH,OW} */
TSB_API int tsb_conv2d_i8_output_shape(const tsb_conv_plan *plan, int shape[4]);
/*
 * TSB_KERNEL_DIRECT or TSB_KERNEL_TCGEN05: what the plan resolved to.  A TSB_KERNEL_AUTO plan takes the CUDA-core
 * kernel only for what the tensor-core kernel cannot express (a non-zero padding_value, filters beyond the tensor
 * map limits); it is many times slower, so a host should check this once per plan and say so in its log --
 * tsb_conv2d_i8_plan_describe gives the reason.
 */
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
 * A residual block's expansion convolution and its projection shortcut in ONE launch.  In a TenniS graph the two are
 *   add( add_bias(dequantize(conv2d_quantized(x, w))), add_bias(dequantize(conv2d_quantized(x_shortcut, w_shortcut))) )
 * followed by the activation (src/kernels/cpu/math_cpu.cpp add; doc/zh_CN/operators.md conv2d_quantized): `shortcut` is
 * the plan of the projection -- a 1x1 convolution of any stride without padding whose output shape equals `plan`'s --
 * and its dequantized (+ shortcut_bias, may be NULL) fp32 result takes the place of epilogue->residual (which must be
 * NULL; residual_after_activation keeps its meaning).  Every fp32 step is rounded separately, as when the projection is
 * run on its own and handed over as a residual tensor, so the results are the same bits; the projection's fp32 output is
 * never written to or read from global memory.  Both inputs are NHWC_PAD int8, 16-byte aligned; the outputs are
 * pixel-major fp32 and / or NHWC_PAD int8 with half-away rounding (one requantize scale or one per image); both plans
 * have had tsb_conv2d_i8_set_weights.  shortcut_dequantize_scales and shortcut_bias are device arrays of O floats.
 * tile_channels: 0 = the library chooses, 128 or 256 = output channels per tile (a tuning override for tests).
 * Returns TSB_ERR_UNSUPPORTED for anything else; the caller then runs the two convolutions one after the other.
 */
TSB_API int tsb_conv2d_i8_run_projected(tsb_conv_plan *plan, const int8_t *x, tsb_conv_plan *shortcut,
                                        const int8_t *x_shortcut, const float *shortcut_dequantize_scales,
                                        const float *shortcut_bias, const tsb_conv_epilogue *epilogue, int tile_channels,
                                        void *workspace, size_t workspace_bytes, void *stream);
/*
 * A convolution over the channel concatenation of two int8 tensors without materialising the concatenation
 * (`concat` followed by `conv2d_quantized` in a graph: the transition of a cross-stage-partial block).  The weight tensor
 * [O][C_first + C_rest][KH][KW] is split along its channel axis into two plans: `first` (a 1x1 convolution of any stride
 * without padding over x_first, the leading C_first channels) and `plan` (over x, the remaining channels; its epilogue,
 * dequantize scales and bias are those of the whole convolution).  Both parts sum into one int32 accumulator -- int32
 * sums are exact in any order -- so the result is bit-identical to concatenating first.  Both inputs must have been
 * quantized with the same scales (as a concatenated tensor would have been).  Layout rules, tile_channels and the
 * TSB_ERR_UNSUPPORTED fallback are those of tsb_conv2d_i8_run_projected; epilogue->residual must be NULL.
 */
TSB_API int tsb_conv2d_i8_run_concat(tsb_conv_plan *plan, const int8_t *x, tsb_conv_plan *first, const int8_t *x_first,
                                     const tsb_conv_epilogue *epilogue, int tile_channels, void *workspace,
                                     size_t workspace_bytes, void *stream);

/*
 * Failure detection.  Every wait inside the tensor-core kernel is bounded; a wait that runs out makes the kernel
 * write a code (1..6, which wait) into the status word at the start of the workspace, release what it holds and
 * return, so the CUDA context stays usable but that run's outputs are invalid.
 *  - tsb_conv2d_i8_status: copies the word back, synchronises the stream and returns TSB_OK or
 *    TSB_ERR_DEVICE_TIMEOUT (tsb_last_error names the wait); a reported time-out is cleared again.
 *  - tsb_conv2d_i8_status_async: only enqueues the 4-byte copy into `status_word_host` (pinned memory) on the
 *    stream -- no wait; the caller looks at the word once the stream has passed that point (an event, or its next
 *    synchronisation) and turns it into a status and message with tsb_conv2d_i8_status_decode.  This is how the
 *  - tsb_conv2d_i8_set_status_word: the kernels of this plan report into `*device_visible_word` instead of the
 *    workspace's first word (NULL: back to the workspace).  The word must be writable by the device for as long as the
 *    plan runs: device memory, or -- what the TenniS operator does -- the device pointer of MAPPED pinned host memory
 *    (cudaHostAlloc with cudaHostAllocMapped): nothing is written to it unless a wait gives up, and the host reads it as
 *    plain memory, so checking costs neither a copy nor an event per run.  The caller zeroes the word before the first
 *    run and after reporting a time-out; tsb_conv2d_i8_status / _status_async keep reading the workspace word.
 * tsb_conv2d_quantized_host (the waiting form) checks the word itself.
 */
TSB_API int tsb_conv2d_i8_status(tsb_conv_plan *plan, void *workspace, void *stream);
TSB_API int tsb_conv2d_i8_set_status_word(tsb_conv_plan *plan, int *device_visible_word);
TSB_API int tsb_conv2d_i8_status_async(tsb_conv_plan *plan, void *workspace, int *status_word_host, void *stream);
TSB_API int tsb_conv2d_i8_status_decode(int status_word);

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
 *  - max pooling (operator "pooling2d", type max; src/kernels/gpu/pooling2d_core.cu, src/kernels/cpu/pooling2d_core.cpp:47-93)
 *    on int8 NHWC_PAD: because quantize is monotonic, pooling the int8 tensor equals quantizing the pooled fp32 tensor
 *    with the same scale.  The output extent is the reference's: tsb_pool_out_dim = ceil((x + pad_lo + pad_hi - k) /
 *    float(stride) + 1) (include/backend/common_function.h:13-20) -- CEIL, unlike the convolution's floor -- and every
 *    window is clipped to the image, so padding never takes part in the maximum.  (A ResNet stem pool written for
 *    floor semantics, 112 -> 56 with k 3, stride 2, reaches TenniS as padding {top 1, bottom 0, left 1, right 0}.)
 *    Geometries in which a whole window falls into the padding are rejected: the reference's value there is whatever
 *    lies at the clamped start index;
 *  - global average pooling ("global_pooling2d", type avg) on fp32 [N][pixels][C] -> [N][C];
 *  - inner product ("inner_prod"; the reference calls cuBLAS SGEMM) y[n][o] = sum_k x[n][k] * w[o][k] + bias[o].
 * The two fp32 reductions sum in a fixed order that differs from the CPU reference's, so they agree to rounding
 * (1e-5 relative), not bit for bit.
 */
TSB_API int tsb_pool_out_dim(int x, int pad_lo, int pad_hi, int k, int stride);
TSB_API int tsb_maxpool_i8_nhwc(const int8_t *x, int8_t *y, int n, int h, int w, int channels, int k, int stride, int pad_top,
                                int pad_bottom, int pad_left, int pad_right, void *stream);
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

#ifdef TSB_ENABLE_TRACE
/* Profiling builds only (compile the library with -DTSB_ENABLE_TRACE; release builds carry neither this symbol nor the
 * stamps): while a device buffer of 2048 bytes is set, CTA 0 of each tensor-core convolution launch records a
 * timeline (eight nanosecond stamps per tile for its first 32 tiles) into it.  NULL switches it off. */
TSB_API int tsb_debug_set_trace_buffer(void *device_buffer);
#endif

/* Number of kernels this library has launched on the calling process since load (bench bookkeeping). */
TSB_API int64_t tsb_kernel_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* TENNIS_B200_H */
