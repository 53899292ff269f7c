// extern "C" entry points of libtennis_b200.so (declared in include/tennis_b200.h) and the convolution plan.
#include "common.cuh"
#include "conv_common.cuh"
#include "conv_tc.h"

#include <cstdlib>
#include <cstring>
#include <new>

namespace tsb {

std::string &last_error() {
    static thread_local std::string e;
    return e;
}
std::atomic<int64_t> g_launches{0};

// quantize.cu
int quantize_f32_i8(const float *, int8_t *, int64_t, const float *, int, cudaStream_t);
int quantize_f64_i8(const double *, int8_t *, int64_t, const float *, int, cudaStream_t);
int quantize_f32_i8_static(const float *, int8_t *, int64_t, const float *, int, cudaStream_t);
int quantize_f32_nchw_to_nhwc(const float *, int8_t *, int, int, int, int, const float *, int, cudaStream_t);
int quantize_stage(const float *, int8_t *, int, int, int, int, int, int, int, int, const float *, int, cudaStream_t);
int repack_i8_nchw_to_nhwc(const int8_t *, int8_t *, int, int, int, int, cudaStream_t);
int repack_i8_nhwc_to_nchw(const int8_t *, int8_t *, int, int, int, int, cudaStream_t);
int add_bias_f32_nchw(const float *, float *, int, int, int, const float *, cudaStream_t);
int activation_f32(const float *, float *, int64_t, int, float, cudaStream_t);
// netops.cu
int pool_out_dim(int, int, int, int, int);
int maxpool_i8_nhwc(const int8_t *, int8_t *, int, int, int, int, int, int, int, int, int, int, cudaStream_t);
int global_avgpool_f32_nhwc(const float *, float *, int, int, int, cudaStream_t);
int inner_prod_f32(const float *, const float *, const float *, float *, int, int, int, cudaStream_t);
int concat_i8_nhwc(const int8_t *, int, const int8_t *, int, int8_t *, int64_t, cudaStream_t);

namespace {

size_t align256(size_t v) { return (v + 255) & ~size_t(255); }

}  // namespace
}  // namespace tsb

struct tsb_conv_plan {
    tsb_conv_desc desc;
    tsb::ConvGeom geom;
    int kernel;                      // resolved TSB_KERNEL_*
    tsb::tc::Tuning tune;            // heuristic overrides taken from the descriptor
    const char *why_not_tc;
    tsb::tc::View view;
    tsb::tc::Config cfg;             // configuration with all shared memory given to the pipeline
    tsb::tc::Config cfg_alt;         // the other orientation (alt_valid): taken when the epilogue is pixel-major fp32 and no
    int alt_valid;                   // staged configuration fits
    tsb::tc::Config cfg_stg[3];      // [1], [2]: configurations that set shared memory aside for the staged epilogue
    int stg_valid[3];
    int *status_word = nullptr;      // where the kernels report a wait that gave up, when not the workspace's first word
    size_t off_weights, off_stage, ws_bytes;
    // state bound by set_weights / run
    const int8_t *weights_oihw;      // direct kernel reads the caller's tensor
    const void *weights_ws;          // workspace the packed weights live in
    CUtensorMap map_b, map_b_alt, map_b_stg[3];
    const int8_t *map_a_ptr, *map_a_alt_ptr, *map_a_stg_ptr[3];
    CUtensorMap map_a, map_a_alt, map_a_stg[3];
    // tsb_conv2d_i8_run_projected: configuration and tensor maps of the last pair, reused while the four pointers, the
    // shortcut plan and the tile override stay the same
    struct {
        const void *x = nullptr, *x2 = nullptr, *w = nullptr, *w2 = nullptr;
        const tsb_conv_plan *shortcut = nullptr;
        tsb_conv_desc shortcut_desc;            // (a later plan at the same address may describe another convolution)
        int tile = -1;
        tsb::tc::Config cfg;
        CUtensorMap map_a, map_b, map_a2, map_b2;
    } pair;
};

using namespace tsb;

extern "C" {

const char *tsb_last_error(void) { return last_error().c_str(); }

const char *tsb_status_string(int status) {
    switch (status) {
        case TSB_OK: return "ok";
        case TSB_ERR_INVALID_ARGUMENT: return "invalid argument";
        case TSB_ERR_UNSUPPORTED: return "unsupported";
        case TSB_ERR_WORKSPACE_TOO_SMALL: return "workspace too small";
        case TSB_ERR_DEVICE_TIMEOUT: return "a device-side wait ran out";
        default: return status > 0 ? cudaGetErrorString((cudaError_t)status) : "unknown status";
    }
}

int tsb_version(void) { return 100; }

int tsb_padded_channels(int channels) {
    if (channels <= 16) return 16;
    return round_up(channels, 64);
}

int64_t tsb_kernel_launch_count(void) { return g_launches.load(); }

#ifdef TSB_ENABLE_TRACE
int tsb_debug_set_trace_buffer(void *device_buffer) {
    tc::set_trace_buffer(static_cast<unsigned long long *>(device_buffer));
    return TSB_OK;
}
#endif

int tsb_quantize_f32_i8(const float *x, int8_t *y, int64_t count, const float *scales_host, int nscales, void *stream) {
    return quantize_f32_i8(x, y, count, scales_host, nscales, (cudaStream_t)stream);
}
int tsb_quantize_f64_i8(const double *x, int8_t *y, int64_t count, const float *scales_host, int nscales, void *stream) {
    return quantize_f64_i8(x, y, count, scales_host, nscales, (cudaStream_t)stream);
}
int tsb_quantize_f32_i8_static(const float *x, int8_t *y, int64_t count, const float *scales_host, int nscales,
                               void *stream) {
    return quantize_f32_i8_static(x, y, count, scales_host, nscales, (cudaStream_t)stream);
}
int tsb_quantize_f32_nchw_to_nhwc(const float *x, int8_t *y, int n, int c, int h, int w, const float *scales_host,
                                  int nscales, void *stream) {
    return quantize_f32_nchw_to_nhwc(x, y, n, c, h, w, scales_host, nscales, (cudaStream_t)stream);
}
int tsb_repack_i8_nchw_to_nhwc(const int8_t *x, int8_t *y, int n, int c, int h, int w, void *stream) {
    return repack_i8_nchw_to_nhwc(x, y, n, c, h, w, (cudaStream_t)stream);
}
int tsb_repack_i8_nhwc_to_nchw(const int8_t *x, int8_t *y, int n, int c, int h, int w, void *stream) {
    return repack_i8_nhwc_to_nchw(x, y, n, c, h, w, (cudaStream_t)stream);
}
int tsb_add_bias_f32_nchw(const float *x, float *y, int n, int c, int hw, const float *bias, void *stream) {
    return add_bias_f32_nchw(x, y, n, c, hw, bias, (cudaStream_t)stream);
}
int tsb_relu_f32(const float *x, float *y, int64_t count, void *stream) {
    return activation_f32(x, y, count, TSB_ACT_RELU, 0.0f, (cudaStream_t)stream);
}
int tsb_leaky_relu_f32(const float *x, float *y, int64_t count, float scale, void *stream) {
    return activation_f32(x, y, count, TSB_ACT_LEAKY_RELU, scale, (cudaStream_t)stream);
}

int tsb_pool_out_dim(int x, int pad_lo, int pad_hi, int k, int stride) {
    if (x < 1 || k < 1 || stride < 1 || pad_lo < 0 || pad_hi < 0) return fail(TSB_ERR_INVALID_ARGUMENT, "pool_out_dim: bad geometry");
    return pool_out_dim(x, pad_lo, pad_hi, k, stride);
}
int tsb_maxpool_i8_nhwc(const int8_t *x, int8_t *y, int n, int h, int w, int channels, int k, int stride, int pad_top,
                        int pad_bottom, int pad_left, int pad_right, void *stream) {
    return maxpool_i8_nhwc(x, y, n, h, w, channels, k, stride, pad_top, pad_bottom, pad_left, pad_right, (cudaStream_t)stream);
}
int tsb_global_avgpool_f32_nhwc(const float *x, float *y, int n, int pixels, int channels, void *stream) {
    return global_avgpool_f32_nhwc(x, y, n, pixels, channels, (cudaStream_t)stream);
}
int tsb_inner_prod_f32(const float *x, const float *w, const float *bias, float *y, int n, int k, int o, void *stream) {
    return inner_prod_f32(x, w, bias, y, n, k, o, (cudaStream_t)stream);
}
int tsb_concat_i8_nhwc(const int8_t *a, int channels_a, const int8_t *b, int channels_b, int8_t *y, int64_t pixels, void *stream) {
    return concat_i8_nhwc(a, channels_a, b, channels_b, y, pixels, (cudaStream_t)stream);
}

int tsb_conv2d_i8_plan_create(const tsb_conv_desc *d, tsb_conv_plan **out) {
    if (!d || !out) return fail(TSB_ERR_INVALID_ARGUMENT, "plan_create: null pointer");
    *out = nullptr;
    if (d->n < 1 || d->c < 1 || d->h < 1 || d->w < 1 || d->o < 1 || d->kh < 1 || d->kw < 1)
        return fail(TSB_ERR_INVALID_ARGUMENT, "plan_create: bad extents x=[%d,%d,%d,%d] w=[%d,%d,%d,%d]", d->n, d->c, d->h,
                    d->w, d->o, d->c, d->kh, d->kw);
    if (d->stride_h < 1 || d->stride_w < 1 || d->dilation_h < 1 || d->dilation_w < 1)
        return fail(TSB_ERR_INVALID_ARGUMENT, "plan_create: stride and dilation must be positive");
    if (d->pad_top < 0 || d->pad_bottom < 0 || d->pad_left < 0 || d->pad_right < 0)
        return fail(TSB_ERR_INVALID_ARGUMENT, "plan_create: negative padding");
    if (d->kernel < TSB_KERNEL_AUTO || d->kernel > TSB_KERNEL_TCGEN05)
        return fail(TSB_ERR_INVALID_ARGUMENT, "plan_create: unknown kernel selector %d", d->kernel);
    if (d->mma_orientation < 0 || d->mma_orientation > 2 || d->raw_row_mode < 0 || d->raw_row_mode > 2 || d->patch_mode < 0 ||
        d->patch_mode > 2)
        return fail(TSB_ERR_INVALID_ARGUMENT, "plan_create: mma_orientation, raw_row_mode and patch_mode take TSB_TUNE_AUTO, _OFF or _ON");
    const int OH = conv_out_dim(d->h, d->pad_top, d->pad_bottom, d->kh, d->stride_h, d->dilation_h);
    const int OW = conv_out_dim(d->w, d->pad_left, d->pad_right, d->kw, d->stride_w, d->dilation_w);
    if (OH < 1 || OW < 1 || d->h + d->pad_top + d->pad_bottom < d->dilation_h * (d->kh - 1) + 1 ||
        d->w + d->pad_left + d->pad_right < d->dilation_w * (d->kw - 1) + 1)
        return fail(TSB_ERR_INVALID_ARGUMENT, "plan_create: the filter does not fit the padded input");
    if ((int64_t)d->n * d->o * OH * OW > INT32_MAX || (int64_t)d->n * tsb_padded_channels(d->c) * d->h * d->w > INT32_MAX)
        return fail(TSB_ERR_UNSUPPORTED, "plan_create: tensors beyond 2^31 elements (TenniS counts are 32-bit)");

    tsb_conv_plan *p = new (std::nothrow) tsb_conv_plan();
    if (!p) return fail(TSB_ERR_INVALID_ARGUMENT, "plan_create: out of host memory");
    p->desc = *d;
    ConvGeom &g = p->geom;
    g.N = d->n; g.C = d->c; g.H = d->h; g.W = d->w;
    g.O = d->o; g.KH = d->kh; g.KW = d->kw;
    g.OH = OH; g.OW = OW;
    g.pad_t = d->pad_top; g.pad_l = d->pad_left;
    g.sh = d->stride_h; g.sw = d->stride_w; g.dh = d->dilation_h; g.dw = d->dilation_w;
    g.Cp = tsb_padded_channels(d->c);
    g.pad_value = (int)(int8_t)d->padding_value;  // T(padding_value) of the reference's im2col call
    p->why_not_tc = "";
    p->tune.orientation = d->mma_orientation;
    p->tune.rows = d->raw_row_mode;
    p->tune.patch = d->patch_mode;
    const bool tc_ok = tc::make_view(g, p->tune, &p->view, &p->why_not_tc);
    if (d->kernel == TSB_KERNEL_TCGEN05 && !tc_ok) {
        int st = fail(TSB_ERR_UNSUPPORTED, "plan_create: tcgen05 kernel not available: %s", p->why_not_tc);
        delete p;
        return st;
    }
    p->kernel = (d->kernel == TSB_KERNEL_DIRECT || !tc_ok) ? TSB_KERNEL_DIRECT : TSB_KERNEL_TCGEN05;
    p->off_weights = 256;
    size_t end = 256;
    if (p->kernel == TSB_KERNEL_TCGEN05) {
        int sms = 148, dev = 0;
        if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (sms <= 0) sms = 148;
        p->cfg = tc::choose_config(p->view, p->tune, sms, -1);
        p->cfg_alt = tc::choose_config(p->view, p->tune, sms, p->cfg.swap ? 0 : 1);
        // a forced orientation is final: the run-time choice by epilogue is only made between the library's own two plans
        p->alt_valid = p->cfg_alt.swap != p->cfg.swap && p->tune.orientation == 0;
        for (int level = 1; level <= 2; ++level) {
            p->cfg_stg[level] = tc::choose_config(p->view, p->tune, sms, -1, level);
            const tc::Config &c = p->cfg_stg[level];
            p->stg_valid[level] = c.staging == level && c.stages >= 2 && c.dyn_smem <= 227u * 1024u && (!p->view.rows || c.b_resident);
            p->map_a_stg_ptr[level] = nullptr;
        }
        end = p->off_weights + align256(p->view.weight_bytes);
    }
    p->off_stage = end;
    // NHWC_PAD staging of an operator-visible NCHW input (either kernel can read NHWC_PAD; only the tensor-core
    // kernel needs it)
    if (p->kernel == TSB_KERNEL_TCGEN05) end += align256(p->view.stage_bytes);
    else end += align256((size_t)g.N * g.C * g.H * g.W);
    p->ws_bytes = end;
    p->weights_oihw = nullptr;
    p->weights_ws = nullptr;
    p->map_a_ptr = nullptr;
    p->map_a_alt_ptr = nullptr;
    if (p->kernel != TSB_KERNEL_TCGEN05) p->stg_valid[1] = p->stg_valid[2] = 0;
    *out = p;
    return TSB_OK;
}

int tsb_conv2d_i8_plan_destroy(tsb_conv_plan *plan) {
    delete plan;
    return TSB_OK;
}

int tsb_conv2d_i8_output_shape(const tsb_conv_plan *plan, int shape[4]) {
    if (!plan || !shape) return fail(TSB_ERR_INVALID_ARGUMENT, "output_shape: null pointer");
    shape[0] = plan->geom.N; shape[1] = plan->geom.O; shape[2] = plan->geom.OH; shape[3] = plan->geom.OW;
    return TSB_OK;
}

int tsb_conv2d_i8_kernel(const tsb_conv_plan *plan) { return plan ? plan->kernel : TSB_ERR_INVALID_ARGUMENT; }

int tsb_conv2d_i8_plan_describe(const tsb_conv_plan *plan, char *text, size_t text_bytes) {
    if (!plan || !text || text_bytes < 2) return fail(TSB_ERR_INVALID_ARGUMENT, "plan_describe: null pointer");
    auto one = [&](const tc::Config &c, char *dst, size_t n) {
        const char *mode = c.patch ? "patch" : (plan->view.rows ? "rows" : (plan->view.a_tiled ? "tiled" : (plan->view.fold ? "fold" : "im2col")));
        return snprintf(dst, n, "mode=%s swap=%d bn=%d bk=%d pix=%d tiles=%dx%d grid=%d stages=%d kgroup=%d resident=%d smem=%u", mode, c.swap,
                        c.bn, c.bk, c.pix, c.num_m_tiles, c.num_n_tiles, c.grid, c.stages, c.kgroup, c.b_resident, c.dyn_smem);
    };
    int len;
    if (plan->kernel != TSB_KERNEL_TCGEN05) {
        len = snprintf(text, text_bytes, "kernel=direct (%s)", plan->why_not_tc);
    } else {
        len = snprintf(text, text_bytes, "kernel=tcgen05 ");
        if (plan->view.fold && len > 0 && (size_t)len < text_bytes) len += snprintf(text + len, text_bytes - len, "cpix=%d ", plan->view.cpix);
        if (len > 0 && (size_t)len < text_bytes) len += one(plan->cfg, text + len, text_bytes - len);
        if (plan->alt_valid && len > 0 && (size_t)len < text_bytes) {
            len += snprintf(text + len, text_bytes - len, " | alt: ");
            if ((size_t)len < text_bytes) len += one(plan->cfg_alt, text + len, text_bytes - len);
        }
        for (int level = 1; level <= 2; ++level)
            if (plan->stg_valid[level] && len > 0 && (size_t)len < text_bytes) {
                len += snprintf(text + len, text_bytes - len, " | staged%d: ", level);
                if ((size_t)len < text_bytes) len += one(plan->cfg_stg[level], text + len, text_bytes - len);
            }
    }
    if (len < 0) return fail(TSB_ERR_INVALID_ARGUMENT, "plan_describe: formatting failed");
    return (size_t)len < text_bytes ? len : (int)text_bytes - 1;
}

size_t tsb_conv2d_i8_workspace_bytes(const tsb_conv_plan *plan) { return plan ? plan->ws_bytes : 0; }

int tsb_conv2d_i8_set_weights(tsb_conv_plan *plan, const int8_t *w_oihw, void *workspace, size_t workspace_bytes,
                              void *stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    if (!plan || !w_oihw || !workspace) return fail(TSB_ERR_INVALID_ARGUMENT, "set_weights: null pointer");
    if (workspace_bytes < plan->ws_bytes) return fail(TSB_ERR_WORKSPACE_TOO_SMALL, "set_weights: workspace %zu < %zu", workspace_bytes, plan->ws_bytes);
    if (reinterpret_cast<uintptr_t>(workspace) % 256) return fail(TSB_ERR_INVALID_ARGUMENT, "set_weights: workspace must be 256-byte aligned");
    TSB_CUDA(cudaMemsetAsync(workspace, 0, 256, stream));  // status word
    plan->weights_oihw = w_oihw;
    plan->weights_ws = workspace;
    if (plan->kernel == TSB_KERNEL_TCGEN05) {
        int8_t *wp = static_cast<int8_t *>(workspace) + plan->off_weights;
        int st0 = tc::pack_weights(plan->view, w_oihw, wp, stream);
        if (st0 != TSB_OK) return st0;
        int st = tc::encode_weight_map(plan->view, plan->cfg, wp, &plan->map_b);
        if (st != TSB_OK) return st;
        if (plan->alt_valid) {
            st = tc::encode_weight_map(plan->view, plan->cfg_alt, wp, &plan->map_b_alt);
            if (st != TSB_OK) return st;
        }
        for (int level = 1; level <= 2; ++level)
            if (plan->stg_valid[level]) {
                st = tc::encode_weight_map(plan->view, plan->cfg_stg[level], wp, &plan->map_b_stg[level]);
                if (st != TSB_OK) return st;
            }
    }
    return TSB_OK;
}

static int build_epilogue(const tsb_conv_plan *plan, const tsb_conv_epilogue *e, EpiParams *out) {
    const ConvGeom &g = plan->geom;
    if (!e->dequantize_scales) return fail(TSB_ERR_INVALID_ARGUMENT, "run: dequantize_scales is required");
    if (!e->out_f32 && !e->out_i8 && !e->out_acc) return fail(TSB_ERR_INVALID_ARGUMENT, "run: no output requested");
    if (e->activation < TSB_ACT_NONE || e->activation > TSB_ACT_LEAKY_RELU) return fail(TSB_ERR_INVALID_ARGUMENT, "run: unknown activation %d", e->activation);
    if (e->out_f32_layout != TSB_LAYOUT_NCHW && e->out_f32_layout != TSB_LAYOUT_NHWC_PAD) return fail(TSB_ERR_INVALID_ARGUMENT, "run: unknown out_f32_layout");
    if (e->out_i8_layout != TSB_LAYOUT_NCHW && e->out_i8_layout != TSB_LAYOUT_NHWC_PAD) return fail(TSB_ERR_INVALID_ARGUMENT, "run: unknown out_i8_layout");
    EpiParams &p = *out;
    p.dq = e->dequantize_scales;
    p.bias = e->bias;
    p.residual = e->residual;
    p.out_f32 = e->out_f32;
    p.out_i8 = e->out_i8;
    p.out_acc = e->out_acc;
    p.activation = e->activation;
    p.leaky = e->leaky_scale;
    p.res_after = (e->residual && e->residual_after_activation) ? 1 : 0;
    p.f32_nhwc = e->out_f32_layout == TSB_LAYOUT_NHWC_PAD;
    p.i8_nhwc = e->out_i8_layout == TSB_LAYOUT_NHWC_PAD;
    p.out_cp = tsb_padded_channels(g.O);
    p.O = g.O;
    p.P = g.OH * g.OW;
    p.rne_limit = 0; p.group_len = 1; p.nscales = 1;
    p.rq_scales[0] = 1.0f;
    if (e->out_i8) {
        if (!e->requant_scales_host || e->n_requant_scales < 1) return fail(TSB_ERR_INVALID_ARGUMENT, "run: out_i8 needs requantize scales");
        if (e->n_requant_scales > kMaxRequantScales) return fail(TSB_ERR_UNSUPPORTED, "run: at most %d requantize scales", kMaxRequantScales);
        if (p.i8_nhwc && reinterpret_cast<uintptr_t>(e->out_i8) % 16) return fail(TSB_ERR_INVALID_ARGUMENT, "run: NHWC out_i8 must be 16-byte aligned");
        QuantRule r = make_quant_rule((int64_t)g.N * g.O * g.OH * g.OW, e->n_requant_scales);
        p.rne_limit = (uint32_t)r.rne_limit;
        p.group_len = (uint32_t)r.group_len;
        p.nscales = r.nscales;
        for (int i = 0; i < e->n_requant_scales; ++i) p.rq_scales[i] = e->requant_scales_host[i];
    }
    return TSB_OK;
}

int tsb_conv2d_i8_quantize_input(tsb_conv_plan *plan, const float *x_f32_nchw, const float *scales_host, int nscales,
                                 void *workspace, size_t workspace_bytes, void *stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    if (!plan || !x_f32_nchw || !workspace) return fail(TSB_ERR_INVALID_ARGUMENT, "quantize_input: null pointer");
    if (workspace_bytes < plan->ws_bytes) return fail(TSB_ERR_WORKSPACE_TOO_SMALL, "quantize_input: workspace %zu < %zu", workspace_bytes, plan->ws_bytes);
    if (reinterpret_cast<uintptr_t>(workspace) % 256) return fail(TSB_ERR_INVALID_ARGUMENT, "quantize_input: workspace must be 256-byte aligned");
    const ConvGeom &g = plan->geom;
    int8_t *stage = static_cast<int8_t *>(workspace) + plan->off_stage;
    if (plan->kernel == TSB_KERNEL_TCGEN05 && plan->view.fold)
        return quantize_stage(x_f32_nchw, stage, g.N, g.C, g.H, g.W, 1, plan->view.Wp, plan->view.cpix, g.pad_l, scales_host, nscales, stream);
    if (plan->kernel == TSB_KERNEL_TCGEN05)
        return quantize_stage(x_f32_nchw, stage, g.N, g.C, g.H, g.W, 0, 0, 0, 0, scales_host, nscales, stream);
    return quantize_f32_i8(x_f32_nchw, stage, (int64_t)g.N * g.C * g.H * g.W, scales_host, nscales, stream);  // direct kernel: NCHW
}

int tsb_conv2d_i8_run(tsb_conv_plan *plan, const int8_t *x, int x_layout, const tsb_conv_epilogue *epilogue,
                      void *workspace, size_t workspace_bytes, void *stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    if (!plan || !epilogue || !workspace) return fail(TSB_ERR_INVALID_ARGUMENT, "run: null pointer");
    if (x_layout != TSB_LAYOUT_NCHW && x_layout != TSB_LAYOUT_NHWC_PAD && x_layout != TSB_LAYOUT_STAGED) return fail(TSB_ERR_INVALID_ARGUMENT, "run: unknown x_layout %d", x_layout);
    if (!x && x_layout != TSB_LAYOUT_STAGED) return fail(TSB_ERR_INVALID_ARGUMENT, "run: null input");
    if (workspace_bytes < plan->ws_bytes) return fail(TSB_ERR_WORKSPACE_TOO_SMALL, "run: workspace %zu < %zu", workspace_bytes, plan->ws_bytes);
    if (plan->weights_ws != workspace || !plan->weights_oihw) return fail(TSB_ERR_INVALID_ARGUMENT, "run: tsb_conv2d_i8_set_weights was not called with this workspace");
    EpiParams epi;
    int st = build_epilogue(plan, epilogue, &epi);
    if (st != TSB_OK) return st;
    const ConvGeom &g = plan->geom;
    int8_t *stage = static_cast<int8_t *>(workspace) + plan->off_stage;
    if (plan->kernel == TSB_KERNEL_DIRECT) {
        if (x_layout == TSB_LAYOUT_STAGED) return launch_conv_direct(g, stage, 0, plan->weights_oihw, epi, stream);
        return launch_conv_direct(g, x, x_layout == TSB_LAYOUT_NHWC_PAD, plan->weights_oihw, epi, stream);
    }

    const int8_t *x_tc = x;
    if (x_layout == TSB_LAYOUT_STAGED) {
        x_tc = stage;
    } else if (plan->view.fold) {
        st = tc::stage_folded(plan->view, x, x_layout == TSB_LAYOUT_NHWC_PAD, stage, stream);
        if (st != TSB_OK) return st;
        x_tc = stage;
    } else if (x_layout == TSB_LAYOUT_NCHW) {
        st = repack_i8_nchw_to_nhwc(x, stage, g.N, g.C, g.H, g.W, stream);
        if (st != TSB_OK) return st;
        x_tc = stage;
    }
    // Outputs that can go through shared-memory tiles and tensor-map stores (int8 NHWC_PAD, pixel-major fp32 with or
    // without a residual) take the configuration that sets the tiles' shared memory aside.
    const int level = tc::staging_level(plan->view, epi);
    if (level != 0 && plan->stg_valid[level]) {
        if (plan->map_a_stg_ptr[level] != x_tc) {
            st = tc::encode_activation_map(plan->view, plan->cfg_stg[level], x_tc, &plan->map_a_stg[level]);
            if (st != TSB_OK) return st;
            plan->map_a_stg_ptr[level] = x_tc;
        }
        return tc::launch_conv_tc(plan->view, plan->cfg_stg[level], plan->map_a_stg[level], plan->map_b_stg[level], x_tc, epi,
                                  plan->status_word ? plan->status_word : static_cast<int *>(workspace), stream);
    }
    // Otherwise pixel-major fp32 tensors (a network's residuals and block outputs) are stored coalesced when a thread owns
    // a channel, i.e. in the swapped orientation; everything else follows the geometry heuristic.
    const bool want_swap = (epi.out_f32 || epi.residual) && epi.f32_nhwc && !epi.out_acc;
    // (the swapped patch-mode kernel has no fast path for pixel-major fp32 tensors)
    const bool use_alt = plan->alt_valid && (want_swap != (plan->cfg.swap != 0)) && (want_swap ? plan->cfg_alt.swap : 0) &&
                         !plan->cfg_alt.patch;
    if (use_alt) {
        if (plan->map_a_alt_ptr != x_tc) {
            st = tc::encode_activation_map(plan->view, plan->cfg_alt, x_tc, &plan->map_a_alt);
            if (st != TSB_OK) return st;
            plan->map_a_alt_ptr = x_tc;
        }
        return tc::launch_conv_tc(plan->view, plan->cfg_alt, plan->map_a_alt, plan->map_b_alt, x_tc, epi, plan->status_word ? plan->status_word : static_cast<int *>(workspace), stream);
    }
    if (plan->map_a_ptr != x_tc) {
        st = tc::encode_activation_map(plan->view, plan->cfg, x_tc, &plan->map_a);
        if (st != TSB_OK) return st;
        plan->map_a_ptr = x_tc;
    }
    return tc::launch_conv_tc(plan->view, plan->cfg, plan->map_a, plan->map_b, x_tc, epi, plan->status_word ? plan->status_word : static_cast<int *>(workspace), stream);
}

// Two convolutions in one launch (conv_tc.cu, DUAL instances).  concat == false: `shortcut` is a projection whose dequantized
// (+ bias) result is the residual of `plan`.  concat == true: `shortcut` convolves the leading channels of a concatenated
// input and `plan` the rest; both sum into one accumulator.
static int run_pair(tsb_conv_plan *plan, const int8_t *x, tsb_conv_plan *shortcut, const int8_t *x_shortcut,
                    const float *shortcut_dequantize_scales, const float *shortcut_bias, const tsb_conv_epilogue *epilogue,
                    int tile_channels, void *workspace, size_t workspace_bytes, void *stream_, bool concat) {
    cudaStream_t stream = (cudaStream_t)stream_;
    if (!plan || !shortcut || !x || !x_shortcut || (!concat && !shortcut_dequantize_scales) || !epilogue || !workspace)
        return fail(TSB_ERR_INVALID_ARGUMENT, "run_projected: null pointer");
    if (workspace_bytes < plan->ws_bytes) return fail(TSB_ERR_WORKSPACE_TOO_SMALL, "run_projected: workspace %zu < %zu", workspace_bytes, plan->ws_bytes);
    if (plan->weights_ws != workspace || !plan->weights_oihw || !shortcut->weights_ws || !shortcut->weights_oihw)
        return fail(TSB_ERR_INVALID_ARGUMENT, "run_projected: tsb_conv2d_i8_set_weights was not called on both plans");
    if (tile_channels != 0 && tile_channels != 128 && tile_channels != 256) return fail(TSB_ERR_INVALID_ARGUMENT, "run_projected: tile_channels takes 0, 128 or 256");
    if (plan->kernel != TSB_KERNEL_TCGEN05 || shortcut->kernel != TSB_KERNEL_TCGEN05)
        return fail(TSB_ERR_UNSUPPORTED, "run_projected: both convolutions must run on the tcgen05 kernel");
    if (epilogue->residual) return fail(TSB_ERR_INVALID_ARGUMENT, "run_projected: the projection is the residual; epilogue->residual must be null");
    const char *why = "";
    if (!tc::dual_supported(plan->view, shortcut->view, &why)) return fail(TSB_ERR_UNSUPPORTED, "run_projected: %s", why);
    if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(x_shortcut)) % 16) return fail(TSB_ERR_INVALID_ARGUMENT, "run_projected: inputs must be 16-byte aligned");
    EpiParams epi;
    int st = build_epilogue(plan, epilogue, &epi);
    if (st != TSB_OK) return st;
    epi.res_after = (!concat && epilogue->residual_after_activation) ? 1 : 0;
    int sms = 148, dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms <= 0) sms = 148;
    const int8_t *wp = static_cast<const int8_t *>(workspace) + plan->off_weights;
    const int8_t *wp2 = static_cast<const int8_t *>(shortcut->weights_ws) + shortcut->off_weights;
    auto &pr = plan->pair;
    const int tile_key = tile_channels + (concat ? 1000 : 0);      // the two modes never share a configuration
    if (pr.x != x || pr.x2 != x_shortcut || pr.w != wp || pr.w2 != wp2 || pr.shortcut != shortcut || pr.tile != tile_key ||
        memcmp(&pr.shortcut_desc, &shortcut->desc, sizeof(tsb_conv_desc)) != 0) {
        pr.x = nullptr;     // invalid until every map is encoded
        pr.cfg = tc::choose_config_dual(plan->view, shortcut->view, sms, tile_channels, concat);
        if (pr.cfg.stages < 2 || pr.cfg.dyn_smem > 227u * 1024u) return fail(TSB_ERR_UNSUPPORTED, "run_projected: the pair does not fit shared memory");
        if ((st = tc::encode_activation_map(plan->view, pr.cfg, x, &pr.map_a)) != TSB_OK) return st;
        if ((st = tc::encode_weight_map(plan->view, pr.cfg, wp, &pr.map_b)) != TSB_OK) return st;
        if ((st = tc::encode_activation_map(shortcut->view, pr.cfg, x_shortcut, &pr.map_a2)) != TSB_OK) return st;
        if ((st = tc::encode_weight_map(shortcut->view, pr.cfg, wp2, &pr.map_b2)) != TSB_OK) return st;
        pr.x = x; pr.x2 = x_shortcut; pr.w = wp; pr.w2 = wp2; pr.shortcut = shortcut; pr.tile = tile_key;
        pr.shortcut_desc = shortcut->desc;
    }
    tc::DualArgs dual;
    dual.view = &shortcut->view;
    dual.map_a = pr.map_a2;
    dual.map_b = pr.map_b2;
    dual.dq = concat ? nullptr : shortcut_dequantize_scales;
    dual.bias = concat ? nullptr : shortcut_bias;
    return tc::launch_conv_tc(plan->view, pr.cfg, pr.map_a, pr.map_b, x, epi, plan->status_word ? plan->status_word : static_cast<int *>(workspace), stream, &dual);
}

int tsb_conv2d_i8_run_projected(tsb_conv_plan *plan, const int8_t *x, tsb_conv_plan *shortcut, const int8_t *x_shortcut,
                                const float *shortcut_dequantize_scales, const float *shortcut_bias,
                                const tsb_conv_epilogue *epilogue, int tile_channels, void *workspace, size_t workspace_bytes,
                                void *stream) {
    return run_pair(plan, x, shortcut, x_shortcut, shortcut_dequantize_scales, shortcut_bias, epilogue, tile_channels, workspace,
                    workspace_bytes, stream, false);
}

int tsb_conv2d_i8_run_concat(tsb_conv_plan *plan, const int8_t *x, tsb_conv_plan *first, const int8_t *x_first,
                             const tsb_conv_epilogue *epilogue, int tile_channels, void *workspace, size_t workspace_bytes,
                             void *stream) {
    return run_pair(plan, x, first, x_first, nullptr, nullptr, epilogue, tile_channels, workspace, workspace_bytes, stream, true);
}

// what each code of the status word means (the kernel's bounded waits, conv_tc.cu)
static const char *wait_name(int code) {
    switch (code) {
        case 1: return "producer: pipeline stage free";
        case 2: return "MMA issuer: accumulator buffer free";
        case 3: return "MMA issuer: tile loaded";
        case 4: return "epilogue: accumulator ready";
        case 5: return "producer: resident weight tile free";
        case 6: return "MMA issuer: resident weight tile loaded";
        case 7: return "epilogue: staged residual tile loaded";
        default: return "unknown wait";
    }
}

// Reads the status word (after everything enqueued on the stream) and, when a wait ran out, clears it again so that
// one reported time-out does not stick to later runs.
static int read_status(void *workspace, cudaStream_t stream, const char *who) {
    int word = 0;
    TSB_CUDA(cudaMemcpyAsync(&word, workspace, sizeof(int), cudaMemcpyDeviceToHost, stream));
    TSB_CUDA(cudaStreamSynchronize(stream));
    if (word == 0) return TSB_OK;
    TSB_CUDA(cudaMemsetAsync(workspace, 0, sizeof(int), stream));
    return fail(TSB_ERR_DEVICE_TIMEOUT, "%s: conv kernel gave up on bounded wait %d (%s); the outputs of that run are invalid", who, word,
                wait_name(word));
}

int tsb_conv2d_i8_status(tsb_conv_plan *plan, void *workspace, void *stream_) {
    if (!plan || !workspace) return fail(TSB_ERR_INVALID_ARGUMENT, "status: null pointer");
    return read_status(workspace, (cudaStream_t)stream_, "status");
}

int tsb_conv2d_i8_status_async(tsb_conv_plan *plan, void *workspace, int *status_word_host, void *stream_) {
    if (!plan || !workspace || !status_word_host) return fail(TSB_ERR_INVALID_ARGUMENT, "status_async: null pointer");
    TSB_CUDA(cudaMemcpyAsync(status_word_host, workspace, sizeof(int), cudaMemcpyDeviceToHost, (cudaStream_t)stream_));
    return TSB_OK;
}

int tsb_conv2d_i8_set_status_word(tsb_conv_plan *plan, int *device_visible_word) {
    if (!plan) return fail(TSB_ERR_INVALID_ARGUMENT, "set_status_word: null plan");
    plan->status_word = device_visible_word;
    return TSB_OK;
}

int tsb_conv2d_i8_status_decode(int status_word) {
    if (status_word == 0) return TSB_OK;
    return fail(TSB_ERR_DEVICE_TIMEOUT, "conv kernel gave up on bounded wait %d (%s); the outputs of that run are invalid", status_word,
                wait_name(status_word));
}

// ---- host-buffer convenience --------------------------------------------------------------------------
namespace {
struct HostScratch {
    size_t x_f32, w, dq, bias, out, ws, total;
};
HostScratch host_layout(const tsb_conv_plan *p) {
    const ConvGeom &g = p->geom;
    HostScratch s;
    size_t off = 0;
    s.x_f32 = off; off += align256((size_t)g.N * g.C * g.H * g.W * 4);
    s.w = off;     off += align256((size_t)g.O * g.C * g.KH * g.KW);
    s.dq = off;    off += align256((size_t)g.O * 4);
    s.bias = off;  off += align256((size_t)g.O * 4);
    s.out = off;   off += align256((size_t)g.N * g.O * g.OH * g.OW * 4);
    s.ws = off;    off += align256(p->ws_bytes);
    s.total = off;
    return s;
}
}  // namespace

size_t tsb_conv2d_host_scratch_bytes(const tsb_conv_plan *plan) { return plan ? host_layout(plan).total : 0; }

static int conv2d_quantized_host(tsb_conv_plan *plan, const float *x_host, const float *qscales_host, int nq,
                                 const int8_t *w_host, const float *dq_host, const float *bias_host, int activation,
                                 float leaky, float *out_host, void *scratch, size_t scratch_bytes, int weights_resident,
                                 cudaStream_t stream, bool wait) {
    if (!plan || !x_host || !qscales_host || !out_host || !scratch) return fail(TSB_ERR_INVALID_ARGUMENT, "conv2d_quantized_host: null pointer");
    if (!weights_resident && (!w_host || !dq_host)) return fail(TSB_ERR_INVALID_ARGUMENT, "conv2d_quantized_host: weights and dequantize scales are required");
    const HostScratch L = host_layout(plan);
    if (scratch_bytes < L.total) return fail(TSB_ERR_WORKSPACE_TOO_SMALL, "conv2d_quantized_host: scratch %zu < %zu", scratch_bytes, L.total);
    if (reinterpret_cast<uintptr_t>(scratch) % 256) return fail(TSB_ERR_INVALID_ARGUMENT, "conv2d_quantized_host: scratch must be 256-byte aligned");
    const ConvGeom &g = plan->geom;
    if (nq != g.N) return fail(TSB_ERR_INVALID_ARGUMENT, "conv2d_quantized_host: %d quantize scales for batch %d (one per sample, base_quantize.cpp:26)", nq, g.N);
    char *base = static_cast<char *>(scratch);
    float *d_x = reinterpret_cast<float *>(base + L.x_f32);
    int8_t *d_w = reinterpret_cast<int8_t *>(base + L.w);
    float *d_dq = reinterpret_cast<float *>(base + L.dq);
    float *d_bias = reinterpret_cast<float *>(base + L.bias);
    float *d_out = reinterpret_cast<float *>(base + L.out);
    void *ws = base + L.ws;
    TSB_CUDA(cudaMemcpyAsync(d_x, x_host, (size_t)g.N * g.C * g.H * g.W * 4, cudaMemcpyHostToDevice, stream));
    int st;
    if (!weights_resident) {
        TSB_CUDA(cudaMemcpyAsync(d_w, w_host, (size_t)g.O * g.C * g.KH * g.KW, cudaMemcpyHostToDevice, stream));
        TSB_CUDA(cudaMemcpyAsync(d_dq, dq_host, (size_t)g.O * 4, cudaMemcpyHostToDevice, stream));
        if (bias_host) TSB_CUDA(cudaMemcpyAsync(d_bias, bias_host, (size_t)g.O * 4, cudaMemcpyHostToDevice, stream));
        st = tsb_conv2d_i8_set_weights(plan, d_w, ws, plan->ws_bytes, stream);
        if (st != TSB_OK) return st;
    }
    st = tsb_conv2d_i8_quantize_input(plan, d_x, qscales_host, nq, ws, plan->ws_bytes, stream);
    if (st != TSB_OK) return st;
    tsb_conv_epilogue e;
    std::memset(&e, 0, sizeof(e));
    e.dequantize_scales = d_dq;
    e.bias = bias_host ? d_bias : nullptr;
    e.activation = activation;
    e.leaky_scale = leaky;
    e.out_f32 = d_out;
    e.out_f32_layout = TSB_LAYOUT_NCHW;
    st = tsb_conv2d_i8_run(plan, nullptr, TSB_LAYOUT_STAGED, &e, ws, plan->ws_bytes, stream);
    if (st != TSB_OK) return st;
    TSB_CUDA(cudaMemcpyAsync(out_host, d_out, (size_t)g.N * g.O * g.OH * g.OW * 4, cudaMemcpyDeviceToHost, stream));
    // the waiting form also reports a kernel that gave up on one of its bounded waits (the non-waiting form cannot:
    // its caller asks tsb_conv2d_i8_status after synchronising)
    if (wait && plan->kernel == TSB_KERNEL_TCGEN05) return read_status(ws, stream, "conv2d_quantized_host");
    if (wait) TSB_CUDA(cudaStreamSynchronize(stream));
    return TSB_OK;
}

int tsb_conv2d_quantized_host(tsb_conv_plan *plan, const float *x_host, const float *qscales_host, int nq,
                              const int8_t *w_host, const float *dq_host, const float *bias_host, int activation,
                              float leaky, float *out_host, void *scratch, size_t scratch_bytes, int weights_resident,
                              void *stream) {
    return conv2d_quantized_host(plan, x_host, qscales_host, nq, w_host, dq_host, bias_host, activation, leaky, out_host,
                                 scratch, scratch_bytes, weights_resident, (cudaStream_t)stream, true);
}

int tsb_conv2d_quantized_host_async(tsb_conv_plan *plan, const float *x_host, const float *qscales_host, int nq,
                                    const int8_t *w_host, const float *dq_host, const float *bias_host, int activation,
                                    float leaky, float *out_host, void *scratch, size_t scratch_bytes,
                                    int weights_resident, void *stream) {
    return conv2d_quantized_host(plan, x_host, qscales_host, nq, w_host, dq_host, bias_host, activation, leaky, out_host,
                                 scratch, scratch_bytes, weights_resident, (cudaStream_t)stream, false);
}

}  // extern "C"
