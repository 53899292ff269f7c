// Data shared by the two convolution kernels: the problem geometry and the epilogue description as the
// kernels see them, and the element-wise epilogue that turns one int32 accumulator into its outputs.
#pragma once

#include "common.cuh"

namespace tsb {

constexpr int kMaxRequantScales = TSB_MAX_REQUANT_SCALES;

struct ConvGeom {
    int N, C, H, W;
    int O, KH, KW;
    int OH, OW;
    int pad_t, pad_l;
    int sh, sw, dh, dw;
    int Cp;             // channels of the NHWC_PAD input
    int pad_value;      // int8(padding_value)
};

struct EpiParams {
    const float *dq;
    const float *bias;
    const float *residual;
    float *out_f32;
    int8_t *out_i8;
    int32_t *out_acc;
    int activation;
    float leaky;
    int res_after;      // the residual is added after the activation instead of before it
    int f32_nhwc;       // out_f32 / residual are [N][P][O] instead of NCHW
    int i8_nhwc;        // out_i8 is NHWC_PAD with out_cp channels
    int out_cp;
    int O, P;           // output channels, OH*OW
    // requantize
    uint32_t rne_limit;
    uint32_t group_len;
    int nscales;
    float rq_scales[kMaxRequantScales];
};

#ifdef __CUDACC__
// One output element (image n, channel o, pixel p) with the residual value handed in.
__device__ __forceinline__ void epilogue_store_value(const EpiParams &e, int n, int o, int p, int acc, float res, bool has_res) {
    const uint32_t nchw = (uint32_t)(n * e.O + o) * (uint32_t)e.P + (uint32_t)p;
    const uint32_t nhwc = (uint32_t)(n * e.P + p) * (uint32_t)e.O + (uint32_t)o;
    if (e.out_acc) e.out_acc[nchw] = acc;
    if (!e.out_f32 && !e.out_i8) return;
    EpilogueMath math{e.activation, e.leaky};
    const uint32_t fidx = e.f32_nhwc ? nhwc : nchw;
    const float v = math(acc, e.dq[o], e.bias ? e.bias[o] : 0.0f, e.bias != nullptr, res, has_res, e.res_after != 0);
    if (e.out_f32) e.out_f32[fidx] = v;
    if (e.out_i8) {
        const uint32_t g = e.nscales == 1 ? 0u : nchw / e.group_len;
        if (g < (uint32_t)e.nscales) {
            const int q = q8(v, e.rq_scales[g], nchw < e.rne_limit);
            const size_t qidx = e.i8_nhwc ? (size_t)(n * e.P + p) * e.out_cp + o : (size_t)nchw;
            e.out_i8[qidx] = (int8_t)q;
        }
    }
}
// One output element (image n, channel o, pixel p); the residual, if any, read from e.residual.
__device__ __forceinline__ void epilogue_store_one(const EpiParams &e, int n, int o, int p, int acc) {
    const uint32_t fidx = e.f32_nhwc ? (uint32_t)(n * e.P + p) * (uint32_t)e.O + (uint32_t)o : (uint32_t)(n * e.O + o) * (uint32_t)e.P + (uint32_t)p;
    epilogue_store_value(e, n, o, p, acc, e.residual ? e.residual[fidx] : 0.0f, e.residual != nullptr);
}
#endif

struct tsb_conv_plan_impl;

// conv_direct.cu
int launch_conv_direct(const ConvGeom &g, const int8_t *x, int x_nhwc, const int8_t *w_oihw, const EpiParams &epi,
                       cudaStream_t stream);

}  // namespace tsb
