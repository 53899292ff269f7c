// Direct int8 convolution on CUDA cores.  It takes every geometry the operator accepts (any padding, a
// non-zero padding_value, tiny channel counts, any alignment) and is the kernel behind plans that the
// tcgen05 implicit-GEMM kernel does not cover.  One thread owns one output pixel and kOT output channels;
// the weights of those channels are staged through shared memory in channel chunks.
#include "conv_common.cuh"

namespace tsb {
namespace {

constexpr int kPix = 128;  // threads per block = output pixels per block
constexpr int kOT = 8;     // output channels per block
constexpr int kWeightSmem = 32 * 1024;

__global__ void __launch_bounds__(kPix)
conv_direct_kernel(ConvGeom g, const int8_t *__restrict__ x, int x_nhwc, const int8_t *__restrict__ w,
                   const __grid_constant__ EpiParams epi, int chunk_c) {
    extern __shared__ int8_t wsm[];  // [kOT][chunk_c*KH*KW]
    const int n = blockIdx.z;
    const int o0 = blockIdx.y * kOT;
    const int p = blockIdx.x * kPix + threadIdx.x;
    const int P = g.OH * g.OW;
    const bool live = p < P;
    const int oh = live ? p / g.OW : 0, ow = live ? p % g.OW : 0;
    const int taps = g.KH * g.KW;
    const int ih0 = oh * g.sh - g.pad_t, iw0 = ow * g.sw - g.pad_l;
    int acc[kOT];
#pragma unroll
    for (int j = 0; j < kOT; ++j) acc[j] = 0;

    for (int c0 = 0; c0 < g.C; c0 += chunk_c) {
        const int cc = min(chunk_c, g.C - c0);
        const int per_o = cc * taps;
        __syncthreads();
        for (int i = threadIdx.x; i < kOT * per_o; i += kPix) {
            const int j = i / per_o, r = i - j * per_o;
            wsm[i] = (o0 + j < g.O) ? w[((size_t)(o0 + j) * g.C + c0) * taps + r] : (int8_t)0;
        }
        __syncthreads();
        if (!live) continue;
        for (int c = 0; c < cc; ++c) {
            for (int kh = 0; kh < g.KH; ++kh) {
                const int ih = ih0 + kh * g.dh;
                const bool row_ok = (unsigned)ih < (unsigned)g.H;
                for (int kw = 0; kw < g.KW; ++kw) {
                    const int iw = iw0 + kw * g.dw;
                    int xv = g.pad_value;
                    if (row_ok && (unsigned)iw < (unsigned)g.W) {
                        const size_t xi = x_nhwc ? ((size_t)(n * g.H + ih) * g.W + iw) * g.Cp + (c0 + c)
                                                 : ((size_t)(n * g.C + c0 + c) * g.H + ih) * g.W + iw;
                        xv = x[xi];
                    }
                    const int wi = (c * g.KH + kh) * g.KW + kw;
#pragma unroll
                    for (int j = 0; j < kOT; ++j) acc[j] += xv * (int)wsm[j * per_o + wi];
                }
            }
        }
    }
    if (!live) return;
#pragma unroll
    for (int j = 0; j < kOT; ++j)
        if (o0 + j < g.O) epilogue_store_one(epi, n, o0 + j, p, acc[j]);
    // padding channels of an NHWC_PAD int8 output stay zero so the next layer can consume it as is
    if (epi.out_i8 && epi.i8_nhwc && blockIdx.y == gridDim.y - 1)
        for (int o = g.O; o < epi.out_cp; ++o) epi.out_i8[(size_t)(n * P + p) * epi.out_cp + o] = 0;
}

}  // namespace

int launch_conv_direct(const ConvGeom &g, const int8_t *x, int x_nhwc, const int8_t *w_oihw, const EpiParams &epi,
                       cudaStream_t stream) {
    const int taps = g.KH * g.KW;
    int chunk_c = kWeightSmem / (kOT * taps);
    if (chunk_c < 1) return fail(TSB_ERR_UNSUPPORTED, "conv direct: a %dx%d filter does not fit the weight tile", g.KH, g.KW);
    if (chunk_c > g.C) chunk_c = g.C;
    if (g.N > 65535 || ceil_div(g.O, kOT) > 65535) return fail(TSB_ERR_UNSUPPORTED, "conv direct: grid too large");
    dim3 grid(ceil_div(g.OH * g.OW, kPix), ceil_div(g.O, kOT), g.N);
    const size_t smem = (size_t)kOT * chunk_c * taps;
    conv_direct_kernel<<<grid, kPix, smem, stream>>>(g, x, x_nhwc, w_oihw, epi, chunk_c);
    TSB_LAUNCHED("conv_direct_kernel");
    return TSB_OK;
}

}  // namespace tsb
