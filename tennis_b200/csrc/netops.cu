// The non-convolution operators a quantized ResNet-style network needs between and after its convolutions,
// on the layouts the convolution path keeps activations in.  All are memory-bound byte / float movers.
//   pooling2d (max)       src/kernels/gpu/pooling2d_core.cu, src/backend/base/base_pooling2d.cpp
//   global_pooling2d (avg) src/kernels/gpu/global_pooling2d.cu
//   inner_prod             src/kernels/gpu/inner_prod.cu (cuBLAS SGEMM in the reference)
#include "common.cuh"

#include <algorithm>
#include <cmath>

namespace tsb {
namespace {

constexpr int kThreads = 256;

// int8 NHWC_PAD max pooling; a window is clipped to the image, as the reference's kernels clip it
// (src/kernels/cpu/pooling2d_core.cpp:47-93, src/kernels/gpu/pooling2d_core.cu), so taps in the padding never count.
// quantize is monotonic, so pooling the int8 tensor gives exactly quantize(pool(x)) for the same scale.  One thread
// produces 16 channels of one output pixel.  KFIX > 0: a KFIX x KFIX window as straight-line code -- every tap is loaded
// (from a clamped address when it lies outside the image, and replaced by -128 afterwards), so all the loads of a thread
// are in flight together; KFIX = 0: any window, taps outside the image skipped.
template <int KFIX>
__global__ void __launch_bounds__(kThreads)
maxpool_i8_nhwc_kernel(const int8_t *__restrict__ x, int8_t *__restrict__ y, int N, int H, int W, int Cp, int OH, int OW,
                       int K, int S, int pad_t, int pad_l) {
    pdl_sync();
    // (the host checks that the tensors have fewer than 2^31 16-byte units: 32-bit index arithmetic, no 64-bit divisions)
    const uint32_t units = (uint32_t)Cp / 16u;
    const uint32_t total = (uint32_t)N * (uint32_t)OH * (uint32_t)OW * units;
    for (uint32_t i = blockIdx.x * kThreads + threadIdx.x; i < total; i += gridDim.x * kThreads) {
        const int u = (int)(i % units);
        const uint32_t pix = i / units;
        const uint32_t prow = pix / (uint32_t)OW;
        const int ow = (int)(pix - prow * (uint32_t)OW), n = (int)(prow / (uint32_t)OH), oh = (int)(prow - (uint32_t)n * (uint32_t)OH);
        // four int8 lanes per 32-bit word, compared with the per-byte signed maximum
        uint32_t w4[4] = {0x80808080u, 0x80808080u, 0x80808080u, 0x80808080u};
        if (KFIX > 0) {
            const int8_t *img = x + (size_t)n * H * W * Cp + u * 16;
            constexpr int kTaps = KFIX > 0 ? KFIX * KFIX : 1;
            int4 v[kTaps];
            bool ok[kTaps];
#pragma unroll
            for (int kh = 0; kh < KFIX; ++kh) {
                const int ih = oh * S - pad_t + kh;
                const int ihc = min(max(ih, 0), H - 1);
#pragma unroll
                for (int kw = 0; kw < KFIX; ++kw) {
                    const int iw = ow * S - pad_l + kw;
                    const int iwc = min(max(iw, 0), W - 1);
                    ok[kh * KFIX + kw] = ih == ihc && iw == iwc;
                    v[kh * KFIX + kw] = __ldg(reinterpret_cast<const int4 *>(img + ((uint32_t)ihc * (uint32_t)W + (uint32_t)iwc) * (uint32_t)Cp));
                }
            }
#pragma unroll
            for (int t = 0; t < KFIX * KFIX; ++t) {
                if (!ok[t]) v[t] = make_int4((int)0x80808080u, (int)0x80808080u, (int)0x80808080u, (int)0x80808080u);
                w4[0] = __vmaxs4(w4[0], (uint32_t)v[t].x);
                w4[1] = __vmaxs4(w4[1], (uint32_t)v[t].y);
                w4[2] = __vmaxs4(w4[2], (uint32_t)v[t].z);
                w4[3] = __vmaxs4(w4[3], (uint32_t)v[t].w);
            }
        } else
        for (int kh = 0; kh < K; ++kh) {
            const int ih = oh * S - pad_t + kh;
            if ((unsigned)ih >= (unsigned)H) continue;
            const int8_t *row = x + (((int64_t)n * H + ih) * W) * Cp + u * 16;
#pragma unroll 3
            for (int kw = 0; kw < K; ++kw) {
                const int iw = ow * S - pad_l + kw;
                if ((unsigned)iw >= (unsigned)W) continue;
                const int4 v = __ldg(reinterpret_cast<const int4 *>(row + (int64_t)iw * Cp));
                w4[0] = __vmaxs4(w4[0], (uint32_t)v.x);
                w4[1] = __vmaxs4(w4[1], (uint32_t)v.y);
                w4[2] = __vmaxs4(w4[2], (uint32_t)v.z);
                w4[3] = __vmaxs4(w4[3], (uint32_t)v.w);
            }
        }
        *reinterpret_cast<int4 *>(y + (size_t)pix * Cp + u * 16) = make_int4(w4[0], w4[1], w4[2], w4[3]);
    }
}

// fp32 [N][P][C] -> [N][C]: sum over the P pixels in index order, one multiply by 1/P... no: divided by P as the
// reference's average pooling does (sum / count).
__global__ void __launch_bounds__(kThreads)
global_avgpool_f32_nhwc_kernel(const float *__restrict__ x, float *__restrict__ y, int N, int P, int C) {
    pdl_sync();
    const int64_t total = (int64_t)N * C;
    for (int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x; i < total; i += (int64_t)gridDim.x * kThreads) {
        const int c = (int)(i % C), n = (int)(i / C);
        // eight loads in flight, added in pixel order (the sum is a plain left-to-right fp32 sum)
        const float *col = x + (int64_t)n * P * C + c;
        float s = 0.0f;
        for (int p0 = 0; p0 < P; p0 += 8) {
            float v[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = p0 + j < P ? __ldg(col + (int64_t)(p0 + j) * C) : 0.0f;
#pragma unroll
            for (int j = 0; j < 8; ++j)
                if (p0 + j < P) s = __fadd_rn(s, v[j]);
        }
        y[i] = __fdiv_rn(s, (float)P);
    }
}

// y[n][o] = sum_k x[n][k] * w[o][k] + bias[o].  A warp owns a block of kIpN images x kIpO outputs: per step of 32 k's it
// loads kIpN + kIpO values and does kIpN * kIpO multiply-adds, so every loaded value is used several times.  Each output
// is summed in a fixed order (lane l of K slice s takes its k's in sequence, then a butterfly over the lanes, then the
// slices in order), whatever the block shape.
constexpr int kIpN = 4, kIpO = 8;
// VEC = 4: every lane reads four consecutive k per step as one 16-byte load (rows 16-byte aligned, K a multiple of 4)
constexpr int kIpKS = 2;     // warps that share one block of outputs, each on every kIpKS-th step along K
template <int VEC>
__global__ void __launch_bounds__(kThreads)
inner_prod_f32_kernel(const float *__restrict__ x, const float *__restrict__ w, const float *__restrict__ bias,
                      float *__restrict__ y, int N, int K, int O) {
    static_assert(kIpN * kIpO == 32, "the final sum gives one output to every lane");
    __shared__ float part[kThreads / 32][kIpN * kIpO];
    pdl_sync();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int slots = kThreads / 32 / kIpKS;              // output blocks a thread block works on at a time
    const int slot = warp / kIpKS, ks = warp % kIpKS;
    const int n_blocks = (N + kIpN - 1) / kIpN, o_blocks = (O + kIpO - 1) / kIpO;
    const int64_t total = (int64_t)n_blocks * o_blocks;
    const int64_t per_round = (int64_t)gridDim.x * slots;
    for (int64_t base = 0; base < total; base += per_round) {     // the same number of rounds for every thread (barriers inside)
        const int64_t i = base + (int64_t)blockIdx.x * slots + slot;
        const bool active = i < total;
        // neighbouring warps (of one block) take the same rows of w and different rows of x: w comes from HBM once
        const int ob = active ? (int)(i / n_blocks) : 0, nb = active ? (int)(i % n_blocks) : 0;
        if (active) {
            const float *xr[kIpN];
            const float *wr[kIpO];
#pragma unroll
            for (int a = 0; a < kIpN; ++a) xr[a] = x + (int64_t)min(nb * kIpN + a, N - 1) * K;   // clamped: extra rows are not stored
#pragma unroll
            for (int b = 0; b < kIpO; ++b) wr[b] = w + (int64_t)min(ob * kIpO + b, O - 1) * K;
            float s[kIpN][kIpO];
#pragma unroll
            for (int a = 0; a < kIpN; ++a)
#pragma unroll
                for (int b = 0; b < kIpO; ++b) s[a][b] = 0.0f;
            if (VEC == 4) {
                for (int k = (ks * 32 + lane) * 4; k < K; k += 128 * kIpKS) {
                    float4 xv[kIpN], wv[kIpO];
#pragma unroll
                    for (int a = 0; a < kIpN; ++a) xv[a] = __ldg(reinterpret_cast<const float4 *>(xr[a] + k));
#pragma unroll
                    for (int b = 0; b < kIpO; ++b) wv[b] = __ldg(reinterpret_cast<const float4 *>(wr[b] + k));
#pragma unroll
                    for (int a = 0; a < kIpN; ++a)
#pragma unroll
                        for (int b = 0; b < kIpO; ++b) {
                            float t = s[a][b];
                            t = fmaf(xv[a].x, wv[b].x, t);
                            t = fmaf(xv[a].y, wv[b].y, t);
                            t = fmaf(xv[a].z, wv[b].z, t);
                            t = fmaf(xv[a].w, wv[b].w, t);
                            s[a][b] = t;
                        }
                }
            } else {
                for (int k = ks * 32 + lane; k < K; k += 32 * kIpKS) {
                    float xv[kIpN], wv[kIpO];
#pragma unroll
                    for (int a = 0; a < kIpN; ++a) xv[a] = __ldg(xr[a] + k);
#pragma unroll
                    for (int b = 0; b < kIpO; ++b) wv[b] = __ldg(wr[b] + k);
#pragma unroll
                    for (int a = 0; a < kIpN; ++a)
#pragma unroll
                        for (int b = 0; b < kIpO; ++b) s[a][b] = fmaf(xv[a], wv[b], s[a][b]);
                }
            }
#pragma unroll
            for (int a = 0; a < kIpN; ++a)
#pragma unroll
                for (int b = 0; b < kIpO; ++b) {
                    float t = s[a][b];
#pragma unroll
                    for (int off = 16; off > 0; off >>= 1) t += __shfl_xor_sync(0xffffffffu, t, off);
                    if (lane == 0) part[warp][a * kIpO + b] = t;
                }
        }
        __syncthreads();
        if (active && ks == 0) {
            // lane l adds the K slices of output (l / kIpO, l % kIpO) in a fixed order
            float t = part[warp][lane];
#pragma unroll
            for (int q = 1; q < kIpKS; ++q) t += part[warp + q][lane];
            const int n = nb * kIpN + lane / kIpO, o = ob * kIpO + lane % kIpO;
            if (n < N && o < O) y[(int64_t)n * O + o] = bias ? t + bias[o] : t;
        }
        __syncthreads();
    }
}

// y[pixel] = [a[pixel][0..ca) | b[pixel][0..cb) | zeros up to cy]; ca_p, cb_p, cy are the padded channel counts
__global__ void __launch_bounds__(kThreads)
concat_i8_nhwc_kernel(const int8_t *__restrict__ a, int ca, int ca_p, const int8_t *__restrict__ b, int cb, int cb_p,
                      int8_t *__restrict__ y, int cy, int64_t pixels, int vec) {
    pdl_sync();
    if (vec) {   // ca and cb are multiples of 16: whole 16-byte units
        const int units = cy / 16, ua = ca / 16, ub = cb / 16;
        const int64_t total = pixels * units;
        for (int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x; i < total; i += (int64_t)gridDim.x * kThreads) {
            const int u = (int)(i % units);
            const int64_t px = i / units;
            int4 v = make_int4(0, 0, 0, 0);
            if (u < ua) v = __ldg(reinterpret_cast<const int4 *>(a + px * ca_p) + u);
            else if (u < ua + ub) v = __ldg(reinterpret_cast<const int4 *>(b + px * cb_p) + (u - ua));
            reinterpret_cast<int4 *>(y + px * cy)[u] = v;
        }
    } else {
        const int64_t total = pixels * cy;
        for (int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x; i < total; i += (int64_t)gridDim.x * kThreads) {
            const int c = (int)(i % cy);
            const int64_t px = i / cy;
            int8_t v = 0;
            if (c < ca) v = a[px * ca_p + c];
            else if (c < ca + cb) v = b[px * cb_p + (c - ca)];
            y[i] = v;
        }
    }
}

int grid_for(int64_t items, int per_block) {
    int64_t blocks = (items + per_block - 1) / per_block;
    if (blocks < 1) blocks = 1;
    return (int)(blocks < 148 * 16 ? blocks : 148 * 16);
}

}  // namespace

// Output extent of the reference's pooling2d: ceil((x + pad_lo + pad_hi - k) / float(stride) + 1), evaluated in fp32
// (include/backend/common_function.h:13-20, src/runtime/inferer/factory.cpp:221-223).
int pool_out_dim(int x, int pad_lo, int pad_hi, int k, int stride) {
    return (int)std::ceil((float)(x + pad_lo + pad_hi - k) / (float)stride + 1.0f);
}

int maxpool_i8_nhwc(const int8_t *x, int8_t *y, int n, int h, int w, int channels, int k, int stride, int pad_top,
                    int pad_bottom, int pad_left, int pad_right, cudaStream_t stream) {
    if (!x || !y) return fail(TSB_ERR_INVALID_ARGUMENT, "maxpool: null pointer");
    if (n < 1 || h < 1 || w < 1 || channels < 1 || k < 1 || stride < 1 || pad_top < 0 || pad_bottom < 0 || pad_left < 0 ||
        pad_right < 0)
        return fail(TSB_ERR_INVALID_ARGUMENT, "maxpool: bad geometry");
    const int cp = tsb_padded_channels(channels);
    const int oh = pool_out_dim(h, pad_top, pad_bottom, k, stride), ow = pool_out_dim(w, pad_left, pad_right, k, stride);
    if (oh < 1 || ow < 1) return fail(TSB_ERR_INVALID_ARGUMENT, "maxpool: empty output");
    // Every window must meet the image.  Where the ceil-mode extent adds a window that starts at or beyond the image
    // edge (or ends before it), the reference reads whatever lies at the clamped start index -- the next channel
    // plane or memory past the tensor -- which no layout-independent kernel can reproduce.
    if ((oh - 1) * stride - pad_top >= h || (ow - 1) * stride - pad_left >= w || k - pad_top < 1 || k - pad_left < 1)
        return fail(TSB_ERR_UNSUPPORTED, "maxpool: a pooling window lies entirely in the padding (the reference's result there is undefined)");
    if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) % 16) return fail(TSB_ERR_INVALID_ARGUMENT, "maxpool: tensors must be 16-byte aligned");
    const int64_t items = (int64_t)n * oh * ow * (cp / 16);
    if (items >= (int64_t)1 << 31 || (int64_t)n * h * w * (cp / 16) >= (int64_t)1 << 31) return fail(TSB_ERR_UNSUPPORTED, "maxpool: tensor too large");
    auto kernel = k == 3 ? maxpool_i8_nhwc_kernel<3> : (k == 2 ? maxpool_i8_nhwc_kernel<2> : maxpool_i8_nhwc_kernel<0>);
    // one item per thread (up to 148 x 64 blocks): the block scheduler evens out what a grid-stride loop of 1.3 rounds would not
    const int blocks = (int)std::min<int64_t>((items + kThreads - 1) / kThreads, 148 * 64);
    TSB_CUDA(launch_pdl(kernel, dim3(blocks), dim3(kThreads), 0, stream, x, y, n, h, w, cp, oh, ow, k, stride,
                        pad_top, pad_left));
    TSB_LAUNCHED("maxpool_i8_nhwc_kernel");
    return TSB_OK;
}

int global_avgpool_f32_nhwc(const float *x, float *y, int n, int pixels, int channels, cudaStream_t stream) {
    if (!x || !y) return fail(TSB_ERR_INVALID_ARGUMENT, "global_avgpool: null pointer");
    if (n < 1 || pixels < 1 || channels < 1) return fail(TSB_ERR_INVALID_ARGUMENT, "global_avgpool: bad shape");
    TSB_CUDA(launch_pdl(global_avgpool_f32_nhwc_kernel, dim3(grid_for((int64_t)n * channels, kThreads)), dim3(kThreads), 0, stream, x, y, n, pixels, channels));
    TSB_LAUNCHED("global_avgpool_f32_nhwc_kernel");
    return TSB_OK;
}

int inner_prod_f32(const float *x, const float *w, const float *bias, float *y, int n, int k, int o, cudaStream_t stream) {
    if (!x || !w || !y) return fail(TSB_ERR_INVALID_ARGUMENT, "inner_prod: null pointer");
    if (n < 1 || k < 1 || o < 1) return fail(TSB_ERR_INVALID_ARGUMENT, "inner_prod: bad shape");
    const dim3 grid(grid_for((int64_t)((n + kIpN - 1) / kIpN) * ((o + kIpO - 1) / kIpO), kThreads / 32 / kIpKS));
    const bool vec = k % 4 == 0 && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w)) & 15) == 0;
    if (vec) TSB_CUDA(launch_pdl(inner_prod_f32_kernel<4>, grid, dim3(kThreads), 0, stream, x, w, bias, y, n, k, o));
    else TSB_CUDA(launch_pdl(inner_prod_f32_kernel<1>, grid, dim3(kThreads), 0, stream, x, w, bias, y, n, k, o));
    TSB_LAUNCHED("inner_prod_f32_kernel");
    return TSB_OK;
}

int concat_i8_nhwc(const int8_t *a, int ca, const int8_t *b, int cb, int8_t *y, int64_t pixels, cudaStream_t stream) {
    if (!a || !b || !y) return fail(TSB_ERR_INVALID_ARGUMENT, "concat: null pointer");
    if (ca < 1 || cb < 1 || pixels < 1) return fail(TSB_ERR_INVALID_ARGUMENT, "concat: bad extents");
    if ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(y)) % 16)
        return fail(TSB_ERR_INVALID_ARGUMENT, "concat: tensors must be 16-byte aligned");
    const int ca_p = tsb_padded_channels(ca), cb_p = tsb_padded_channels(cb), cy = tsb_padded_channels(ca + cb);
    const int vec = (ca % 16 == 0 && cb % 16 == 0) ? 1 : 0;
    const int64_t items = vec ? pixels * (cy / 16) : pixels * cy;
    TSB_CUDA(launch_pdl(concat_i8_nhwc_kernel, dim3(grid_for(items, kThreads)), dim3(kThreads), 0, stream, a, ca, ca_p, b, cb, cb_p, y, cy,
                        pixels, vec));
    TSB_LAUNCHED("concat_i8_nhwc_kernel");
    return TSB_OK;
}

}  // namespace tsb
