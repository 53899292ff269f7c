// quantize (fp32 -> int8) and the layout staging kernels.  All of them are HBM-bound byte movers: wide
// coalesced loads/stores, grid sized as a multiple of the SM count, no tensor cores.
#include "common.cuh"

#include <algorithm>
#include <atomic>
#include <cmath>
#include <mutex>

namespace tsb {

QuantRule make_quant_rule(int64_t count, int nscales) {
    QuantRule r;
    r.nscales = nscales;
    if (nscales == 1) {
        r.rne_limit = (count >> 3) << 3;  // AVX body of the reference; the tail rounds half-away
        r.group_len = count > 0 ? count : 1;
    } else {
        r.rne_limit = 0;
        // int(std::ceil(static_cast<float>(count) / quantize_group)) evaluated in fp32, as the reference does
        float len = std::ceil(static_cast<float>(static_cast<int>(count)) / static_cast<float>(static_cast<size_t>(nscales)));
        r.group_len = static_cast<int64_t>(static_cast<int>(len));
        if (r.group_len < 1) r.group_len = 1;
    }
    return r;
}

constexpr int kInlineScales = 64;
struct ScaleArg {
    const float *dev;             // used when nscales > kInlineScales
    float inl[kInlineScales];
    __device__ __forceinline__ float get(int g) const { return dev ? dev[g] : inl[g]; }
};

// Scale table of tsb_quantize_f32_i8_static: fixed device storage that exists from the moment the library is loaded
// on a GPU until the process exits (16 KiB per GPU), so that entry point never has to ask the driver for memory.
constexpr int kStaticScaleCapacity = 4096;
static __device__ __align__(256) float g_static_scale_table[kStaticScaleCapacity];

namespace {

constexpr int kThreads = 256;

// 16 consecutive elements of this thread, streamed once
__device__ __forceinline__ void load16(const float *src, float (&f)[16]) {
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const float4 t = __ldcs(reinterpret_cast<const float4 *>(src) + k);
        f[4 * k + 0] = t.x; f[4 * k + 1] = t.y; f[4 * k + 2] = t.z; f[4 * k + 3] = t.w;
    }
}
__device__ __forceinline__ void load16(const double *src, double (&f)[16]) {
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        const double2 t = __ldcs(reinterpret_cast<const double2 *>(src) + k);
        f[2 * k + 0] = t.x; f[2 * k + 1] = t.y;
    }
}

// 16 consecutive elements per thread: 4 x float4 (8 x double2) in, one 16-byte store out.
template <typename TIn>
__global__ void __launch_bounds__(kThreads)
quantize_vec16_kernel(const TIn *__restrict__ x, int8_t *__restrict__ y, uint32_t count, QuantRule rule,
                      ScaleArg scales) {
    const uint32_t nvec = count >> 4;
    const uint32_t rne_limit = (uint32_t)rule.rne_limit;
    const uint32_t group_len = (uint32_t)rule.group_len;
    const int nscales = rule.nscales;
    for (uint32_t v = blockIdx.x * kThreads + threadIdx.x; v < nvec; v += gridDim.x * kThreads) {
        const uint32_t i0 = v << 4;
        TIn f[16];
        load16(x + i0, f);
        uint32_t g0 = nscales == 1 ? 0u : i0 / group_len;
        uint32_t g1 = nscales == 1 ? 0u : (i0 + 15u) / group_len;
        uint32_t packed[4];
        if (g1 >= (uint32_t)nscales || g0 != g1 || (i0 < rne_limit && i0 + 16u > rne_limit)) {
            // a scale-group boundary, the end of the scale list or the rounding switch falls inside this vector
            int4 old = *reinterpret_cast<const int4 *>(y + i0);
            const int8_t *oldb = reinterpret_cast<const int8_t *>(&old);
            int8_t *pb = reinterpret_cast<int8_t *>(packed);
#pragma unroll
            for (int k = 0; k < 16; ++k) {
                uint32_t i = i0 + k;
                uint32_t g = nscales == 1 ? 0u : i / group_len;
                pb[k] = g < (uint32_t)nscales ? (int8_t)q8(f[k], scales.get(g), i < rne_limit) : oldb[k];
            }
        } else {
            const float s = scales.get(g0);
            const bool he = i0 < rne_limit;
            bool done = false;
            if (sizeof(TIn) == 4) {
                // fp32: product, rounding and ONE saturating conversion per value, one range test per sixteen (NaN and
                // |v| >= 2^31 convert to -128 on the reference's CPU, which a saturating conversion does not give: such a
                // vector takes the exact form below)
                float worst = 0.0f;
                bool odd = false;
#pragma unroll
                for (int k = 0; k < 16; ++k) {
                    const float v = __fmul_rn((float)f[k], s);
                    worst = fmaxf(worst, fabsf(v));
                    odd = odd || (v != v);
                    int q;
                    if (he) {
                        asm("cvt.rni.sat.s8.f32 %0, %1;" : "=r"(q) : "f"(v));
                    } else {
                        const float mag = __fadd_rz(fabsf(v), 0.5f);
                        const float sm = __int_as_float((__float_as_int(mag) & 0x7fffffff) | (__float_as_int(v) & 0x80000000));
                        asm("cvt.rzi.sat.s8.f32 %0, %1;" : "=r"(q) : "f"(sm));
                    }
                    if ((k & 3) == 0) packed[k >> 2] = (uint32_t)(q & 0xff);
                    else packed[k >> 2] |= (uint32_t)(q & 0xff) << (8 * (k & 3));
                }
                done = !(odd || !(worst < 2147483648.0f));
            }
            if (!done) {
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    int a = q8(f[4 * k + 0], s, he), b = q8(f[4 * k + 1], s, he);
                    int c = q8(f[4 * k + 2], s, he), d = q8(f[4 * k + 3], s, he);
                    packed[k] = (a & 0xff) | ((b & 0xff) << 8) | ((c & 0xff) << 16) | ((uint32_t)(d & 0xff) << 24);
                }
            }
        }
        __stcs(reinterpret_cast<int4 *>(y + i0), make_int4(packed[0], packed[1], packed[2], packed[3]));
    }
}

// element-at-a-time: misaligned tensors and the < 16 element tail
template <typename TIn>
__global__ void __launch_bounds__(kThreads)
quantize_scalar_kernel(const TIn *__restrict__ x, int8_t *__restrict__ y, uint32_t begin, uint32_t count,
                       QuantRule rule, ScaleArg scales) {
    const uint32_t rne_limit = (uint32_t)rule.rne_limit;
    const uint32_t group_len = (uint32_t)rule.group_len;
    for (uint32_t i = begin + blockIdx.x * kThreads + threadIdx.x; i < count; i += gridDim.x * kThreads) {
        uint32_t g = rule.nscales == 1 ? 0u : i / group_len;
        if (g < (uint32_t)rule.nscales) y[i] = (int8_t)q8(x[i], scales.get(g), i < rne_limit);
    }
}

// [N][C][HW] (fp32, quantized on the fly, or int8) -> [N][HW][Cp] int8, padding channels zero.
// One block moves a 64-pixel x 64-channel tile through shared memory: reads are coalesced along pixels,
// writes are 16-byte vectors along channels.  grid = (pixel tiles, channel chunks, N).
template <typename TIn>
__global__ void __launch_bounds__(kThreads)
nchw_to_nhwc_kernel(const TIn *__restrict__ x, int8_t *__restrict__ y, int C, int Cp, int HW, QuantRule rule,
                    ScaleArg scales) {
    __shared__ int8_t tile[64][64 + 4];
    const int n = blockIdx.z;
    const int p0 = blockIdx.x * 64;
    const int c0 = blockIdx.y * 64;
    const uint32_t rne_limit = (uint32_t)rule.rne_limit;
    const uint32_t group_len = (uint32_t)rule.group_len;
    const int pl = threadIdx.x & 63, cl = threadIdx.x >> 6;
    const int sp = threadIdx.x >> 2, sq = threadIdx.x & 3;
    const int cw = min(64, Cp - c0);
#pragma unroll 4
    for (int i = 0; i < 16; ++i) {
        const int ci = cl + 4 * i;
        if (ci < cw) {
            const int c = c0 + ci, p = p0 + pl;
            int8_t v = 0;
            if (c < C && p < HW) {
                const uint32_t idx = (uint32_t)(n * C + c) * (uint32_t)HW + (uint32_t)p;
                if (sizeof(TIn) == 1) {
                    v = (int8_t)x[idx];
                } else {
                    uint32_t g = rule.nscales == 1 ? 0u : idx / group_len;
                    v = g < (uint32_t)rule.nscales ? (int8_t)q8((float)x[idx], scales.get(g), idx < rne_limit) : 0;
                }
            }
            tile[ci][pl] = v;
        }
    }
    __syncthreads();
    if (16 * sq < cw && p0 + sp < HW) {
        uint32_t w[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            uint32_t b0 = (uint8_t)tile[16 * sq + 4 * k + 0][sp], b1 = (uint8_t)tile[16 * sq + 4 * k + 1][sp];
            uint32_t b2 = (uint8_t)tile[16 * sq + 4 * k + 2][sp], b3 = (uint8_t)tile[16 * sq + 4 * k + 3][sp];
            w[k] = b0 | (b1 << 8) | (b2 << 16) | (b3 << 24);
        }
        int8_t *dst = y + ((size_t)n * HW + p0 + sp) * Cp + c0 + 16 * sq;
        *reinterpret_cast<int4 *>(dst) = make_int4(w[0], w[1], w[2], w[3]);
    }
}

// [N][HW][Cp] int8 -> [N][C][HW] int8
__global__ void __launch_bounds__(kThreads)
nhwc_to_nchw_kernel(const int8_t *__restrict__ x, int8_t *__restrict__ y, int C, int Cp, int HW) {
    __shared__ int8_t tile[64][64 + 4];  // [p][c]
    const int n = blockIdx.y;
    const int p0 = blockIdx.x * 64;
    const int a = threadIdx.x & 63, b = threadIdx.x >> 6;
    for (int c0 = 0; c0 < C; c0 += 64) {
        for (int i = 0; i < 16; ++i) {
            const int pi = b + 4 * i;
            int8_t v = 0;
            if (p0 + pi < HW && c0 + a < Cp) v = x[((size_t)n * HW + p0 + pi) * Cp + c0 + a];
            tile[pi][a] = v;
        }
        __syncthreads();
        for (int i = 0; i < 16; ++i) {
            const int ci = b + 4 * i;
            if (c0 + ci < C && p0 + a < HW) y[((size_t)n * C + c0 + ci) * HW + p0 + a] = tile[a][ci];
        }
        __syncthreads();
    }
}

// fp32 NCHW -> int8 in the layout a convolution consumes, quantized on the way.  One thread produces 16 output
// bytes: 16 channels of one pixel (NHWC_PAD, or the folded layout with 16 bytes per pixel) or 8 channels of two
// neighbouring pixels (folded layout with 8 bytes per pixel).  Consecutive threads read consecutive pixels of each
// channel plane (full 32-byte sectors) and write consecutive 16-byte units (fully coalesced), so no shared memory
// is needed.  Rounding and scale groups follow the NCHW element index.
struct StageDesc {
    int N, C, H, W;
    int folded;      // 0: [N][H][W][Cp]; 1: [N][H][Wp][cpix] with pixel w at column w + pad_l
    int Cp;          // NHWC_PAD channels
    int Wp, cpix, pad_l;
};

__global__ void __launch_bounds__(kThreads)
quantize_stage_kernel(const float *__restrict__ x, int8_t *__restrict__ y, StageDesc d, uint32_t units, QuantRule rule,
                      ScaleArg scales) {
    pdl_sync();
    const uint32_t rne_limit = (uint32_t)rule.rne_limit;
    const uint32_t group_len = (uint32_t)rule.group_len;
    const uint32_t HW = (uint32_t)(d.H * d.W);
    const uint32_t CHW = (uint32_t)d.C * HW;
    const bool per_sample = rule.nscales > 1 && group_len == CHW;   // the usual case: one scale per image
    const uint32_t upp = (uint32_t)d.Cp / 16u;                       // NHWC_PAD: 16-byte units per pixel
    const uint32_t upr = d.folded ? (uint32_t)(d.Wp * d.cpix) / 16u : 1u;  // folded: units per staged row
    for (uint32_t t = blockIdx.x * kThreads + threadIdx.x; t < units; t += gridDim.x * kThreads) {
        // Thread -> output unit.  NHWC_PAD: the 32 lanes of a warp take 32 consecutive pixels of one 16-channel group,
        // so every load instruction reads 128 contiguous bytes of one channel plane.
        uint32_t u, n, h, c0;
        int w0;
        if (!d.folded) {
            const uint32_t lane = t & 31u, grp = t >> 5;
            const uint32_t cg = grp % upp, pblock = grp / upp;
            const uint32_t pix = pblock * 32u + lane;
            const uint32_t npix_total = (uint32_t)d.N * HW;
            if (pix >= npix_total) continue;
            u = pix * upp + cg;
            n = pix / HW;
            const uint32_t p = pix - n * HW;
            h = p / (uint32_t)d.W;
            w0 = (int)(p - h * (uint32_t)d.W);
            c0 = cg * 16u;
        } else {
            u = t;
            const uint32_t ur = t % upr, row = t / upr;
            h = row % (uint32_t)d.H;
            n = row / (uint32_t)d.H;
            w0 = (int)(ur * (16u / (uint32_t)d.cpix)) - d.pad_l;
            c0 = 0;
        }
        const bool two_pixels = d.folded && d.cpix == 8;
        const uint32_t base = (n * (uint32_t)d.C * (uint32_t)d.H + h) * (uint32_t)d.W;   // + c*H*W + w
        // all sixteen loads first (indices clamped so they can be issued unconditionally), arithmetic afterwards
        float val[16];
        uint32_t idx[16];
        bool ok[16];
#pragma unroll
        for (int b = 0; b < 16; ++b) {
            const int pi = two_pixels ? (b >> 3) : 0;
            const uint32_t c = c0 + (uint32_t)(two_pixels ? (b & 7) : b);
            const int w = w0 + pi;
            ok[b] = c < (uint32_t)d.C && (unsigned)w < (unsigned)d.W && (!d.folded || (two_pixels ? (b & 7) : b) < d.cpix);
            idx[b] = ok[b] ? base + c * HW + (uint32_t)w : 0u;
            val[b] = __ldg(x + idx[b]);
        }
        const float sample_scale = scales.get(per_sample ? (int)n : 0);
        uint32_t word[4] = {0, 0, 0, 0};
#pragma unroll
        for (int b = 0; b < 16; ++b) {
            int q = 0;
            if (ok[b]) {
                float s = sample_scale;
                bool in_range = true;
                if (rule.nscales != 1 && !per_sample) {
                    const uint32_t g = idx[b] / group_len;
                    in_range = g < (uint32_t)rule.nscales;
                    s = in_range ? scales.get((int)g) : 0.0f;
                }
                if (in_range) q = q8(val[b], s, idx[b] < rne_limit);
            }
            word[b >> 2] |= (uint32_t)(q & 0xff) << (8 * (b & 3));
        }
        *reinterpret_cast<int4 *>(y + (size_t)u * 16) = make_int4(word[0], word[1], word[2], word[3]);
    }
}

// NHWC_PAD staging of tensors with 64-channel groups (Cp a multiple of 64), through a shared-memory tile of 32 pixels x 64
// channels: warp w reads channels 8w .. 8w+7 of the tile's 32 consecutive pixels (every load instruction 128 contiguous
// bytes of one channel plane), packs its 8 bytes per pixel into the pixel's row of the tile, and the tile leaves as 16-byte
// units -- four lanes write the 64 contiguous bytes of a pixel, so every store fills whole sectors.  (The kernel above
// writes a pixel's bytes 16 at a time from lanes that sit a whole pixel row apart.)  Two tiles alternate: one barrier per
// tile.  Rounding and scale groups follow the NCHW element index.
__global__ void __launch_bounds__(kThreads)
quantize_stage_tile_kernel(const float *__restrict__ x, int8_t *__restrict__ y, StageDesc d, uint32_t tiles, QuantRule rule,
                           ScaleArg scales) {
    pdl_sync();
    constexpr int kRow = 72;                                      // bytes per pixel row of the tile: 64 + 8 (bank spread)
    __shared__ __align__(16) uint8_t tile[2][32 * kRow];
    const uint32_t rne_limit = (uint32_t)rule.rne_limit;
    const uint32_t group_len = (uint32_t)rule.group_len;
    const uint32_t HW = (uint32_t)(d.H * d.W);
    const uint32_t CHW = (uint32_t)d.C * HW;
    const bool per_sample = rule.nscales > 1 && group_len == CHW;
    const bool simple = rule.nscales == 1 || per_sample;
    const uint32_t npix = (uint32_t)d.N * HW;
    const uint32_t groups = (uint32_t)d.Cp / 64u;                 // channel groups per pixel tile
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    uint32_t buf = 0;
    for (uint32_t t = blockIdx.x; t < tiles; t += gridDim.x, buf ^= 1u) {
        const uint32_t ptile = t / groups, cg = t - ptile * groups;
        const uint32_t pix = ptile * 32u + lane;
        const bool live = pix < npix;
        const uint32_t n = live ? pix / HW : 0u, p = live ? pix - n * HW : 0u;
        const uint32_t c0 = cg * 64u + warp * 8u;
        float val[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const uint32_t c = c0 + (uint32_t)j;
            val[j] = (live && c < (uint32_t)d.C) ? __ldg(x + (n * (uint32_t)d.C + c) * HW + p) : 0.0f;
        }
        const float sample_scale = scales.get(per_sample ? (int)n : 0);
        uint32_t lo = 0, hi = 0;
        // Fast forms for whole groups of eight live channels under one scale: the product, the rounding and a saturating
        // conversion per value, one range test per eight (NaN and |v| >= 2^31 convert to -128 on the reference's CPU, not to
        // what a saturating conversion gives: such a group falls through to the exact form below)
        const uint32_t idx0 = (n * (uint32_t)d.C + c0) * HW + p;
        const bool full = live && c0 + 8u <= (uint32_t)d.C && simple;
        bool done = false;
        if (full && (rne_limit == 0u || idx0 + 7u * HW < rne_limit)) {
            const bool even = rne_limit != 0u;
            float worst = 0.0f;
            bool odd = false;
            int q[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float v = __fmul_rn(val[j], sample_scale);
                worst = fmaxf(worst, fabsf(v));     // (fmaxf drops a NaN operand: tested on its own)
                odd = odd || (v != v);
                if (even) {
                    asm("cvt.rni.sat.s8.f32 %0, %1;" : "=r"(q[j]) : "f"(v));
                } else {
                    const float mag = __fadd_rz(fabsf(v), 0.5f);
                    const float sm = __int_as_float((__float_as_int(mag) & 0x7fffffff) | (__float_as_int(v) & 0x80000000));
                    asm("cvt.rzi.sat.s8.f32 %0, %1;" : "=r"(q[j]) : "f"(sm));
                }
            }
            odd = odd || !(worst < 2147483648.0f);
            if (!odd) {
                lo = (uint32_t)(q[0] & 0xff) | ((uint32_t)(q[1] & 0xff) << 8) | ((uint32_t)(q[2] & 0xff) << 16) | ((uint32_t)(q[3] & 0xff) << 24);
                hi = (uint32_t)(q[4] & 0xff) | ((uint32_t)(q[5] & 0xff) << 8) | ((uint32_t)(q[6] & 0xff) << 16) | ((uint32_t)(q[7] & 0xff) << 24);
                done = true;
            }
        }
        if (!done)
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const uint32_t c = c0 + (uint32_t)j;
            int q = 0;
            if (live && c < (uint32_t)d.C) {
                const uint32_t idx = (n * (uint32_t)d.C + c) * HW + p;
                float sc = sample_scale;
                bool in_range = true;
                if (!simple) {
                    const uint32_t g = idx / group_len;
                    in_range = g < (uint32_t)rule.nscales;
                    sc = in_range ? scales.get((int)g) : 0.0f;
                }
                if (in_range) q = q8(val[j], sc, idx < rne_limit);
            }
            if (j < 4) lo |= (uint32_t)(q & 0xff) << (8 * j);
            else hi |= (uint32_t)(q & 0xff) << (8 * (j - 4));
        }
        *reinterpret_cast<uint2 *>(&tile[buf][lane * kRow + warp * 8]) = make_uint2(lo, hi);
        __syncthreads();
        // 32 pixels x 4 units of 16 bytes: the first 128 threads carry one unit each
        if (threadIdx.x < 128) {
            const uint32_t pr = threadIdx.x >> 2, u = threadIdx.x & 3u;
            const uint32_t opix = ptile * 32u + pr;
            if (opix < npix) {
                const uint2 a = *reinterpret_cast<const uint2 *>(&tile[buf][pr * kRow + u * 16]);
                const uint2 b = *reinterpret_cast<const uint2 *>(&tile[buf][pr * kRow + u * 16 + 8]);
                *reinterpret_cast<int4 *>(y + (size_t)opix * d.Cp + cg * 64u + u * 16u) = make_int4((int)a.x, (int)a.y, (int)b.x, (int)b.y);
            }
        }
        // (the other tile is written next; this one is rewritten only after the next barrier)
    }
}

// Folded staging of inputs with at most four channels (the RGB stems of the benchmark networks): a thread produces 32
// consecutive output bytes -- four staged pixels of 8 bytes, or two of 16 -- from exactly the CC x pixels values that are
// live, so no load is wasted on padding channels; loads of a warp cover consecutive pixels of each channel plane, stores are
// two 16-byte vectors per thread, contiguous over the warp.  One scale per tensor or per sample (the host checks).
template <int CC, int CPIX, bool VEC>
__global__ void __launch_bounds__(kThreads)
quantize_stage_small_kernel(const float *__restrict__ x, int8_t *__restrict__ y, StageDesc d, uint32_t units, QuantRule rule,
                            ScaleArg scales) {
    pdl_sync();
    constexpr int PPT = 32 / CPIX;                       // pixels per thread
    const uint32_t rne_limit = (uint32_t)rule.rne_limit;
    const uint32_t HW = (uint32_t)(d.H * d.W);
    const uint32_t upr = (uint32_t)(d.Wp * CPIX) / 32u;  // 32-byte units per staged row (Wp * CPIX is a multiple of 32 here)
    (void)units;
    // block: 64 units x 4 rows; grid: x over the units of a row, y over (a stride of) the rows -- no division per unit
    for (uint32_t row = blockIdx.y * 4 + threadIdx.y; row < (uint32_t)(d.N * d.H); row += gridDim.y * 4)
    for (uint32_t ur = blockIdx.x * 64 + threadIdx.x; ur < upr; ur += gridDim.x * 64) {
        const uint32_t t = row * upr + ur;
        const uint32_t n = row / (uint32_t)d.H, h = row - n * (uint32_t)d.H;
        const int w0 = (int)(ur * PPT) - d.pad_l;
        const uint32_t base = (n * (uint32_t)CC * (uint32_t)d.H + h) * (uint32_t)d.W;
        float val[PPT][CC];
        if (VEC) {
            // W is a multiple of 4 and x is 16-byte aligned: the four pixels lie in two aligned groups of four, each wholly
            // inside or wholly outside the row; every thread of the grid has the same offset into its first group
            static_assert(!VEC || PPT == 4, "the 16-byte loads serve four pixels per thread");
            const int g0 = (w0 + 4096) / 4 - 1024;           // floor(w0 / 4); w0 >= -pad_l > -4096
            const int r = w0 - g0 * 4;                       // 0..3
            const int groups = d.W >> 2;
#pragma unroll
            for (int c = 0; c < CC; ++c) {
                const float4 *src = reinterpret_cast<const float4 *>(x + base + (uint32_t)c * HW);
                const float4 zero = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                const float4 a = (unsigned)g0 < (unsigned)groups ? __ldg(src + g0) : zero;
                const float4 b = (r != 0 && (unsigned)(g0 + 1) < (unsigned)groups) ? __ldg(src + g0 + 1) : zero;
                if (r == 0)      { val[0][c] = a.x; val[1][c] = a.y; val[2][c] = a.z; val[3][c] = a.w; }
                else if (r == 1) { val[0][c] = a.y; val[1][c] = a.z; val[2][c] = a.w; val[3][c] = b.x; }
                else if (r == 2) { val[0][c] = a.z; val[1][c] = a.w; val[2][c] = b.x; val[3][c] = b.y; }
                else             { val[0][c] = a.w; val[1][c] = b.x; val[2][c] = b.y; val[3][c] = b.z; }
            }
        } else {
#pragma unroll
            for (int p = 0; p < PPT; ++p) {
                const int w = w0 + p;
                const bool in = (unsigned)w < (unsigned)d.W;
#pragma unroll
                for (int c = 0; c < CC; ++c) val[p][c] = in ? __ldg(x + base + (uint32_t)c * HW + (uint32_t)w) : 0.0f;
            }
        }
        const float s = scales.get(rule.nscales == 1 ? 0 : (int)n);
        uint32_t word[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        bool done = false;
        if (rne_limit == 0u) {
            // everything rounds half away from zero (the multi-scale rule): product, rounding and a saturating conversion
            // per value, one range test per thread (NaN and |v| >= 2^31 convert to -128 on the reference's CPU: the exact
            // form below takes the thread then); values outside the row are zeros and stay zeros
            float worst = 0.0f;
            bool odd = false;
#pragma unroll
            for (int p = 0; p < PPT; ++p)
#pragma unroll
                for (int c = 0; c < CC; ++c) {
                    const float v = __fmul_rn(val[p][c], s);
                    worst = fmaxf(worst, fabsf(v));
                    odd = odd || (v != v);
                    const float mag = __fadd_rz(fabsf(v), 0.5f);
                    const float sm = __int_as_float((__float_as_int(mag) & 0x7fffffff) | (__float_as_int(v) & 0x80000000));
                    int q;
                    asm("cvt.rzi.sat.s8.f32 %0, %1;" : "=r"(q) : "f"(sm));
                    const bool in = (unsigned)(w0 + p) < (unsigned)d.W;
                    word[(p * CPIX + c) >> 2] |= in ? (uint32_t)(q & 0xff) << (8 * (c & 3)) : 0u;
                }
            done = !(odd || !(worst < 2147483648.0f));
            if (!done) {
#pragma unroll
                for (int k = 0; k < 8; ++k) word[k] = 0u;
            }
        }
        if (!done)
#pragma unroll
        for (int p = 0; p < PPT; ++p) {
            const int w = w0 + p;
            if ((unsigned)w < (unsigned)d.W) {
#pragma unroll
                for (int c = 0; c < CC; ++c) {
                    const uint32_t idx = base + (uint32_t)c * HW + (uint32_t)w;
                    const int q = q8(val[p][c], s, idx < rne_limit);
                    word[(p * CPIX + c) >> 2] |= (uint32_t)(q & 0xff) << (8 * (c & 3));
                }
            }
        }
        int4 *dst = reinterpret_cast<int4 *>(y + (size_t)t * 32);
        __stcs(dst, make_int4(word[0], word[1], word[2], word[3]));
        __stcs(dst + 1, make_int4(word[4], word[5], word[6], word[7]));
    }
}

__global__ void __launch_bounds__(kThreads)
add_bias_nchw_kernel(const float *__restrict__ x, float *__restrict__ y, int C, int HW, int64_t count,
                     const float *__restrict__ bias) {
    for (int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x; i < count; i += (int64_t)gridDim.x * kThreads) {
        const int c = (int)((i / HW) % C);
        y[i] = __fadd_rn(x[i], bias[c]);
    }
}

// The same with 16-byte accesses: a block works inside one (sample, channel) plane, so the bias is a per-block scalar
// and no index arithmetic is left in the loop.  planes = N*C, vec = HW/4 float4 per plane, chunks = blocks per plane.
__global__ void __launch_bounds__(kThreads)
add_bias_nchw_vec4_kernel(const float4 *__restrict__ x, float4 *__restrict__ y, int C, int vec, int chunks, int planes,
                          const float *__restrict__ bias) {
    for (int blk = blockIdx.x; blk < planes * chunks; blk += gridDim.x) {
        const int plane = blk / chunks, chunk = blk - plane * chunks;
        const float b = bias[plane % C];
        const float4 *src = x + (size_t)plane * vec;
        float4 *dst = y + (size_t)plane * vec;
        for (int i = chunk * kThreads + threadIdx.x; i < vec; i += chunks * kThreads) {
            float4 v = __ldcs(src + i);
            v.x = __fadd_rn(v.x, b); v.y = __fadd_rn(v.y, b); v.z = __fadd_rn(v.z, b); v.w = __fadd_rn(v.w, b);
            __stcs(dst + i, v);
        }
    }
}

// 16-byte accesses for the activations as well (count a multiple of 4, both tensors 16-byte aligned)
__global__ void __launch_bounds__(kThreads)
activation_vec4_kernel(const float4 *__restrict__ x, float4 *__restrict__ y, int64_t vec, int activation, float leaky) {
    for (int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x; i < vec; i += (int64_t)gridDim.x * kThreads) {
        float4 v = __ldcs(x + i);
        float *f = reinterpret_cast<float *>(&v);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            if (activation == TSB_ACT_RELU) f[k] = f[k] > 0.0f ? f[k] : 0.0f;
            else if (activation == TSB_ACT_LEAKY_RELU) f[k] = f[k] > 0.0f ? f[k] : __fmul_rn(f[k], leaky);
        }
        __stcs(y + i, v);
    }
}

__global__ void __launch_bounds__(kThreads)
activation_kernel(const float *__restrict__ x, float *__restrict__ y, int64_t count, int activation, float leaky) {
    for (int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x; i < count; i += (int64_t)gridDim.x * kThreads) {
        float v = x[i];
        if (activation == TSB_ACT_RELU) v = v > 0.0f ? v : 0.0f;
        else if (activation == TSB_ACT_LEAKY_RELU) v = v > 0.0f ? v : __fmul_rn(v, leaky);
        y[i] = v;
    }
}

// SM count of the CURRENT device (one process may drive several GPUs; remembered per device)
int sm_count() {
    constexpr int kMaxDevices = 64;
    static std::atomic<int> cached[kMaxDevices] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 148;
    int sms = cached[dev].load(std::memory_order_relaxed);
    if (!sms) {
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
        cached[dev].store(sms, std::memory_order_relaxed);
    }
    return sms;
}

int grid_for(int64_t work_items) {
    int64_t blocks = ceil_div64(work_items, kThreads);
    int64_t cap = (int64_t)sm_count() * 8;  // a whole number of waves of resident blocks
    if (blocks < 1) blocks = 1;
    return (int)(blocks < cap ? blocks : cap);
}

}  // namespace

// Builds the scale argument.  More than kInlineScales scales (weight quantization at compile time, one scale
// per output channel) go through a stream-ordered temporary; *tmp must be freed by the caller after launch.
int make_scale_arg(const float *scales_host, int nscales, cudaStream_t stream, ScaleArg *arg, float **tmp) {
    *tmp = nullptr;
    arg->dev = nullptr;
    if (nscales <= kInlineScales) {
        for (int i = 0; i < nscales; ++i) arg->inl[i] = scales_host[i];
        return TSB_OK;
    }
    TSB_CUDA(cudaMallocAsync((void **)tmp, sizeof(float) * (size_t)nscales, stream));
    cudaError_t e = cudaMemcpyAsync(*tmp, scales_host, sizeof(float) * (size_t)nscales, cudaMemcpyHostToDevice, stream);
    if (e != cudaSuccess) { cudaFreeAsync(*tmp, stream); *tmp = nullptr; return cuda_fail(e, "copy of quantize scales"); }
    arg->dev = *tmp;
    return TSB_OK;
}

template <typename TIn>
static int quantize_any_i8(const TIn *x, int8_t *y, int64_t count, const float *scales_host, int nscales,
                           cudaStream_t stream) {
    if (!x || !y || !scales_host) return fail(TSB_ERR_INVALID_ARGUMENT, "quantize: null pointer");
    if (nscales < 1) return fail(TSB_ERR_INVALID_ARGUMENT, "quantize: needs at least one scale");
    if (count < 0 || count > INT32_MAX) return fail(TSB_ERR_INVALID_ARGUMENT, "quantize: count %lld out of range", (long long)count);
    if (count == 0) return TSB_OK;
    QuantRule rule = make_quant_rule(count, nscales);
    ScaleArg arg;
    float *tmp = nullptr;
    int st = make_scale_arg(scales_host, nscales, stream, &arg, &tmp);
    if (st != TSB_OK) return st;
    const bool aligned = (reinterpret_cast<uintptr_t>(x) % 16 == 0) && (reinterpret_cast<uintptr_t>(y) % 16 == 0);
    uint32_t done = 0;
    if (aligned && count >= 16) {
        quantize_vec16_kernel<TIn><<<grid_for(count >> 4), kThreads, 0, stream>>>(x, y, (uint32_t)count, rule, arg);
        TSB_LAUNCHED("quantize_vec16_kernel");
        done = (uint32_t)((count >> 4) << 4);
    }
    if (done < count) {
        quantize_scalar_kernel<TIn><<<grid_for(count - done), kThreads, 0, stream>>>(x, y, done, (uint32_t)count, rule, arg);
        TSB_LAUNCHED("quantize_scalar_kernel");
    }
    if (tmp) TSB_CUDA(cudaFreeAsync(tmp, stream));
    return TSB_OK;
}

int quantize_f32_i8(const float *x, int8_t *y, int64_t count, const float *scales_host, int nscales, cudaStream_t stream) {
    return quantize_any_i8<float>(x, y, count, scales_host, nscales, stream);
}

int quantize_f64_i8(const double *x, int8_t *y, int64_t count, const float *scales_host, int nscales, cudaStream_t stream) {
    return quantize_any_i8<double>(x, y, count, scales_host, nscales, stream);
}

static int check_nchw(const void *x, const void *y, int n, int c, int h, int w, const char *who) {
    if (!x || !y) return fail(TSB_ERR_INVALID_ARGUMENT, "%s: null pointer", who);
    if (n < 1 || c < 1 || h < 1 || w < 1) return fail(TSB_ERR_INVALID_ARGUMENT, "%s: bad shape [%d,%d,%d,%d]", who, n, c, h, w);
    if ((int64_t)n * tsb_padded_channels(c) * h * w > INT32_MAX) return fail(TSB_ERR_INVALID_ARGUMENT, "%s: tensor too large", who);
    if (n > 65535) return fail(TSB_ERR_INVALID_ARGUMENT, "%s: batch %d too large", who, n);
    return TSB_OK;
}

// fp32 NCHW -> staged int8.  folded == 0: NHWC_PAD with tsb_padded_channels(c) channels; folded == 1: rows of wp
// pixels of cpix bytes, pixel w at column w + pad_l.
int quantize_stage(const float *x, int8_t *y, int n, int c, int h, int w, int folded, int wp, int cpix, int pad_l,
                   const float *scales_host, int nscales, cudaStream_t stream) {
    int st = check_nchw(x, y, n, c, h, w, "quantize_stage");
    if (st != TSB_OK) return st;
    if (!scales_host || nscales < 1) return fail(TSB_ERR_INVALID_ARGUMENT, "quantize_stage: needs scales");
    if (reinterpret_cast<uintptr_t>(y) % 16) return fail(TSB_ERR_INVALID_ARGUMENT, "quantize_stage: output must be 16-byte aligned");
    if (folded && (c > cpix || (cpix != 8 && cpix != 16) || (wp * cpix) % 16 != 0))
        return fail(TSB_ERR_INVALID_ARGUMENT, "quantize_stage: bad folded layout");
    QuantRule rule = make_quant_rule((int64_t)n * c * h * w, nscales);
    ScaleArg arg;
    float *tmp = nullptr;
    st = make_scale_arg(scales_host, nscales, stream, &arg, &tmp);
    if (st != TSB_OK) return st;
    StageDesc d;
    d.N = n; d.C = c; d.H = h; d.W = w;
    d.folded = folded;
    d.Cp = tsb_padded_channels(c);
    d.Wp = wp; d.cpix = cpix; d.pad_l = pad_l;
    // NHWC_PAD: threads are laid out in groups of 32 pixels x (Cp/16) channel groups (the last group may be partial)
    const int64_t units = folded ? (int64_t)n * h * (wp * cpix / 16)
                                 : ceil_div64((int64_t)n * h * w, 32) * 32 * (d.Cp / 16);
    if (units > (int64_t)UINT32_MAX) return fail(TSB_ERR_UNSUPPORTED, "quantize_stage: tensor too large");
    // few input channels, one scale per tensor or per sample, rows made of whole 32-byte units: the lean kernel
    const bool per_sample = rule.nscales > 1 && rule.nscales == n && rule.group_len == (int64_t)c * h * w;
    if (folded && c <= 4 && (wp * cpix) % 32 == 0 && (rule.nscales == 1 || per_sample)) {
        const uint32_t units32 = (uint32_t)((int64_t)n * h * (wp * cpix / 32));
        cudaError_t e = cudaSuccess;
        const dim3 small_grid((unsigned)ceil_div(wp * cpix / 32, 64), (unsigned)std::min(ceil_div(n * h, 4), 65535));
        // 16-byte loads where every row of every plane starts on a 16-byte boundary
        const bool vec = cpix == 8 && w % 4 == 0 && reinterpret_cast<uintptr_t>(x) % 16 == 0 && pad_l < 4096;
#define TSB_STAGE_SMALL(CC_, CPIX_, VEC_)                                                                                 \
        if (c == CC_ && cpix == CPIX_ && vec == VEC_)                                                                     \
            e = launch_pdl(quantize_stage_small_kernel<CC_, CPIX_, VEC_>, small_grid, dim3(64, 4), 0, stream, x, y, d, units32, rule, arg)
        TSB_STAGE_SMALL(1, 8, true); TSB_STAGE_SMALL(2, 8, true); TSB_STAGE_SMALL(3, 8, true); TSB_STAGE_SMALL(4, 8, true);
        TSB_STAGE_SMALL(1, 8, false); TSB_STAGE_SMALL(2, 8, false); TSB_STAGE_SMALL(3, 8, false); TSB_STAGE_SMALL(4, 8, false);
        TSB_STAGE_SMALL(1, 16, false); TSB_STAGE_SMALL(2, 16, false); TSB_STAGE_SMALL(3, 16, false); TSB_STAGE_SMALL(4, 16, false);
#undef TSB_STAGE_SMALL
        TSB_CUDA(e);
        TSB_LAUNCHED("quantize_stage_small_kernel");
        if (tmp) TSB_CUDA(cudaFreeAsync(tmp, stream));
        return TSB_OK;
    }
    if (!folded && d.Cp % 64 == 0) {
        const int64_t tiles = ceil_div64((int64_t)n * h * w, 32) * (d.Cp / 64);
        if (tiles <= (int64_t)UINT32_MAX) {
            const int blocks = (int)std::min<int64_t>(tiles, (int64_t)sm_count() * 8);
            TSB_CUDA(launch_pdl(quantize_stage_tile_kernel, dim3(blocks), dim3(kThreads), 0, stream, x, y, d, (uint32_t)tiles, rule, arg));
            TSB_LAUNCHED("quantize_stage_tile_kernel");
            if (tmp) TSB_CUDA(cudaFreeAsync(tmp, stream));
            return TSB_OK;
        }
    }
    TSB_CUDA(launch_pdl(quantize_stage_kernel, dim3(grid_for(units)), dim3(kThreads), 0, stream, x, y, d, (uint32_t)units, rule, arg));
    TSB_LAUNCHED("quantize_stage_kernel");
    if (tmp) TSB_CUDA(cudaFreeAsync(tmp, stream));
    return TSB_OK;
}

int quantize_f32_nchw_to_nhwc(const float *x, int8_t *y, int n, int c, int h, int w, const float *scales_host,
                              int nscales, cudaStream_t stream) {
    return quantize_stage(x, y, n, c, h, w, 0, 0, 0, 0, scales_host, nscales, stream);
}

int repack_i8_nchw_to_nhwc(const int8_t *x, int8_t *y, int n, int c, int h, int w, cudaStream_t stream) {
    int st = check_nchw(x, y, n, c, h, w, "repack_nchw_to_nhwc");
    if (st != TSB_OK) return st;
    if (reinterpret_cast<uintptr_t>(y) % 16) return fail(TSB_ERR_INVALID_ARGUMENT, "repack_nchw_to_nhwc: output must be 16-byte aligned");
    QuantRule rule = make_quant_rule(1, 1);
    ScaleArg arg;
    arg.dev = nullptr;
    dim3 grid(ceil_div(h * w, 64), ceil_div(tsb_padded_channels(c), 64), n);
    nchw_to_nhwc_kernel<int8_t><<<grid, kThreads, 0, stream>>>(x, y, c, tsb_padded_channels(c), h * w, rule, arg);
    TSB_LAUNCHED("nchw_to_nhwc_kernel<int8_t>");
    return TSB_OK;
}

int repack_i8_nhwc_to_nchw(const int8_t *x, int8_t *y, int n, int c, int h, int w, cudaStream_t stream) {
    int st = check_nchw(x, y, n, c, h, w, "repack_nhwc_to_nchw");
    if (st != TSB_OK) return st;
    dim3 grid(ceil_div(h * w, 64), n);
    nhwc_to_nchw_kernel<<<grid, kThreads, 0, stream>>>(x, y, c, tsb_padded_channels(c), h * w);
    TSB_LAUNCHED("nhwc_to_nchw_kernel");
    return TSB_OK;
}

int add_bias_f32_nchw(const float *x, float *y, int n, int c, int hw, const float *bias, cudaStream_t stream) {
    if (!x || !y || !bias) return fail(TSB_ERR_INVALID_ARGUMENT, "add_bias: null pointer");
    if (n < 1 || c < 1 || hw < 1) return fail(TSB_ERR_INVALID_ARGUMENT, "add_bias: bad shape");
    const int64_t count = (int64_t)n * c * hw;
    const bool aligned = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) % 16) == 0;
    if (aligned && hw % 4 == 0 && (int64_t)n * c <= INT32_MAX / 64) {
        const int vec = hw / 4, planes = n * c;
        // enough blocks per plane to fill the GPU even when there are few planes, at most one per 256 float4
        const int chunks = std::max(1, std::min(ceil_div(vec, kThreads), ceil_div(sm_count() * 8, planes)));
        const int blocks = (int)std::min<int64_t>((int64_t)planes * chunks, (int64_t)sm_count() * 16);
        add_bias_nchw_vec4_kernel<<<blocks, kThreads, 0, stream>>>(reinterpret_cast<const float4 *>(x), reinterpret_cast<float4 *>(y), c, vec,
                                                                    chunks, planes, bias);
        TSB_LAUNCHED("add_bias_nchw_vec4_kernel");
        return TSB_OK;
    }
    add_bias_nchw_kernel<<<grid_for(count), kThreads, 0, stream>>>(x, y, c, hw, count, bias);
    TSB_LAUNCHED("add_bias_nchw_kernel");
    return TSB_OK;
}

int activation_f32(const float *x, float *y, int64_t count, int activation, float leaky, cudaStream_t stream) {
    if (!x || !y) return fail(TSB_ERR_INVALID_ARGUMENT, "activation: null pointer");
    if (count < 0) return fail(TSB_ERR_INVALID_ARGUMENT, "activation: negative count");
    if (count == 0) return TSB_OK;
    if (count % 4 == 0 && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) % 16) == 0) {
        activation_vec4_kernel<<<grid_for(count / 4), kThreads, 0, stream>>>(reinterpret_cast<const float4 *>(x), reinterpret_cast<float4 *>(y),
                                                                             count / 4, activation, leaky);
        TSB_LAUNCHED("activation_vec4_kernel");
        return TSB_OK;
    }
    activation_kernel<<<grid_for(count), kThreads, 0, stream>>>(x, y, count, activation, leaky);
    TSB_LAUNCHED("activation_kernel");
    return TSB_OK;
}

// quantize for callers that must not allocate: identical arithmetic and kernels to quantize_f32_i8, but the scale
// list always travels through g_static_scale_table instead of kernel arguments or a stream-ordered temporary.
//
// In host code the array's name is only a handle; the device address comes from cudaGetSymbolAddress, asked once per
// device (with that device current) on the first call made there and remembered.
int quantize_f32_i8_static(const float *x, int8_t *y, int64_t count, const float *scales_host, int nscales,
                           cudaStream_t stream) {
    if (!x || !y || !scales_host) return fail(TSB_ERR_INVALID_ARGUMENT, "quantize_static: null pointer");
    if (nscales < 1) return fail(TSB_ERR_INVALID_ARGUMENT, "quantize_static: needs at least one scale");
    if (nscales > kStaticScaleCapacity)
        return fail(TSB_ERR_UNSUPPORTED, "quantize_static: %d scales exceed the built-in table of %d; use tsb_quantize_f32_i8",
                    nscales, kStaticScaleCapacity);
    if (count < 0 || count > INT32_MAX) return fail(TSB_ERR_INVALID_ARGUMENT, "quantize_static: count %lld out of range", (long long)count);
    if (count == 0) return TSB_OK;

    constexpr int kMaxDevices = 64;
    static float *table_on_device[kMaxDevices] = {};
    static std::mutex table_lock;
    int dev = -1;
    TSB_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return fail(TSB_ERR_UNSUPPORTED, "quantize_static: device index %d not supported", dev);
    float *table = nullptr;
    {
        std::lock_guard<std::mutex> guard(table_lock);
        if (!table_on_device[dev]) {
            void *addr = nullptr;
            TSB_CUDA(cudaGetSymbolAddress(&addr, g_static_scale_table));
            table_on_device[dev] = static_cast<float *>(addr);
        }
        table = table_on_device[dev];
    }
    // every call overwrites the part of the table it uses; nothing has to start at zero
    TSB_CUDA(cudaMemcpyAsync(table, scales_host, sizeof(float) * (size_t)nscales, cudaMemcpyHostToDevice, stream));

    QuantRule rule = make_quant_rule(count, nscales);
    ScaleArg arg;
    arg.dev = table;
    const bool aligned = (reinterpret_cast<uintptr_t>(x) % 16 == 0) && (reinterpret_cast<uintptr_t>(y) % 16 == 0);
    uint32_t done = 0;
    if (aligned && count >= 16) {
        quantize_vec16_kernel<float><<<grid_for(count >> 4), kThreads, 0, stream>>>(x, y, (uint32_t)count, rule, arg);
        TSB_LAUNCHED("quantize_vec16_kernel");
        done = (uint32_t)((count >> 4) << 4);
    }
    if (done < count) {
        quantize_scalar_kernel<float><<<grid_for(count - done), kThreads, 0, stream>>>(x, y, done, (uint32_t)count, rule, arg);
        TSB_LAUNCHED("quantize_scalar_kernel");
    }
    return TSB_OK;
}

}  // namespace tsb
