// int8 x int8 -> int32 convolution as an implicit GEMM on the sm_100a tensor cores.
//
//   GEMM view   M = N*OH*OW output pixels, N = O output channels, K = KH*KW*Cp  (k ordered kh, kw, c)
//   A operand   activations, int8 [N][H][W][Cp]; one TMA im2col load per (filter tap, channel block) brings the
//               128 x BK tile of a 128-pixel run of output positions -- halo, stride, dilation and zero padding
//               are resolved by the tensor map, nothing is materialised in memory
//   B operand   weights, int8 [O][KH][KW][Cp]; plain 2-D TMA tiles of BN x BK
//   MMA         tcgen05.mma kind::i8, 128 x BN x 32 per instruction, int32 accumulators in tensor memory,
//               issued by one thread; two accumulator buffers so the epilogue of tile i overlaps the
//               main loop of tile i+1
//   epilogue    sixteen warps read the accumulators with tcgen05.ld and apply dequantize / bias / residual /
//               activation / requantize in registers, then store fp32 (NCHW or NHWC) and/or int8
//
// Warp roles in a CTA of 576 threads: warp 0 = TMA producer, warp 1 = tensor-memory owner + MMA issuer,
// warps 2..17 = epilogue.  The kernel is persistent: gridDim.x CTAs walk the tile list with stride gridDim.x.
//
// Every wait on an mbarrier is bounded; a wait that runs out records a code in *status, raises a CTA-wide
// abort flag and all roles fall through to the common exit, where tensor memory is released.
#include "conv_common.cuh"
#include "conv_tc.h"

#include <cuda.h>
#include <cudaTypedefs.h>

#include <algorithm>
#include <atomic>
#include <type_traits>
#include <cstdlib>

namespace tsb {
namespace tc {

constexpr int kBM = 128;
constexpr int kIssuers = 2;                              // warps that issue MMAs, on alternate tiles
constexpr int kEpiWarp0 = 1 + kIssuers;                  // first epilogue warp
constexpr int kEpiThreads = 512;
constexpr int kThreads = 32 * kEpiWarp0 + kEpiThreads;   // producer warp, issuer warps, sixteen epilogue warps
constexpr int kMaxAccBufs = 4;                           // accumulator buffers in tensor memory (512 columns / BN, at most 4)
constexpr uint32_t kSmemBudget = 200 * 1024;  // stages; the rest holds barriers and epilogue tables

// ---------------------------------------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}

// Bounded wait.  Returns false when the CTA is aborting or ~2 s of polling went by.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    for (uint32_t spin = 0;; ++spin) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((spin & 255u) == 255u) {
            if (*abort_flag) return false;
            if (clock64() - t0 > 4000000000LL) return false;
        }
    }
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y) : "memory");
}

// plain (untiled) bulk copy global -> shared; both addresses and the size are multiples of 16 bytes
__device__ __forceinline__ void bulk_load(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 :: "r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int c, int w, int h, int n) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c), "r"(w), "r"(h), "r"(n) : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int c, int w, int h) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c), "r"(w), "r"(h) : "memory");
}
// tile stores shared -> global (bulk async group of the issuing thread); out-of-range parts of the box are not written
__device__ __forceinline__ void tma_store_2d(const CUtensorMap *map, uint32_t src, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(map), "r"(src), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tma_store_3d(const CUtensorMap *map, uint32_t src, int x, int y, int z) {
    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(map), "r"(src), "r"(x), "r"(y), "r"(z) : "memory");
}
__device__ __forceinline__ void tma_store_4d(const CUtensorMap *map, uint32_t src, int x, int y, int z, int w) {
    asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];" ::"l"(map), "r"(src), "r"(x), "r"(y), "r"(z), "r"(w) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// the stores of this thread's groups have finished READING shared memory (the source may be overwritten)
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
// generic-proxy writes to shared memory become visible to the async proxy (TMA) of this CTA
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
// named barrier over `threads` threads that also ORs a predicate over them
__device__ __forceinline__ bool bar_or(int id, int threads, bool pred) {
    uint32_t r;
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t"
        "setp.ne.b32 p, %1, 0;\n\t"
        "bar.red.or.pred q, %2, %3, p;\n\t"
        "selp.u32 %0, 1, 0, q;\n\t}"
        : "=r"(r) : "r"((uint32_t)pred), "r"(id), "r"(threads) : "memory");
    return r != 0;
}
__device__ __forceinline__ void tma_load_im2col_4d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int c, int w,
                                                   int h, int n, uint16_t off_w, uint16_t off_h) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.im2col.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4, %5, %6}], [%2], {%7, %8};"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c), "r"(w), "r"(h), "r"(n), "h"(off_w), "h"(off_h) : "memory");
}

// Brings a box of a tensor into L2 without a destination in shared memory (no barrier, nothing to wait for).
__device__ __forceinline__ void tma_prefetch_l2_2d(const CUtensorMap *map, int x, int y) {
    asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];" ::"l"(map), "r"(x), "r"(y) : "memory");
}

__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mma_i8(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// The same, executed only when `on` is non-zero -- a predicated instruction, not a branch.  The issuing thread runs
// alone in its warp and pays tens of cycles for every branch or dependent instruction, so its MMA sequences are
// straight-line code in which inactive slots (a filter row outside the image, a k block beyond the group) are switched
// off by predicate.
__device__ __forceinline__ void mma_i8_if(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate, uint32_t on) {
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "setp.ne.b32 q, %5, 0;\n\t"
        "@q tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(on));
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, int (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
          "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
          "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor of a K-major tile whose rows are one swizzle span (BK bytes) wide:
// 8-row groups are 8*BK bytes apart (stride byte offset); version 1; swizzle 128B (2) or 64B (4).
template <int BK>
__device__ __forceinline__ uint64_t smem_desc(uint32_t saddr) {
    constexpr uint64_t layout = BK == 128 ? 2 : (BK == 64 ? 4 : 6);
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
    d |= (uint64_t)1 << 16;                       // leading byte offset: unused for swizzled K-major
    d |= (uint64_t)((8 * BK) >> 4) << 32;         // stride byte offset
    d |= (uint64_t)1 << 46;                       // descriptor version of this architecture
    d |= layout << 61;
    return d;
}

// The same with a run-time stride between 8-row groups and a start that need not be 1024-byte aligned (patch mode).
// The swizzle is a function of the absolute shared-memory address (measured: any 128-byte-aligned start and any group
// stride read back what a tensor-map copy with the same swizzle wrote; the base-offset field stays 0).
template <int BK>
__device__ __forceinline__ uint64_t smem_desc_strided(uint32_t saddr, uint32_t group_stride_bytes) {
    constexpr uint64_t layout = BK == 128 ? 2 : (BK == 64 ? 4 : 6);
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(group_stride_bytes >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= layout << 61;
    return d;
}

// The same descriptors split for the issuing thread's inner loops: everything but the 14-bit start-address field is
// loop-invariant, so a loop keeps the invariant part in a register and ORs in (address >> 4) -- shared-memory addresses
// stay below 2^18, so the field never overflows into its neighbours, and stepping along K inside a swizzle span or to
// another filter tap is a plain add on that field.
template <int BK>
__device__ __forceinline__ constexpr uint64_t smem_desc_hi(uint32_t group_stride_bytes) {
    return ((uint64_t)1 << 16) | ((uint64_t)(group_stride_bytes >> 4) << 32) | ((uint64_t)1 << 46) |
           ((uint64_t)(BK == 128 ? 2 : (BK == 64 ? 4 : 6)) << 61);
}

// A descriptor from its two 32-bit halves (a register pair: no instruction).  The issuing thread keeps the high half and
// the leading-offset bits of the low half loop-invariant and steps only the 14-bit address field: `lo` below is
// (address >> 4) | (1 << 16), and adding a few 16-byte units to it never carries out of the field.
__device__ __forceinline__ uint64_t desc_pair(uint32_t hi, uint32_t lo) { return ((uint64_t)hi << 32) | (uint64_t)lo; }
constexpr uint32_t kDescLbo = 1u << 16;   // leading byte offset 16 (unused for swizzled K-major operands, set as before)

// Descriptor of a pixel operand whose rows OVERLAP in shared memory (raw-row mode): no swizzle, K-major.  In that canonical
// layout row r, 16-byte K chunk j sits at (r % 8) * 16 + (r / 8) * SBO + j * LBO; with SBO = 128 and LBO = 16 that is
// r * 16 + j * 16: pixel r reads the bytes that start 16 bytes after pixel r-1's, which is exactly a convolution window
// sliding by one pixel stride over one staged image row.
__device__ __forceinline__ uint64_t smem_desc_sliding(uint32_t saddr) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
    d |= (uint64_t)(16 >> 4) << 16;               // leading byte offset: next 16-byte chunk along K
    d |= (uint64_t)(128 >> 4) << 32;              // stride byte offset: next group of 8 rows
    d |= (uint64_t)1 << 46;                       // descriptor version of this architecture
    return d;                                     // layout 0: no swizzle
}

// Instruction descriptor: int32 accumulate, signed 8-bit A and B, both K-major, M = 128, N = BN.
template <int BN>
__device__ __forceinline__ constexpr uint32_t instr_desc() {
    return (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(kBM >> 4) << 24);
}


// ---------------------------------------------------------------------------------------------------------
// epilogue: 32 accumulator columns of one output pixel (one thread) at a time
// ---------------------------------------------------------------------------------------------------------
constexpr int kEpiGeneric = 0;   // any combination of outputs, element by element
constexpr int kEpiF32Nchw = 1;   // fp32 NCHW output only (the operator's own output)
constexpr int kEpiI8Nhwc = 2;    // requantized int8 NHWC_PAD output only, half-away rounding, one scale per sample
constexpr int kEpiNhwc = 3;      // fp32 [N][P][O] residual in and/or fp32 [N][P][O] out and/or int8 NHWC_PAD out (normal orientation)
constexpr int kEpiStaged = 4;    // the same outputs through shared-memory tiles and tensor-map loads / stores (normal orientation)
constexpr uint32_t kStageF32Bytes = kBM * 32 * 4;   // one staged fp32 tile: 128 pixels x 32 channels, 128-byte rows, swizzle 128B
constexpr uint32_t kStageI8Bytes = kBM * 32;        // one staged int8 tile: 128 pixels x 32 channels, 32-byte rows
constexpr int kQuads = 4;                           // the sixteen epilogue warps form four quads of one warp per lane quarter

template <int ACT, bool HAS_BIAS>
__device__ __forceinline__ float epi_value(int acc, float dq, float bias, float leaky) {
    float f = __fmul_rn(__int2float_rn(acc), dq);
    if (HAS_BIAS) f = __fadd_rn(f, bias);
    if (ACT == TSB_ACT_RELU) f = fmaxf(f, 0.0f);   // finite values only: same result as x > 0 ? x : 0
    if (ACT == TSB_ACT_LEAKY_RELU) f = f > 0.0f ? f : __fmul_rn(f, leaky);
    return f;
}

// Round-half-away of an already scaled value t, as a signed 32-bit integer (three instructions per value):
// floor(|t| + 0.5) is obtained exactly as trunc(round_toward_zero(|t| + 0.5)) -- a round-to-nearest sum would be wrong
// for |t| just below 0.5 -- and the sign is put back before the (saturating) conversion.
__device__ __forceinline__ int half_away_s32(float t) {
    const float mag = __fadd_rz(fabsf(t), 0.5f);
    const float signed_mag = __int_as_float((__float_as_int(mag) & 0x7fffffff) | (__float_as_int(t) & 0x80000000));
    return __float2int_rz(signed_mag);
}

// four signed integers -> four int8 with saturation to [-128,127], v0 in the lowest byte
__device__ __forceinline__ uint32_t pack_sat_s8(int v0, int v1, int v2, int v3) {
    uint32_t hi, out;
    asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(hi) : "r"(v3), "r"(v2), "r"(0));
    asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(out) : "r"(v1), "r"(v0), "r"(hi));
    return out;
}

// max that keeps a NaN once it has seen one
__device__ __forceinline__ float max_nan(float a, float b) {
    float r;
    asm("max.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
    return r;
}

// the same over three values (one instruction on this architecture)
__device__ __forceinline__ float max3_nan(float a, float b, float c) {
    float r;
    asm("max.NaN.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}

// ---- fast paths, normal orientation: the thread owns one PIXEL (its tensor-memory lane) and 32 consecutive channels
template <int ACT, bool HAS_BIAS, int W>
__device__ __forceinline__ void store_f32_nchw_t(const int (&v)[W], const float *__restrict__ dq,
                                                 const float *__restrict__ bias, float leaky, float *__restrict__ dst,
                                                 uint32_t stride) {
#pragma unroll
    for (int j4 = 0; j4 < W / 4; ++j4) {
        const float4 d4 = *reinterpret_cast<const float4 *>(dq + 4 * j4);
        const float4 b4 = *reinterpret_cast<const float4 *>(bias + 4 * j4);
        dst[(uint32_t)(4 * j4 + 0) * stride] = epi_value<ACT, HAS_BIAS>(v[4 * j4 + 0], d4.x, b4.x, leaky);
        dst[(uint32_t)(4 * j4 + 1) * stride] = epi_value<ACT, HAS_BIAS>(v[4 * j4 + 1], d4.y, b4.y, leaky);
        dst[(uint32_t)(4 * j4 + 2) * stride] = epi_value<ACT, HAS_BIAS>(v[4 * j4 + 2], d4.z, b4.z, leaky);
        dst[(uint32_t)(4 * j4 + 3) * stride] = epi_value<ACT, HAS_BIAS>(v[4 * j4 + 3], d4.w, b4.w, leaky);
    }
}

// The same with an fp32 NCHW residual (operator "add" between add_bias and the activation, or after the activation): the
// residual is read where the result is written, so a warp's 32 pixels make one coalesced line per channel either way.
template <int ACT, bool HAS_BIAS, int W, bool AFTER>
__device__ __forceinline__ void store_f32_nchw_res_t(const int (&v)[W], const float *__restrict__ dq,
                                                     const float *__restrict__ bias, float leaky, const float *__restrict__ res,
                                                     float *__restrict__ dst, uint32_t stride) {
#pragma unroll
    for (int j8 = 0; j8 < W / 8; ++j8) {
        float r[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) r[k] = __ldg(res + (uint32_t)(8 * j8 + k) * stride);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const int j = 8 * j8 + k;
            float t = __fmul_rn(__int2float_rn(v[j]), dq[j]);
            if (HAS_BIAS) t = __fadd_rn(t, bias[j]);
            if (!AFTER) t = __fadd_rn(t, r[k]);
            if (ACT == TSB_ACT_RELU) t = fmaxf(t, 0.0f);
            if (ACT == TSB_ACT_LEAKY_RELU) t = t > 0.0f ? t : __fmul_rn(t, leaky);
            if (AFTER) t = __fadd_rn(t, r[k]);
            dst[(uint32_t)j * stride] = t;
        }
    }
}

// Requantized int8 output.  Returns false when a scaled value was NaN or beyond the int32 range -- those quantize to
// -128 in the reference (x86 integer-indefinite), which the saturating fast path does not reproduce; the caller
// then redoes the chunk element by element.
template <int ACT, bool HAS_BIAS, int W>
__device__ __forceinline__ bool store_i8_nhwc_t(const int (&v)[W], const float *__restrict__ dq,
                                                const float *__restrict__ bias, float leaky, float rs,
                                                int8_t *__restrict__ dst) {
    uint32_t q[W / 4];
    float worst = 0.0f;
#pragma unroll
    for (int j4 = 0; j4 < W / 4; ++j4) {
        const float4 d4 = *reinterpret_cast<const float4 *>(dq + 4 * j4);
        const float4 b4 = *reinterpret_cast<const float4 *>(bias + 4 * j4);
        const float t0 = __fmul_rn(epi_value<ACT, HAS_BIAS>(v[4 * j4 + 0], d4.x, b4.x, leaky), rs);
        const float t1 = __fmul_rn(epi_value<ACT, HAS_BIAS>(v[4 * j4 + 1], d4.y, b4.y, leaky), rs);
        const float t2 = __fmul_rn(epi_value<ACT, HAS_BIAS>(v[4 * j4 + 2], d4.z, b4.z, leaky), rs);
        const float t3 = __fmul_rn(epi_value<ACT, HAS_BIAS>(v[4 * j4 + 3], d4.w, b4.w, leaky), rs);
        worst = max3_nan(max3_nan(worst, fabsf(t0), fabsf(t1)), fabsf(t2), fabsf(t3));
        q[j4] = pack_sat_s8(half_away_s32(t0), half_away_s32(t1), half_away_s32(t2), half_away_s32(t3));
    }
    if (!(worst < 2147483648.0f)) return false;
#pragma unroll
    for (int h = 0; h < W / 16; ++h) *reinterpret_cast<int4 *>(dst + 16 * h) = make_int4(q[4 * h], q[4 * h + 1], q[4 * h + 2], q[4 * h + 3]);
    return true;
}

// Block-output epilogue of a residual network: v = act(dq*acc + bias + residual); fp32 copy for the next residual and
// int8 copy for the next convolution.  Each pointer may be null.  All three tensors are pixel-major, so the thread's 32
// channels are contiguous: 16-byte loads and stores.
template <int ACT, bool HAS_BIAS, int W, bool AFTER>
__device__ __forceinline__ bool store_nhwc_t(const int (&v)[W], const float *__restrict__ dq, const float *__restrict__ bias,
                                             float leaky, const float *__restrict__ res, float *__restrict__ out_f32,
                                             int8_t *__restrict__ out_i8, float rs) {
    uint32_t q[W / 4];
    float worst = 0.0f;
#pragma unroll
    for (int j4 = 0; j4 < W / 4; ++j4) {
        const float4 d4 = *reinterpret_cast<const float4 *>(dq + 4 * j4);
        const float4 b4 = *reinterpret_cast<const float4 *>(bias + 4 * j4);
        float4 r4 = make_float4(0.f, 0.f, 0.f, 0.f);
        if (res) r4 = __ldg(reinterpret_cast<const float4 *>(res) + j4);
        float f[4];
        const float dd[4] = {d4.x, d4.y, d4.z, d4.w}, bb[4] = {b4.x, b4.y, b4.z, b4.w}, rr[4] = {r4.x, r4.y, r4.z, r4.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            float t = __fmul_rn(__int2float_rn(v[4 * j4 + k]), dd[k]);
            if (HAS_BIAS) t = __fadd_rn(t, bb[k]);
            if (res && !AFTER) t = __fadd_rn(t, rr[k]);
            if (ACT == TSB_ACT_RELU) t = fmaxf(t, 0.0f);
            if (ACT == TSB_ACT_LEAKY_RELU) t = t > 0.0f ? t : __fmul_rn(t, leaky);
            if (res && AFTER) t = __fadd_rn(t, rr[k]);
            f[k] = t;
        }
        if (out_f32) reinterpret_cast<float4 *>(out_f32)[j4] = make_float4(f[0], f[1], f[2], f[3]);
        if (out_i8) {
            const float t0 = __fmul_rn(f[0], rs), t1 = __fmul_rn(f[1], rs), t2 = __fmul_rn(f[2], rs), t3 = __fmul_rn(f[3], rs);
            worst = max3_nan(max3_nan(worst, fabsf(t0), fabsf(t1)), fabsf(t2), fabsf(t3));
            q[j4] = pack_sat_s8(half_away_s32(t0), half_away_s32(t1), half_away_s32(t2), half_away_s32(t3));
        }
    }
    if (out_i8) {
        if (!(worst < 2147483648.0f)) return false;
#pragma unroll
        for (int h = 0; h < W / 16; ++h) *reinterpret_cast<int4 *>(out_i8 + 16 * h) = make_int4(q[4 * h], q[4 * h + 1], q[4 * h + 2], q[4 * h + 3]);
    }
    return true;
}

// Staged form of the same block epilogue: the thread's 32 channels of residual come from its row of a shared-memory tile
// that a tensor-map load filled (128-byte rows, 128B swizzle: 16-byte chunk i of row r sits at chunk i ^ (r & 7)), the
// fp32 results go back into the same places and the int8 results into the thread's 32-byte row of a second tile; tensor-
// map stores carry both tiles to global memory.  No global address arithmetic, every shared-memory access 16 bytes wide.
template <int ACT, bool HAS_BIAS, bool AFTER>
__device__ __forceinline__ bool staged_chunk_t(const int (&v)[32], const float *__restrict__ dq, const float *__restrict__ bias,
                                               float leaky, float4 *__restrict__ r_row, int key, bool has_res, bool has_f32,
                                               int4 *__restrict__ q_row, bool has_i8, float rs) {
    uint32_t q[8];
    float worst = 0.0f;
#pragma unroll
    for (int j4 = 0; j4 < 8; ++j4) {
        const float4 d4 = *reinterpret_cast<const float4 *>(dq + 4 * j4);
        const float4 b4 = *reinterpret_cast<const float4 *>(bias + 4 * j4);
        float4 r4 = make_float4(0.f, 0.f, 0.f, 0.f);
        if (has_res) r4 = r_row[j4 ^ key];
        float f[4];
        const float dd[4] = {d4.x, d4.y, d4.z, d4.w}, bb[4] = {b4.x, b4.y, b4.z, b4.w}, rr[4] = {r4.x, r4.y, r4.z, r4.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            float t = __fmul_rn(__int2float_rn(v[4 * j4 + k]), dd[k]);
            if (HAS_BIAS) t = __fadd_rn(t, bb[k]);
            // without a residual rr is zero: adding it changes nothing but the sign of a negative zero, which the
            // operators' results are compared up to anyway (relu and leaky_relu do not pin it either)
            if (!AFTER) t = __fadd_rn(t, rr[k]);
            if (ACT == TSB_ACT_RELU) t = fmaxf(t, 0.0f);
            if (ACT == TSB_ACT_LEAKY_RELU) t = t > 0.0f ? t : __fmul_rn(t, leaky);
            if (AFTER) t = __fadd_rn(t, rr[k]);
            f[k] = t;
        }
        if (has_f32) r_row[j4 ^ key] = make_float4(f[0], f[1], f[2], f[3]);
        if (has_i8) {
            const float t0 = __fmul_rn(f[0], rs), t1 = __fmul_rn(f[1], rs), t2 = __fmul_rn(f[2], rs), t3 = __fmul_rn(f[3], rs);
            worst = max3_nan(max3_nan(worst, fabsf(t0), fabsf(t1)), fabsf(t2), fabsf(t3));
            q[j4] = pack_sat_s8(half_away_s32(t0), half_away_s32(t1), half_away_s32(t2), half_away_s32(t3));
        }
    }
    if (has_i8) {
        if (!(worst < 2147483648.0f)) return false;
        q_row[0] = make_int4(q[0], q[1], q[2], q[3]);
        q_row[1] = make_int4(q[4], q[5], q[6], q[7]);
    }
    return true;
}

// ---- fast paths, swapped orientation: the thread owns one CHANNEL (its lane) and 32 consecutive pixels; dq and bias
// are per-thread scalars
template <int ACT, bool HAS_BIAS>
__device__ __forceinline__ void swap_f32_run(const int (&v)[32], float dq, float bias, float leaky, float *__restrict__ dst) {
    // 32 consecutive pixels of one channel plane: 128 contiguous bytes
    if ((reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
#pragma unroll
        for (int j4 = 0; j4 < 8; ++j4) {
            float4 o;
            o.x = epi_value<ACT, HAS_BIAS>(v[4 * j4 + 0], dq, bias, leaky);
            o.y = epi_value<ACT, HAS_BIAS>(v[4 * j4 + 1], dq, bias, leaky);
            o.z = epi_value<ACT, HAS_BIAS>(v[4 * j4 + 2], dq, bias, leaky);
            o.w = epi_value<ACT, HAS_BIAS>(v[4 * j4 + 3], dq, bias, leaky);
            reinterpret_cast<float4 *>(dst)[j4] = o;
        }
    } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) dst[j] = epi_value<ACT, HAS_BIAS>(v[j], dq, bias, leaky);
    }
}

// int8 NHWC_PAD output: for one pixel the 32 lanes of the warp hold 32 consecutive channels, so each byte store
// instruction of the warp writes one full 32-byte sector.  The first `split` pixels use rs0, the rest rs1 (the chunk
// crosses at most one image boundary).
// Returns false if a value needs the slow path (NaN / beyond int32); the decision is uniform over the warp.
template <int ACT, bool HAS_BIAS>
__device__ __forceinline__ bool swap_i8_run(const int (&v)[32], float dq, float bias, float leaky, float rs0, float rs1,
                                            int split, bool write, int8_t *__restrict__ dst, uint32_t pixel_stride) {
    float worst = 0.0f;
    int q[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) {
        const float t = __fmul_rn(epi_value<ACT, HAS_BIAS>(v[j], dq, bias, leaky), j < split ? rs0 : rs1);
        worst = max_nan(worst, fabsf(t));
        const float mag = __fadd_rz(fabsf(t), 0.5f);
        const float sm = __int_as_float((__float_as_int(mag) & 0x7fffffff) | (__float_as_int(t) & 0x80000000));
        asm("cvt.rzi.s8.f32 %0, %1;" : "=r"(q[j]) : "f"(sm));  // float -> int8 conversions saturate
    }
    if (__any_sync(0xffffffffu, !(worst < 2147483648.0f))) return false;
    if (write) {
#pragma unroll
        for (int j = 0; j < 32; ++j) dst[(uint32_t)j * pixel_stride] = (int8_t)q[j];
    }
    return true;
}

// Patch mode, swapped orientation: the 32 accumulators of a chunk are 4 tile rows of 8 pixels of one channel.
// rows_live / cols_live say how much of that 4 x 8 block lies inside the image (uniform over the warp).
template <int ACT, bool HAS_BIAS>
__device__ __forceinline__ bool patch_i8_run(const int (&v)[32], float dq, float bias, float leaky, float rs, bool write,
                                             int8_t *__restrict__ dst, uint32_t pixel_stride, uint32_t row_stride,
                                             int rows_live, int cols_live) {
    float worst = 0.0f;
    int q[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) {
        const float t = __fmul_rn(epi_value<ACT, HAS_BIAS>(v[j], dq, bias, leaky), rs);
        const bool live = (j >> 3) < rows_live && (j & 7) < cols_live;
        worst = max_nan(worst, live ? fabsf(t) : 0.0f);
        const float mag = __fadd_rz(fabsf(t), 0.5f);
        const float sm = __int_as_float((__float_as_int(mag) & 0x7fffffff) | (__float_as_int(t) & 0x80000000));
        asm("cvt.rzi.s8.f32 %0, %1;" : "=r"(q[j]) : "f"(sm));
    }
    if (__any_sync(0xffffffffu, !(worst < 2147483648.0f))) return false;
    if (write) {
#pragma unroll
        for (int j = 0; j < 32; ++j)
            if ((j >> 3) < rows_live && (j & 7) < cols_live) dst[(uint32_t)(j >> 3) * row_stride + (uint32_t)(j & 7) * pixel_stride] = (int8_t)q[j];
    }
    return true;
}
template <int ACT, bool HAS_BIAS>
__device__ __forceinline__ void patch_f32_run(const int (&v)[32], float dq, float bias, float leaky, float *__restrict__ dst,
                                              uint32_t row_stride, int rows_live, int cols_live) {
    // fp32 NCHW: each tile row is 8 consecutive floats of one channel plane
    const bool vec = cols_live == 8 && ((reinterpret_cast<uintptr_t>(dst) | ((uintptr_t)row_stride * 4)) & 15) == 0;
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        if (r >= rows_live) break;
        float *row = dst + (size_t)r * row_stride;
        if (vec) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                float4 o;
                o.x = epi_value<ACT, HAS_BIAS>(v[8 * r + 4 * h + 0], dq, bias, leaky);
                o.y = epi_value<ACT, HAS_BIAS>(v[8 * r + 4 * h + 1], dq, bias, leaky);
                o.z = epi_value<ACT, HAS_BIAS>(v[8 * r + 4 * h + 2], dq, bias, leaky);
                o.w = epi_value<ACT, HAS_BIAS>(v[8 * r + 4 * h + 3], dq, bias, leaky);
                reinterpret_cast<float4 *>(row)[h] = o;
            }
        } else {
#pragma unroll
            for (int cidx = 0; cidx < 8; ++cidx)
                if (cidx < cols_live) row[cidx] = epi_value<ACT, HAS_BIAS>(v[8 * r + cidx], dq, bias, leaky);
        }
    }
}

// Pixel-major fp32 tensors in the swapped orientation: for one pixel the warp's 32 lanes touch 32 consecutive floats
// (residual read, fp32 write) and 32 consecutive int8 (requantized write): every access is one coalesced line.
template <int ACT, bool HAS_BIAS, bool AFTER>
__device__ __forceinline__ bool swap_nhwc_run(const int (&v)[32], float dq, float bias, float leaky,
                                              const float *__restrict__ res, float *__restrict__ out_f32,
                                              int8_t *__restrict__ out_i8, bool write_i8, float rs0, float rs1, int split,
                                              uint32_t O, uint32_t out_cp, bool ch_live) {
    float worst = 0.0f;
#pragma unroll
    for (int j0 = 0; j0 < 32; j0 += 8) {
        float r[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) r[k] = (res && ch_live) ? __ldg(res + (uint32_t)(j0 + k) * O) : 0.0f;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const int j = j0 + k;
            float t = __fmul_rn(__int2float_rn(v[j]), dq);
            if (HAS_BIAS) t = __fadd_rn(t, bias);
            if (res && !AFTER) t = __fadd_rn(t, r[k]);
            if (ACT == TSB_ACT_RELU) t = fmaxf(t, 0.0f);
            if (ACT == TSB_ACT_LEAKY_RELU) t = t > 0.0f ? t : __fmul_rn(t, leaky);
            if (res && AFTER) t = __fadd_rn(t, r[k]);
            if (out_f32 && ch_live) out_f32[(uint32_t)j * O] = t;
            if (out_i8) {
                const float u = __fmul_rn(t, j < split ? rs0 : rs1);
                worst = max_nan(worst, fabsf(u));
                const float mag = __fadd_rz(fabsf(u), 0.5f);
                const float sm = __int_as_float((__float_as_int(mag) & 0x7fffffff) | (__float_as_int(u) & 0x80000000));
                int q;
                asm("cvt.rzi.s8.f32 %0, %1;" : "=r"(q) : "f"(sm));
                if (write_i8) out_i8[(uint32_t)j * out_cp] = (int8_t)q;   // redone by the caller if the check below fails
            }
        }
    }
    return !__any_sync(0xffffffffu, !(worst < 2147483648.0f));
}

// run FN<activation, has_bias>(args...) for the runtime activation / bias combination
#define TSB_EPI_DISPATCH_W(RESULT, FN, W_, ...)                                                           \
    do {                                                                                                  \
        if (has_bias) {                                                                                   \
            if (act == TSB_ACT_RELU) RESULT FN<TSB_ACT_RELU, true, W_>(__VA_ARGS__);                      \
            else if (act == TSB_ACT_LEAKY_RELU) RESULT FN<TSB_ACT_LEAKY_RELU, true, W_>(__VA_ARGS__);     \
            else RESULT FN<TSB_ACT_NONE, true, W_>(__VA_ARGS__);                                          \
        } else {                                                                                          \
            if (act == TSB_ACT_RELU) RESULT FN<TSB_ACT_RELU, false, W_>(__VA_ARGS__);                     \
            else if (act == TSB_ACT_LEAKY_RELU) RESULT FN<TSB_ACT_LEAKY_RELU, false, W_>(__VA_ARGS__);    \
            else RESULT FN<TSB_ACT_NONE, false, W_>(__VA_ARGS__);                                         \
        }                                                                                                 \
    } while (0)
// the two residual epilogues: a second instantiation for "residual after the activation"
#define TSB_EPI_DISPATCH_RES_W(RESULT, FN, W_, ...)                                                       \
    do {                                                                                                  \
        if (epi.res_after) TSB_EPI_DISPATCH_W(RESULT, FN, W_ TSB_COMMA true, __VA_ARGS__);                \
        else TSB_EPI_DISPATCH_W(RESULT, FN, W_ TSB_COMMA false, __VA_ARGS__);                             \
    } while (0)
#define TSB_COMMA ,
#define TSB_EPI_DISPATCH_SWAPRES(RESULT, FN, ...)                                                         \
    do {                                                                                                  \
        if (epi.res_after) TSB_EPI_DISPATCH_W(RESULT, FN, true, __VA_ARGS__);                             \
        else TSB_EPI_DISPATCH_W(RESULT, FN, false, __VA_ARGS__);                                          \
    } while (0)
#define TSB_EPI_DISPATCH(RESULT, FN, ...)                                                                 \
    do {                                                                                                  \
        if (has_bias) {                                                                                   \
            if (act == TSB_ACT_RELU) RESULT FN<TSB_ACT_RELU, true>(__VA_ARGS__);                          \
            else if (act == TSB_ACT_LEAKY_RELU) RESULT FN<TSB_ACT_LEAKY_RELU, true>(__VA_ARGS__);         \
            else RESULT FN<TSB_ACT_NONE, true>(__VA_ARGS__);                                              \
        } else {                                                                                          \
            if (act == TSB_ACT_RELU) RESULT FN<TSB_ACT_RELU, false>(__VA_ARGS__);                         \
            else if (act == TSB_ACT_LEAKY_RELU) RESULT FN<TSB_ACT_LEAKY_RELU, false>(__VA_ARGS__);        \
            else RESULT FN<TSB_ACT_NONE, false>(__VA_ARGS__);                                             \
        }                                                                                                 \
    } while (0)

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, int (&v)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ldw(uint32_t taddr, int (&v)[32]) { tmem_ld32(taddr, v); }
__device__ __forceinline__ void tmem_ldw(uint32_t taddr, int (&v)[16]) { tmem_ld16(taddr, v); }

// one tensor-memory column of this warp's 32 lanes (used by the rolled, element-by-element paths)
__device__ __forceinline__ int tmem_ld1(uint32_t taddr) {
    int r;
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x1.b32 {%0}, [%1];" : "=r"(r) : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
    return r;
}

// ---------------------------------------------------------------------------------------------------------
// kernel
// ---------------------------------------------------------------------------------------------------------
// Division by a divisor known at launch time as multiply-high, add and shift (round-up method for 32-bit unsigned
// numerators below 2^31): the role threads divide once or twice per tile and a hardware-less 32-bit division costs them
// more than a hundred cycles each.
struct FastDiv {
    uint32_t mul = 0, shr = 0;
    FastDiv() = default;
    explicit FastDiv(uint32_t d) {
        uint32_t l = 0;
        while ((1ull << l) < d) ++l;
        shr = l;
        mul = (uint32_t)((((1ull << 32) * ((1ull << l) - d)) / d) + 1);
    }
    __device__ __forceinline__ int div(int n) const {
        return (int)(((uint64_t)__umulhi((uint32_t)n, mul) + (uint32_t)n) >> shr);
    }
};

struct KernelParams {
    int M_total;     // N*OH*OW
    int OW, P;       // P = OH*OW
    int KH, KW;
    int sh, sw, dh, dw, pad_t, pad_l;
    int Cp;          // channels of the staged input per filter tap
    int num_m_tiles, num_n_tiles;   // pixel tiles, channel tiles
    FastDiv d_P, d_OW, d_m_tiles, d_n_tiles, d_segs, d_OH, d_dh;   // dividers by P, OW, num_m_tiles, num_n_tiles, rows_segs, rows_OH, dh
    int per_sample_scale;  // requantize: scale index = image index
    int epi_mode;          // kEpi*: which epilogue code path full 32-column chunks take
    int a_tiled;           // activations are a plain [M][Cp] matrix (1x1, stride 1, no padding): 2-D tile loads
    // shared-memory plan (bytes from the 1024-aligned base)
    int stages;            // pipeline stages (<= kMaxStages)
    uint32_t stage_bytes;  // one stage: kgroup units of (pixel tile, followed by the weight tile unless the weights are resident)
    int kgroup;            // general mode: K blocks per stage (1, 2 or 4; divides the K blocks of a tile): one barrier wait
                           // and one commit of the MMA issuer serve kgroup * BK/32 MMAs
    uint32_t unit_bytes;   // one K block inside a stage
    int b_resident;        // all K blocks of this CTA's weight tile stay in shared memory; only activations stream
    uint32_t b_off;        // offset of the resident weights
    uint32_t bar_off;      // offset of the mbarriers; tensor-memory slot, abort flag and epilogue tables follow
    uint32_t stg_off;      // staged epilogue: offset of the four quads' tiles (1024-aligned); per quad an fp32 tile (when
    int stg_f32;           // stg_f32) followed by an int8 tile
    // raw-row mode (rows_segs > 0): a tile is up to 128 consecutive pixels of ONE output row; per filter row the
    // producer copies the staged bytes under those pixels once, and the MMA reads them through a sliding descriptor
    int rows_segs;         // tiles per output row (0: mode off)
    int rows_OH, rows_H;   // output rows per image, staged input rows per image
    uint32_t rows_bytes;   // bytes copied per tile and filter row
    long long rows_stride_h, rows_stride_n;   // bytes between staged rows / images
    const int8_t *rows_x;  // the folded staging
    // patch mode (patch != 0; stride-1 filters with several taps): a tile is 8 pixels wide and PIX/8 pixels high; ONE
    // tiled tensor-map load per channel block brings the input patch under it, halo included, and every filter tap reads
    // its shifted window out of that patch through a descriptor whose start is moved by whole pixels
    int patch;
    int patch_tiles_w, patch_tiles_hw;        // tiles across an image, tiles per image
    int patch_pw;                             // patch width in pixels: 8 + (KW-1)*dw
    uint32_t patch_bytes;                     // bytes of one patch (one channel block)
    int OH;
    FastDiv d_tiles_w, d_tiles_hw;
    int res_prefetch;      // the residual tensor has a tensor map (map_r): the epilogue prefetches its boxes into L2 two
                           // chunks ahead of the loads, so that those find the data on chip
    int *status;     // device word: 0 ok, else the code of the wait that ran out
    unsigned long long *trace;  // profiling builds: timeline of CTA 0, 8 stamps per tile, 32 tiles (null otherwise)
};

__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
#ifdef TSB_ENABLE_TRACE
#define TSB_TRACE(tile_index, slot)                                                              \
    do {                                                                                         \
        if (kp.trace && blockIdx.x == 0 && (tile_index) < 32) kp.trace[(tile_index) * 8 + (slot)] = global_ns(); \
    } while (0)
// cycle accounting of the MMA issuer (profiling builds): where its time goes, summed over the CTA's tiles
#define TSB_CYC_DECL long long cyc_full = 0, cyc_tempty = 0, cyc_issue = 0, cyc_commit = 0, cyc_t0 = clock64(), cyc_tmp = 0; int cyc_waits = 0
#define TSB_CYC_START cyc_tmp = clock64()
#define TSB_CYC_ADD(which) do { which += clock64() - cyc_tmp; } while (0)
#define TSB_CYC_REPORT(ntiles)                                                                   \
    do {                                                                                         \
        if (kp.trace && blockIdx.x == 0) {                                                       \
            kp.trace[31 * 8 + 0] = (unsigned long long)(clock64() - cyc_t0);                     \
            kp.trace[31 * 8 + 1] = (unsigned long long)cyc_full;                                 \
            kp.trace[31 * 8 + 2] = (unsigned long long)cyc_tempty;                               \
            kp.trace[31 * 8 + 3] = (unsigned long long)(ntiles);                                 \
            kp.trace[31 * 8 + 4] = (unsigned long long)cyc_waits;                                \
            kp.trace[31 * 8 + 5] = (unsigned long long)cyc_issue;                                \
            kp.trace[31 * 8 + 6] = (unsigned long long)cyc_commit;                               \
        }                                                                                        \
    } while (0)
#else
#define TSB_TRACE(tile_index, slot) do { } while (0)
#define TSB_CYC_DECL do { } while (0)
#define TSB_CYC_START do { } while (0)
#define TSB_CYC_ADD(which) do { } while (0)
#define TSB_CYC_REPORT(ntiles) do { } while (0)
#endif

// raw-row mode: the filter rows kh_lo..kh_hi that meet an input row for output row oh (a contiguous, non-empty range)
__device__ __forceinline__ void rows_span(const KernelParams &kp, int oh, int &kh_lo, int &kh_hi) {
    const int top = oh * kp.sh - kp.pad_t;                 // input row under filter row 0
    kh_lo = top >= 0 ? 0 : kp.d_dh.div(-top + kp.dh - 1);
    kh_hi = min(kp.KH - 1, kp.d_dh.div(kp.rows_H - 1 - top));
}

constexpr int kModeGeneral = 0, kModeRows = 1, kModePatch = 2;

// Projected-shortcut kernels (DUAL): a second, 1x1 convolution over the same output pixels (the projection shortcut of a
// residual block: its own input, weights, dequantize scales and bias) runs in the same tile, into a second accumulator,
// ahead of the main convolution; the epilogue dequantizes it (+ bias) and uses the result as the main convolution's
// residual.  The projection's fp32 output never exists in global memory.
struct alignas(64) DualParams {
    CUtensorMap map_a2, map_b2;   // the projection's activations ([M][Cp2] tiles or a 1x1 im2col walk with its stride) and weights
    const float *dq2, *bias2;     // its dequantize scales and (optional) bias, per output channel
    int k2_iters;                 // its K blocks per tile: Cp2 / BK
    int Cp2, a2_tiled, sh2, sw2;
    int concat;                   // 1: no second accumulator and no residual -- the second convolution's K blocks are summed into
                                  // the main accumulator, i.e. ONE convolution over the channel concatenation of the two inputs
                                  // (int32 sums are exact in any order); dq2 / bias2 are unused
};
struct NoDual {};
constexpr int kMaxStages = 24;
constexpr uint32_t kMaxDynamicSmem = 227 * 1024;

// barriers: full[stages], empty[stages], tmem_full[4], tmem_empty[4], b_full, b_free, staged_residual[4]
__host__ __device__ constexpr uint32_t num_barriers(int stages) { return 2u * (uint32_t)stages + 2u * kMaxAccBufs + 2u + 4u; }

// PIX pixels x CH channels per tile.  Normal orientation: the pixel tile is the MMA's A operand (M = 128 pixels), the
// weight tile its B operand (N = BN channels).  Swapped orientation: the weight tile is A (M = 128 channels, rows
// beyond O zero-filled by the tensor map) and the pixel tile is B (N = BN pixels).  An MMA instruction takes the same
// 128 cycles whatever its N, so layers with at most 128 output channels run swapped: N = 256 pixels fills the
// instruction where N = O would leave it half or three-quarters empty.
// MODE: how activations reach shared memory -- kModeGeneral (im2col or plain 2-D tile loads), kModeRows (raw-row), kModePatch.
// A compile-time parameter: the role loops of each mode stay short and keep their registers.
template <int BN, int BK, bool SWAP, int MODE, bool DUAL = false>
__global__ void __launch_bounds__(kThreads, 1)
conv_i8_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                  const __grid_constant__ CUtensorMap map_r, const __grid_constant__ CUtensorMap map_of,
                  const __grid_constant__ CUtensorMap map_oi, const __grid_constant__ KernelParams kp,
                  const __grid_constant__ EpiParams epi,
                  const __grid_constant__ std::conditional_t<DUAL, DualParams, NoDual> dual) {
    static_assert(!DUAL || (!SWAP && MODE == kModeGeneral), "projected-shortcut kernels: normal orientation, general mode");
    constexpr int PIX = SWAP ? BN : kBM;      // pixels per tile
    constexpr int CH = SWAP ? kBM : BN;       // output channels per tile
    constexpr uint32_t kPixBytes = PIX * BK, kWgtBytes = CH * BK;
    constexpr int kBufs = 512 / BN < kMaxAccBufs ? 512 / BN : kMaxAccBufs;   // accumulator buffers: 2 for BN = 256, else 4
    constexpr uint32_t kTmemCols = 512;                                       // one CTA per SM: all of tensor memory
    const int kStages = kp.stages;

    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t *base_ptr = smem_raw + (base - raw);
    const uint32_t bar_full = base + kp.bar_off;
    const uint32_t bar_empty = bar_full + 8 * kStages;
    const uint32_t bar_tfull = bar_empty + 8 * kStages;
    const uint32_t bar_tempty = bar_tfull + 8 * kMaxAccBufs;
    const uint32_t bar_bfull = bar_tempty + 8 * kMaxAccBufs;
    const uint32_t bar_bfree = bar_bfull + 8;
    const uint32_t bar_stg = bar_bfree + 8;     // one per epilogue quad: a staged residual tile has landed
    const uint32_t slot_off = kp.bar_off + 8 * num_barriers(kStages);
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(base_ptr + slot_off);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(base_ptr + slot_off + 4);
    float *table = reinterpret_cast<float *>(base_ptr + ((slot_off + 8 + 15) & ~15u));
    // patch mode: (byte offset >> 4) of every filter tap's window inside a patch, for the MMA issuer
    uint32_t *tap16 = reinterpret_cast<uint32_t *>(table + kMaxAccBufs * 2 * BN);
    const uint32_t w_res = base + kp.b_off;   // resident weights

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int total_tiles = kp.num_m_tiles * kp.num_n_tiles;
    const int k_iters = kp.KH * kp.KW * (kp.Cp / BK);
    int k_sc = 0;                              // K blocks of the projection, which come first in every tile
    bool concat = false;
    if constexpr (DUAL) { k_sc = dual.k2_iters; concat = dual.concat != 0; }
    // This CTA's tiles.  Streaming weights: tiles blockIdx.x, +gridDim.x, ... with the channel tile running fastest.
    // Resident weights: one contiguous range of the channel-major tile order, so the weight tile changes at most a
    // few times.
    const int tile_lo = kp.b_resident ? (int)((long long)blockIdx.x * total_tiles / gridDim.x) : 0;
    const int tile_hi = kp.b_resident ? (int)((long long)(blockIdx.x + 1) * total_tiles / gridDim.x) : 0;
    const int my_tiles = kp.b_resident ? tile_hi - tile_lo : (total_tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;
    // Accumulator buffers in use = epilogue groups: as many as tensor memory holds (kBufs), but no more than this CTA has
    // tiles -- a CTA with a single tile puts all sixteen epilogue warps on it.
    // (a projected-shortcut tile holds two accumulators: buffers 2a and 2a+1 of logical buffer a)
    const int nbuf = DUAL ? ((kBufs >= 4 && my_tiles >= 2) ? 2 : 1) : (my_tiles >= 4 && kBufs >= 4 ? 4 : (my_tiles >= 2 ? 2 : 1));
    auto decode = [&](int i, int &m_tile, int &n_tile) {   // m_tile: pixel tile, n_tile: channel tile
        if (kp.b_resident) {
            const int t = tile_lo + i;
            n_tile = kp.d_m_tiles.div(t); m_tile = t - n_tile * kp.num_m_tiles;
        } else {
            const int t = (int)blockIdx.x + i * (int)gridDim.x;
            m_tile = kp.d_n_tiles.div(t); n_tile = t - m_tile * kp.num_n_tiles;
        }
    };

    if (threadIdx.x == 0) {
        TSB_TRACE(0, 7);
        for (int s = 0; s < kStages; ++s) { mbar_init(bar_full + 8 * s, 1); mbar_init(bar_empty + 8 * s, 1); }
        for (int a = 0; a < kMaxAccBufs; ++a) { mbar_init(bar_tfull + 8 * a, 1); mbar_init(bar_tempty + 8 * a, kEpiThreads / nbuf); }
        mbar_init(bar_bfull, 1);
        mbar_init(bar_bfree, 1);
        for (int q = 0; q < kQuads; ++q) mbar_init(bar_stg + 8 * q, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(const_cast<uint32_t *>(tmem_slot)), kTmemCols);
        tmem_relinquish();
    }
    if (MODE == kModePatch && threadIdx.x >= 32 * kEpiWarp0) {
        for (int t = (int)threadIdx.x - 32 * kEpiWarp0; t < kp.KH * kp.KW; t += kEpiThreads) {
            const int kh = t / kp.KW, kw = t - kh * kp.KW;
            tap16[t] = (uint32_t)((kh * kp.dh * kp.patch_pw + kw * kp.dw) * BK) >> 4;
        }
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    pdl_sync();   // everything above touched only shared and tensor memory

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            int stage = 0; uint32_t phase = 0;
            bool ok = true;
            int cur_n = -1, w_loads = 0;
            for (int i = 0; i < my_tiles && ok; ++i) {
                TSB_TRACE(i, 0);
                int m_tile, n_tile;
                decode(i, m_tile, n_tile);
                const int m0 = m_tile * PIX;
                const int img = kp.d_P.div(m0), rem = m0 - img * kp.P;
                const int oh = kp.d_OW.div(rem), ow = rem - oh * kp.OW;
                const int wc = ow * kp.sw - kp.pad_l, hc = oh * kp.sh - kp.pad_t;
                if (kp.b_resident && n_tile != cur_n) {
                    // (re)load the whole weight tile; wait until the MMAs that read the previous one are done
                    if (w_loads > 0 && !mbar_wait(bar_bfree, (uint32_t)(w_loads - 1) & 1u, abort_flag)) {
                        if (!*abort_flag) { *abort_flag = 1; atomicExch(kp.status, 5); }
                        break;
                    }
                    mbar_arrive_expect_tx(bar_bfull, (uint32_t)(k_iters + k_sc) * kWgtBytes);
                    if constexpr (DUAL)
                        for (int it = 0; it < k_sc; ++it)
                            tma_load_2d(w_res + (uint32_t)it * kWgtBytes, &dual.map_b2, bar_bfull, it * BK, n_tile * CH);
                    for (int it = 0; it < k_iters; ++it)
                        tma_load_2d(w_res + (uint32_t)(k_sc + it) * kWgtBytes, &map_b, bar_bfull, it * BK, n_tile * CH);
                    cur_n = n_tile;
                    ++w_loads;
                }
                if (MODE == kModePatch) {
                    const int p_img = kp.d_tiles_hw.div(m_tile), p_rem = m_tile - p_img * kp.patch_tiles_hw;
                    const int p_r = kp.d_tiles_w.div(p_rem), p_c = p_rem - p_r * kp.patch_tiles_w;
                    const int h0 = p_r * (PIX / 8) - kp.pad_t, w0 = p_c * 8 - kp.pad_l;
                    for (int cb = 0; cb < kp.Cp && ok; cb += BK) {
                        if (!mbar_wait(bar_empty + 8 * stage, phase ^ 1u, abort_flag)) {
                            if (!*abort_flag) { *abort_flag = 1; atomicExch(kp.status, 1); }
                            ok = false;
                            break;
                        }
                        mbar_arrive_expect_tx(bar_full + 8 * stage, kp.patch_bytes);
                        tma_load_4d(base + stage * kp.stage_bytes, &map_a, bar_full + 8 * stage, cb, w0, h0, p_img);
                        if (++stage == kStages) { stage = 0; phase ^= 1u; }
                    }
                } else if (MODE == kModeRows) {
                    // One copy per output row (per run of its segments that this CTA owns): the staged bytes from the
                    // first to the last input row the filter meets, from this segment to the end of the row.  The
                    // following tiles of the same output row read the same stage at +2048 bytes per segment.
                    const int row_id = kp.d_segs.div(m_tile), seg = m_tile - row_id * kp.rows_segs;
                    if (seg == 0 || i == 0) {
                        const int r_img = kp.d_OH.div(row_id), r_oh = row_id - r_img * kp.rows_OH;
                        int kh_lo, kh_hi;
                        rows_span(kp, r_oh, kh_lo, kh_hi);
                        if (!mbar_wait(bar_empty + 8 * stage, phase ^ 1u, abort_flag)) {
                            if (!*abort_flag) { *abort_flag = 1; atomicExch(kp.status, 1); }
                            break;
                        }
                        const int ih_lo = r_oh * kp.sh - kp.pad_t + kh_lo * kp.dh;
                        const uint32_t bytes = (uint32_t)((kh_hi - kh_lo) * kp.dh) * (uint32_t)kp.rows_stride_h +
                                               (uint32_t)(kp.rows_segs - 1 - seg) * (PIX * 16) + kp.rows_bytes;
                        mbar_arrive_expect_tx(bar_full + 8 * stage, bytes);
                        bulk_load(base + stage * kp.stage_bytes,
                                  kp.rows_x + r_img * kp.rows_stride_n + ih_lo * kp.rows_stride_h + (long long)seg * (PIX * 16),
                                  bytes, bar_full + 8 * stage);
                        if (++stage == kStages) { stage = 0; phase ^= 1u; }
                    }
                } else {
                    int gk = 0;   // K block inside the current stage
                    if constexpr (DUAL) {
                        const int wc2 = ow * dual.sw2, hc2 = oh * dual.sh2;   // the projection: 1x1, no padding
                        for (int cb = 0; cb < dual.Cp2; cb += BK) {
                            if (gk == 0) {
                                if (!mbar_wait(bar_empty + 8 * stage, phase ^ 1u, abort_flag)) {
                                    if (!*abort_flag) { *abort_flag = 1; atomicExch(kp.status, 1); }
                                    ok = false;
                                    break;
                                }
                                mbar_arrive_expect_tx(bar_full + 8 * stage, (uint32_t)kp.kgroup * (kp.b_resident ? kPixBytes : kPixBytes + kWgtBytes));
                            }
                            const uint32_t sp = base + stage * kp.stage_bytes + (uint32_t)gk * kp.unit_bytes, sw = sp + kPixBytes;
                            if (dual.a2_tiled) tma_load_2d(sp, &dual.map_a2, bar_full + 8 * stage, cb, m0);
                            else tma_load_im2col_4d(sp, &dual.map_a2, bar_full + 8 * stage, cb, wc2, hc2, img, (uint16_t)0, (uint16_t)0);
                            if (!kp.b_resident) tma_load_2d(sw, &dual.map_b2, bar_full + 8 * stage, cb, n_tile * CH);
                            if (++gk == kp.kgroup) {
                                gk = 0;
                                if (++stage == kStages) { stage = 0; phase ^= 1u; }
                            }
                        }
                    }
                    for (int kh = 0; kh < kp.KH && ok; ++kh)
                        for (int kw = 0; kw < kp.KW && ok; ++kw)
                            for (int cb = 0; cb < kp.Cp; cb += BK) {
                                if (gk == 0) {
                                    if (!mbar_wait(bar_empty + 8 * stage, phase ^ 1u, abort_flag)) {
                                        if (!*abort_flag) { *abort_flag = 1; atomicExch(kp.status, 1); }
                                        ok = false;
                                        break;
                                    }
                                    mbar_arrive_expect_tx(bar_full + 8 * stage, (uint32_t)kp.kgroup * (kp.b_resident ? kPixBytes : kPixBytes + kWgtBytes));
                                }
                                const uint32_t sp = base + stage * kp.stage_bytes + (uint32_t)gk * kp.unit_bytes, sw = sp + kPixBytes;
                                if (kp.a_tiled)
                                    tma_load_2d(sp, &map_a, bar_full + 8 * stage, cb, m0);
                                else
                                    tma_load_im2col_4d(sp, &map_a, bar_full + 8 * stage, cb, wc, hc, img,
                                                       (uint16_t)(kw * kp.dw), (uint16_t)(kh * kp.dh));
                                if (!kp.b_resident)
                                    tma_load_2d(sw, &map_b, bar_full + 8 * stage, (kh * kp.KW + kw) * kp.Cp + cb, n_tile * CH);
                                if (++gk == kp.kgroup) {
                                    gk = 0;
                                    if (++stage == kStages) { stage = 0; phase ^= 1u; }
                                }
                            }
                }
                TSB_TRACE(i, 1);
            }
        }
    } else if (warp <= kIssuers) {
        // ------------------------------------------------------------------ MMA issuers
        // One thread feeds the tensor core.  An MMA with N = 64 executes in 48 cycles, while a thread that runs alone in
        // its warp pays tens of cycles for every branch, shared-memory load or dependent instruction (measured: a loop
        // that computes a descriptor per MMA issues one every 80-180 cycles, straight-line code with the operands in
        // registers one every 48-55).  So: the MMAs of a stage are straight-line code; descriptors are a loop-invariant
        // high word plus a 14-bit address field (in 16-byte units) that takes one add; per-tap offsets sit in registers;
        // slots that do not apply are switched off by predicate; and one barrier wait / one commit serve as many MMAs as
        // the stage holds.
        // Issuing costs the thread far more than an MMA with a small N takes to execute, and what it spends between two
        // MMAs is not hidden behind the tensor core's work on the earlier one (measured: ~125 cycles per MMA at N = 64,
        // ~190 at N = 256).  So kIssuers warps issue, each for every kIssuers-th tile of the CTA: while one computes
        // descriptors, waits and commits, the tensor core runs the other's MMAs.  A tile's stages, accumulator buffer and
        // barriers belong to the issuer of that tile alone.  Where tiles share state that one thread has to order -- a
        // raw-row stage shared by the segments of an output row, or resident weights that are replaced inside this CTA's
        // tile range -- the first issuer takes every tile.
        if (lane == 0) {
            constexpr uint32_t idesc = instr_desc<BN>();
            constexpr uint64_t dhi = smem_desc_hi<BK>(8 * BK);
            constexpr uint32_t kWgt16 = kWgtBytes >> 4, kPix16 = kPixBytes >> 4;
            constexpr int kMmaPerBlock = BK / 32;
            const uint32_t base16 = base >> 4, stage16 = kp.stage_bytes >> 4, wres16 = w_res >> 4, unit16 = kp.unit_bytes >> 4;
            const int resident = kp.b_resident;
            bool ok = true;
            int rows_seg_first = 0;
            int first_m = 0, first_n = 0, last_m = 0, last_n = 0;
            if (my_tiles > 0) { decode(0, first_m, first_n); decode(my_tiles - 1, last_m, last_n); }
            // pipeline stages a tile consumes
            const int spt = MODE == kModePatch ? kp.Cp / BK : (MODE == kModeRows ? 1 : (k_iters + k_sc) / kp.kgroup);
            // A barrier wait names a phase by its parity only, so a waiter must never be two rounds of the stage ring away
            // from the phase it means.  With several issuers that holds when the ring has room for one tile of each
            // (kStages >= issuers * spt): the round before the one an issuer waits for then lies in tiles that were
            // loaded before its own previous tile, whose loads it has seen complete.
            const bool shared_state = (MODE == kModeRows && kp.rows_segs > 1) || (resident && first_n != last_n);
            // (an issuer must also own its accumulator buffers: with a single logical buffer one thread takes every tile)
            const int issuers = (shared_state || kStages < kIssuers * spt || (DUAL && nbuf < kIssuers)) ? 1 : kIssuers;
            const int me = warp - 1;
            int stage = 0; uint32_t phase = 0;
            auto advance = [&](int n) {      // move n stages on (n >= 0)
                stage += n;
                while (stage >= kStages) { stage -= kStages; phase ^= 1u; }
            };
            advance(me * spt);
            int w_loads = resident ? 1 : 0;   // without shared state the resident weights are loaded exactly once
            int cur_n = -1;
            // patch mode with up to nine filter taps (3x3, 1x3 ...): the taps' window offsets live in registers
            const int taps = kp.KH * kp.KW;
            uint32_t tapreg[9];
#pragma unroll
            for (int t = 0; t < 9; ++t) tapreg[t] = (MODE == kModePatch && t < taps) ? tap16[t] : 0u;
            TSB_CYC_DECL;
            for (int local = me; local < my_tiles && ok && me < issuers; local += issuers) {
                int m_tile, n_tile;
                decode(local, m_tile, n_tile);
                uint32_t st16 = base16 + (uint32_t)stage * stage16;    // (address >> 4) of the current stage
                const int acc = local & (nbuf - 1);
                const uint32_t acc_phase = (uint32_t)(local / nbuf) & 1u;
                TSB_CYC_START;
                if (!mbar_wait(bar_tempty + 8 * acc, acc_phase ^ 1u, abort_flag)) {
                    if (!*abort_flag) { *abort_flag = 1; atomicExch(kp.status, 2); }
                    break;
                }
                TSB_CYC_ADD(cyc_tempty);
                if (resident && n_tile != cur_n) {
                    // the (w_loads)-th load of resident weights: completes phase (w_loads - 1) of its barrier
                    if (!mbar_wait(bar_bfull, (uint32_t)(w_loads - 1) & 1u, abort_flag)) {
                        if (!*abort_flag) { *abort_flag = 1; atomicExch(kp.status, 6); }
                        break;
                    }
                    cur_n = n_tile;
                    ++w_loads;
                }
                tc_fence_after();
                if (me == 0) TSB_TRACE(local, 2);
                uint32_t d_tmem = tmem_base + (uint32_t)(DUAL ? (2 * acc + (concat ? 0 : 1)) * BN : acc * BN);   // DUAL: the projection's accumulator first
                uint32_t accumulate = 0;
                if (MODE == kModePatch) {
                    const int n_cb = kp.Cp / BK;
                    const uint64_t dhi_patch = smem_desc_hi<BK>((uint32_t)kp.patch_pw * BK);   // next tile row = next patch row
                    const uint32_t hi_patch = (uint32_t)(dhi_patch >> 32), hi_plain = (uint32_t)(dhi >> 32);
                    const uint32_t wtap16 = (uint32_t)n_cb * kWgt16;                          // next tap of the resident weights
                    for (int cbi = 0; cbi < n_cb && ok; ++cbi) {
                        TSB_CYC_START;
                        if (!mbar_wait(bar_full + 8 * stage, phase, abort_flag)) {
                            if (!*abort_flag) { *abort_flag = 1; atomicExch(kp.status, 3); }
                            ok = false;
                            break;
                        }
                        TSB_CYC_ADD(cyc_full);
                        tc_fence_after();
                        if (cbi == 0 && me == 0) TSB_TRACE(local, 3);
                        uint32_t w16 = wres16 + (uint32_t)cbi * kWgt16;
                        TSB_CYC_START;
                        if (taps == 9) {
                            // 3x3: eighteen or thirty-six MMAs, two adds each
                            const uint32_t p_lo = st16 | kDescLbo;
#pragma unroll
                            for (int t = 0; t < 9; ++t) {
                                const uint32_t a_lo = p_lo + tapreg[t], w_lo = (w16 | kDescLbo) + (uint32_t)t * wtap16;
#pragma unroll
                                for (int k = 0; k < kMmaPerBlock; ++k) {
                                    const uint64_t dp = desc_pair(hi_patch, a_lo + 2u * k), dw = desc_pair(hi_plain, w_lo + 2u * k);
                                    mma_i8(d_tmem, SWAP ? dw : dp, SWAP ? dp : dw, idesc, (t | k) ? 1u : accumulate);
                                }
                            }
                            accumulate = 1u;
                        } else if (taps < 9) {
#pragma unroll
                            for (int t = 0; t < 9; ++t) {
                                const uint64_t dp = dhi_patch | (uint64_t)(st16 + tapreg[t]);
                                const uint64_t dw = dhi | (uint64_t)w16;
                                const uint64_t da = SWAP ? dw : dp, db = SWAP ? dp : dw;
                                const uint32_t on = t < taps ? 1u : 0u;
#pragma unroll
                                for (int k = 0; k < kMmaPerBlock; ++k)
                                    mma_i8_if(d_tmem, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc, (t | k) ? 1u : accumulate, on);
                                w16 += wtap16;
                            }
                            accumulate = 1u;
                        } else {
                            for (int t = 0; t < taps; ++t) {
                                const uint64_t dp = dhi_patch | (uint64_t)(st16 + tap16[t]);
                                const uint64_t dw = dhi | (uint64_t)w16;
                                const uint64_t da = SWAP ? dw : dp, db = SWAP ? dp : dw;
#pragma unroll
                                for (int k = 0; k < kMmaPerBlock; ++k) {
                                    mma_i8(d_tmem, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc, accumulate);
                                    accumulate = 1u;
                                }
                                w16 += wtap16;
                            }
                        }
                        TSB_CYC_ADD(cyc_issue);
                        TSB_CYC_START;
                        tc_commit(bar_empty + 8 * stage);
                        TSB_CYC_ADD(cyc_commit);
                        st16 += stage16;
                        if (++stage == kStages) { stage = 0; phase ^= 1u; st16 = base16; }
                    }
                } else if (!SWAP && MODE == kModeRows) {
                    const int row_id = kp.d_segs.div(m_tile), seg = m_tile - row_id * kp.rows_segs;
                    int kh_lo, kh_hi;
                    rows_span(kp, row_id - kp.d_OH.div(row_id) * kp.rows_OH, kh_lo, kh_hi);
                    if (seg == 0 || local == me) {     // the stage of this output row: loaded once, used by all its segments
                        TSB_CYC_START;
                        if (!mbar_wait(bar_full + 8 * stage, phase, abort_flag)) {
                            if (!*abort_flag) { *abort_flag = 1; atomicExch(kp.status, 3); }
                            break;
                        }
                        TSB_CYC_ADD(cyc_full);
                        tc_fence_after();
                        rows_seg_first = seg;
                    }
                    if (me == 0) TSB_TRACE(local, 3);
                    // sliding descriptor (no swizzle, LBO 16, SBO 128): only its address field changes from row to row
                    const uint64_t dslide = smem_desc_sliding(0);
                    const uint32_t row16 = (uint32_t)kp.dh * (uint32_t)(kp.rows_stride_h >> 4);
                    // filter row kh reads the staged row (kh - kh_lo); rows outside [kh_lo, kh_hi] meet no input row
                    const uint32_t a16_0 = st16 + (uint32_t)(seg - rows_seg_first) * PIX - (uint32_t)kh_lo * row16;
                    if (kp.KH <= 8) {
                        // straight-line code for the filter heights in use (a predicated-off MMA still costs the issuing
                        // thread some 50 cycles, so the sequence is as long as the filter is high, not always eight)
                        auto issue_rows = [&](auto height) {
                            constexpr int kH = decltype(height)::value;
                            if (kh_lo == 0 && kh_hi == kH - 1) {
                                // every filter row meets an input row (all output rows but those at the image's edge): no
                                // predicates, accumulate flags known at compile time
#pragma unroll
                                for (int kh = 0; kh < kH; ++kh) {
                                    const uint64_t da = dslide | (uint64_t)((a16_0 + (uint32_t)kh * row16) & 0x3FFFu);
                                    const uint64_t db = dhi | (uint64_t)(wres16 + (uint32_t)kh * kWgt16);
#pragma unroll
                                    for (int k = 0; k < kMmaPerBlock; ++k)
                                        mma_i8(d_tmem, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc, (kh | k) ? 1u : 0u);
                                }
                                return;
                            }
#pragma unroll
                            for (int kh = 0; kh < kH; ++kh) {
                                const uint64_t da = dslide | (uint64_t)((a16_0 + (uint32_t)kh * row16) & 0x3FFFu);
                                const uint64_t db = dhi | (uint64_t)(wres16 + (uint32_t)kh * kWgt16);
                                const uint32_t on = (kh >= kh_lo && kh <= kh_hi && kh < kp.KH) ? 1u : 0u;
#pragma unroll
                                for (int k = 0; k < kMmaPerBlock; ++k)
                                    mma_i8_if(d_tmem, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc, (kh > kh_lo || k > 0) ? 1u : 0u, on);
                            }
                        };
                        if (kp.KH <= 3) issue_rows(std::integral_constant<int, 3>());
                        else if (kp.KH <= 5) issue_rows(std::integral_constant<int, 5>());
                        else if (kp.KH <= 7) issue_rows(std::integral_constant<int, 7>());
                        else issue_rows(std::integral_constant<int, 8>());
                    } else {
                        for (int kh = kh_lo; kh <= kh_hi; ++kh) {
                            const uint64_t da = dslide | (uint64_t)(a16_0 + (uint32_t)kh * row16);
                            const uint64_t db = dhi | (uint64_t)(wres16 + (uint32_t)kh * kWgt16);
#pragma unroll
                            for (int k = 0; k < kMmaPerBlock; ++k) {
                                mma_i8(d_tmem, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc, accumulate);
                                accumulate = 1u;
                            }
                        }
                    }
                    if (seg == kp.rows_segs - 1 || local == my_tiles - 1) {
                        tc_commit(bar_empty + 8 * stage);
                        advance(1);
                    }
                } else {
                    // general mode: a stage holds kgroup K blocks; one wait, kgroup * BK/32 MMAs in a row, one commit
                    uint32_t w16 = wres16;
                    const int G = kp.kgroup;
                    const uint32_t hi_plain = (uint32_t)(dhi >> 32);
                    auto issue_stage = [&](auto group) {      // the MMAs of one stage as straight-line code
                        constexpr int kG = decltype(group)::value;
#pragma unroll
                        for (int g = 0; g < kG; ++g) {
                            const uint32_t a_lo = (st16 | kDescLbo) + (uint32_t)g * unit16;
                            const uint32_t w_lo = resident ? (w16 | kDescLbo) + (uint32_t)g * kWgt16 : a_lo + kPix16;
#pragma unroll
                            for (int k = 0; k < kMmaPerBlock; ++k) {
                                // +32 bytes along K = +2 in the descriptor's 16-byte address units (inside the swizzle span)
                                const uint64_t dp = desc_pair(hi_plain, a_lo + 2u * k), dw = desc_pair(hi_plain, w_lo + 2u * k);
                                mma_i8(d_tmem, SWAP ? dw : dp, SWAP ? dp : dw, idesc, (g | k) ? 1u : accumulate);
                            }
                        }
                    };
                    for (int it = 0; it < k_iters + k_sc; it += G) {
                        if (DUAL && it == k_sc && !concat) { d_tmem -= BN; accumulate = 0u; }   // the main convolution's accumulator
                        TSB_CYC_START;
                        if (!mbar_wait(bar_full + 8 * stage, phase, abort_flag)) {
                            if (!*abort_flag) { *abort_flag = 1; atomicExch(kp.status, 3); }
                            ok = false;
                            break;
                        }
                        TSB_CYC_ADD(cyc_full);
                        tc_fence_after();
                        if (it == 0 && me == 0) TSB_TRACE(local, 3);
                        TSB_CYC_START;
                        if (G == 4) issue_stage(std::integral_constant<int, 4>());
                        else if (G == 2) issue_stage(std::integral_constant<int, 2>());
                        else issue_stage(std::integral_constant<int, 1>());
                        TSB_CYC_ADD(cyc_issue);
                        accumulate = 1u;
                        TSB_CYC_START;
                        tc_commit(bar_empty + 8 * stage);  // frees the stage once these MMAs have read it
                        TSB_CYC_ADD(cyc_commit);
                        w16 += (uint32_t)G * kWgt16;
                        st16 += stage16;
                        if (++stage == kStages) { stage = 0; phase ^= 1u; st16 = base16; }
                    }
                }
                TSB_CYC_START;
                if (ok) tc_commit(bar_tfull + 8 * acc);  // accumulator complete
                TSB_CYC_ADD(cyc_commit);
                if (ok && resident && issuers == 1) {
                    int nm = 0, nn = -1;
                    if (local + 1 < my_tiles) decode(local + 1, nm, nn);
                    if (nn != cur_n) tc_commit(bar_bfree);  // the resident weights may be replaced
                }
                advance((issuers - 1) * spt);             // skip the stages of the other issuers' tiles
                if (me == 0) TSB_TRACE(local, 4);
            }
            if (me == 0) TSB_CYC_REPORT((my_tiles + issuers - 1) / issuers);
        }
    } else {
        // ------------------------------------------------------------------ epilogue (the last sixteen warps)
        // A warp may read only the 32 tensor-memory lanes of its quarter (warp id mod 4); four warps share a
        // quarter and split the tile's columns between them in chunks of 32.
        // The sixteen warps form nbuf groups (of four, eight or all sixteen warps); group g owns accumulator buffer g and
        // takes the tiles local = g, g + nbuf, ...  One tile's epilogue is a chain of latencies (barrier, tensor-memory
        // load, arithmetic, stores); with the groups on different tiles those chains overlap.
        const int group_warps = 16 / nbuf;                       // 4, 8 or 16
        const int group_threads = 32 * group_warps;
        const int parts = group_warps / 4;                       // warps of a group per lane quarter: 1, 2 or 4
        const int quarter = warp & 3;
        const int group = (warp - kEpiWarp0) / group_warps;
        const int part = ((warp - kEpiWarp0) % group_warps) >> 2;        // 0 .. parts-1
        const int et = (int)threadIdx.x - 32 * kEpiWarp0 - group * group_threads;   // thread index inside the group
        const int row = quarter * 32 + lane;     // tensor-memory lane this thread reads
        constexpr int kChunks = BN / 32;
        constexpr int CW = 32;                   // normal orientation: columns a warp takes per step
        const bool has_bias = epi.bias != nullptr;
        const int act = epi.activation;
        uint32_t stg_phase[1] = {0u};            // staged epilogue: phase of this quad's residual barrier
        int table_n = -1;                        // channel tile this group's scale / bias table holds
        for (int local = group; local < my_tiles; local += nbuf) {
            const int acc = group;
            const uint32_t acc_phase = (uint32_t)(local / nbuf) & 1u;
            int m_tile, n_tile;
            decode(local, m_tile, n_tile);
            const int o_base = n_tile * CH;
            const int slot = DUAL ? 2 * acc : acc;          // first accumulator buffer (and table) of this tile
            float *t_dq = table + slot * 2 * BN, *t_bias = t_dq + BN;
            if (!SWAP && n_tile != table_n) {
                // this group's table of per-channel scales and biases: rebuilt only when the channel tile changes (never, for
                // layers of at most BN channels), between two barriers of the group
                if (table_n >= 0) asm volatile("bar.sync %0, %1;" ::"r"(1 + group), "r"(group_threads) : "memory");
                for (int j = et; j < BN; j += group_threads) {
                    const int o = o_base + j;
                    t_dq[j] = o < epi.O ? epi.dq[o] : 0.0f;
                    t_bias[j] = (o < epi.O && epi.bias) ? epi.bias[o] : 0.0f;
                    if constexpr (DUAL) {                   // the projection's table: the next slot
                        t_dq[2 * BN + j] = (o < epi.O && dual.dq2) ? dual.dq2[o] : 0.0f;
                        t_dq[3 * BN + j] = (o < epi.O && dual.bias2) ? dual.bias2[o] : 0.0f;
                    }
                }
                asm volatile("bar.sync %0, %1;" ::"r"(1 + group), "r"(group_threads) : "memory");
                table_n = n_tile;
            }
            // every warp waits for the accumulator on its own; one that gives up raises the CTA's abort flag, which ends
            // the other warps' waits as well
            if (!mbar_wait(bar_tfull + 8 * acc, acc_phase, abort_flag)) {
                if (!*abort_flag) { *abort_flag = 1; atomicExch(kp.status, 4); }
                break;
            }
            tc_fence_after();
            if (et == 0 && local < 32) TSB_TRACE(local, 5);
#ifdef TSB_ENABLE_TRACE
            // profiling experiment: with trace[255] set, the epilogue warps hand the accumulator back without touching it
            // (outputs are then garbage) -- shows how fast the other two roles run when left alone
            if (kp.trace && kp.trace[255] != 0) { tc_fence_before(); mbar_arrive(bar_tempty + 8 * acc); continue; }
#endif
            const uint32_t taddr0 = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(slot * BN);
            if (!SWAP) {
                int m = m_tile * PIX + row;
                bool live = m < kp.M_total;
                if (MODE == kModeRows) {
                    const int row_id = kp.d_segs.div(m_tile), ow = (m_tile - row_id * kp.rows_segs) * PIX + row;
                    live = ow < kp.OW;
                    m = row_id * kp.OW + ow;
                }
                if (MODE == kModePatch) {
                    const int p_img = kp.d_tiles_hw.div(m_tile), p_rem = m_tile - p_img * kp.patch_tiles_hw;
                    const int p_r = kp.d_tiles_w.div(p_rem), p_c = p_rem - p_r * kp.patch_tiles_w;
                    const int oh = p_r * (PIX / 8) + (row >> 3), ow = p_c * 8 + (row & 7);
                    live = oh < kp.OH && ow < kp.OW;
                    m = p_img * kp.P + oh * kp.OW + ow;
                }
                const int img = live ? kp.d_P.div(m) : 0;
                const int p = live ? m - img * kp.P : 0;
                if (kp.epi_mode == kEpiStaged) {
                    // ---- staged epilogue: residual in by tensor-map load, fp32 / int8 tiles out by tensor-map stores.
                    // A quad (the four warps of this group that share `part`, one per lane quarter = the tile's 128
                    // pixels) owns one fp32 tile and one int8 tile in shared memory and works through its 32-channel
                    // chunks; the warp of lane quarter 0 issues the quad's copies.
                    const int quad = group * parts + part;
                    const int bar_id = 5 + quad;                                   // named barriers 1..4 belong to the groups
                    const uint32_t stg = base + kp.stg_off + (uint32_t)quad * ((kp.stg_f32 ? kStageF32Bytes : 0u) + kStageI8Bytes);
                    float4 *r_tile = reinterpret_cast<float4 *>(base_ptr + (stg - base));
                    int4 *q_tile = reinterpret_cast<int4 *>(base_ptr + (stg - base) + (kp.stg_f32 ? kStageF32Bytes : 0u));
                    const uint32_t q_addr = stg + (kp.stg_f32 ? kStageF32Bytes : 0u);
                    const uint32_t rbar = bar_stg + 8 * quad;
                    const bool leader = quarter == 0 && lane == 0;
                    const bool has_res = epi.residual != nullptr, has_f32 = epi.out_f32 != nullptr, has_i8 = epi.out_i8 != nullptr;
                    // tile coordinates of the three tensor maps (innermost coordinate: the channel)
                    int c1 = m_tile * PIX, c2 = 0, c3 = 0;                          // general: [pixel][channel]
                    if (MODE == kModeRows) {                                      // [image row][ow][channel]
                        const int row_id = kp.d_segs.div(m_tile);
                        c1 = (m_tile - row_id * kp.rows_segs) * PIX; c2 = row_id;
                    }
                    if (MODE == kModePatch) {                                     // [image][oh][ow][channel]
                        const int p_img = kp.d_tiles_hw.div(m_tile), p_rem = m_tile - p_img * kp.patch_tiles_hw;
                        const int p_r = kp.d_tiles_w.div(p_rem), p_c = p_rem - p_r * kp.patch_tiles_w;
                        c1 = p_c * 8; c2 = p_r * (PIX / 8); c3 = p_img;
                    }
                    auto load_res = [&](int ch) {
                        mbar_arrive_expect_tx(rbar, kStageF32Bytes);
                        if (MODE == kModePatch) tma_load_4d(stg, &map_r, rbar, ch, c1, c2, c3);
                        else if (MODE == kModeRows) tma_load_3d(stg, &map_r, rbar, ch, c1, c2);
                        else tma_load_2d(stg, &map_r, rbar, ch, c1);
                    };
                    auto store_tile = [&](const CUtensorMap *map, uint32_t src, int ch) {
                        if (MODE == kModePatch) tma_store_4d(map, src, ch, c1, c2, c3);
                        else if (MODE == kModeRows) tma_store_3d(map, src, ch, c1, c2);
                        else tma_store_2d(map, src, ch, c1);
                    };
                    // channels this tile has to cover: the real ones, and for an int8 output its zero padding as well
                    const int ch_end = min(o_base + BN, max(epi.O, has_i8 ? epi.out_cp : 0));
                    const int nchunks = ch_end > o_base ? (ch_end - o_base + 31) >> 5 : 0;
                    const float rs = epi.nscales == 1 ? epi.rq_scales[0] : epi.rq_scales[min(img, epi.nscales - 1)];
                    const int key = row & 7;
                    float4 *r_row = r_tile + row * 8;
                    int4 *q_row = q_tile + row * 2;
                    if (leader && has_res && part < nchunks && o_base + part * 32 < epi.O) {
                        load_res(o_base + part * 32);
                        if (MODE == kModeGeneral && part + parts < nchunks && o_base + (part + parts) * 32 < epi.O)
                            tma_prefetch_l2_2d(&map_r, o_base + (part + parts) * 32, c1);
                    }
                    bool stg_ok = true;
#pragma unroll 1
                    for (int c = part; c < nchunks; c += parts) {
                        const int col0 = c * 32;
                        const bool real = o_base + col0 < epi.O;      // false: nothing but the int8 output's channel padding
                        int v[32];
                        if constexpr (DUAL) {
                            // the projection's 32 channels of this pixel, dequantized (+ bias), into the thread's own row of
                            // the fp32 tile -- where a tensor-map load would have put a residual
                            if (real && !concat) {
                                tmem_ld32(taddr0 + (uint32_t)(BN + col0), v);
                                tmem_ld_wait();
                                const bool bias2 = dual.bias2 != nullptr;
#pragma unroll
                                for (int j4 = 0; j4 < 8; ++j4) {
                                    const float4 d4 = *reinterpret_cast<const float4 *>(t_dq + 2 * BN + col0 + 4 * j4);
                                    const float4 b4 = *reinterpret_cast<const float4 *>(t_dq + 3 * BN + col0 + 4 * j4);
                                    float4 f;
                                    f.x = __fmul_rn(__int2float_rn(v[4 * j4 + 0]), d4.x);
                                    f.y = __fmul_rn(__int2float_rn(v[4 * j4 + 1]), d4.y);
                                    f.z = __fmul_rn(__int2float_rn(v[4 * j4 + 2]), d4.z);
                                    f.w = __fmul_rn(__int2float_rn(v[4 * j4 + 3]), d4.w);
                                    if (bias2) { f.x = __fadd_rn(f.x, b4.x); f.y = __fadd_rn(f.y, b4.y); f.z = __fadd_rn(f.z, b4.z); f.w = __fadd_rn(f.w, b4.w); }
                                    r_row[j4 ^ key] = f;
                                }
                            }
                        }
                        if (real) tmem_ld32(taddr0 + (uint32_t)col0, v);
                        else {
#pragma unroll
                            for (int j = 0; j < 32; ++j) v[j] = 0;
                        }
                        if (real && has_res) {
                            if (!mbar_wait(rbar, stg_phase[0], abort_flag)) { stg_ok = false; }
                            stg_phase[0] ^= 1u;
                        }
                        if (real) tmem_ld_wait();
                        bool fine = true;
                        if (stg_ok) {
                            if (epi.res_after) TSB_EPI_DISPATCH_W(fine =, staged_chunk_t, true, v, t_dq + col0, t_bias + col0, epi.leaky, r_row, key, real && (has_res || (DUAL && !concat)), has_f32, q_row, has_i8, rs);
                            else TSB_EPI_DISPATCH_W(fine =, staged_chunk_t, false, v, t_dq + col0, t_bias + col0, epi.leaky, r_row, key, real && (has_res || (DUAL && !concat)), has_f32, q_row, has_i8, rs);
                        }
                        fence_async_smem();
                        // all four warps have written their rows; the OR says whether any value needs the exact slow path
                        const bool redo = bar_or(bar_id, 128, !fine || !stg_ok);
                        if (leader) {
                            if (!redo) {
                                if (has_f32 && real) store_tile(&map_of, stg, o_base + col0);
                                if (has_i8) store_tile(&map_oi, q_addr, o_base + col0);
                                bulk_commit();
                            }
                            bulk_wait_read();                                        // the tiles may be overwritten
                            const int cn = c + parts;
                            if (has_res && cn < nchunks && o_base + cn * 32 < epi.O) load_res(o_base + cn * 32);
                            // and the residual box after that one on its way into L2
                            const int cp = cn + parts;
                            if (has_res && MODE == kModeGeneral && cp < nchunks && o_base + cp * 32 < epi.O) tma_prefetch_l2_2d(&map_r, o_base + cp * 32, c1);
                        }
                        if (redo) {
                            // NaN or a value beyond the int32 range (they quantize to -128 in the reference), or a load that
                            // did not arrive: this chunk goes element by element, straight to global memory
                            for (int j = 0; j < 32; ++j) {
                                const int o = o_base + col0 + j;
                                const int a = real ? tmem_ld1(taddr0 + (uint32_t)(col0 + j)) : 0;
                                int a2 = 0;
                                if constexpr (DUAL) a2 = (real && !concat) ? tmem_ld1(taddr0 + (uint32_t)(BN + col0 + j)) : 0;
                                if (!live) continue;
                                if (DUAL && !concat && o < epi.O) {
                                    float r = __fmul_rn(__int2float_rn(a2), t_dq[2 * BN + col0 + j]);
                                    if constexpr (DUAL) { if (dual.bias2) r = __fadd_rn(r, t_dq[3 * BN + col0 + j]); }
                                    epilogue_store_value(epi, img, o, p, a, r, true);
                                } else if (o < epi.O) epilogue_store_one(epi, img, o, p, a);
                                else if (has_i8 && epi.i8_nhwc && o < epi.out_cp) epi.out_i8[(size_t)m * epi.out_cp + o] = 0;
                            }
                        }
                        // the next chunk's writes must not overtake the leader's wait above; with a residual the load it
                        // issues afterwards orders them, otherwise a second barrier does
                        if (!(has_res && c + parts < nchunks && o_base + (c + parts) * 32 < epi.O)) asm volatile("bar.sync %0, 128;" ::"r"(bar_id) : "memory");
                    }
                    if (!stg_ok && !*abort_flag) { *abort_flag = 1; atomicExch(kp.status, 7); }
                } else {
                // residual boxes of this thread quad ({32 channels, 128 pixels} each), two chunks ahead of their use
                const bool prefetcher = kp.res_prefetch && MODE != kModePatch && MODE != kModeRows && quarter == 0 && lane == 0;
                if (prefetcher) {
                    if (o_base + part * CW < epi.O) tma_prefetch_l2_2d(&map_r, o_base + part * CW, m_tile * PIX);
                    if (part + parts < BN / CW && o_base + (part + parts) * CW < epi.O) tma_prefetch_l2_2d(&map_r, o_base + (part + parts) * CW, m_tile * PIX);
                }
#pragma unroll 1
                for (int c = part; c < BN / CW; c += parts) {
                    const int col0 = c * CW;
                    if (prefetcher && c + 2 * parts < BN / CW && o_base + (c + 2 * parts) * CW < epi.O)
                        tma_prefetch_l2_2d(&map_r, o_base + (c + 2 * parts) * CW, m_tile * PIX);
                    if (o_base + col0 >= epi.O) {
                        // nothing but channel padding in this step: no accumulators to read, only the zero bytes the
                        // NHWC_PAD layout wants in its padding channels
                        if (live && epi.out_i8 && epi.i8_nhwc) {
#pragma unroll
                            for (int u = 0; u < CW; u += 16)
                                if (o_base + col0 + u < epi.out_cp)
                                    *reinterpret_cast<int4 *>(epi.out_i8 + (size_t)m * epi.out_cp + o_base + col0 + u) = make_int4(0, 0, 0, 0);
                        }
                        continue;
                    }
                    const bool full = o_base + col0 + CW <= epi.O;
                    bool done = false;
                    if (full && kp.epi_mode != kEpiGeneric) {
                        int v[CW];
                        tmem_ldw(taddr0 + (uint32_t)col0, v);
                        tmem_ld_wait();
                        if (kp.epi_mode == kEpiF32Nchw) {
                            if (live) {
                                const size_t off = (size_t)(img * epi.O + o_base + col0) * (size_t)epi.P + (size_t)p;
                                float *dst = epi.out_f32 + off;
                                if (epi.residual) TSB_EPI_DISPATCH_RES_W(, store_f32_nchw_res_t, CW, v, t_dq + col0, t_bias + col0, epi.leaky, epi.residual + off, dst, (uint32_t)epi.P);
                                else TSB_EPI_DISPATCH_W(, store_f32_nchw_t, CW, v, t_dq + col0, t_bias + col0, epi.leaky, dst, (uint32_t)epi.P);
                            }
                            done = true;
                        } else if (kp.epi_mode == kEpiI8Nhwc) {
                            const float rs = epi.nscales == 1 ? epi.rq_scales[0] : epi.rq_scales[img];
                            int8_t *dst = epi.out_i8 + (size_t)m * epi.out_cp + o_base + col0;
                            bool fine = true;
                            if (live) TSB_EPI_DISPATCH_W(fine =, store_i8_nhwc_t, CW, v, t_dq + col0, t_bias + col0, epi.leaky, rs, dst);
                            done = !__any_sync(0xffffffffu, !fine);
                        } else {
                            const float rs = epi.nscales == 1 ? epi.rq_scales[0] : epi.rq_scales[img];
                            const size_t f_off = (size_t)m * epi.O + o_base + col0;
                            const float *res = epi.residual ? epi.residual + f_off : nullptr;
                            float *of = epi.out_f32 ? epi.out_f32 + f_off : nullptr;
                            int8_t *oi = epi.out_i8 ? epi.out_i8 + (size_t)m * epi.out_cp + o_base + col0 : nullptr;
                            bool fine = true;
                            if (live) TSB_EPI_DISPATCH_RES_W(fine =, store_nhwc_t, CW, v, t_dq + col0, t_bias + col0, epi.leaky, res, of, oi, rs);
                            done = !__any_sync(0xffffffffu, !fine);
                        }
                    }
                    if (!done) {
                        // element by element: any combination of outputs, residual, partial channel chunks
                        for (int j = 0; j < CW; ++j) {
                            const int a = tmem_ld1(taddr0 + (uint32_t)(col0 + j));
                            const int o = o_base + col0 + j;
                            if (!live) continue;
                            if (o < epi.O) epilogue_store_one(epi, img, o, p, a);
                            else if (epi.out_i8 && epi.i8_nhwc && o < epi.out_cp) epi.out_i8[(size_t)m * epi.out_cp + o] = 0;
                        }
                    }
                }
                }   // not staged
            } else {
                // this thread's channel; its scale and bias live in registers
                const int o = o_base + row;
                const bool ch_live = o < epi.O;
                const bool quarter_live = o_base + quarter * 32 < max(epi.O, epi.out_i8 && epi.i8_nhwc ? epi.out_cp : 0);
                const float my_dq = ch_live ? epi.dq[o] : 0.0f;
                const float my_bias = (ch_live && epi.bias) ? epi.bias[o] : 0.0f;
                int p_img = 0, p_r = 0, p_c = 0;
                if (MODE == kModePatch) {
                    p_img = kp.d_tiles_hw.div(m_tile);
                    const int p_rem = m_tile - p_img * kp.patch_tiles_hw;
                    p_r = kp.d_tiles_w.div(p_rem);
                    p_c = p_rem - p_r * kp.patch_tiles_w;
                }
                // residual boxes of this thread quad ({128 channels, 32 pixels} each), two chunks ahead of their use
                const bool prefetcher = kp.res_prefetch && MODE != kModePatch && quarter == 0 && lane == 0;
                if (prefetcher) {
                    if (m_tile * PIX + part * 32 < kp.M_total) tma_prefetch_l2_2d(&map_r, o_base, m_tile * PIX + part * 32);
                    if (part + parts < kChunks && m_tile * PIX + (part + parts) * 32 < kp.M_total) tma_prefetch_l2_2d(&map_r, o_base, m_tile * PIX + (part + parts) * 32);
                }
#pragma unroll 1
                for (int c = part; c < kChunks && quarter_live; c += parts) {
                    const int col0 = c * 32;
                    if (prefetcher && c + 2 * parts < kChunks && m_tile * PIX + (c + 2 * parts) * 32 < kp.M_total)
                        tma_prefetch_l2_2d(&map_r, o_base, m_tile * PIX + (c + 2 * parts) * 32);
                    if (MODE == kModePatch) {
                        // this chunk: tile rows col0/8 .. col0/8+3, 8 pixels each
                        const int oh0 = p_r * (PIX / 8) + (col0 >> 3), ow0 = p_c * 8;
                        if (oh0 >= kp.OH) break;                         // uniform over the warp; later chunks lie lower still
                        const int rows_live = min(4, kp.OH - oh0), cols_live = min(8, kp.OW - ow0);
                        const int p0 = oh0 * kp.OW + ow0;
                        bool done = false;
                        if (kp.epi_mode == kEpiF32Nchw || kp.epi_mode == kEpiI8Nhwc) {
                            int v[32];
                            tmem_ld32(taddr0 + (uint32_t)col0, v);
                            tmem_ld_wait();
                            if (kp.epi_mode == kEpiF32Nchw) {
                                if (ch_live) {
                                    float *dst = epi.out_f32 + ((size_t)(p_img * epi.O + o) * (size_t)epi.P + (size_t)p0);
                                    TSB_EPI_DISPATCH(, patch_f32_run, v, my_dq, my_bias, epi.leaky, dst, (uint32_t)kp.OW, rows_live, cols_live);
                                }
                                done = true;
                            } else {
                                const float rs = epi.nscales == 1 ? epi.rq_scales[0] : epi.rq_scales[p_img];
                                int8_t *dst = epi.out_i8 + ((size_t)p_img * epi.P + p0) * epi.out_cp + o;
                                TSB_EPI_DISPATCH(done =, patch_i8_run, v, my_dq, my_bias, epi.leaky, rs, o < epi.out_cp, dst, (uint32_t)epi.out_cp,
                                                 (uint32_t)(kp.OW * epi.out_cp), rows_live, cols_live);
                            }
                        }
                        if (!done) {
                            for (int j = 0; j < 32; ++j) {
                                if ((j >> 3) >= rows_live || (j & 7) >= cols_live) continue;   // uniform over the warp
                                const int a = tmem_ld1(taddr0 + (uint32_t)(col0 + j));
                                const int pj = p0 + (j >> 3) * kp.OW + (j & 7);
                                if (ch_live) epilogue_store_one(epi, p_img, o, pj, a);
                                else if (epi.out_i8 && epi.i8_nhwc && o < epi.out_cp)
                                    epi.out_i8[((size_t)p_img * epi.P + pj) * epi.out_cp + o] = 0;
                            }
                        }
                        continue;
                    }
                    const int mfirst = m_tile * PIX + col0;              // first pixel of this chunk
                    if (mfirst >= kp.M_total) break;                     // uniform over the warp
                    const int npix = min(32, kp.M_total - mfirst);
                    const int img0 = kp.d_P.div(mfirst), p0 = mfirst - img0 * kp.P;
                    const int split = kp.P - p0;                           // pixels j >= split belong to the next image
                    const bool one_image = npix == 32 && split >= 32;
                    // pixel-major outputs are linear in the pixel index: an image boundary inside the chunk only switches
                    // the requantize scale (at most once when an image has at least 32 pixels)
                    const bool linear_ok = npix == 32 && kp.P >= 32;
                    bool done = false;
                    if (kp.epi_mode != kEpiGeneric && (kp.epi_mode == kEpiF32Nchw ? one_image : linear_ok)) {
                        int v[32];
                        tmem_ld32(taddr0 + (uint32_t)col0, v);
                        tmem_ld_wait();
                        const float rs0 = epi.nscales == 1 ? epi.rq_scales[0] : epi.rq_scales[img0];
                        const float rs1 = epi.nscales == 1 ? rs0 : epi.rq_scales[min(img0 + 1, epi.nscales - 1)];
                        if (kp.epi_mode == kEpiF32Nchw) {
                            if (ch_live) {
                                float *dst = epi.out_f32 + ((size_t)(img0 * epi.O + o) * (size_t)epi.P + (size_t)p0);
                                TSB_EPI_DISPATCH(, swap_f32_run, v, my_dq, my_bias, epi.leaky, dst);
                            }
                            done = true;
                        } else if (kp.epi_mode == kEpiI8Nhwc) {
                            int8_t *dst = epi.out_i8 + (size_t)mfirst * epi.out_cp + o;
                            TSB_EPI_DISPATCH(done =, swap_i8_run, v, my_dq, my_bias, epi.leaky, rs0, rs1, split, o < epi.out_cp, dst, (uint32_t)epi.out_cp);
                        } else {
                            const size_t f_off = (size_t)mfirst * epi.O + (ch_live ? o : 0);
                            const float *res = epi.residual ? epi.residual + f_off : nullptr;
                            float *of = epi.out_f32 ? epi.out_f32 + f_off : nullptr;
                            int8_t *oi = epi.out_i8 ? epi.out_i8 + (size_t)mfirst * epi.out_cp + o : nullptr;
                            TSB_EPI_DISPATCH_SWAPRES(done =, swap_nhwc_run, v, my_dq, my_bias, epi.leaky, res, of, oi, o < epi.out_cp, rs0, rs1, split,
                                             (uint32_t)epi.O, (uint32_t)epi.out_cp, ch_live);
                        }
                    }
                    if (!done) {
                        int img = img0, p = p0;
                        for (int j = 0; j < npix; ++j) {
                            const int a = tmem_ld1(taddr0 + (uint32_t)(col0 + j));
                            if (ch_live) epilogue_store_one(epi, img, o, p, a);
                            else if (epi.out_i8 && epi.i8_nhwc && o < epi.out_cp)
                                epi.out_i8[(size_t)(img * epi.P + p) * epi.out_cp + o] = 0;
                            if (++p == kp.P) { p = 0; ++img; }
                        }
                    }
                }
            }
            tc_fence_before();
            mbar_arrive(bar_tempty + 8 * acc);
            if (et == 0) TSB_TRACE(local, 6);
        }
    }

    // common exit: everybody meets here, then the allocating warp releases tensor memory
    if (*abort_flag) {
        // give copies that may still be in flight time to land before shared memory is released
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000LL) { __nanosleep(1000); }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

// ---------------------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------------------
namespace {

#ifdef TSB_ENABLE_TRACE
unsigned long long *g_trace = nullptr;  // set through set_trace_buffer()
#endif
PFN_cuTensorMapEncodeTiled_v12000 g_encode_tiled = nullptr;
PFN_cuTensorMapEncodeIm2col_v12000 g_encode_im2col = nullptr;

int load_driver() {
    if (g_encode_tiled && g_encode_im2col) return TSB_OK;
    cudaDriverEntryPointQueryResult q;
    void *fn = nullptr;
    TSB_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q));
    if (q != cudaDriverEntryPointSuccess || !fn) return fail(TSB_ERR_UNSUPPORTED, "driver lacks cuTensorMapEncodeTiled");
    g_encode_tiled = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(fn);
    TSB_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeIm2col", &fn, cudaEnableDefault, &q));
    if (q != cudaDriverEntryPointSuccess || !fn) return fail(TSB_ERR_UNSUPPORTED, "driver lacks cuTensorMapEncodeIm2col");
    g_encode_im2col = reinterpret_cast<PFN_cuTensorMapEncodeIm2col_v12000>(fn);
    return TSB_OK;
}

CUtensorMapSwizzle swizzle_for(int bk) {
    return bk == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : (bk == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B);
}

template <int BN, int BK, bool SWAP, int MODE, bool DUAL = false>
int launch(const Config &cfg, const CUtensorMap &ma, const CUtensorMap &mb, const CUtensorMap &mr, const CUtensorMap &mof,
           const CUtensorMap &moi, const KernelParams &kp, const EpiParams &epi, cudaStream_t stream,
           const std::conditional_t<DUAL, DualParams, NoDual> &dual = {}) {
    // The shared-memory limit of a kernel is a per-device attribute: one process may drive several GPUs (one TenniS
    // Workbench per device, each on its own thread), so the "already raised" note is kept per device.
    static std::atomic<uint64_t> configured{0};
    auto kernel = conv_i8_tc_kernel<BN, BK, SWAP, MODE, DUAL>;
    int dev = 0;
    TSB_CUDA(cudaGetDevice(&dev));
    const uint64_t bit = dev >= 0 && dev < 64 ? 1ull << dev : 0;
    if (!(configured.load(std::memory_order_acquire) & bit)) {
        TSB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kMaxDynamicSmem));
        configured.fetch_or(bit, std::memory_order_release);
    }
    TSB_CUDA(launch_pdl(kernel, dim3(cfg.grid), dim3(kThreads), cfg.dyn_smem, stream, ma, mb, mr, mof, moi, kp, epi, dual));
    TSB_LAUNCHED("conv_i8_tc_kernel");
    return TSB_OK;
}

}  // namespace

#ifdef TSB_ENABLE_TRACE
void set_trace_buffer(unsigned long long *device_buffer) { g_trace = device_buffer; }
#endif

bool make_view(const ConvGeom &g, const Tuning &tune, View *view, const char **why) {
    *why = "";
    View v;
    v.real = g;
    v.g = g;
    if (g.pad_value != 0) { *why = "non-zero padding_value"; return false; }
    if (g.C <= 16) {
        // fold the filter row into the channel dimension
        const int cpix = (g.C <= 8 && g.sw % 2 == 0) ? 8 : 16;
        const int span = (g.KW - 1) * g.dw + 1;
        const int bkf = round_up(span * cpix, 64);
        if (bkf > 128) { *why = "filter row too wide to fold into one K block"; return false; }
        const int unit = 32 / cpix;  // pixels per 32 bytes: rows of the staging are whole 32-byte units (what one thread of
                                     // the staging quantize writes)
        const int need = std::max(g.W + g.pad_l, (g.OW - 1) * g.sw + bkf / cpix);
        v.fold = 1;
        v.cpix = cpix;
        v.Wp = round_up(need, unit);
        v.g.C = bkf; v.g.Cp = bkf; v.g.W = g.OW; v.g.KW = 1; v.g.sw = 1; v.g.dw = 1; v.g.pad_l = 0;
        v.stride_w = (uint64_t)g.sw * cpix;
        v.stride_h = (uint64_t)v.Wp * cpix;
        v.stride_n = v.stride_h * g.H;
        v.stage_bytes = (size_t)v.stride_n * g.N;
        // raw-row mode: pixel stride of exactly one 16-byte unit, every output row meets at least one input row, and
        // output rows long enough to fill most of a 128-pixel tile (tune.rows forces it on/off where it is possible)
        bool rows_ok = v.stride_w == 16 && (size_t)g.KH * bkf * std::min(round_up(g.O, 64), 256) <= 96 * 1024 &&
                       (size_t)(g.KH - 1) * g.dh * v.stride_h + (size_t)ceil_div(g.OW, kBM) * kBM * 16 + 2048 <= 48 * 1024;
        for (int oh = 0; oh < g.OH && rows_ok; ++oh) {
            bool any = false;
            for (int kh = 0; kh < g.KH; ++kh) {
                const int ih = oh * g.sh - g.pad_t + kh * g.dh;
                any = any || (ih >= 0 && ih < g.H);
            }
            rows_ok = any;
        }
        const int segs = ceil_div(g.OW, kBM);
        const bool rows_pay = (double)g.OW / (double)(segs * kBM) >= 0.75;
        if (rows_ok && (tune.rows ? tune.rows == 2 : rows_pay)) {
            v.rows = 1;
            v.rows_segs = segs;
            v.stage_bytes += (size_t)kBM * 16 + 256;   // the copy under the last tile of the last row runs past the row's end
        }
    } else {
        if (g.Cp % 64 != 0) { *why = "channel padding is not a multiple of 64"; return false; }
        v.stride_w = (uint64_t)g.Cp;
        v.stride_h = (uint64_t)g.Cp * g.W;
        v.stride_n = v.stride_h * g.H;
        v.stage_bytes = (size_t)v.stride_n * g.N;
    }
    v.a_tiled = (!v.fold && g.KH == 1 && g.KW == 1 && g.sh == 1 && g.sw == 1 && g.pad_t == 0 && g.pad_l == 0 &&
                 g.OH == g.H && g.OW == g.W) ? 1 : 0;
    v.patch = (!v.fold && !v.a_tiled && g.sh == 1 && g.sw == 1 && g.KH * g.KW > 1 && (g.KW - 1) * g.dw + 8 <= 256 &&
               (g.KH - 1) * g.dh + 32 <= 256 && tune.patch != 1) ? 1 : 0;
    const ConvGeom &t = v.g;
    v.weight_bytes = (size_t)t.O * t.KH * t.KW * t.Cp;
    // im2col tensor maps take box corners in [-128,127], filter offsets in [0,255] and traversal strides up to 8
    const int up_w = (t.OW - 1) * t.sw - t.pad_l - (t.W - 1);
    const int up_h = (t.OH - 1) * t.sh - t.pad_t - (t.H - 1);
    if (t.pad_t > 128 || t.pad_l > 128 || t.pad_t < 0 || t.pad_l < 0 || up_w < -128 || up_w > 127 || up_h < -128 || up_h > 127) {
        *why = "padding beyond the im2col corner range";
        return false;
    }
    if ((t.KW - 1) * t.dw > 255 || (t.KH - 1) * t.dh > 255) { *why = "filter extent beyond the im2col offset range"; return false; }
    if (t.sh > 8 || t.sw > 8) { *why = "stride beyond the traversal-stride range"; return false; }
    if ((int64_t)t.N * t.OH * t.OW > INT32_MAX - 256) { *why = "too many output pixels"; return false; }
    if ((int64_t)t.N * t.O * t.OH * t.OW > UINT32_MAX) { *why = "output too large for 32-bit indexing"; return false; }
    if (v.stage_bytes > (size_t)INT32_MAX) { *why = "staged input too large"; return false; }
    *view = v;
    return true;
}

int staging_level(const View &v, const EpiParams &epi) {
    const ConvGeom &g = v.real;
    if (epi.out_acc) return 0;
    const bool per_sample = epi.nscales > 1 && epi.nscales == g.N && epi.group_len == (uint32_t)(g.O * g.OH * g.OW);
    if (epi.out_i8 && !(epi.i8_nhwc && epi.rne_limit == 0 && (epi.nscales == 1 || per_sample))) return 0;
    if (epi.out_i8 && reinterpret_cast<uintptr_t>(epi.out_i8) % 16) return 0;
    const bool f32_tiles = (epi.out_f32 || epi.residual) && epi.f32_nhwc;
    if (f32_tiles) {
        // tensor maps over [pixels][O] fp32: rows must be whole 16-byte units, the tensors 16-byte aligned and distinct
        if (g.O % 4 != 0 || (const void *)epi.residual == (const void *)epi.out_f32) return 0;
        if ((reinterpret_cast<uintptr_t>(epi.out_f32) | reinterpret_cast<uintptr_t>(epi.residual)) % 16) return 0;
        return 2;
    }
    // fp32 NCHW output, or int8 NHWC_PAD alone: the direct paths (a thread's 32 int8 channels are one 32-byte sector,
    // which two 16-byte stores write as well as a tile store would)
    return 0;
}

Config choose_config(const View &v, const Tuning &tune, int sm_count, int orientation, int staging) {
    const ConvGeom &g = v.g;
    Config c;
    c.bk = (g.Cp % 128 == 0) ? 128 : 64;
    const int64_t M = (int64_t)g.N * g.OH * g.OW;
    const uint32_t stg_bytes = staging == 2 ? kQuads * (kStageF32Bytes + kStageI8Bytes) : (staging == 1 ? kQuads * kStageI8Bytes : 0u);
    const uint32_t budget = kSmemBudget - stg_bytes;
    // An MMA instruction costs the same 128 cycles for any N up to 256, so N should be 256 whenever possible.
    // Normal orientation: 128 pixels on M, up to 256 output channels on N.  Swapped orientation: channels on M,
    // 256 (or 128) pixels on N -- it halves the MMA count of narrow layers but its epilogue (one channel per thread)
    // is dearer, so it is taken where it measured faster: multi-tap filters with at most 64 output channels.
    // patch mode under a given tile shape: most of each 8 x (pix/8) tile inside the image, and the whole weight tile
    // in shared memory beside at least two patches (tune.patch == 2 drops the first condition)
    auto patch_fits = [&](int pix, int ch) {
        if (!v.patch) return false;
        const int th = pix / 8;
        const int tiles_w = ceil_div(g.OW, 8), tiles_h = ceil_div(g.OH, th);
        const int pw = 8 + (g.KW - 1) * g.dw, ph = th + (g.KH - 1) * g.dh;
        const double eff = (double)(g.OH * g.OW) / ((double)tiles_w * tiles_h * pix);
        const uint64_t patch_bytes = (uint64_t)round_up(pw * ph * c.bk, 1024);
        const uint64_t w_all = (uint64_t)g.KH * g.KW * g.Cp * (uint64_t)ch;
        return (eff >= 0.7 || tune.patch == 2) && w_all + 2 * patch_bytes <= budget;
    };
    const int bn_normal = g.O > 128 ? 256 : (g.O > 64 ? 128 : 64);
    if (v.rows) c.swap = 0;
    else if (orientation >= 0) c.swap = orientation;
    else if (tune.orientation) c.swap = tune.orientation == 2 && g.O <= 128;
    // narrow multi-tap layers: swapped fills the MMA's N, but where patch mode applies the normal orientation with its
    // cheaper epilogue (16 warps, 16-byte stores) measured faster
    else c.swap = g.O <= 64 && g.KH * g.KW >= 9 && !v.fold && !patch_fits(kBM, bn_normal);
    if (c.swap) {
        c.ch = kBM;
        c.bn = 256;
        if (ceil_div64(M, 256) < sm_count && ceil_div64(M, 128) > ceil_div64(M, 256)) c.bn = 128;  // few pixels: more, smaller tiles
        c.pix = c.bn;
    } else {
        c.bn = g.O > 128 ? 256 : (g.O > 64 ? 128 : 64);
        // the staged block epilogue over plain [pixels][channels] tiles (the 1x1 expansions of residual blocks) measured 3-5 %
        // faster with four 128-channel accumulators, one tile per epilogue quad, than with two 256-channel ones
        if (staging == 2 && v.a_tiled && c.bn == 256) c.bn = 128;
        const int m_tiles128 = (int)ceil_div64(M, kBM);
        // a narrower N tile when the wide one leaves most SMs idle or the last wave nearly empty
        while (c.bn > 64) {
            const int64_t tiles = (int64_t)m_tiles128 * ceil_div(g.O, c.bn);
            const int64_t waves = ceil_div64(tiles, sm_count);
            const double eff = (double)tiles / (double)(waves * sm_count);
            if (eff >= 0.8) break;
            const int64_t tiles2 = (int64_t)m_tiles128 * ceil_div(g.O, c.bn / 2);
            const double eff2 = (double)tiles2 / (double)(ceil_div64(tiles2, sm_count) * sm_count);
            if (eff2 <= eff) break;
            c.bn /= 2;
        }
        c.pix = kBM;
        c.ch = c.bn;
    }
    c.num_m_tiles = v.rows ? g.N * g.OH * v.rows_segs : (int)ceil_div64(M, c.pix);
    c.num_n_tiles = ceil_div(g.O, c.ch);
    if (patch_fits(c.pix, c.ch)) {
        const int th = c.pix / 8;
        c.patch = 1;
        c.patch_tiles_w = ceil_div(g.OW, 8); c.patch_tiles_h = ceil_div(g.OH, th);
        c.patch_pw = 8 + (g.KW - 1) * g.dw; c.patch_ph = th + (g.KH - 1) * g.dh;
        c.num_m_tiles = g.N * c.patch_tiles_w * c.patch_tiles_h;
    }
    const int64_t tiles = (int64_t)c.num_m_tiles * c.num_n_tiles;
    c.grid = (int)(tiles < sm_count ? tiles : sm_count);
    // shared-memory plan: keep the CTA's whole weight tile resident when it is small enough to leave room for
    // at least four activation stages; otherwise stream activations and weights together
    // raw-row mode stages, per output row, the KH staged image rows under all its segments of 128 sliding windows
    // (127 pixel strides of 16 bytes plus one window in the last segment)
    const uint32_t p_bytes = c.patch ? (uint32_t)round_up(c.patch_pw * c.patch_ph * c.bk, 1024) : v.rows ? (uint32_t)round_up((g.KH - 1) * g.dh * (int)v.stride_h + (v.rows_segs - 1) * kBM * 16 + (kBM - 1) * 16 + c.bk, 128)
                                    : (uint32_t)c.pix * c.bk;
    const uint32_t w_bytes = (uint32_t)c.ch * c.bk;
    const uint32_t k_iters = (uint32_t)g.KH * g.KW * (g.Cp / c.bk);
    const uint32_t w_total = k_iters * w_bytes;
    const bool want_resident = v.rows || c.patch || tiles > c.grid;  // pays off only when a CTA runs several tiles
    // (raw-row mode always keeps its weights resident; make_view admitted it only where two row stages fit beside them)
    const uint32_t min_stages = v.rows ? 2 : 4;
    // K blocks per stage (im2col / tiled loads only): the MMA issuer pays a barrier wait and a commit per stage, which
    // costs it more than the MMAs of one K block take when N is small, so short K blocks are grouped -- as long as the
    // group divides the K blocks of a tile, stays within 48 KB and leaves at least three stages.
    auto group_for = [&](uint32_t unit, uint32_t room) {
        if (c.patch || v.rows) return 1;
        for (int gsz = 4; gsz >= 2; gsz /= 2)
            if (k_iters % (uint32_t)gsz == 0 && (uint32_t)gsz * unit <= 48 * 1024 && room / ((uint32_t)gsz * unit) >= 3) return gsz;
        return 1;
    };
    if (c.patch || (want_resident && w_total <= 128 * 1024 && w_total < budget && (budget - w_total) / p_bytes >= min_stages)) {
        c.b_resident = 1;
        c.unit_bytes = p_bytes;
        c.kgroup = group_for(p_bytes, budget - w_total);
        c.stage_bytes = (uint32_t)c.kgroup * p_bytes;
        c.stages = std::min<int>(kMaxStages, (int)((budget - w_total) / c.stage_bytes));
        c.b_off = (uint32_t)c.stages * c.stage_bytes;
        c.bar_off = c.b_off + w_total;
    } else {
        c.b_resident = 0;
        c.unit_bytes = p_bytes + w_bytes;
        c.kgroup = group_for(c.unit_bytes, budget);
        c.stage_bytes = (uint32_t)c.kgroup * c.unit_bytes;
        c.stages = std::min<int>(kMaxStages, (int)(budget / c.stage_bytes));
        c.b_off = 0;
        c.bar_off = (uint32_t)c.stages * c.stage_bytes;
    }
    // the staged epilogue's tiles (1024-byte aligned for the 128B swizzle) sit between the pipeline and the barriers
    c.staging = c.swap ? 0 : staging;
    if (c.staging) {
        c.stg_off = (c.bar_off + 1023u) & ~1023u;
        c.bar_off = c.stg_off + stg_bytes;
    }
    const uint32_t tables = ((c.bar_off + 8 * num_barriers(c.stages) + 8 + 15) & ~15u) + kMaxAccBufs * 2 * (uint32_t)c.bn * 4 +
                            (c.patch ? 4 * (uint32_t)(g.KH * g.KW) : 0);   // epilogue tables, then patch mode's tap table
    c.dyn_smem = tables + 1024;  // slack to align the tiles to 1024 bytes
    return c;
}

bool dual_supported(const View &v, const View &sc, const char **why) {
    const ConvGeom &g = v.g, &s = sc.g;
    *why = "";
    if (v.fold || v.rows || sc.fold || sc.rows) { *why = "folded inputs (at most 16 channels)"; return false; }
    if (s.KH != 1 || s.KW != 1 || s.pad_t != 0 || s.pad_l != 0) { *why = "the projection must be a 1x1 convolution without padding"; return false; }
    if (s.N != g.N || s.O != g.O || s.OH != g.OH || s.OW != g.OW) { *why = "the projection's output shape differs"; return false; }
    if ((s.H - 1) / s.sh + 1 != s.OH || (s.W - 1) / s.sw + 1 != s.OW) { *why = "the projection's padding is not zero on every side"; return false; }
    if (g.O % 4 != 0) { *why = "output channels not a multiple of 4"; return false; }
    return true;
}

Config choose_config_dual(const View &v, const View &sc, int sm_count, int bn, bool concat) {
    const ConvGeom &g = v.g, &s = sc.g;
    Config c;
    c.bk = (g.Cp % 128 == 0 && s.Cp % 128 == 0) ? 128 : 64;
    c.swap = 0;
    // 128 channels per tile: four accumulator buffers hold two tiles, so the MMAs of one tile run under the epilogue of
    // the other (256 would fill tensor memory with a single tile; measured 10-25 % slower on the ResNet-50 shapes)
    c.bn = bn == 128 || bn == 256 ? bn : 128;
    if (concat && bn == 0 && g.O <= 64) c.bn = 64;      // one accumulator per tile: a narrow layer keeps its narrow tile
    c.pix = kBM;
    c.ch = c.bn;
    const int64_t M = (int64_t)g.N * g.OH * g.OW;
    c.num_m_tiles = (int)ceil_div64(M, c.pix);
    c.num_n_tiles = ceil_div(g.O, c.ch);
    const int64_t tiles = (int64_t)c.num_m_tiles * c.num_n_tiles;
    c.grid = (int)(tiles < sm_count ? tiles : sm_count);
    const uint32_t stg_bytes = kQuads * (kStageF32Bytes + kStageI8Bytes);
    const uint32_t budget = kSmemBudget - stg_bytes;
    const uint32_t p_bytes = (uint32_t)c.pix * c.bk, w_bytes = (uint32_t)c.ch * c.bk;
    const uint32_t k1 = (uint32_t)g.KH * g.KW * (g.Cp / c.bk), k2 = (uint32_t)(s.Cp / c.bk);
    const uint32_t w_total = (k1 + k2) * w_bytes;
    // K blocks per stage: a stage never mixes the two convolutions, so the group divides both block counts
    auto group_for = [&](uint32_t unit, uint32_t room) {
        for (int gsz = 4; gsz >= 2; gsz /= 2)
            if (k1 % (uint32_t)gsz == 0 && k2 % (uint32_t)gsz == 0 && (uint32_t)gsz * unit <= 48 * 1024 && room / ((uint32_t)gsz * unit) >= 3) return gsz;
        return 1;
    };
    if (tiles > c.grid && w_total <= 128 * 1024 && w_total < budget && (budget - w_total) / p_bytes >= 4) {
        c.b_resident = 1;
        c.unit_bytes = p_bytes;
        c.kgroup = group_for(p_bytes, budget - w_total);
        c.stage_bytes = (uint32_t)c.kgroup * p_bytes;
        c.stages = std::min<int>(kMaxStages, (int)((budget - w_total) / c.stage_bytes));
        c.b_off = (uint32_t)c.stages * c.stage_bytes;
        c.bar_off = c.b_off + w_total;
    } else {
        c.b_resident = 0;
        c.unit_bytes = p_bytes + w_bytes;
        c.kgroup = group_for(c.unit_bytes, budget);
        c.stage_bytes = (uint32_t)c.kgroup * c.unit_bytes;
        c.stages = std::min<int>(kMaxStages, (int)(budget / c.stage_bytes));
        c.b_off = 0;
        c.bar_off = (uint32_t)c.stages * c.stage_bytes;
    }
    c.staging = 2;
    c.stg_off = (c.bar_off + 1023u) & ~1023u;
    c.bar_off = c.stg_off + stg_bytes;
    const uint32_t tables = ((c.bar_off + 8 * num_barriers(c.stages) + 8 + 15) & ~15u) + kMaxAccBufs * 2 * (uint32_t)c.bn * 4;
    c.dyn_smem = tables + 1024;
    return c;
}

int encode_weight_map(const View &v, const Config &cfg, const int8_t *w_packed, CUtensorMap *map) {
    int st = load_driver();
    if (st != TSB_OK) return st;
    const ConvGeom &g = v.g;
    const cuuint64_t ktot = (cuuint64_t)g.KH * g.KW * g.Cp;
    cuuint64_t dims[2] = {ktot, (cuuint64_t)g.O};
    cuuint64_t strides[1] = {ktot};
    cuuint32_t box[2] = {(cuuint32_t)cfg.bk, (cuuint32_t)cfg.ch};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = g_encode_tiled(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<int8_t *>(w_packed), dims, strides, box,
                                estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle_for(cfg.bk),
                                CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(TSB_ERR_UNSUPPORTED, "cuTensorMapEncodeTiled(weights) failed with %d", (int)r);
    return TSB_OK;
}

int encode_activation_map(const View &v, const Config &cfg, const int8_t *x, CUtensorMap *map) {
    int st = load_driver();
    if (st != TSB_OK) return st;
    if (reinterpret_cast<uintptr_t>(x) % 16) return fail(TSB_ERR_INVALID_ARGUMENT, "staged activations must be 16-byte aligned");
    const ConvGeom &g = v.g;
    if (cfg.patch) {
        cuuint64_t dims4[4] = {(cuuint64_t)g.Cp, (cuuint64_t)g.W, (cuuint64_t)g.H, (cuuint64_t)g.N};
        cuuint64_t strides4[3] = {v.stride_w, v.stride_h, v.stride_n};
        cuuint32_t box4[4] = {(cuuint32_t)cfg.bk, (cuuint32_t)cfg.patch_pw, (cuuint32_t)cfg.patch_ph, 1};
        cuuint32_t estr4[4] = {1, 1, 1, 1};
        CUresult r4 = g_encode_tiled(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<int8_t *>(x), dims4, strides4, box4,
                                     estr4, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle_for(cfg.bk),
                                     CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r4 != CUDA_SUCCESS) return fail(TSB_ERR_UNSUPPORTED, "cuTensorMapEncodeTiled(activation patches) failed with %d", (int)r4);
        return TSB_OK;
    }
    if (v.a_tiled) {
        cuuint64_t dims2[2] = {(cuuint64_t)g.Cp, (cuuint64_t)g.N * g.H * g.W};
        cuuint64_t strides2[1] = {(cuuint64_t)g.Cp};
        cuuint32_t box2[2] = {(cuuint32_t)cfg.bk, (cuuint32_t)cfg.pix};
        cuuint32_t estr2[2] = {1, 1};
        CUresult r2 = g_encode_tiled(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<int8_t *>(x), dims2, strides2, box2,
                                     estr2, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle_for(cfg.bk),
                                     CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r2 != CUDA_SUCCESS) return fail(TSB_ERR_UNSUPPORTED, "cuTensorMapEncodeTiled(activations) failed with %d", (int)r2);
        return TSB_OK;
    }
    cuuint64_t dims[4] = {(cuuint64_t)g.Cp, (cuuint64_t)g.W, (cuuint64_t)g.H, (cuuint64_t)g.N};
    cuuint64_t strides[3] = {v.stride_w, v.stride_h, v.stride_n};
    // The box of base pixels: from -pad to the last position a filter can start at.  The far corner is chosen so
    // that exactly OW x OH positions are visited with the traversal stride (floor semantics of the operator).
    int lower[2] = {-g.pad_l, -g.pad_t};
    int upper[2] = {(g.OW - 1) * g.sw - g.pad_l - (g.W - 1), (g.OH - 1) * g.sh - g.pad_t - (g.H - 1)};
    cuuint32_t estr[4] = {1, (cuuint32_t)g.sw, (cuuint32_t)g.sh, 1};
    CUresult r = g_encode_im2col(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<int8_t *>(x), dims, strides, lower,
                                 upper, (cuuint32_t)cfg.bk, (cuuint32_t)cfg.pix, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                 swizzle_for(cfg.bk), CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                                 CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(TSB_ERR_UNSUPPORTED, "cuTensorMapEncodeIm2col failed with %d", (int)r);
    // Tensors under 128 KiB: drivers up to 13.1 set a descriptor bit that makes im2col loads of such small tensors
    // misbehave; clearing it is the documented remedy used by NVIDIA's open-source templates.
    int driver = 0;
    cudaDriverGetVersion(&driver);
    if (driver <= 13010 && v.stage_bytes < 131072)
        reinterpret_cast<uint64_t *>(map)[1] &= ~(1ull << 21);
    return TSB_OK;
}

namespace {

// [O][C][KH][KW] -> [O][KH][KW][Cp], padding channels zero
__global__ void pack_weights_kernel(const int8_t *__restrict__ w, int8_t *__restrict__ wp, int O, int C, int Cp, int taps) {
    const int64_t total = (int64_t)O * taps * Cp;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int c = (int)(i % Cp);
        const int t = (int)((i / Cp) % taps);
        const int o = (int)(i / ((int64_t)Cp * taps));
        wp[i] = c < C ? w[((int64_t)o * C + c) * taps + t] : (int8_t)0;
    }
}

// [O][C][KH][KW] -> [O][KH][bkf]: byte j of a filter row belongs to pixel offset j / cpix and channel j % cpix
__global__ void pack_weights_folded_kernel(const int8_t *__restrict__ w, int8_t *__restrict__ wp, int O, int C, int KH,
                                           int KW, int dw, int cpix, int bkf) {
    const int64_t total = (int64_t)O * KH * bkf;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int j = (int)(i % bkf);
        const int kh = (int)((i / bkf) % KH);
        const int o = (int)(i / ((int64_t)bkf * KH));
        const int pj = j / cpix, c = j % cpix;
        int8_t val = 0;
        if (c < C && pj % dw == 0 && pj / dw < KW) val = w[(((int64_t)o * C + c) * KH + kh) * KW + pj / dw];
        wp[i] = val;
    }
}

// int8 [N][C][H][W] (or NHWC_PAD [N][H][W][Cp]) -> [N][H][Wp][cpix]; one thread writes 16 bytes
__global__ void stage_folded_kernel(const int8_t *__restrict__ x, int x_nhwc, int Cp, int8_t *__restrict__ y, int N, int C,
                                    int H, int W, int Wp, int cpix, int pad_l) {
    const int units_per_row = Wp * cpix / 16;
    const int64_t total = (int64_t)N * H * units_per_row;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int u = (int)(i % units_per_row);
        const int h = (int)((i / units_per_row) % H);
        const int n = (int)(i / ((int64_t)units_per_row * H));
        uint32_t word[4] = {0, 0, 0, 0};
#pragma unroll
        for (int b = 0; b < 16; ++b) {
            const int byte = u * 16 + b;
            const int wp = byte / cpix, c = byte % cpix;
            const int wi = wp - pad_l;
            int8_t v = 0;
            if (c < C && wi >= 0 && wi < W)
                v = x_nhwc ? x[(((int64_t)n * H + h) * W + wi) * Cp + c] : x[(((int64_t)n * C + c) * H + h) * W + wi];
            word[b >> 2] |= (uint32_t)(uint8_t)v << (8 * (b & 3));
        }
        *reinterpret_cast<int4 *>(y + i * 16) = make_int4(word[0], word[1], word[2], word[3]);
    }
}

}  // namespace

int pack_weights(const View &v, const int8_t *w_oihw, int8_t *w_packed, cudaStream_t stream) {
    const ConvGeom &r = v.real;
    const int64_t total = (int64_t)v.weight_bytes;
    const int blocks = (int)std::min<int64_t>(ceil_div64(total, 256), 148 * 8);
    if (v.fold) {
        pack_weights_folded_kernel<<<blocks, 256, 0, stream>>>(w_oihw, w_packed, r.O, r.C, r.KH, r.KW, r.dw, v.cpix, v.g.Cp);
        TSB_LAUNCHED("pack_weights_folded_kernel");
    } else {
        pack_weights_kernel<<<blocks, 256, 0, stream>>>(w_oihw, w_packed, r.O, r.C, r.Cp, r.KH * r.KW);
        TSB_LAUNCHED("pack_weights_kernel");
    }
    return TSB_OK;
}

int stage_folded(const View &v, const int8_t *x, int x_nhwc, int8_t *staged, cudaStream_t stream) {
    const ConvGeom &r = v.real;
    const int64_t total = (int64_t)v.stage_bytes / 16;
    const int blocks = (int)std::min<int64_t>(ceil_div64(total, 256), 148 * 16);
    stage_folded_kernel<<<blocks, 256, 0, stream>>>(x, x_nhwc, r.Cp, staged, r.N, r.C, r.H, r.W, v.Wp, v.cpix, r.pad_l);
    TSB_LAUNCHED("stage_folded_kernel");
    return TSB_OK;
}

int launch_conv_tc(const View &v, const Config &cfg, const CUtensorMap &map_a, const CUtensorMap &map_b,
                   const int8_t *x_staged, const EpiParams &epi, int *status_word, cudaStream_t stream, const DualArgs *dual) {
    const ConvGeom &g = v.g;
    if (dual) {
        // the projected-shortcut kernels exist for the staged block epilogue only
        const bool i8_ok = !epi.out_i8 || (epi.i8_nhwc && epi.rne_limit == 0 && reinterpret_cast<uintptr_t>(epi.out_i8) % 16 == 0 &&
                                           (epi.nscales == 1 || (epi.nscales == g.N && epi.group_len == (uint32_t)(g.O * g.OH * g.OW))));
        const bool f32_ok = !epi.out_f32 || (epi.f32_nhwc && reinterpret_cast<uintptr_t>(epi.out_f32) % 16 == 0);
        if (epi.out_acc || epi.residual || !i8_ok || !f32_ok || g.O % 4 != 0 || cfg.swap || cfg.patch || v.rows || v.fold || cfg.staging != 2)
            return fail(TSB_ERR_UNSUPPORTED, "projected shortcut: needs pixel-major fp32 / NHWC_PAD int8 outputs with half-away rounding, no residual tensor, O %% 4 == 0");
    }
    KernelParams kp;
    kp.M_total = g.N * g.OH * g.OW;
    kp.OW = g.OW;
    kp.P = g.OH * g.OW;
    kp.KH = g.KH; kp.KW = g.KW;
    kp.sh = g.sh; kp.sw = g.sw; kp.dh = g.dh; kp.dw = g.dw; kp.pad_t = g.pad_t; kp.pad_l = g.pad_l;
    kp.Cp = g.Cp;
    kp.num_m_tiles = cfg.num_m_tiles;
    kp.num_n_tiles = cfg.num_n_tiles;
    kp.d_P = FastDiv((uint32_t)kp.P); kp.d_OW = FastDiv((uint32_t)kp.OW);
    kp.d_m_tiles = FastDiv((uint32_t)cfg.num_m_tiles); kp.d_n_tiles = FastDiv((uint32_t)cfg.num_n_tiles);
    kp.d_segs = FastDiv((uint32_t)std::max(1, v.rows_segs)); kp.d_OH = FastDiv((uint32_t)g.OH); kp.d_dh = FastDiv((uint32_t)g.dh);
    kp.per_sample_scale = (epi.nscales > 1 && epi.nscales == g.N && epi.group_len == (uint32_t)(g.O * g.OH * g.OW)) ? 1 : 0;
    kp.status = status_word;
#ifdef TSB_ENABLE_TRACE
    kp.trace = g_trace;
#else
    kp.trace = nullptr;
#endif
    kp.a_tiled = v.a_tiled;
    kp.stages = cfg.stages; kp.stage_bytes = cfg.stage_bytes; kp.b_resident = cfg.b_resident;
    kp.kgroup = cfg.kgroup; kp.unit_bytes = cfg.unit_bytes;
    kp.b_off = cfg.b_off; kp.bar_off = cfg.bar_off;
    kp.rows_segs = 0; kp.rows_OH = g.OH; kp.rows_H = g.H; kp.rows_bytes = 0; kp.rows_stride_h = 0; kp.rows_stride_n = 0;
    kp.rows_x = nullptr;
    kp.patch = cfg.patch; kp.OH = g.OH;
    kp.patch_tiles_w = std::max(1, cfg.patch_tiles_w); kp.patch_tiles_hw = std::max(1, cfg.patch_tiles_w * cfg.patch_tiles_h);
    kp.patch_pw = cfg.patch_pw; kp.patch_bytes = (uint32_t)(cfg.patch_pw * cfg.patch_ph * cfg.bk);
    kp.d_tiles_w = FastDiv((uint32_t)kp.patch_tiles_w); kp.d_tiles_hw = FastDiv((uint32_t)kp.patch_tiles_hw);
    if (cfg.patch && !cfg.b_resident) return fail(TSB_ERR_UNSUPPORTED, "patch mode needs resident weights");
    if (v.rows) {
        if (cfg.swap || !cfg.b_resident || !x_staged) return fail(TSB_ERR_UNSUPPORTED, "raw-row mode needs the normal orientation and resident weights");
        kp.rows_segs = v.rows_segs;
        kp.rows_bytes = (uint32_t)round_up((kBM - 1) * 16 + cfg.bk, 16);
        kp.rows_stride_h = (long long)v.stride_h;
        kp.rows_stride_n = (long long)v.stride_n;
        kp.rows_x = x_staged;
    }
    if (cfg.dyn_smem > kMaxDynamicSmem) return fail(TSB_ERR_UNSUPPORTED, "shared-memory plan of %u bytes does not fit", cfg.dyn_smem);
    const bool plain = !epi.out_acc && !epi.residual;
    kp.epi_mode = kEpiGeneric;
    if (plain && epi.out_f32 && !epi.f32_nhwc && !epi.out_i8) kp.epi_mode = kEpiF32Nchw;
    // ... and with an fp32 NCHW residual (a shortcut folded into the convolution by the graph rewrite), where a thread owns a pixel
    if (!cfg.swap && !epi.out_acc && epi.residual && epi.out_f32 && !epi.f32_nhwc && !epi.out_i8 && (const void *)epi.residual != (const void *)epi.out_f32)
        kp.epi_mode = kEpiF32Nchw;
    const bool i8_fast = !epi.out_i8 || (epi.i8_nhwc && epi.rne_limit == 0 && (epi.nscales == 1 || kp.per_sample_scale));
    if (plain && epi.out_i8 && !epi.out_f32 && i8_fast) kp.epi_mode = kEpiI8Nhwc;
    // pixel-major fp32 tensors (block outputs and residuals of a network): 16-byte accesses need O % 4 == 0
    if (!epi.out_acc && (epi.out_f32 || epi.residual) && epi.f32_nhwc && i8_fast && (const void *)epi.residual != (const void *)epi.out_f32 &&
        (cfg.swap || (g.O % 4 == 0 && ((reinterpret_cast<uintptr_t>(epi.out_f32) | reinterpret_cast<uintptr_t>(epi.residual)) & 15) == 0)))
        kp.epi_mode = kEpiNhwc;
    const int mode = cfg.patch ? kModePatch : (v.rows ? kModeRows : kModeGeneral);
    // Pixel-major fp32 residual (the shortcut of a residual block, as large as the output): a tensor map over it lets the
    // epilogue prefetch the boxes it is about to read into L2.  The map is not used for loads, so a failure to encode one
    // only switches the prefetch off.
    CUtensorMap map_r = map_b;
    kp.res_prefetch = 0;
    if (kp.epi_mode == kEpiNhwc && epi.residual && mode == kModeGeneral && g.O % 4 == 0 && reinterpret_cast<uintptr_t>(epi.residual) % 16 == 0 &&
        load_driver() == TSB_OK) {
        cuuint64_t dims[2] = {(cuuint64_t)g.O, (cuuint64_t)kp.M_total};
        cuuint64_t strides[1] = {(cuuint64_t)g.O * 4};
        cuuint32_t box[2] = {cfg.swap ? (cuuint32_t)std::min(g.O, kBM) : 32u, cfg.swap ? 32u : (cuuint32_t)kBM};
        cuuint32_t estr[2] = {1, 1};
        if (g_encode_tiled(&map_r, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float *>(epi.residual), dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS)
            kp.res_prefetch = 1;
        else
            map_r = map_b;
    }
    // Staged epilogue (normal orientation, shared memory set aside by the configuration): tensor maps over the residual,
    // the fp32 output and the int8 output whose boxes are one quad's tile -- 32 channels x the tile's 128 pixels, shaped
    // like the pixel tile of the load mode (a run of pixels, a run inside one output row, or an 8 x 16 block).
    CUtensorMap map_of = map_b, map_oi = map_b;
    kp.stg_off = cfg.stg_off;
    kp.stg_f32 = cfg.staging == 2 ? 1 : 0;
    // (a projection needs the staged epilogue, whose fp32 tile receives its result; a concatenation takes whatever epilogue
    // its outputs would take in a plain run -- int8 alone goes out through the direct path, which is faster for it)
    const bool dual_concat = dual && dual->dq == nullptr;
    const int want_staging = (dual && !dual_concat) ? 2 : (cfg.swap ? 0 : staging_level(v, epi));
    if (want_staging != 0 && cfg.staging >= want_staging && load_driver() == TSB_OK) {
        const ConvGeom &r = v.real;
        auto encode = [&](CUtensorMap *map, const void *ptr, bool is_f32, uint64_t channels) -> bool {
            const uint64_t es = is_f32 ? 4 : 1;
            const CUtensorMapDataType dt = is_f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_UINT8;
            const CUtensorMapSwizzle sw = is_f32 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE;
            cuuint32_t estr[4] = {1, 1, 1, 1};
            CUresult rc;
            if (mode == kModePatch) {
                cuuint64_t dims[4] = {channels, (cuuint64_t)r.OW, (cuuint64_t)r.OH, (cuuint64_t)r.N};
                cuuint64_t strides[3] = {channels * es, channels * es * r.OW, channels * es * r.OW * r.OH};
                cuuint32_t box[4] = {32, 8, (cuuint32_t)(kBM / 8), 1};
                rc = g_encode_tiled(map, dt, 4, const_cast<void *>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            } else if (mode == kModeRows) {
                cuuint64_t dims[3] = {channels, (cuuint64_t)r.OW, (cuuint64_t)r.N * r.OH};
                cuuint64_t strides[2] = {channels * es, channels * es * r.OW};
                cuuint32_t box[3] = {32, (cuuint32_t)kBM, 1};
                rc = g_encode_tiled(map, dt, 3, const_cast<void *>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            } else {
                cuuint64_t dims[2] = {channels, (cuuint64_t)kp.M_total};
                cuuint64_t strides[1] = {channels * es};
                cuuint32_t box[2] = {32, (cuuint32_t)kBM};
                rc = g_encode_tiled(map, dt, 2, const_cast<void *>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            }
            return rc == CUDA_SUCCESS;
        };
        bool ok_maps = true;
        if (epi.residual) ok_maps = ok_maps && encode(&map_r, epi.residual, true, (uint64_t)r.O);
        if (epi.out_f32) ok_maps = ok_maps && encode(&map_of, epi.out_f32, true, (uint64_t)r.O);
        if (epi.out_i8) ok_maps = ok_maps && encode(&map_oi, epi.out_i8, false, (uint64_t)epi.out_cp);
        if (ok_maps) {
            kp.epi_mode = kEpiStaged;
            kp.res_prefetch = 0;
            kp.stg_f32 = cfg.staging == 2 ? 1 : 0;
        }
    }
    if (dual) {
        if (!dual_concat && kp.epi_mode != kEpiStaged) return fail(TSB_ERR_UNSUPPORTED, "projected shortcut: the output tensor maps could not be encoded");
        if (dual_concat && kp.epi_mode != kEpiStaged && kp.epi_mode != kEpiI8Nhwc && kp.epi_mode != kEpiNhwc)
            return fail(TSB_ERR_UNSUPPORTED, "concatenated input: outputs must be pixel-major fp32 and / or NHWC_PAD int8 with half-away rounding");
        const ConvGeom &s = dual->view->g;
        DualParams dp;
        dp.map_a2 = dual->map_a; dp.map_b2 = dual->map_b;
        dp.dq2 = dual->dq; dp.bias2 = dual->bias;
        dp.concat = dual->dq == nullptr ? 1 : 0;
        dp.k2_iters = s.Cp / cfg.bk; dp.Cp2 = s.Cp; dp.a2_tiled = dual->view->a_tiled; dp.sh2 = s.sh; dp.sw2 = s.sw;
        if (cfg.bn == 256 && cfg.bk == 64) return launch<256, 64, false, kModeGeneral, true>(cfg, map_a, map_b, map_r, map_of, map_oi, kp, epi, stream, dp);
        if (cfg.bn == 256 && cfg.bk == 128) return launch<256, 128, false, kModeGeneral, true>(cfg, map_a, map_b, map_r, map_of, map_oi, kp, epi, stream, dp);
        if (cfg.bn == 128 && cfg.bk == 64) return launch<128, 64, false, kModeGeneral, true>(cfg, map_a, map_b, map_r, map_of, map_oi, kp, epi, stream, dp);
        if (cfg.bn == 128 && cfg.bk == 128) return launch<128, 128, false, kModeGeneral, true>(cfg, map_a, map_b, map_r, map_of, map_oi, kp, epi, stream, dp);
        if (cfg.bn == 64 && cfg.bk == 64 && dual_concat) return launch<64, 64, false, kModeGeneral, true>(cfg, map_a, map_b, map_r, map_of, map_oi, kp, epi, stream, dp);
        if (cfg.bn == 64 && cfg.bk == 128 && dual_concat) return launch<64, 128, false, kModeGeneral, true>(cfg, map_a, map_b, map_r, map_of, map_oi, kp, epi, stream, dp);
        return fail(TSB_ERR_UNSUPPORTED, "no projected-shortcut kernel for tile %dx%d", cfg.bn, cfg.bk);
    }
#define TSB_TC_CASE(BN_, BK_, SWAP_, MODE_) \
    if (cfg.bn == BN_ && cfg.bk == BK_ && (cfg.swap != 0) == SWAP_ && mode == MODE_) return launch<BN_, BK_, SWAP_, MODE_>(cfg, map_a, map_b, map_r, map_of, map_oi, kp, epi, stream)
#define TSB_TC_BOTH(BN_, BK_, MODE_) TSB_TC_CASE(BN_, BK_, false, MODE_); TSB_TC_CASE(BN_, BK_, true, MODE_)
    TSB_TC_CASE(64, 64, false, kModeGeneral); TSB_TC_CASE(64, 128, false, kModeGeneral);
    TSB_TC_BOTH(128, 64, kModeGeneral); TSB_TC_BOTH(256, 64, kModeGeneral);
    TSB_TC_BOTH(128, 128, kModeGeneral); TSB_TC_BOTH(256, 128, kModeGeneral);
    TSB_TC_CASE(64, 64, false, kModePatch); TSB_TC_CASE(64, 128, false, kModePatch);
    TSB_TC_BOTH(128, 64, kModePatch); TSB_TC_BOTH(256, 64, kModePatch);
    TSB_TC_BOTH(128, 128, kModePatch); TSB_TC_BOTH(256, 128, kModePatch);
    TSB_TC_CASE(64, 64, false, kModeRows); TSB_TC_CASE(128, 64, false, kModeRows); TSB_TC_CASE(256, 64, false, kModeRows);
    TSB_TC_CASE(64, 128, false, kModeRows); TSB_TC_CASE(128, 128, false, kModeRows); TSB_TC_CASE(256, 128, false, kModeRows);
#undef TSB_TC_BOTH
#undef TSB_TC_CASE
    return fail(TSB_ERR_UNSUPPORTED, "no tcgen05 kernel for tile %dx%d", cfg.bn, cfg.bk);
}

}  // namespace tc
}  // namespace tsb
