// Shared host/device helpers of the tennis_b200 library: status handling, launch bookkeeping and the exact
// fp32/int8 arithmetic every kernel must agree on.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <string>

#include "../../include/tennis_b200.h"

namespace tsb {

// ---------------------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------------------
std::string &last_error();
extern std::atomic<int64_t> g_launches;

inline int fail(int status, const char *fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    last_error() = buf;
    return status;
}

inline int cuda_fail(cudaError_t e, const char *what) {
    return fail(int(e), "%s: %s", what, cudaGetErrorString(e));
}

#define TSB_CUDA(call)                                                  \
    do {                                                                \
        cudaError_t e__ = (call);                                       \
        if (e__ != cudaSuccess) return ::tsb::cuda_fail(e__, #call);    \
    } while (0)

// after every kernel launch
#define TSB_LAUNCHED(name)                                              \
    do {                                                                \
        ::tsb::g_launches.fetch_add(1, std::memory_order_relaxed);      \
        cudaError_t e__ = cudaGetLastError();                           \
        if (e__ != cudaSuccess) return ::tsb::cuda_fail(e__, name);     \
    } while (0)

// Launch with programmatic stream serialization: the grid may start while the previous kernel of the stream is still
// draining, so its prologue overlaps that kernel's tail.  Only for kernels whose every thread executes pdl_sync() before
// its first access to global memory.
#ifdef __CUDACC__
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args &&...args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}
// Waits until the kernels this grid depends on have completed and their writes are visible, then lets the next grid of
// the stream start its own prologue.
__device__ __forceinline__ void pdl_sync() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
#endif

inline int ceil_div(int a, int b) { return (a + b - 1) / b; }
inline int64_t ceil_div64(int64_t a, int64_t b) { return (a + b - 1) / b; }
inline int round_up(int a, int b) { return ceil_div(a, b) * b; }

// Output extent of a convolution: integer division that truncates toward zero, then +1
// (include/backend/common_function.h:30-40 of the reference).
inline int conv_out_dim(int x, int pad_lo, int pad_hi, int k, int stride, int dilation) {
    return (x + pad_lo + pad_hi - (dilation * (k - 1) + 1)) / stride + 1;
}

// Rounding rule of a quantize over `count` elements with `nscales` scales, as data for the kernels.
struct QuantRule {
    int64_t rne_limit;   // elements with NCHW index below this round half-to-even, the rest half-away
    int64_t group_len;   // elements per scale group (>= 1)
    int nscales;
};
QuantRule make_quant_rule(int64_t count, int nscales);

// ---------------------------------------------------------------------------------------------------------
// device side: the arithmetic contract
// ---------------------------------------------------------------------------------------------------------
#ifdef __CUDACC__

// fp32 -> int8 with the reference's two rounding modes.  A product that is NaN or outside the int32 range
// converts to INT32_MIN on x86 (cvtps2dq / cvttss2si "integer indefinite") and therefore clamps to -128.
__device__ __forceinline__ int q8_half_even(float v) {
    if (!(fabsf(v) < 2147483648.0f)) return -128;
    int r = __float2int_rn(v);
    return max(-128, min(127, r));
}
__device__ __forceinline__ int q8_half_away(float v) {
    if (!(fabsf(v) < 2147483648.0f)) return -128;
    // floor(|v| + 0.5) computed exactly: the sum is rounded toward zero, so it can never reach the next integer early
    // (a round-to-nearest sum would for |v| just below 0.5); then the sign is put back
    const float mag = __fadd_rz(fabsf(v), 0.5f);
    const int r = __float2int_rz(copysignf(mag, v));
    return max(-128, min(127, r));
}
__device__ __forceinline__ int q8(float x, float scale, bool half_even) {
    const float v = __fmul_rn(x, scale);  // one rounding, never contracted
    return half_even ? q8_half_even(v) : q8_half_away(v);
}

// fp64 input (src/kernels/cpu/quantize.cpp:30-36,38-67,134 of the reference): the product is formed in double (the
// fp32 scale is promoted), rounded half away from zero and converted the x86 way -- for every element, whatever the
// number of scales (the fp64 path has no half-to-even vector body).
__device__ __forceinline__ int q8(double x, float scale, bool /*half_even*/) {
    const double r = round(__dmul_rn(x, (double)scale));
    if (!(fabs(r) < 2147483648.0)) return -128;    // NaN or beyond int32: "integer indefinite", then the clamp
    return max(-128, min(127, (int)r));
}

// dequantize -> add_bias -> (+residual) -> activation (-> +residual when it follows the activation), one rounding per step.
struct EpilogueMath {
    int activation;
    float leaky;
    __device__ __forceinline__ float operator()(int acc, float dq, float bias, bool has_bias, float residual,
                                                bool has_residual, bool residual_after = false) const {
        float v = __fmul_rn(__int2float_rn(acc), dq);
        if (has_bias) v = __fadd_rn(v, bias);
        if (has_residual && !residual_after) v = __fadd_rn(v, residual);
        if (activation == TSB_ACT_RELU) v = v > 0.0f ? v : 0.0f;
        else if (activation == TSB_ACT_LEAKY_RELU) v = v > 0.0f ? v : __fmul_rn(v, leaky);
        if (has_residual && residual_after) v = __fadd_rn(v, residual);
        return v;
    }
};

#endif  // __CUDACC__

}  // namespace tsb
