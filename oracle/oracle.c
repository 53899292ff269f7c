/*
 * CPU restatement of the reference's int8 quantized-convolution arithmetic.
 *
 * TEST INFRASTRUCTURE ONLY.  Nothing in the product path may call into this file: it exists so that the
 * tests, the smoke check and the benchmark's CPU arm have a checker.  Parity of this restatement is PINNED
 * by running it against the reference's own compiled CPU operators (oracle/_ref, built by the Makefile in
 * this directory) and against the fixtures under tests/golden/ that were generated from those operators.
 *
 * Every function names the reference source it follows (paths relative to the reference tree).
 * Build: gcc -O2 -fopenmp -ffp-contract=off  (no FMA contraction: the reference performs a separate
 * multiply and a separate add wherever two operators follow one another).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* fp32 -> int32 as x86 cvt(t)ps2dq does it: out-of-range and NaN give INT32_MIN ("integer indefinite"). */
static int32_t cvt_rne_x86(float v) {
    if (!(v >= -2147483648.0f && v < 2147483648.0f)) return INT32_MIN;
    return (int32_t)lrintf(v); /* current rounding mode: round-half-to-even */
}
static int32_t cvt_trunc_x86(float v) {
    if (!(v >= -2147483648.0f && v < 2147483648.0f)) return INT32_MIN;
    return (int32_t)v;
}
static int8_t clamp_i8(int32_t v) {
    if (v > 127) return 127;
    if (v < -128) return -128;
    return (int8_t)v;
}

/* to_int8<float>: src/kernels/cpu/quantize.cpp:22-28 -- int32_t(round(src)), round = half away from zero. */
static int8_t to_int8_half_away(float v) { return clamp_i8(cvt_trunc_x86(roundf(v))); }
/* AVX body: src/kernels/cpu/quantize.cpp:84-97 with include/kernels/common/simd_def/simd_avx_def.h:273-275
 * (_mm256_cvtps_epi32, round-half-to-even), then to_int8<int32_t> clamp (:15-20). */
static int8_t to_int8_half_even(float v) { return clamp_i8(cvt_rne_x86(v)); }

/* Group length of the multi-scale path: src/kernels/cpu/quantize.cpp:113
 * int(std::ceil(static_cast<float>(count) / quantize_group)) -- evaluated in fp32. */
int orc_quantize_group_len(int count, int nscales) {
    return (int)ceilf((float)count / (float)(size_t)nscales);
}

/*
 * cpu_quantize_compute_run<float>: src/kernels/cpu/quantize.cpp:69-125.
 *  one scale : first (count>>3)<<3 elements through the AVX body (half-to-even), the tail through
 *              to_int8<float> (half-away);
 *  G scales  : consecutive groups of ceil(count/G) elements, to_int8<float> everywhere; elements past
 *              G*group_len (only possible when the fp32 ceil under-estimates) are left untouched.
 */
void orc_quantize_f32(const float *x, int count, const float *scales, int nscales, int8_t *y) {
    if (nscales == 1) {
        const float s = scales[0];
        const int body = (count >> 3) << 3;
        for (int i = 0; i < body; ++i) y[i] = to_int8_half_even(x[i] * s);
        for (int i = body; i < count; ++i) y[i] = to_int8_half_away(x[i] * s);
    } else {
        const int len = orc_quantize_group_len(count, nscales);
        int index = 0;
        for (int g = 0; g < nscales; ++g) {
            const float s = scales[g];
            int left = len;
            while (index < count && left) {
                y[index] = to_int8_half_away(x[index] * s);
                ++index;
                --left;
            }
        }
    }
}

/* to_int8<double>: src/kernels/cpu/quantize.cpp:30-36 -- int32_t(round(src)) on a double (cvttsd2si: out-of-range
 * and NaN give INT32_MIN). */
static int8_t to_int8_f64(double v) {
    const double r = round(v);
    if (!(r >= -2147483648.0 && r < 2147483648.0)) return clamp_i8(INT32_MIN);
    return clamp_i8((int32_t)r);
}

/*
 * cpu_quantize_compute_run<double> (the generic template): src/kernels/cpu/quantize.cpp:38-67, dispatched at :134.
 * The product is double * float -> double; every element goes through to_int8<double> (half away), with one scale or
 * with G groups of ceil(count/G) elements.
 */
void orc_quantize_f64(const double *x, int count, const float *scales, int nscales, int8_t *y) {
    if (nscales == 1) {
        const float s = scales[0];
        for (int i = 0; i < count; ++i) y[i] = to_int8_f64(x[i] * s);
    } else {
        const int len = orc_quantize_group_len(count, nscales);
        int index = 0;
        for (int g = 0; g < nscales; ++g) {
            const float s = scales[g];
            int left = len;
            while (index < count && left) {
                y[index] = to_int8_f64(x[index] * s);
                ++index;
                --left;
            }
        }
    }
}

/* pooling2d_forward: include/backend/common_function.h:13-20 -- ceil of an fp32 quotient. */
int orc_pool_out_dim(int x, int pad_lo, int pad_hi, int k, int stride) {
    return (int)ceilf((float)(x + pad_lo + pad_hi - k) / (float)stride + 1.0f);
}

/*
 * cpu_max_pooling: src/kernels/cpu/pooling2d_core.cpp:47-93 (the generic kernel; the k3s2 / k2s2 special cases of
 * pooling_algorithm.h compute the same maxima).  NCHW fp32; each window is clipped to the image and the maximum
 * starts from the window's first element.  Windows that miss the image altogether are outside this restatement
 * (the reference reads past the plane there); returns -1 for such a geometry.
 */
int orc_max_pooling2d(const float *x, int N, int C, int H, int W, int k, int stride, int pt, int pb, int pl, int pr,
                      float *y) {
    const int OH = orc_pool_out_dim(H, pt, pb, k, stride), OW = orc_pool_out_dim(W, pl, pr, k, stride);
    if (OH < 1 || OW < 1 || (OH - 1) * stride - pt >= H || (OW - 1) * stride - pl >= W || k - pt < 1 || k - pl < 1) return -1;
    for (int nc = 0; nc < N * C; ++nc) {
        const float *in = x + (size_t)nc * H * W;
        float *out = y + (size_t)nc * OH * OW;
        for (int oh = 0; oh < OH; ++oh) {
            int h0 = oh * stride - pt, h1 = h0 + k < H ? h0 + k : H;
            if (h0 < 0) h0 = 0;
            for (int ow = 0; ow < OW; ++ow) {
                int w0 = ow * stride - pl, w1 = w0 + k < W ? w0 + k : W;
                if (w0 < 0) w0 = 0;
                float m = in[h0 * W + w0];
                for (int ih = h0; ih < h1; ++ih)
                    for (int iw = w0; iw < w1; ++iw)
                        if (in[ih * W + iw] > m) m = in[ih * W + iw];
                out[oh * OW + ow] = m;
            }
        }
    }
    return 0;
}

/* conv2d_forward: include/backend/common_function.h:30-40 (integer division, then floor of an integer). */
int orc_conv_out_dim(int x, int pad_lo, int pad_hi, int k, int stride, int dilation) {
    return (x + pad_lo + pad_hi - (dilation * (k - 1) + 1)) / stride + 1;
}

/* im2col_cpu<int8_t>: src/kernels/cpu/im2col.cpp:36-111.  col is [C*KH*KW][OH*OW]. */
void orc_im2col_i8(const int8_t *im, int C, int H, int W, int KH, int KW, int pt, int pb, int pl, int pr,
                   int sh, int sw, int dh, int dw, int8_t *col, int8_t padding_value) {
    const int OH = orc_conv_out_dim(H, pt, pb, KH, sh, dh);
    const int OW = orc_conv_out_dim(W, pl, pr, KW, sw, dw);
    for (int c = 0; c < C; ++c) {
        const int8_t *src = im + (size_t)c * H * W;
        int8_t *dst = col + (size_t)c * KH * KW * OH * OW;
        for (int kh = 0; kh < KH; ++kh)
            for (int kw = 0; kw < KW; ++kw) {
                int ih = -pt + kh * dh;
                for (int oh = 0; oh < OH; ++oh, ih += sh) {
                    if ((unsigned)ih >= (unsigned)H) {
                        for (int ow = 0; ow < OW; ++ow) *dst++ = padding_value;
                        continue;
                    }
                    int iw = -pl + kw * dw;
                    for (int ow = 0; ow < OW; ++ow, iw += sw)
                        *dst++ = ((unsigned)iw < (unsigned)W) ? src[ih * W + iw] : padding_value;
                }
            }
    }
}

/* math<int8_t,int32_t>::gemm(NoTrans, NoTrans, M, N, K, 1, A, B, 0, C): src/kernels/cpu/math_cpu.cpp:237-244,
 * 142-210, inline_dot :29-46.  Exact int32 sums, so the loop order here (row of B innermost, cache friendly)
 * gives the same bits as the reference's strided dot products. */
void orc_gemm_i8_i32(int M, int N, int K, const int8_t *A, const int8_t *B, int32_t *Cm) {
#pragma omp parallel for schedule(static)
    for (int i = 0; i < M; ++i) {
        int32_t *c = Cm + (size_t)i * N;
        memset(c, 0, (size_t)N * sizeof(int32_t));
        for (int k = 0; k < K; ++k) {
            const int32_t a = A[(size_t)i * K + k];
            const int8_t *b = B + (size_t)k * N;
            for (int j = 0; j < N; ++j) c[j] += a * (int32_t)b[j];
        }
    }
}

/*
 * cpu_conv2d_nchw_compute_run<int8_t>: src/kernels/cpu/quantized/conv2d_quantized_core.cpp:18-126.
 * Per image: im2col (skipped for 1x1 / stride 1 / no padding, :46-49) then the int8 GEMM into an int32
 * scratch, then y = float(acc) * dequantize_scales[o] (:80-107: _mm256_cvtepi32_ps + one fp32 multiply).
 * acc_out (optional) receives the int32 accumulators, NCHW.
 * Returns 0, or -1 when the output would be empty.
 */
int orc_conv2d_quantized(const int8_t *x, int N, int C, int H, int W, const int8_t *w, int O, int KH, int KW,
                         int pt, int pb, int pl, int pr, float padding_value, int sh, int sw, int dh, int dw,
                         const float *dq, float *out, int32_t *acc_out) {
    const int OH = orc_conv_out_dim(H, pt, pb, KH, sh, dh);
    const int OW = orc_conv_out_dim(W, pl, pr, KW, sw, dw);
    if (OH <= 0 || OW <= 0) return -1;
    const int K = C * KH * KW, P = OH * OW;
    const int is_1x1 = sh == 1 && sw == 1 && KH == 1 && KW == 1 && pt == 0 && pb == 0 && pl == 0 && pr == 0;
    int8_t *col = is_1x1 ? NULL : (int8_t *)malloc((size_t)K * P);
    int32_t *acc = acc_out ? acc_out : (int32_t *)malloc((size_t)N * O * P * sizeof(int32_t));
    for (int n = 0; n < N; ++n) {
        const int8_t *xin = x + (size_t)n * C * H * W;
        const int8_t *b = xin;
        if (!is_1x1) {
            memset(col, 0, (size_t)K * P);
            orc_im2col_i8(xin, C, H, W, KH, KW, pt, pb, pl, pr, sh, sw, dh, dw, col, (int8_t)padding_value);
            b = col;
        }
        orc_gemm_i8_i32(O, P, K, w, b, acc + (size_t)n * O * P);
    }
    if (out) {
#pragma omp parallel for schedule(static)
        for (int no = 0; no < N * O; ++no) {
            const float s = dq[no % O];
            const int32_t *a = acc + (size_t)no * P;
            float *y = out + (size_t)no * P;
            for (int p = 0; p < P; ++p) y[p] = (float)a[p] * s;
        }
    }
    free(col);
    if (!acc_out) free(acc);
    return 0;
}

/* cpu_add_bias_compute_run<float>, dim = 1 (NCHW): src/kernels/cpu/add_bias.cpp:47-85 -- one fp32 add. */
void orc_add_bias_nchw(const float *x, int N, int C, int P, const float *bias, float *y) {
#pragma omp parallel for schedule(static)
    for (int nc = 0; nc < N * C; ++nc) {
        const float b = bias[nc % C];
        for (int p = 0; p < P; ++p) y[(size_t)nc * P + p] = x[(size_t)nc * P + p] + b;
    }
}

/* cpu_relu_compute_run<float>: src/kernels/cpu/relu.cpp:30-52 -- max(x, 0). */
void orc_relu(const float *x, size_t count, float *y) {
    for (size_t i = 0; i < count; ++i) y[i] = x[i] > 0.0f ? x[i] : 0.0f;
}

/* cpu_leay_relu_compute_run<float>: src/kernels/cpu/leaky_relu.cpp:39-67.
 * SIMD body: max(x,0) + scale*min(x,0); scalar tail: x > 0 ? x : x*scale.  Both give x for x > 0 and the
 * single product x*scale for x < 0; they can differ only in the sign of a zero result. */
void orc_leaky_relu(const float *x, size_t count, float scale, float *y) {
    for (size_t i = 0; i < count; ++i) y[i] = x[i] > 0.0f ? x[i] : x[i] * scale;
}
