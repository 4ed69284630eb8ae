/* CPU restatement of the quantized linear-layer arithmetic of StartLux-Prism.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker that the CUDA kernels are compared with; the product path
 * never links, loads or calls it.  Every function names the reference file:line whose arithmetic it restates.
 * Parity status: pinned.  The functions are checked (tests/test_oracle.py) against vectors produced by the
 * reference's own CPU-runnable code (tests/golden/make_golden.py): w4a8.quantize_ref / gemm_ref, w8a8.weight_from_q8,
 * mxfp4.pack / dequant_packed / the activation quantizer, gguf_weights' k-quant dequantizers, and against the
 * literal known-answer grid of tests/test_mxfp4.py:34-38.  The W8A8 GEMM epilogue, the per-token quantizer and the
 * fold have no CPU implementation in the reference (Triton / CUDA only); they are restated from the kernel source and
 * pinned by the float64 exact-product bound of tests/test_cuda_gemm.py:50,66-67.
 *
 * Build: gcc -O2 -fopenmp -ffp-contract=off -shared -fPIC (see oracle/Makefile).  -ffp-contract=off matters: every
 * fp32 product and sum below must round on its own, as the reference's explicit mul_rn / add_rn do.
 */
#include <math.h>
#include <stdlib.h>
#include <stdint.h>
#include <string.h>

static inline uint16_t f32_to_bf16_rne(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40); /* NaN stays NaN */
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

static inline float bf16_to_f32(uint16_t h) {
    uint32_t u = (uint32_t)h << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

/* ---------------------------------------------------------------------------------------------------- W8A8 GEMM
 * kernels/w8a8.py:31-98 (_w8a8_kernel): per scale group g of gk inputs an exact int32 dot product, then
 *   acc += mul_rn(mul_rn(float(acci), sa[m, g]), sw[n, g])          (w8a8.py:76)
 * for g ascending from acc = 0.  epi 0 stores bf16(acc) (w8a8.py:79-80), epi 1 stores add_rn(out, acc)
 * (w8a8.py:85), epi 3 stores the raw int32 sum over all of K (w8a8.py:54-63).  Rows >= live are left untouched
 * (w8a8.py:77, csrc/w8a8_gemm.cu:411-413).  With gk == K this is csrc/w8a8_gemm.cu:334-339,370-371.
 * a [M, K] int8, a_s [M, K/gk] fp32, w [N, K] int8, w_s [N, K/gk] fp32; out row stride ldo elements. */
void orc_w8a8_gemm(const int8_t *a, const float *a_s, const int8_t *w, const float *w_s, void *out, long ldo,
                   int live, int N, int K, int gk, int epi) {
    int G = K / gk;
#pragma omp parallel for schedule(static)
    for (long idx = 0; idx < (long)live * N; ++idx) {
        int m = (int)(idx / N), n = (int)(idx % N);
        const int8_t *ar = a + (long)m * K, *wr = w + (long)n * K;
        if (epi == 3) {
            int32_t tot = 0;
            for (int k = 0; k < K; ++k) tot += (int32_t)ar[k] * (int32_t)wr[k];
            ((int32_t *)out)[(long)m * ldo + n] = tot;
            continue;
        }
        float acc = 0.0f;
        for (int g = 0; g < G; ++g) {
            int32_t ai = 0;
            for (int k = g * gk; k < (g + 1) * gk; ++k) ai += (int32_t)ar[k] * (int32_t)wr[k];
            float t = (float)ai * a_s[(long)m * G + g];
            if (epi == 4) {
                /* the vocabulary head, kernels/decode.py:136-160 (_head_q8_kernel): `acc += (ai * sa) * sw` written
                 * without mul_rn / add_rn, which the reference's compiler contracts into one fused multiply-add */
                acc = fmaf(t, w_s[(long)n * G + g], acc);
                continue;
            }
            t = t * w_s[(long)n * G + g];
            acc = acc + t;
        }
        if (epi == 4) {
            ((float *)out)[(long)m * ldo + n] = acc;
            continue;
        }
        if (epi == 0)
            ((uint16_t *)out)[(long)m * ldo + n] = f32_to_bf16_rne(acc);
        else {
            float *p = (float *)out + (long)m * ldo + n;
            *p = *p + acc;
        }
    }
}

/* The fused SwiGLU epilogue, kernels/w8a8.py:86-98 (EPI 2), one scale group over K: the weight rows come in tiles of
 * bn rows, bn / 2 gate rows then the matching up rows (interleave_gate_up, w8a8.py:289-294).  Per row and tile:
 *   acc = mul_rn(mul_rn(float(acci), sa[m]), sw[n]);  act = gate / (1 + exp(-gate)) * up;
 *   scale = max(max|act|, 1e-10) / 127;  q = rint(act / scale).
 * q [M, N / 2] int8, s [M, N / bn] fp32.  exp is the C library's expf here: kernels are compared within one int8 step. */
void orc_w8a8_swiglu_epi(const int8_t *a, const float *a_s, const int8_t *w, const float *w_s, int8_t *q, float *s,
                         int live, int N, int K, int bn) {
    int hb = bn / 2, tiles = N / bn;
#pragma omp parallel for schedule(static)
    for (long idx = 0; idx < (long)live * tiles; ++idx) {
        int m = (int)(idx / tiles), t = (int)(idx % tiles);
        const int8_t *ar = a + (long)m * K;
        float act[128];
        float amax = 0.0f;
        for (int c = 0; c < hb; ++c) {
            const int8_t *gr = w + (long)(t * bn + c) * K, *ur = w + (long)(t * bn + hb + c) * K;
            int32_t gi = 0, ui = 0;
            for (int k = 0; k < K; ++k) {
                gi += (int32_t)ar[k] * (int32_t)gr[k];
                ui += (int32_t)ar[k] * (int32_t)ur[k];
            }
            float g = (float)gi * a_s[m];
            g = g * w_s[t * bn + c];
            float u = (float)ui * a_s[m];
            u = u * w_s[t * bn + hb + c];
            float v = g / (1.0f + expf(-g));
            v = v * u;
            act[c] = v;
            if (fabsf(v) > amax) amax = fabsf(v);
        }
        float scale = (amax > 1e-10f ? amax : 1e-10f) / 127.0f;
        for (int c = 0; c < hb; ++c) q[(long)m * (N / 2) + (long)t * hb + c] = (int8_t)nearbyintf(act[c] / scale);
        s[(long)m * tiles + t] = scale;
    }
}

/* ------------------------------------------------------------------------------------------- deferred residual add
 * kernels/quant.py:128-141 (_fold_parts), :434-446 (_fold_kernel): tot = sum over slots (int32, exact);
 * h = add_rn(h, mul_rn(mul_rn(float(tot), a_s[r]), w_s[c])).  slots [S, rows, N] with slot stride `ss` elements. */
void orc_fold(float *h, long ldh, const int32_t *slots, long ss, int S, const float *a_s, const float *w_s, int live,
              int N) {
#pragma omp parallel for schedule(static)
    for (int r = 0; r < live; ++r)
        for (int c = 0; c < N; ++c) {
            int32_t tot = 0;
            for (int p = 0; p < S; ++p) tot += slots[p * ss + (long)r * N + c];
            float v = (float)tot * a_s[r];
            v = v * w_s[c];
            h[(long)r * ldh + c] = h[(long)r * ldh + c] + v;
        }
}

/* -------------------------------------------------------------------------------------- per-token activation quant
 * kernels/quant.py:287-309 (_rows_q8_kernel) and kernels/w8a8.py:101-112 (_quant_rows_kernel):
 *   y = float(x) * inv_s[k]; scale = max(max|y|, 1e-10) / 127; q = rint(y / scale) (half to even) -> int8.
 * One scale per (row, group of gk inputs); gk == K for rows_q8.  Divisions are IEEE (the contract of this build; the
 * reference's Triton `/` is not guaranteed correctly rounded).  x is bf16 (x_is_bf16) or fp32; inv_s may be NULL.
 * amax_in (may be NULL): the row maxima to use instead of the row's own (tensor parallel mode 2, quant.py:303-304:
 * amax = max(amax_in[t], own)); amax_out (may be NULL): the row's own maximum (mode 1, quant.py:301-302). */
void orc_quant_rows(const void *x, int x_is_bf16, const float *inv_s, int8_t *q, float *s, int live, int K, int gk,
                    const float *amax_in, float *amax_out) {
    int G = K / gk;
#pragma omp parallel for schedule(static)
    for (int r = 0; r < live; ++r)
        for (int g = 0; g < G; ++g) {
            float amax = 0.0f;
            for (int k = g * gk; k < (g + 1) * gk; ++k) {
                float v = x_is_bf16 ? bf16_to_f32(((const uint16_t *)x)[(long)r * K + k]) : ((const float *)x)[(long)r * K + k];
                if (inv_s) v = v * inv_s[k];
                float av = fabsf(v);
                if (av > amax) amax = av;
            }
            if (amax_out) amax_out[(long)r * G + g] = amax;
            if (amax_in && amax_in[(long)r * G + g] > amax) amax = amax_in[(long)r * G + g];
            float scale = (amax > 1e-10f ? amax : 1e-10f) / 127.0f;
            for (int k = g * gk; k < (g + 1) * gk; ++k) {
                float v = x_is_bf16 ? bf16_to_f32(((const uint16_t *)x)[(long)r * K + k]) : ((const float *)x)[(long)r * K + k];
                if (inv_s) v = v * inv_s[k];
                q[(long)r * K + k] = (int8_t)nearbyintf(v / scale);
            }
            s[(long)r * G + g] = scale;
        }
}

/* SwiGLU producer, kernels/quant.py:249-284 (_swiglu_piece, _swiglu_q8_kernel):
 *   y = g / (1 + exp(-g)) * u * inv_s[c], then the per-token quantization above.  exp is the C library's expf here;
 * the GPU's differs in the last bits, so tests compare this producer within one int8 step (as the reference's own
 * test does for its fused producers, tests/test_w4a8.py:91-102), never bit for bit. */
void orc_swiglu_q8(const uint16_t *gu, const float *inv_s, int8_t *q, float *s, int live, int FF) {
#pragma omp parallel for schedule(static)
    for (int r = 0; r < live; ++r) {
        const uint16_t *row = gu + (long)r * 2 * FF;
        float amax = 0.0f;
        for (int c = 0; c < FF; ++c) {
            float g = bf16_to_f32(row[c]), u = bf16_to_f32(row[FF + c]);
            float y = g / (1.0f + expf(-g)) * u;
            if (inv_s) y = y * inv_s[c];
            if (fabsf(y) > amax) amax = fabsf(y);
        }
        float scale = (amax > 1e-10f ? amax : 1e-10f) / 127.0f;
        for (int c = 0; c < FF; ++c) {
            float g = bf16_to_f32(row[c]), u = bf16_to_f32(row[FF + c]);
            float y = g / (1.0f + expf(-g)) * u;
            if (inv_s) y = y * inv_s[c];
            q[(long)r * FF + c] = (int8_t)nearbyintf(y / scale);
        }
        s[r] = scale;
    }
}

/* ------------------------------------------------------------------------------------ norm_q8 (RMSNorm + quant)
 * kernels/quant.py:145-171 (_norm_q8_kernel): after the optional deferred add (same roundings as orc_fold),
 *   y = h * rsqrt(sum(h * h) / HID + eps) * w;  scale = max(max|y|, 1e-10) / 127;  q = rint(y / scale).
 * The reference reduces h * h in an order its compiler picks; this restatement adds the squares in double precision
 * (the order-free answer) and rounds once, so kernels are compared with it within one int8 step. */
void orc_norm_q8(float *h, const float *w, int8_t *q, float *s, const int *rows, int live, int HID, float eps,
                 const int32_t *parts, long part_stride, int n_parts, const float *psa, const float *psw) {
#pragma omp parallel for schedule(static)
    for (int i = 0; i < live; ++i) {
        long r = rows ? rows[i] : i;
        float *hr = h + r * HID;
        if (n_parts > 0) {
            for (int c = 0; c < HID; ++c) {
                int32_t tot = 0;
                for (int p = 0; p < n_parts; ++p) tot += parts[p * part_stride + r * HID + c];
                float v = (float)tot * psa[r];
                v = v * psw[c];
                hr[c] = hr[c] + v;
            }
        }
        double ss = 0.0;
        for (int c = 0; c < HID; ++c) ss += (double)hr[c] * (double)hr[c];
        float mean = (float)(ss / HID);
        float rinv = (float)(1.0 / sqrt((double)(mean + eps)));
        float amax = 0.0f;
        for (int c = 0; c < HID; ++c) {
            float y = hr[c] * rinv;
            y = y * w[c];
            if (fabsf(y) > amax) amax = fabsf(y);
        }
        float scale = (amax > 1e-10f ? amax : 1e-10f) / 127.0f;
        for (int c = 0; c < HID; ++c) {
            float y = hr[c] * rinv;
            y = y * w[c];
            q[(long)i * HID + c] = (int8_t)nearbyintf(y / scale);
        }
        s[i] = scale;
    }
}

/* ------------------------------------------------------------------------------------ gated_norm_q8
 * kernels/quant.py:215-246 (_gated_norm_q8_kernel):
 *   y = o * rsqrt(sum_D(o * o) / D + eps) * w[d] * (z / (1 + exp(-z)));  y = y * inv_s;  per-token scale and rint.
 * Sum of squares in double (the reference's order is its compiler's), libm expf: compared within one int8 step. */
void orc_gated_norm_q8(const float *o, const uint16_t *proj, long P, long z_off, const float *w, const float *inv_s,
                       int8_t *q, float *s, int live, int HV, int D, float eps, const float *amax_in, float *amax_out) {
#pragma omp parallel for schedule(static)
    for (int t = 0; t < live; ++t) {
        float amax = 0.0f;
        float *y = (float *)malloc(sizeof(float) * HV * D);
        for (int h = 0; h < HV; ++h) {
            const float *oh = o + ((long)t * HV + h) * D;
            double ss = 0.0;
            for (int d = 0; d < D; ++d) ss += (double)oh[d] * (double)oh[d];
            float mean = (float)(ss / D);
            float rinv = (float)(1.0 / sqrt((double)(mean + eps)));
            for (int d = 0; d < D; ++d) {
                float z = bf16_to_f32(proj[(long)t * P + z_off + (long)h * D + d]);
                float g = z / (1.0f + expf(-z));
                float v = oh[d] * rinv;
                v = v * w[d];
                v = v * g;
                v = v * inv_s[h * D + d];
                y[h * D + d] = v;
                if (fabsf(v) > amax) amax = fabsf(v);
            }
        }
        if (amax_out) amax_out[t] = amax;
        if (amax_in && amax_in[t] > amax) amax = amax_in[t];
        float scale = (amax > 1e-10f ? amax : 1e-10f) / 127.0f;
        for (int i = 0; i < HV * D; ++i) q[(long)t * HV * D + i] = (int8_t)nearbyintf(y[i] / scale);
        s[t] = scale;
        free(y);
    }
}

/* ------------------------------------------------------------------------------------ the producers' fp32 rows
 * y of swiglu (kernels/quant.py:256), RMSNorm (:166) and the gated norm (:236-237) before any quantizer, for the W4A8
 * twins (swiglu_g, norm_g, gated_norm_g: the same rows through the per-256 quantizer orc_quant_g). */
void orc_swiglu_y(const uint16_t *gu, float *y, int live, int FF) {
#pragma omp parallel for schedule(static)
    for (int r = 0; r < live; ++r)
        for (int c = 0; c < FF; ++c) {
            float g = bf16_to_f32(gu[(long)r * 2 * FF + c]), u = bf16_to_f32(gu[(long)r * 2 * FF + FF + c]);
            y[(long)r * FF + c] = g / (1.0f + expf(-g)) * u;
        }
}

void orc_norm_y(const float *h, const float *w, float *y, int live, int HID, float eps) {
#pragma omp parallel for schedule(static)
    for (int r = 0; r < live; ++r) {
        const float *hr = h + (long)r * HID;
        double ss = 0.0;
        for (int c = 0; c < HID; ++c) ss += (double)hr[c] * (double)hr[c];
        float mean = (float)(ss / HID);
        float rinv = (float)(1.0 / sqrt((double)(mean + eps)));
        for (int c = 0; c < HID; ++c) {
            float v = hr[c] * rinv;
            y[(long)r * HID + c] = v * w[c];
        }
    }
}

void orc_gated_norm_y(const float *o, const uint16_t *proj, long P, long z_off, const float *w, float *y, int live,
                      int HV, int D, float eps) {
#pragma omp parallel for schedule(static)
    for (int t = 0; t < live; ++t)
        for (int h = 0; h < HV; ++h) {
            const float *oh = o + ((long)t * HV + h) * D;
            double ss = 0.0;
            for (int d = 0; d < D; ++d) ss += (double)oh[d] * (double)oh[d];
            float mean = (float)(ss / D);
            float rinv = (float)(1.0 / sqrt((double)(mean + eps)));
            for (int d = 0; d < D; ++d) {
                float z = bf16_to_f32(proj[(long)t * P + z_off + (long)h * D + d]);
                float v = oh[d] * rinv;
                v = v * w[d];
                y[((long)t * HV + h) * D + d] = v * (z / (1.0f + expf(-z)));
            }
        }
}

/* ------------------------------------------------------------------------------------ head_quant
 * kernels/decode.py:113-133 (_head_quant_kernel): y = h * rsqrt(sum(h * h) / HID + eps) * w, then per 32 inputs
 * scale = max(max|y|, 1e-10) / 127, q = rint(y / scale).  Sum of squares in double (order-free). */
void orc_head_quant(const float *h, const float *w, int8_t *q, float *s, int live, int HID, float eps) {
#pragma omp parallel for schedule(static)
    for (int r = 0; r < live; ++r) {
        const float *hr = h + (long)r * HID;
        double ss = 0.0;
        for (int c = 0; c < HID; ++c) ss += (double)hr[c] * (double)hr[c];
        float mean = (float)(ss / HID);
        float rinv = (float)(1.0 / sqrt((double)(mean + eps)));
        for (int g = 0; g < HID / 32; ++g) {
            float y[32], amax = 0.0f;
            for (int k = 0; k < 32; ++k) {
                float v = hr[g * 32 + k] * rinv;
                y[k] = v * w[g * 32 + k];
                if (fabsf(y[k]) > amax) amax = fabsf(y[k]);
            }
            float scale = (amax > 1e-10f ? amax : 1e-10f) / 127.0f;
            for (int k = 0; k < 32; ++k) q[(long)r * HID + g * 32 + k] = (int8_t)nearbyintf(y[k] / scale);
            s[(long)r * (HID / 32) + g] = scale;
        }
    }
}

/* ------------------------------------------------------------------------------------ W4A8 activation quant (per 256)
 * kernels/quant.py:314-330 (_store_g) == kernels/w4a8.py:144-155 (quantize_ref):
 *   scale = div_rn(max(max|y|, 1e-10), 127) per 256 inputs; q = rint(div_rn(y, scale));
 *   sums S of each 32 int8 values stored as eight (S & 63) then eight (S >> 6) per 256 inputs.
 * q [M, K]; a [K/256, M] (super-block-major, M = alloc rows); xs [K/256, M, 16]. */
void orc_quant_g(const void *x, int x_is_bf16, int8_t *q, float *a, int8_t *xs, int live, int M, int K) {
    int NB = K / 256;
#pragma omp parallel for schedule(static)
    for (int r = 0; r < live; ++r)
        for (int b = 0; b < NB; ++b) {
            float y[256];
            float amax = 0.0f;
            for (int k = 0; k < 256; ++k) {
                long i = (long)r * K + b * 256 + k;
                y[k] = x_is_bf16 ? bf16_to_f32(((const uint16_t *)x)[i]) : ((const float *)x)[i];
                if (fabsf(y[k]) > amax) amax = fabsf(y[k]);
            }
            float scale = (amax > 1e-10f ? amax : 1e-10f) / 127.0f;
            a[(long)b * M + r] = scale;
            for (int g = 0; g < 8; ++g) {
                int32_t S = 0;
                for (int k = 0; k < 32; ++k) {
                    int8_t v = (int8_t)nearbyintf(y[g * 32 + k] / scale);
                    q[(long)r * K + b * 256 + g * 32 + k] = v;
                    S += v;
                }
                xs[((long)b * M + r) * 16 + g] = (int8_t)(S & 63);
                xs[((long)b * M + r) * 16 + 8 + g] = (int8_t)(S >> 6);
            }
        }
}

/* ------------------------------------------------------------------------------------------------------ W4A8 GEMM
 * kernels/w4a8.py:14-24 (the arithmetic) and :177-199 (gemm_ref), on the repacked operands of w4a8.py:70-94:
 *   Q4_K: q uint8 [n, k/2], byte t of each 16 = q[t] | q[t+16] << 4 per 32 inputs; sc, mn uint8 [k/256, n, 8];
 *         d, dm fp32 [k/256, n].   acc = sum_g sc[g] * (xq . q)_g;  mins = sum_g mn[g] * S_g;
 *         t = d * float(acc); t = fma(-dm, float(mins), t); y = fma(a[m, b], t, y).
 *   Q6_K: q int8 [n, k] (value - 32); sc int8 [k/256, n, 16]; d fp32 [k/256, n].
 *         acc = sum_h sc[h] * (xq . q)_h over 16-input sub-blocks; y = fma(a[m, b], d * float(acc), y).
 * fmaf is a single-rounding fused multiply-add (what w4a8.py:164-174 emulates in float64).
 * epi 0: bf16(y); epi 1: out = add_rn(out, y) (w4a8.py:214-222).  kind 0 = Q4_K, 1 = Q6_K.  Ma = allocated rows of
 * a / xs (their row stride). */
void orc_w4a8_gemm(const int8_t *xq, const float *a, const int8_t *xs, int Ma, const void *wq, const void *wsc,
                   const uint8_t *wmn, const float *wd, const float *wdm, void *out, long ldo, int live, int N,
                   int K, int kind, int epi) {
    int NB = K / 256;
#pragma omp parallel for schedule(static)
    for (long idx = 0; idx < (long)live * N; ++idx) {
        int m = (int)(idx / N), n = (int)(idx % N);
        float y = 0.0f;
        for (int b = 0; b < NB; ++b) {
            const int8_t *xr = xq + (long)m * K + b * 256;
            float t;
            if (kind == 0) {
                const uint8_t *qr = (const uint8_t *)wq + (long)n * (K / 2) + b * 128;
                const uint8_t *sc = (const uint8_t *)wsc + ((long)b * N + n) * 8;
                const uint8_t *mn = wmn + ((long)b * N + n) * 8;
                const int8_t *sx = xs + ((long)b * Ma + m) * 16;
                int32_t acc = 0, mins = 0;
                for (int g = 0; g < 8; ++g) {
                    int32_t dot = 0;
                    for (int i = 0; i < 16; ++i) {
                        dot += (int32_t)xr[g * 32 + i] * (int32_t)(qr[g * 16 + i] & 15);
                        dot += (int32_t)xr[g * 32 + 16 + i] * (int32_t)(qr[g * 16 + i] >> 4);
                    }
                    acc += (int32_t)sc[g] * dot;
                    mins += (int32_t)mn[g] * ((int32_t)sx[g] + 64 * (int32_t)sx[8 + g]);
                }
                t = wd[(long)b * N + n] * (float)acc;
                t = fmaf(-wdm[(long)b * N + n], (float)mins, t);
            } else {
                const int8_t *qr = (const int8_t *)wq + (long)n * K + b * 256;
                const int8_t *sc = (const int8_t *)wsc + ((long)b * N + n) * 16;
                int32_t acc = 0;
                for (int h = 0; h < 16; ++h) {
                    int32_t dot = 0;
                    for (int i = 0; i < 16; ++i) dot += (int32_t)xr[h * 16 + i] * (int32_t)qr[h * 16 + i];
                    acc += (int32_t)sc[h] * dot;
                }
                t = wd[(long)b * N + n] * (float)acc;
            }
            y = fmaf(a[(long)b * Ma + m], t, y);
        }
        if (epi == 0)
            ((uint16_t *)out)[(long)m * ldo + n] = f32_to_bf16_rne(y);
        else {
            float *p = (float *)out + (long)m * ldo + n;
            *p = *p + y;
        }
    }
}

/* --------------------------------------------------------------------------------------------------------- MXFP4
 * kernels/mxfp4.py:40-54 (_e2m1_code) / :106-117 (_code): magnitude code by strict thresholds, sign bit 8 unless
 * the magnitude code is 0 for weights (mxfp4.py:53); the activation kernel sets the sign bit whenever v < 0
 * (mxfp4.py:117) - `neg_zero` selects that variant. */
static inline uint8_t e2m1_code(float v, float sc, int neg_zero) {
    float a = fabsf(v) / sc;
    uint8_t c = 0;
    if (a > 0.25f) c = 1;
    if (a > 0.75f) c = 2;
    if (a > 1.25f) c = 3;
    if (a > 1.75f) c = 4;
    if (a > 2.5f) c = 5;
    if (a > 3.5f) c = 6;
    if (a > 5.0f) c = 7;
    if (v < 0 && (neg_zero || c != 0)) c |= 8;
    return c;
}

/* The block exponent e = clamp(ceil(log2(max(amax, 1e-30) / 6)), -127, 127) (mxfp4.py:66-69 for weights,
 * :133-134 for activations), evaluated exactly: the smallest integer e with 6 * 2^e >= amax. */
static inline int mx_exponent(float amax) {
    if (!(amax > 1e-30f)) amax = 1e-30f;
    int x;
    float m = frexpf(amax, &x); /* amax = m * 2^x, m in [0.5, 1) */
    int e = (m <= 0.75f) ? x - 3 : x - 2;
    if (e < -127) e = -127;
    if (e > 127) e = 127;
    return e;
}

/* kernels/mxfp4.py:119-145 (_quant_kernel), :182-185 (quantize_act): x [n, k] -> q uint8 [n, k/2] (low nibble =
 * even k), s uint8 [n, k/32] = e + 127.  inv (may be NULL): the per-column pre-scale of :148-171. */
void orc_mxfp4_quant(const void *x, int x_is_bf16, const float *inv, uint8_t *q, uint8_t *s, int n, int K,
                     int neg_zero) {
#pragma omp parallel for schedule(static)
    for (int r = 0; r < n; ++r)
        for (int b = 0; b < K / 32; ++b) {
            float v[32], amax = 0.0f;
            for (int k = 0; k < 32; ++k) {
                long i = (long)r * K + b * 32 + k;
                v[k] = x_is_bf16 ? bf16_to_f32(((const uint16_t *)x)[i]) : ((const float *)x)[i];
                if (inv) v[k] = v[k] * inv[b * 32 + k];
                if (fabsf(v[k]) > amax) amax = fabsf(v[k]);
            }
            int e = mx_exponent(amax);
            float sc = ldexpf(1.0f, e);
            for (int k = 0; k < 32; k += 2)
                q[(long)r * (K / 2) + b * 16 + k / 2] =
                    (uint8_t)(e2m1_code(v[k], sc, neg_zero) | (e2m1_code(v[k + 1], sc, neg_zero) << 4));
            s[(long)r * (K / 32) + b] = (uint8_t)(e + 127);
        }
}

static const float E2M1_LUT[16] = {0.f, .5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f, -0.f, -.5f, -1.f, -1.5f, -2.f, -3.f, -4.f, -6.f};

/* kernels/mxfp4.py:89-101 (dequant_packed) and tests/test_mxfp4.py:54-57 (ref_gemm): out = deq(A) deq(W)^T,
 * accumulated in float64 (the tolerance oracle; no reference test pins the MMA's internal summation order).
 * epi 0: bf16 out; epi 1: fp32 out = prev + acc (mxfp4.py:285-287).  out64 (may be NULL) receives the float64 sums. */
void orc_mxfp4_gemm(const uint8_t *aq, const uint8_t *as, const uint8_t *wq, const uint8_t *ws, void *out, long ldo,
                    double *out64, int M, int N, int K, int epi) {
#pragma omp parallel for schedule(static)
    for (long idx = 0; idx < (long)M * N; ++idx) {
        int m = (int)(idx / N), n = (int)(idx % N);
        double acc = 0.0;
        for (int b = 0; b < K / 32; ++b) {
            double part = 0.0;
            for (int i = 0; i < 16; ++i) {
                uint8_t ab = aq[(long)m * (K / 2) + b * 16 + i], wb = wq[(long)n * (K / 2) + b * 16 + i];
                part += (double)E2M1_LUT[ab & 15] * (double)E2M1_LUT[wb & 15];
                part += (double)E2M1_LUT[ab >> 4] * (double)E2M1_LUT[wb >> 4];
            }
            int e = (int)as[(long)m * (K / 32) + b] - 127 + (int)ws[(long)n * (K / 32) + b] - 127;
            acc += ldexp(part, e);
        }
        if (out64) out64[(long)m * N + n] = acc;
        if (!out) continue;
        if (epi == 0)
            ((uint16_t *)out)[(long)m * ldo + n] = f32_to_bf16_rne((float)acc);
        else {
            float *p = (float *)out + (long)m * ldo + n;
            *p = *p + (float)acc;
        }
    }
}

/* ----------------------------------------------------------------------------------- the reference's CPU emulations
 * The timed CPU baseline (not a parity oracle): tests/quant_sim.py:97-107 (int8_rows) and tests/int8_sim.py:75-81
 * fake-quantize x and w to int8 grids and multiply in fp32: out[m, n] = sum_k xq[m, k] * wq[n, k] in fp32.  This is
 * the fp32 product the reference's reference.linear (reference.py:40-41) computes on the fake-quantized operands. */
void orc_fp32_linear(const float *x, const float *w, float *out, int M, int N, int K) {
#pragma omp parallel for schedule(static)
    for (long idx = 0; idx < (long)M * N; ++idx) {
        int m = (int)(idx / N), n = (int)(idx % N);
        const float *xr = x + (long)m * K, *wr = w + (long)n * K;
        float acc = 0.0f;
        for (int k = 0; k < K; ++k) acc += xr[k] * wr[k];
        out[idx] = acc;
    }
}

int orc_version(void) { return 1; }
