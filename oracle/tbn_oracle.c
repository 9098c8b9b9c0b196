/* CPU restatement of the fast-arm-tbcnn hot path.  See tbn_oracle.h.
 *
 * TEST INFRASTRUCTURE ONLY -- never linked into or loaded by the CUDA library.
 * Parity pinned by tests/test_oracle.py against the reference's golden vectors and
 * against the reference sources compiled as oracle/_ref/libtbn_ref.so.
 *
 * Build with -ffp-contract=off: the reference's fp32 loops are separate multiply
 * and add, and a fused multiply-add would change their rounding.
 */
#include "tbn_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>

#define ORC_OK 0
#define ORC_EINVAL (-1)
#define ORC_ENOMEM (-2)
#define ORC_ESHAPE (-7)

static uint32_t round_up_u32(uint32_t v, uint32_t m) { return (v + m - 1) / m * m; }

/* ---------------------------------------------------------------- quantise */

int orc_quantize_to_binary(const float* w, int64_t n, float thr, uint8_t* out) {
    /* quantized_gemm_neon.cpp:553-555: strict '>' so +0, -0 and NaN give 0 (= -1). */
    for (int64_t i = 0; i < n; ++i) out[i] = (w[i] > thr) ? 1 : 0;
    return ORC_OK;
}

int orc_sign_ge0(const float* w, int64_t n, int8_t* out) {
    /* model.hpp:433 and :803: '>= 0' so both zeros give +1, NaN gives -1. */
    for (int64_t i = 0; i < n; ++i) out[i] = (w[i] >= 0.0f) ? 1 : -1;
    return ORC_OK;
}

int orc_quantize_to_ternary(const float* w, int64_t n, float lo, float hi, int8_t* out) {
    /* quantized_gemm_neon.cpp:584-592 */
    for (int64_t i = 0; i < n; ++i) {
        if (w[i] < lo) out[i] = -1;
        else if (w[i] > hi) out[i] = 1;
        else out[i] = 0;
    }
    return ORC_OK;
}

int orc_channel_abs_mean(const float* w, int64_t channels, int64_t per, float* alpha) {
    /* model.hpp:388-394 */
    for (int64_t c = 0; c < channels; ++c) {
        float sum = 0.0f;
        for (int64_t i = 0; i < per; ++i) sum += fabsf(w[c * per + i]);
        alpha[c] = sum / (float)per;
    }
    return ORC_OK;
}

int orc_column_abs_mean(const float* w, int64_t K, int64_t N, float* alpha) {
    for (int64_t n = 0; n < N; ++n) {
        float sum = 0.0f;
        for (int64_t k = 0; k < K; ++k) sum += fabsf(w[k * N + n]);
        alpha[n] = sum / (float)K;
    }
    return ORC_OK;
}

int orc_column_abs_mean_nonzero(const float* w, int64_t K, int64_t N, float lo, float hi,
                                float* alpha) {
    for (int64_t n = 0; n < N; ++n) {
        float sum = 0.0f;
        int64_t cnt = 0;
        for (int64_t k = 0; k < K; ++k) {
            const float v = w[k * N + n];
            if (v < lo || v > hi) {
                sum += fabsf(v);
                ++cnt;
            }
        }
        alpha[n] = cnt ? sum / (float)cnt : 0.0f;
    }
    return ORC_OK;
}

/* -------------------------------------------------------------------- pack */

int orc_binary_pack(const int8_t* data, uint32_t rows, uint32_t cols, uint8_t* bits) {
    /* GeMM.cpp:119-124: shape rules; :131-147: column-major plane, bit set <=> -1. */
    if (rows % 64 != 0 || cols % 8 != 0) return ORC_EINVAL;
    const uint32_t col_bytes = rows / 8;
    memset(bits, 0, (size_t)cols * col_bytes);
    for (uint32_t n = 0; n < cols; ++n) {
        uint8_t* plane = bits + (size_t)n * col_bytes;
        for (uint32_t k = 0; k < rows; ++k) {
            const int8_t v = data[(size_t)k * cols + n];
            if (v == -1) plane[k >> 3] |= (uint8_t)(1u << (k & 7));
            else if (v != 1) return ORC_EINVAL;
        }
    }
    return ORC_OK;
}

int orc_binary_pack_padded(const uint8_t* b, uint32_t K, uint32_t N, uint32_t K_pad,
                           uint32_t N_pad, uint32_t* words) {
    /* quantized_gemm_neon.cpp:199-207: padding value +1 (bit 0); 1 -> +1, else -1. */
    if (K_pad < K || N_pad < N) return ORC_EINVAL;
    int8_t* tmp = (int8_t*)malloc((size_t)K_pad * N_pad);
    if (!tmp) return ORC_ENOMEM;
    memset(tmp, 1, (size_t)K_pad * N_pad);
    for (uint32_t k = 0; k < K; ++k)
        for (uint32_t n = 0; n < N; ++n)
            tmp[(size_t)k * N_pad + n] = (b[(size_t)k * N + n] == 1) ? 1 : -1;
    const int rc = orc_binary_pack(tmp, K_pad, N_pad, (uint8_t*)words);
    free(tmp);
    return rc;
}

int orc_ternary_codes(const int8_t* t, int64_t n, uint8_t* out) {
    /* packed_weights.hpp:53-71: -1 -> 0, 0 -> 1, +1 -> 2, anything else -> 1. */
    memset(out, 0, (size_t)((n + 3) / 4));
    for (int64_t i = 0; i < n; ++i) {
        uint8_t code = 1;
        if (t[i] == -1) code = 0;
        else if (t[i] == 1) code = 2;
        out[i / 4] |= (uint8_t)(code << (2 * (i % 4)));
    }
    return ORC_OK;
}

int orc_ternary_pack(const int8_t* data, uint32_t rows, uint32_t cols, uint8_t* pos, uint8_t* neg) {
    /* GeMM.cpp:34-39 shape rules; :50-66 planes. */
    if (rows % 8 != 0 || cols % 64 != 0) return ORC_EINVAL;
    const uint32_t row_bytes = cols / 8;
    memset(pos, 0, (size_t)rows * row_bytes);
    memset(neg, 0, (size_t)rows * row_bytes);
    for (uint32_t i = 0; i < rows; ++i) {
        for (uint32_t j = 0; j < cols; ++j) {
            const int8_t v = data[(size_t)i * cols + j];
            const uint8_t bit = (uint8_t)(1u << (j & 7));
            if (v == 1) pos[(size_t)i * row_bytes + (j >> 3)] |= bit;
            else if (v == -1) neg[(size_t)i * row_bytes + (j >> 3)] |= bit;
            else if (v != 0) return ORC_EINVAL;
        }
    }
    return ORC_OK;
}

int orc_ternary_pack_from_float(const float* data, uint32_t rows, uint32_t cols, float lo, float hi,
                                uint8_t* pos, uint8_t* neg) {
    /* GeMM.cpp:78-109: '< lo' -> negative plane, else '> hi' -> positive plane. */
    if (rows % 8 != 0 || cols % 64 != 0) return ORC_EINVAL;
    const uint32_t row_bytes = cols / 8;
    memset(pos, 0, (size_t)rows * row_bytes);
    memset(neg, 0, (size_t)rows * row_bytes);
    for (uint32_t i = 0; i < rows; ++i) {
        for (uint32_t j = 0; j < cols; ++j) {
            const float v = data[(size_t)i * cols + j];
            const uint8_t bit = (uint8_t)(1u << (j & 7));
            if (v < lo) neg[(size_t)i * row_bytes + (j >> 3)] |= bit;
            else if (v > hi) pos[(size_t)i * row_bytes + (j >> 3)] |= bit;
        }
    }
    return ORC_OK;
}

/* -------------------------------------------------------------------- GEMM */

int orc_gemm_tbn(const uint8_t* pos, const uint8_t* neg, const uint8_t* bits, uint32_t M, uint32_t K,
                 uint32_t N, int32_t* C) {
    /* GeMM.cpp:233-249: pos = (ap|bc)&(am|~bc), neg = (ap|~bc)&(am|bc), C += pop(pos)-pop(neg).
     * Stated here per 64-bit chunk over the whole K range (GeMM.hpp:24-29 requires K%128==0). */
    if (K % 64 != 0) return ORC_EINVAL;
    const uint32_t kb = K / 8;
    for (uint32_t m = 0; m < M; ++m) {
        for (uint32_t n = 0; n < N; ++n) {
            int32_t acc = 0;
            for (uint32_t w = 0; w < kb; w += 8) {
                uint64_t ap, am, bc;
                memcpy(&ap, pos + (size_t)m * kb + w, 8);
                memcpy(&am, neg + (size_t)m * kb + w, 8);
                memcpy(&bc, bits + (size_t)n * kb + w, 8);
                const uint64_t pm = (ap | bc) & (am | ~bc);
                const uint64_t nm = (ap | ~bc) & (am | bc);
                acc += __builtin_popcountll(pm) - __builtin_popcountll(nm);
            }
            C[(size_t)m * N + n] = acc;
        }
    }
    return ORC_OK;
}

int orc_qlinear_matmul_binary(const float* a, uint32_t M, uint32_t K, const uint8_t* b, uint32_t N,
                              float scale, float lo, float hi, float* C) {
    /* quantized_gemm_neon.cpp:53-55 padding rule, :186-195 ternarise+pack A (zero padded),
     * :199-214 pack B (+1 padded), :217-240 compute, scale, crop. */
    const uint32_t Mp = round_up_u32(M, 16), Kp = round_up_u32(K, 128), Np = round_up_u32(N, 8);
    float* ap = (float*)calloc((size_t)Mp * Kp, sizeof(float));
    uint8_t* pos = (uint8_t*)malloc((size_t)Mp * Kp / 8);
    uint8_t* neg = (uint8_t*)malloc((size_t)Mp * Kp / 8);
    uint32_t* words = (uint32_t*)malloc((size_t)Np * Kp / 8);
    int32_t* acc = (int32_t*)malloc((size_t)Mp * Np * sizeof(int32_t));
    int rc = ORC_ENOMEM;
    if (ap && pos && neg && words && acc) {
        for (uint32_t i = 0; i < M; ++i) memcpy(ap + (size_t)i * Kp, a + (size_t)i * K, K * sizeof(float));
        rc = orc_ternary_pack_from_float(ap, Mp, Kp, lo, hi, pos, neg);
        if (!rc) rc = orc_binary_pack_padded(b, K, N, Kp, Np, words);
        if (!rc) rc = orc_gemm_tbn(pos, neg, (const uint8_t*)words, Mp, Kp, Np, acc);
        if (!rc)
            for (uint32_t i = 0; i < M; ++i)
                for (uint32_t j = 0; j < N; ++j)
                    C[(size_t)i * N + j] = (float)acc[(size_t)i * Np + j] * scale;
    }
    free(ap); free(pos); free(neg); free(words); free(acc);
    return rc;
}

int orc_fxb_naive(const float* a, int64_t M, int64_t K, const uint8_t* b, int64_t N, float scale,
                  float* C) {
    /* quantized_gemm_neon.cpp:77-87 */
    for (int64_t i = 0; i < M; ++i) {
        for (int64_t j = 0; j < N; ++j) {
            float sum = 0.0f;
            for (int64_t k = 0; k < K; ++k) {
                const float sign = (b[k * N + j] == 1) ? 1.0f : -1.0f;
                sum += a[i * K + k] * sign;
            }
            C[i * N + j] = sum * scale;
        }
    }
    return ORC_OK;
}

int orc_gemm_f32(const float* a, int64_t a_rows, int64_t a_cols, const float* b, int64_t b_rows,
                 int64_t b_cols, const float* c, int c_ndim, float alpha, float beta, int transA,
                 int transB, float* out) {
    /* gemm.cpp:46-48 dims, :54-69 initialise, :72-124 blocked accumulate (scalar branch). */
    const int64_t BS = 64;
    const int64_t M = transA ? a_cols : a_rows;
    const int64_t K = transA ? a_rows : a_cols;
    const int64_t N = transB ? b_rows : b_cols;
    const int64_t Kb = transB ? b_cols : b_rows;
    if (K != Kb) return ORC_ESHAPE;
    if (c && c_ndim && beta != 0.0f) {
        for (int64_t i = 0; i < M; ++i)
            for (int64_t j = 0; j < N; ++j)
                out[i * N + j] = beta * (c_ndim == 1 ? c[j] : c[i * N + j]);
    } else {
        memset(out, 0, (size_t)(M * N) * sizeof(float));
    }
    for (int64_t i0 = 0; i0 < M; i0 += BS) {
        const int64_t i1 = i0 + BS < M ? i0 + BS : M;
        for (int64_t j0 = 0; j0 < N; j0 += BS) {
            const int64_t j1 = j0 + BS < N ? j0 + BS : N;
            for (int64_t k0 = 0; k0 < K; k0 += BS) {
                const int64_t k1 = k0 + BS < K ? k0 + BS : K;
                for (int64_t i = i0; i < i1; ++i) {
                    for (int64_t j = j0; j < j1; ++j) {
                        float sum = 0.0f;
                        for (int64_t k = k0; k < k1; ++k) {
                            const float av = transA ? a[k * M + i] : a[i * K + k];
                            const float bv = transB ? b[j * K + k] : b[k * N + j];
                            sum += av * bv;
                        }
                        out[i * N + j] += alpha * sum;
                    }
                }
            }
        }
    }
    return ORC_OK;
}

/* -------------------------------------------------------------------- conv */

int64_t orc_conv_out_dim(int64_t in, int64_t k, int64_t s, int64_t p, int64_t d) {
    return (in + 2 * p - d * (k - 1) - 1) / s + 1;
}

int orc_conv2d_f32(const float* x, int64_t N, int64_t C, int64_t H, int64_t W, const float* w,
                   int64_t M, int64_t kh, int64_t kw, const float* bias, const int64_t* p, float* out) {
    /* conv2d.cpp:114-117 output size, :130-149 bias init, :151-186 accumulate. */
    const int64_t sh = p[0], sw = p[1], ph = p[2], pw = p[3], dh = p[4], dw = p[5];
    const int64_t OH = orc_conv_out_dim(H, kh, sh, ph, dh), OW = orc_conv_out_dim(W, kw, sw, pw, dw);
    if (OH <= 0 || OW <= 0) return ORC_ESHAPE;
    for (int64_t n = 0; n < N; ++n)
        for (int64_t m = 0; m < M; ++m)
            for (int64_t oh = 0; oh < OH; ++oh)
                for (int64_t ow = 0; ow < OW; ++ow) {
                    float acc = bias ? bias[m] : 0.0f;
                    for (int64_t c = 0; c < C; ++c)
                        for (int64_t i = 0; i < kh; ++i)
                            for (int64_t j = 0; j < kw; ++j) {
                                const int64_t ih = oh * sh - ph + i * dh;
                                const int64_t iw = ow * sw - pw + j * dw;
                                if (ih < 0 || ih >= H || iw < 0 || iw >= W) continue;
                                acc += x[((n * C + c) * H + ih) * W + iw] * w[((m * C + c) * kh + i) * kw + j];
                            }
                    out[((n * M + m) * OH + oh) * OW + ow] = acc;
                }
    return ORC_OK;
}

int orc_im2col(const float* x, int64_t N, int64_t C, int64_t H, int64_t W, int64_t kh, int64_t kw,
               const int64_t* p, float* col) {
    /* conv2d.cpp:432-438 shapes, :484-501 general gather (the contiguous fast path
     * :447-481 produces the same values). */
    const int64_t sh = p[0], sw = p[1], ph = p[2], pw = p[3], dh = p[4], dw = p[5];
    const int64_t OH = orc_conv_out_dim(H, kh, sh, ph, dh), OW = orc_conv_out_dim(W, kw, sw, pw, dw);
    const int64_t cols = C * kh * kw;
    for (int64_t n = 0; n < N; ++n)
        for (int64_t oh = 0; oh < OH; ++oh)
            for (int64_t ow = 0; ow < OW; ++ow) {
                float* row = col + ((n * OH + oh) * OW + ow) * cols;
                for (int64_t c = 0; c < C; ++c)
                    for (int64_t i = 0; i < kh; ++i)
                        for (int64_t j = 0; j < kw; ++j) {
                            const int64_t ih = oh * sh - ph + i * dh;
                            const int64_t iw = ow * sw - pw + j * dw;
                            const int inside = ih >= 0 && ih < H && iw >= 0 && iw < W;
                            row[(c * kh + i) * kw + j] = inside ? x[((n * C + c) * H + ih) * W + iw] : 0.0f;
                        }
            }
    return ORC_OK;
}

int orc_im2col_ternary_packed(const float* x, int64_t N, int64_t C, int64_t H, int64_t W, int64_t kh,
                              int64_t kw, const int64_t* p, uint32_t m_padded, uint32_t k_padded,
                              float lo, float hi, uint8_t* pos, uint8_t* neg) {
    /* conv2d.cpp:529-533 zeroed planes, :572-593 general path (fast path :541-569 equal). */
    const int64_t sh = p[0], sw = p[1], ph = p[2], pw = p[3], dh = p[4], dw = p[5];
    const int64_t OH = orc_conv_out_dim(H, kh, sh, ph, dh), OW = orc_conv_out_dim(W, kw, sw, pw, dw);
    const uint32_t row_bytes = k_padded / 8;
    if ((int64_t)m_padded < N * OH * OW || (int64_t)k_padded < C * kh * kw) return ORC_EINVAL;
    memset(pos, 0, (size_t)m_padded * row_bytes);
    memset(neg, 0, (size_t)m_padded * row_bytes);
    for (int64_t n = 0; n < N; ++n)
        for (int64_t oh = 0; oh < OH; ++oh)
            for (int64_t ow = 0; ow < OW; ++ow) {
                const size_t row = (size_t)((n * OH + oh) * OW + ow) * row_bytes;
                for (int64_t c = 0; c < C; ++c)
                    for (int64_t i = 0; i < kh; ++i)
                        for (int64_t j = 0; j < kw; ++j) {
                            const int64_t ih = oh * sh - ph + i * dh;
                            const int64_t iw = ow * sw - pw + j * dw;
                            if (ih < 0 || ih >= H || iw < 0 || iw >= W) continue;
                            const int64_t k = (c * kh + i) * kw + j;
                            const uint8_t bit = (uint8_t)(1u << (k & 7));
                            const float v = x[((n * C + c) * H + ih) * W + iw];
                            if (v < lo) neg[row + (size_t)(k >> 3)] |= bit;
                            else if (v > hi) pos[row + (size_t)(k >> 3)] |= bit;
                        }
            }
    return ORC_OK;
}

int orc_conv2d_tbn_session(const float* x, int64_t N, int64_t C, int64_t H, int64_t W, const float* w,
                           int64_t M, int64_t kh, int64_t kw, const float* bias, const int64_t* p,
                           int use_alpha, float* out) {
    /* model.hpp:388-394 alpha, :433 sign, :464-472 transpose + pad(+1), :474-477 pack,
     * :482-497 fused im2col/ternarise at +-0.1, :500-503 GEMM scale 1, :505-521 reorder,
     * :524-538 + bias, :541-557 * alpha (skipped for alpha == 1). */
    const int64_t sh = p[0], sw = p[1], ph = p[2], pw = p[3], dh = p[4], dw = p[5];
    const int64_t OH = orc_conv_out_dim(H, kh, sh, ph, dh), OW = orc_conv_out_dim(W, kw, sw, pw, dw);
    const int64_t Kc = C * kh * kw;
    const uint32_t Kp = round_up_u32((uint32_t)Kc, 128), Np = round_up_u32((uint32_t)M, 8);
    const uint32_t Mo = (uint32_t)(N * OH * OW), Mp = round_up_u32(Mo, 8);
    float* alpha = (float*)malloc((size_t)M * sizeof(float));
    int8_t* bt = (int8_t*)malloc((size_t)Kp * Np);
    uint8_t* bits = (uint8_t*)malloc((size_t)Kp * Np / 8);
    uint8_t* pos = (uint8_t*)malloc((size_t)Mp * Kp / 8);
    uint8_t* neg = (uint8_t*)malloc((size_t)Mp * Kp / 8);
    int32_t* acc = (int32_t*)malloc((size_t)Mp * Np * sizeof(int32_t));
    int rc = ORC_ENOMEM;
    if (alpha && bt && bits && pos && neg && acc) {
        orc_channel_abs_mean(w, M, Kc, alpha);
        memset(bt, 1, (size_t)Kp * Np);
        for (int64_t m = 0; m < M; ++m)
            for (int64_t k = 0; k < Kc; ++k) bt[(size_t)k * Np + m] = (w[m * Kc + k] >= 0.0f) ? 1 : -1;
        rc = orc_binary_pack(bt, Kp, Np, bits);
        if (!rc) rc = orc_im2col_ternary_packed(x, N, C, H, W, kh, kw, p, Mp, Kp, -0.1f, 0.1f, pos, neg);
        if (!rc) rc = orc_gemm_tbn(pos, neg, bits, Mp, Kp, Np, acc);
        if (!rc)
            for (int64_t n = 0; n < N; ++n)
                for (int64_t m = 0; m < M; ++m)
                    for (int64_t s = 0; s < OH * OW; ++s) {
                        float v = (float)acc[(size_t)(n * OH * OW + s) * Np + m] * 1.0f;
                        if (bias) v += bias[m];
                        if (use_alpha && alpha[m] != 1.0f) v *= alpha[m];
                        out[(n * M + m) * OH * OW + s] = v;
                    }
    }
    free(alpha); free(bt); free(bits); free(pos); free(neg); free(acc);
    return rc;
}

/* -------------------------------------------------------------------- glue */

int64_t orc_pool_out_dim(int64_t in, int64_t k, int64_t s, int64_t p, int ceil_mode) {
    /* pooling.cpp:28-34 */
    return ceil_mode ? (in + 2 * p - k + s - 1) / s + 1 : (in + 2 * p - k) / s + 1;
}

int orc_pool2d(int kind, const float* x, int64_t N, int64_t C, int64_t H, int64_t W, const int64_t* p,
               int ceil_mode, int count_include_pad, float* out) {
    /* pooling.cpp:50-76 (max, out-of-range taps skipped) and :116-143 (avg). */
    const int64_t kh = p[0], kw = p[1], sh = p[2], sw = p[3], ph = p[4], pw = p[5];
    const int64_t OH = orc_pool_out_dim(H, kh, sh, ph, ceil_mode);
    const int64_t OW = orc_pool_out_dim(W, kw, sw, pw, ceil_mode);
    for (int64_t nc = 0; nc < N * C; ++nc)
        for (int64_t oh = 0; oh < OH; ++oh)
            for (int64_t ow = 0; ow < OW; ++ow) {
                float best = -INFINITY, sum = 0.0f;
                int count = 0;
                for (int64_t i = 0; i < kh; ++i)
                    for (int64_t j = 0; j < kw; ++j) {
                        const int64_t ih = oh * sh - ph + i, iw = ow * sw - pw + j;
                        if (ih >= 0 && ih < H && iw >= 0 && iw < W) {
                            const float v = x[(nc * H + ih) * W + iw];
                            best = best > v ? best : v; /* std::max(best, v) */
                            sum += v;
                            ++count;
                        } else if (count_include_pad) {
                            ++count;
                        }
                    }
                out[(nc * OH + oh) * OW + ow] = kind == 0 ? best : (count > 0 ? sum / (float)count : 0.0f);
            }
    return ORC_OK;
}

int orc_global_avgpool2d(const float* x, int64_t N, int64_t C, int64_t H, int64_t W, float* out) {
    /* pooling.cpp:203-213 */
    const int64_t hw = H * W;
    for (int64_t nc = 0; nc < N * C; ++nc) {
        float sum = 0.0f;
        for (int64_t i = 0; i < hw; ++i) sum += x[nc * hw + i];
        out[nc] = sum / (float)hw;
    }
    return ORC_OK;
}

int orc_relu(const float* x, int64_t n, float* out) {
    for (int64_t i = 0; i < n; ++i) out[i] = x[i] > 0.0f ? x[i] : 0.0f;
    return ORC_OK;
}

int orc_add(const float* a, int64_t a_n, const float* b, int64_t b_n, int64_t hw, float* out) {
    if (a_n == b_n) {
        for (int64_t i = 0; i < a_n; ++i) out[i] = a[i] + b[i];
        return ORC_OK;
    }
    if (b_n <= 0 || hw <= 0 || a_n % (b_n * hw) != 0) return ORC_ESHAPE;
    for (int64_t i = 0; i < a_n; ++i) out[i] = a[i] + b[(i / hw) % b_n];
    return ORC_OK;
}
