/* CPU restatement of the fast-arm-tbcnn hot path (plain C11, single thread).
 *
 * TEST INFRASTRUCTURE ONLY: used by tests/, the smoke check and the CPU-baseline
 * leg of the benchmark as the checker.  The CUDA library never links or loads it.
 *
 * Parity is pinned: tests/test_oracle.py checks these functions against the
 * reference's own golden vectors (GeMM/05-final/matrices_to_test.hpp,
 * GeMM/03-blocked/matrices_64x64.hpp, committed as tests/golden/ fixtures) and,
 * differentially, against the reference's sources compiled into
 * oracle/_ref/libtbn_ref.so.
 *
 * Every function cites the reference file:line it restates.  Matrices are
 * row-major.  GEMM dims follow C[M,N] = A[M,K] * B[K,N].
 * Return value: 0 on success, -1 invalid argument, -7 invalid shape
 * (the reference's ErrorCode values, tbn/utils/errors.hpp:10-22).
 */
#ifndef TBN_ORACLE_H
#define TBN_ORACLE_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- weight quantisation -------------------------------------------------- */

/* quantized_gemm_neon.cpp:544-565: out[i] = w[i] > thr ? 1 : 0 (1 means +1). */
int orc_quantize_to_binary(const float* w, int64_t n, float thr, uint8_t* out);

/* model.hpp:433,803: the Session's cached sign, out[i] = w[i] >= 0 ? +1 : -1. */
int orc_sign_ge0(const float* w, int64_t n, int8_t* out);

/* quantized_gemm_neon.cpp:570-597: -1 if w<lo, +1 if w>hi, else 0. */
int orc_quantize_to_ternary(const float* w, int64_t n, float lo, float hi, int8_t* out);

/* model.hpp:388-394: alpha[c] = (sum_i |w[c*per+i]|) / per, fp32 sequential. */
int orc_channel_abs_mean(const float* w, int64_t channels, int64_t per, float* alpha);

/* Per-column variants for a row-major W[K,N] (the training definition,
 * tests/train/mnist/train_tbn_mnist.py:128-139, applied to GEMM columns):
 * alpha[n] = sum_k |W[k,n]| / K, sequential in k. */
int orc_column_abs_mean(const float* w, int64_t K, int64_t N, float* alpha);
/* Ternary: alpha[n] = mean of |W[k,n]| over entries with W<lo or W>hi (0 if none). */
int orc_column_abs_mean_nonzero(const float* w, int64_t K, int64_t N, float lo, float hi,
                                float* alpha);

/* ---- bit packing ---------------------------------------------------------- */

/* GeMM.cpp:114-151 BinaryMatrix::pack: data[rows=K, cols=N] in {-1,+1};
 * bits[n*(K/8) + k/8] bit (k&7) set <=> -1.  rows%64==0, cols%8==0. */
int orc_binary_pack(const int8_t* data, uint32_t rows, uint32_t cols, uint8_t* bits);

/* quantized_gemm_neon.cpp:199-214 / model.hpp:464-477,819-830: BINARY bytes
 * (1 => +1, 0 => -1) of a [K,N] matrix, padded with +1 to [K_pad,N_pad]
 * (K_pad = ceil128(K), N_pad = ceil8(N)), then orc_binary_pack.  Output viewed as
 * little-endian uint32 words: word[n*(K_pad/32) + k/32] bit (k%32). */
int orc_binary_pack_padded(const uint8_t* b, uint32_t K, uint32_t N, uint32_t K_pad,
                           uint32_t N_pad, uint32_t* words);

/* packed_weights.hpp:53-71 TernaryPackedWeights::set_weight over i=0..n-1:
 * 2-bit code 0=-1, 1=0, 2=+1 at byte i/4, shift 2*(i%4).  out: (n+3)/4 bytes. */
int orc_ternary_codes(const int8_t* t, int64_t n, uint8_t* out);

/* GeMM.cpp:29-69 TernaryMatrix::pack (rows%8==0, cols%64==0): row-major planes. */
int orc_ternary_pack(const int8_t* data, uint32_t rows, uint32_t cols, uint8_t* pos, uint8_t* neg);

/* GeMM.cpp:71-112 TernaryMatrix::pack_from_float. */
int orc_ternary_pack_from_float(const float* data, uint32_t rows, uint32_t cols, float lo, float hi,
                                uint8_t* pos, uint8_t* neg);

/* ---- GEMMs ---------------------------------------------------------------- */

/* GeMM.cpp:159-363 GemmEngine::compute: C[m,n] = sum_k a*b with a from two
 * row-major planes [M, K/8], b from column-major bits [N, K/8]; int32 exact, so the
 * reference's tiling does not affect the result and is not restated. */
int orc_gemm_tbn(const uint8_t* pos, const uint8_t* neg, const uint8_t* bits, uint32_t M, uint32_t K,
                 uint32_t N, int32_t* C);

/* quantized_gemm_neon.cpp:165-243 (+ entry 380-430): pad A with zeros to
 * [ceil16(M), ceil128(K)], ternarise at (lo,hi), pad B with +1, integer GEMM,
 * C = float(int32) * scale.  b is BINARY bytes [K,N]. */
int orc_qlinear_matmul_binary(const float* a, uint32_t M, uint32_t K, const uint8_t* b, uint32_t N,
                              float scale, float lo, float hi, float* C);

/* quantized_gemm_neon.cpp:63-90 (the true float x binary product):
 * C[i,j] = scale * sum_k a[i,k] * (b[k,j]==1 ? +1 : -1), fp32, k ascending. */
int orc_fxb_naive(const float* a, int64_t M, int64_t K, const uint8_t* b, int64_t N, float scale,
                  float* C);

/* gemm.cpp:35-129 gemm_float_blocked, scalar branch: out = beta*C (1-D C broadcast
 * over rows) then for 64^3 blocks out[i,j] += alpha * (fp32 partial sum over the k-block).
 * c_ndim: 0 none, 1 C[N], 2 C[M,N]. */
int orc_gemm_f32(const float* a, int64_t a_rows, int64_t a_cols, const float* b, int64_t b_rows,
                 int64_t b_cols, const float* c, int c_ndim, float alpha, float beta, int transA,
                 int transB, float* out);

/* ---- convolution ---------------------------------------------------------- */

/* conv2d.cpp:432-433: out = (in + 2p - d(k-1) - 1)/s + 1. */
int64_t orc_conv_out_dim(int64_t in, int64_t k, int64_t s, int64_t p, int64_t d);

/* conv2d.cpp:78-192 naive direct convolution, accumulator initialised with bias,
 * then sum over (c, kh, kw) in that order.  p = {sh, sw, ph, pw, dh, dw}. */
int orc_conv2d_f32(const float* x, int64_t N, int64_t C, int64_t H, int64_t W, const float* w,
                   int64_t M, int64_t kh, int64_t kw, const float* bias, const int64_t* p, float* out);

/* conv2d.cpp:420-507 im2col: col[(n*OH+oh)*OW+ow][(c*kh+i)*kw+j], zero outside. */
int orc_im2col(const float* x, int64_t N, int64_t C, int64_t H, int64_t W, int64_t kh, int64_t kw,
               const int64_t* p, float* col);

/* conv2d.cpp:511-601 im2col fused with ternarisation into zero-padded planes. */
int orc_im2col_ternary_packed(const float* x, int64_t N, int64_t C, int64_t H, int64_t W, int64_t kh,
                              int64_t kw, const int64_t* p, uint32_t m_padded, uint32_t k_padded,
                              float lo, float hi, uint8_t* pos, uint8_t* neg);

/* model.hpp:375-559 Session::execute_conv cached fast path ("TBN mode"):
 * alpha = per-out-channel mean|w|; sign w>=0; weights -> [K_pad, ceil8(M)] padded +1;
 * activations ternarised at +-0.1 through im2col; int32 GEMM; NCHW reorder;
 * out = (acc + bias) * alpha  (bias BEFORE scale; scale skipped when
 * use_alpha == 0, which mirrors weights that fail the already-binary test). */
int orc_conv2d_tbn_session(const float* x, int64_t N, int64_t C, int64_t H, int64_t W, const float* w,
                           int64_t M, int64_t kh, int64_t kw, const float* bias, const int64_t* p,
                           int use_alpha, float* out);

/* ---- glue ops of the CNN graphs ------------------------------------------ */

/* pooling.cpp:10-80 / 83-148.  p = {kh, kw, sh, sw, ph, pw}; kind 0 max, 1 avg. */
int64_t orc_pool_out_dim(int64_t in, int64_t k, int64_t s, int64_t p, int ceil_mode);
int orc_pool2d(int kind, const float* x, int64_t N, int64_t C, int64_t H, int64_t W, const int64_t* p,
               int ceil_mode, int count_include_pad, float* out);
/* pooling.cpp:184-216: mean over H*W per (n,c), fp32 sequential. */
int orc_global_avgpool2d(const float* x, int64_t N, int64_t C, int64_t H, int64_t W, float* out);
/* model.hpp:1150-1170 */
int orc_relu(const float* x, int64_t n, float* out);
/* model.hpp:921-1036: same-shape add (a_n == b_n) or per-channel [C] broadcast over
 * [N,C,HW] (b_n == C, hw = spatial size) or row broadcast [M,N]+[N] (hw == 1). */
int orc_add(const float* a, int64_t a_n, const float* b, int64_t b_n, int64_t hw, float* out);

#ifdef __cplusplus
}
#endif
#endif /* TBN_ORACLE_H */
