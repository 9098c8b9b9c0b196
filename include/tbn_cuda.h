/* tbn_cuda.h -- C ABI of the B200 (sm_100a) implementation of the fast-arm-tbcnn hot path.
 *
 * The reference (Babushkin05/fast-arm-tbcnn) has no FFI for this path: its boundary is the
 * C++ API in namespace tbn (free operator functions + TBNModel::Session).  This header is the
 * C boundary placed underneath that API: the C++ host layer of this repository (host/include/tbn)
 * and any foreign binding (ctypes, pybind11, cgo ...) call exactly these entry points.
 * Each entry point names the reference function it stands in for (path within the reference
 * project : line).
 *
 * Conventions
 *   - every pointer named d_* (and workspaces) is DEVICE memory on the current CUDA device;
 *     sizes are in elements unless the name says bytes; matrices are row-major;
 *   - GEMM dims follow C[M,N] = A[M,K] * B[K,N];
 *   - `stream` is a cudaStream_t passed as void* (NULL = default stream); all work is
 *     asynchronous on that stream unless stated otherwise;
 *   - the return value is a status: 0 or one of the reference's tbn::ErrorCode values
 *     (tbn/utils/errors.hpp:10-22) or one of the TBN_CUDA_* extensions below;
 *     tbn_cuda_last_error() returns the message of the calling thread's last failure;
 *   - there is no CPU fallback anywhere: without a usable sm_100 device every call fails.
 */
#ifndef TBN_CUDA_H
#define TBN_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes ---------------------------------------------------------------- */
#define TBN_SUCCESS 0
#define TBN_INVALID_ARGUMENT (-1)   /* tbn::ErrorCode::INVALID_ARGUMENT   */
#define TBN_OUT_OF_MEMORY (-2)      /* tbn::ErrorCode::OUT_OF_MEMORY      */
#define TBN_NOT_IMPLEMENTED (-3)    /* tbn::ErrorCode::NOT_IMPLEMENTED    */
#define TBN_RUNTIME_ERROR (-5)      /* tbn::ErrorCode::RUNTIME_ERROR      */
#define TBN_INVALID_SHAPE (-7)      /* tbn::ErrorCode::INVALID_SHAPE      */
#define TBN_DEVICE_NOT_SUPPORTED (-8) /* tbn::ErrorCode::DEVICE_NOT_SUPPORTED */
#define TBN_CUDA_ERROR (-100)       /* a CUDA runtime/driver call failed  */
#define TBN_CUDA_TIMEOUT (-101)     /* a bounded device-side wait expired */

/* ---- numeric modes of the float x {binary,ternary} GEMM ---------------------------- */
/* Weights +-1/0 are exact in bf16; the fp32 activations are split into NPASS bf16 terms
 * (hi [+ mid] [+ lo]) that are multiplied on the tcgen05 tensor cores into one fp32
 * accumulator.  Relative L2 error against the fp32 reference: X3 ~1e-7 (exact split),
 * X2 ~2e-6 (default; inside the 1e-5 bar), X1 ~2e-3 (outside every bar, see TBN_MODE_TC_FP16X1). */
#define TBN_MODE_AUTO 0
#define TBN_MODE_TC_BF16X1 1
#define TBN_MODE_TC_BF16X2 2
#define TBN_MODE_TC_BF16X3 3
#define TBN_MODE_SIMT 4 /* CUDA-core add/subtract-by-sign, fp32, k ascending: bit-equal to
                           qlinear_matmul_binary_naive */
/* The DECLARED lower-precision variant: one tensor-core pass over fp16 activations (11 significant bits,
 * relative L2 error ~2e-4, inside the 1e-3 bar such a variant is allowed) against +-1/0 weights, which are exact
 * in fp16, with fp32 accumulation.  A pre-pass finds max |a| of the call and scales the activations by the power
 * of two that puts it into [2^14, 2^15) -- so no input overflows fp16 and values down to 2^-28 of the largest keep
 * full precision -- and the epilogue multiplies the exact inverse back in.  About twice the throughput of
 * TBN_MODE_TC_BF16X2; never chosen by TBN_MODE_AUTO.  TBN_MODE_TC_BF16X1 (8 significant bits, ~2e-3) is outside
 * every accuracy bar of the float x binary product: it exists for the integer-exact TBN mode, whose ternarised
 * activations bf16 represents exactly, and is kept selectable only for comparison. */
#define TBN_MODE_TC_FP16X1 5

/* ---- epilogue flags -------------------------------------------------------------- */
#define TBN_EPI_RELU 1u
/* (acc*scale + bias[n]) * alpha[n]: the order of Session::execute_conv's cached path
 * (tbn/runtime/model.hpp:523-557).  Default order is acc*alpha[n]*scale + bias[n]. */
#define TBN_EPI_BIAS_BEFORE_ALPHA 2u

/* Convolution only: add a residual tensor (same shape and layout as the output) before the ReLU --
 * the Add + Relu that follows the second convolution of a residual block
 * (Session::execute_add / execute_relu, tbn/runtime/model.hpp:905-1037, 1127-1174). */
#define TBN_EPI_ADD_RESIDUAL 4u

/* ---- weight layouts accepted by the packers ---------------------------------------- */
#define TBN_LAYOUT_KN 0 /* W[K,N] row-major (Gemm B, transB = 0)                          */
#define TBN_LAYOUT_NK 1 /* W[N,K] row-major (conv weights [M_out, C*kh*kw]; Gemm transB=1) */

/* ---- runtime --------------------------------------------------------------------- */

/* Selects `device`, verifies compute capability 10.x and sets up per-device state.
 * Must be called once per device (per process) before any other entry point. */
int32_t tbn_cuda_init(int32_t device);
/* Copies the calling thread's last error message into buf (NUL terminated). Returns its length. */
int32_t tbn_cuda_last_error(char* buf, size_t buf_bytes);
/* Replaces tbn::Tensor's host allocation (tbn/runtime/tensor.hpp:23-28): device buffer, zero-filled. */
int32_t tbn_cuda_malloc(void** d_ptr, size_t bytes);
int32_t tbn_cuda_free(void* d_ptr);
int32_t tbn_cuda_memset(void* d_ptr, int32_t value, size_t bytes, void* stream);
int32_t tbn_cuda_h2d(void* d_dst, const void* h_src, size_t bytes, void* stream);
int32_t tbn_cuda_d2h(void* h_dst, const void* d_src, size_t bytes, void* stream);
int32_t tbn_cuda_d2d(void* d_dst, const void* d_src, size_t bytes, void* stream);
/* Waits for `stream` and reports any device-side error recorded by the kernels
 * (TBN_CUDA_TIMEOUT when a bounded wait expired). */
int32_t tbn_cuda_sync(void* stream);
/* Every wait inside the kernels (on a shared-memory barrier that a TMA copy, an MMA or another warp completes) is
 * bounded: when it has lasted longer than the limit the kernel records a code, every other waiter of the device
 * gives up as well, the kernel frees its tensor memory and returns, and the next tbn_cuda_sync reports
 * TBN_CUDA_TIMEOUT; the context stays usable.  Default 2 s per device; settable between 1 us and 60 s (takes
 * effect for waits that start polling after the call). */
int32_t tbn_cuda_set_wait_limit_ns(uint64_t limit_ns);
/* Launches a one-warp kernel whose only thread waits on a barrier that nothing completes: the wait runs out after
 * the limit above and the following tbn_cuda_sync returns TBN_CUDA_TIMEOUT.  Lets a host check, at start-up and
 * without any fault, that a stuck kernel would be reported instead of hanging the stream.  (No counterpart in the
 * reference.) */
int32_t tbn_cuda_selftest_wait_timeout(void* stream);
/* Number of kernels this library has launched so far in this process. */
int64_t tbn_cuda_launch_count(void);
/* Per-kernel device timing for benchmarks: while enabled, the GEMM entry points bracket their
 * two kernels (activation split, tensor-core GEMM) with CUDA events on the launching stream.
 * tbn_cuda_profile_read waits for the recorded events, returns the accumulated milliseconds and
 * launch counts since the last read, and clears them.  Off by default (no events recorded). */
int32_t tbn_cuda_profile_enable(int32_t enable);
int32_t tbn_cuda_profile_read(double* gemm_ms, int64_t* gemm_launches, double* split_ms,
                              int64_t* split_launches);

/* Tuning switch without a reference counterpart.  A two-term tbn_gemm_fxb / _multi / _host call whose A is
 * 16-byte aligned with lda % 4 == 0 and K % 4 == 0 can let the GEMM kernel read the fp32 rows itself and split
 * them in registers instead of running the activation-split kernel first.  The split is then repeated for every
 * 256-column tile of the weights, so it only pays when there is one such tile (measured at 16384^3, 64 tiles:
 * 23.2 ms fused against 11.4 + 0.35 ms separate).  value 1 (default): fuse when N <= 256; 0: never; 2: always.
 * All three give bit-identical results.  Process-wide; not meant to be flipped while calls are in flight. */
int32_t tbn_cuda_set_fused_split(int32_t value);

/* Per-shape kernel choice of TBN_MODE_AUTO.  Stands in for TilingParams / auto_tune_gemm of the reference
 * (GeMM/05-final/GeMM.hpp:16-43, tbn-runtime/src/operators/gemm.cpp:524-536): instead of tile sizes handed in by
 * the caller, a table measured on the GPU and compiled into the library maps the class of (M, N, K) to
 *   kernel       0 = tcgen05 tensor-core kernel, 1 = CUDA-core add/subtract-by-sign kernel, 2 = tcgen05 on CTA pairs
 *                (cta_group::2: one 256 x 256 tile per pair of SMs, each unpacking half of the weight tile)
 *   bn           column tile of the tensor-core kernel (64 / 128 / 256)
 *   group_m      rasterisation group: m-tiles that share one sweep over the column tiles (L2 reuse)
 *   fused_split  1 = the kernel splits the fp32 activation rows itself instead of a separate pass
 * tbn_gemm_plan reports the choice for a shape (a host may store it beside its packed weights; any out pointer
 * may be NULL).  tbn_gemm_plan_override forces fields for every following call of the process (-1 = as the table
 * says); it is what the tuner (python -m fast_arm_tbcnn_b200.tune) uses to measure the variants. */
int32_t tbn_gemm_plan(int64_t M, int64_t N, int64_t K, int32_t* kernel, int32_t* bn, int32_t* group_m,
                      int32_t* fused_split);
int32_t tbn_gemm_plan_override(int32_t kernel, int32_t bn, int32_t group_m, int32_t fused_split);
/* The column tile the library derives for an (M, N) from a class's tile `preferred`: a class is measured at one
 * representative shape, and a shape whose tile count fills the SMs differently takes the tile a wave model
 * prefers (returns 64, 128 or 256). */
int32_t tbn_gemm_plan_bn(int64_t M, int64_t N, int32_t preferred);

/* Padded dims of the packed layouts: K_pad = ceil128(K), N_pad = ceil8(N)
 * (PaddedDimensions, tbn-runtime/src/operators/quantized_gemm_neon.cpp:38-58). */
int32_t tbn_packed_dims(int64_t K, int64_t N, int64_t* K_pad, int64_t* N_pad);

/* ---- quantise ---------------------------------------------------------------------- */

/* tbn::quantize_to_binary (quantized_gemm_neon.cpp:544-565): out[i] = w[i] > thr ? 1 : 0. */
int32_t tbn_quantize_to_binary(const float* d_w, int64_t n, float thr, uint8_t* d_out, void* stream);
/* tbn::quantize_to_ternary (quantized_gemm_neon.cpp:570-597): -1 / 0 / +1 as int8. */
int32_t tbn_quantize_to_ternary(const float* d_w, int64_t n, float lo, float hi, int8_t* d_out,
                                void* stream);

/* Per-output-channel scale alpha[c] = mean |w[c, :]| of weights [channels, per], summed sequentially in
 * fp32 in memory order: bit-equal to Session::execute_conv (tbn/runtime/model.hpp:388-394).  One thread
 * per channel -- meant for the one-time weight preparation of the bit-exact TBN mode; the packers'
 * d_alpha output is the fast, chunk-summed equivalent. */
int32_t tbn_channel_abs_mean(const float* d_w, int64_t channels, int64_t per, float* d_alpha, void* stream);

/* Bytes of scratch tbn_quant_pack_* needs when d_alpha != NULL (0 otherwise). */
size_t tbn_quant_pack_workspace_bytes(int64_t K, int64_t N, int32_t ternary);

/* Sign-threshold-and-pack in one pass.  Replaces quantize_to_binary + pad(+1) +
 * BinaryMatrix::pack (quantized_gemm_neon.cpp:544-565,199-214; GeMM/05-final/GeMM.cpp:114-151;
 * Session caches tbn/runtime/model.hpp:464-477,819-830).
 *   d_w     fp32 weights; layout KN: element (k,n) at d_w[k*ldw+n]; layout NK: d_w[n*ldw+k]
 *   ge      0: +1 iff w > thr (quantize_to_binary); 1: +1 iff w >= thr (Session caches)
 *   d_words out, uint32 [N_pad][K_pad/32]: word[n*(K_pad/32) + k/32] bit (k%32) set <=> -1;
 *           padding bits are 0 (+1) -- byte-identical to BinaryMatrix::pack's plane.
 *   d_alpha out (nullable), fp32 [N]: mean |w| over k (per-output-channel scale,
 *           model.hpp:388-394; summation is chunked, not bit-equal to the sequential sum). */
int32_t tbn_quant_pack_binary(const float* d_w, int64_t K, int64_t N, int64_t ldw, int32_t layout,
                              float thr, int32_t ge, uint32_t* d_words, float* d_alpha,
                              void* d_workspace, size_t workspace_bytes, void* stream);

/* Same result as tbn_quant_pack_binary, for callers that must not allocate device memory and have
 * no workspace to lend.  (No counterpart in the reference, which only ever uses host memory.)
 * Who needs it: a host that reserves all of its GPU memory when it starts -- an inference server
 * whose tensor arena owns HBM, or a plugin running under another framework's caching allocator --
 * where a cudaMalloc on the request path can fail for lack of free memory and stalls every stream of
 * the device while it runs.  This call takes the scratch for the per-column scale (one partial sum per
 * 128 weight rows and column) from a 4 MiB array built into the library instead.
 *   - limit: ceil(K/128) * N <= 1,048,576 partial sums (e.g. 8192 x 16384); larger shapes are
 *     refused with TBN_INVALID_ARGUMENT and a message naming the limit;
 *   - every GPU that loads the library holds the 4 MiB until the process exits;
 *   - the first call on each device looks up the array's device address (no allocation); make that
 *     first call before any stream capture begins.  The address is kept for the life of the process: after a
 *     cudaDeviceReset the library has to be loaded again.  With CUDA's lazy module loading the first launch of each
 *     kernel variant (small, vectorised, TMA-streamed, [N,K] layout, scale finalisation) also loads its code onto
 *     the device: a host that must see no change in free memory on the request path warms up, during start-up,
 *     one call for every shape class it will use;
 *   - the limit concerns the scale only: with d_alpha == NULL no scratch is used and any size is accepted;
 *   - all calls on a device share the array, so two calls whose kernels may overlap on the GPU
 *     (different streams, different host threads) race on it: issue them on one stream or order
 *     them yourself.  Nothing needs clearing between calls: each call writes every partial sum
 *     before it reads it;
 *   - it calls no cudaMalloc / cudaFree or other allocating routine; inputs, d_words and d_alpha are
 *     the caller's. */
int32_t tbn_quant_pack_binary_noalloc(const float* d_w, int64_t K, int64_t N, int64_t ldw,
                                      int32_t layout, float thr, int32_t ge, uint32_t* d_words,
                                      float* d_alpha, void* stream);

/* Threshold-and-pack for ternary weights.  Replaces quantize_to_ternary
 * (quantized_gemm_neon.cpp:570-597) + the TernaryPackedWeights::set_weight loop
 * (tbn/memory/packed_weights.hpp:53-71) and produces the operand planes of the GEMM.
 *   d_codes out (nullable), uint32 [(K*N+15)/16]: 2-bit code (0=-1, 1=0, 2=+1) of flat element
 *           i = k*N+n at bits 2*(i%16) of word i/16 -- byte-identical to the reference packer.
 *   d_pos/d_neg out, uint32 [N_pad][K_pad/32]: planes in the binary layout above
 *           (bit set in pos <=> +1, in neg <=> -1; padding 0 = weight 0).
 *   d_alpha out (nullable), fp32 [N]: mean |w| over the non-zero entries of the column. */
int32_t tbn_quant_pack_ternary(const float* d_w, int64_t K, int64_t N, int64_t ldw, int32_t layout,
                               float lo, float hi, uint32_t* d_codes, uint32_t* d_pos, uint32_t* d_neg,
                               float* d_alpha, void* d_workspace, size_t workspace_bytes, void* stream);

/* ---- GEMM ---------------------------------------------------------------------------- */

/* Bytes of scratch tbn_gemm_fxb / tbn_gemm_tbn need for the split activations. */
size_t tbn_gemm_workspace_bytes(int64_t M, int64_t K, int32_t mode);

/* Float x binary / float x ternary GEMM:
 *     C[m,n] = (sum_k A[m,k] * w[k,n]) * alpha[n] * scale + bias[n]      (then optional ReLU)
 * with w[k,n] = -1 where the neg plane has its bit set, else +1 (binary: d_pos == NULL) or
 * +1/-1/0 from the pos/neg planes (ternary).  This is the product the reference defines in
 * qlinear_matmul_binary_naive (quantized_gemm_neon.cpp:63-90) and evaluates through
 * tbn::gemm on alpha*sign(W) (gemm.cpp:349-360); it replaces the CPU GEMM engine
 * (GeMM/05-final/GeMM.cpp:303-363) on this path.
 *   d_a [M,K] fp32, row stride lda;  d_c [M,N] fp32, row stride ldc
 *   d_alpha, d_bias: nullable fp32 [N];  mode: TBN_MODE_*;  epilogue: TBN_EPI_* flags */
int32_t tbn_gemm_fxb(const float* d_a, int64_t M, int64_t K, int64_t lda, const uint32_t* d_neg,
                     const uint32_t* d_pos, int64_t N, const float* d_alpha, float scale,
                     const float* d_bias, float* d_c, int64_t ldc, int32_t mode, uint32_t epilogue,
                     void* d_workspace, size_t workspace_bytes, void* stream);

/* tbn_gemm_fxb whose epilogue writes the finished C tile to SEVERAL destinations with the same row
 * stride: d_c_list[0..num_out) is a HOST array of device pointers (1..8), e.g. this GPU's result buffer
 * and the peers' buffers mapped into this GPU's address space, each already offset to the column slab
 * this call produces.  This is the compute + all-gather step of the column-sharded multi-GPU GEMM done
 * in one kernel: every 32 x 32 block of the tile is staged in shared memory and leaves as one tiled TMA store
 * per destination (ordinary stores into local or peer memory; nothing is broadcast by the hardware), rows and
 * columns past the matrix being clipped.  The caller synchronises the GPUs before anyone reads the result.
 * Tensor-core modes only; N and ldc multiples of 4.  (New: the reference is single-device.) */
int32_t tbn_gemm_fxb_multi(const float* d_a, int64_t M, int64_t K, int64_t lda, const uint32_t* d_neg,
                           const uint32_t* d_pos, int64_t N, const float* d_alpha, float scale,
                           const float* d_bias, float* const* d_c_list, int32_t num_out, int64_t ldc,
                           int32_t mode, uint32_t epilogue, void* d_workspace, size_t workspace_bytes,
                           void* stream);

/* tbn_gemm_fxb for callers whose activations and result live in HOST memory, as with the reference's
 * operators (tbn::qlinear_matmul_binary takes and returns host tensors,
 * tbn-runtime/include/tbn/operators/quantized_gemm.hpp:48-57).  h_a [M,K] and h_c [M,N] are host pointers
 * (page-locked memory gives full PCIe speed; pageable memory works, slower); the packed weights, alpha and
 * bias stay on the device.  Rows are processed in chunks so that upload, multiply and download overlap on
 * three internal streams.  All of it is ordered after the work already queued on `stream`, and `stream`
 * waits for the last download: synchronise `stream` before reading h_c.  The internal streams and events are
 * one set per device: calls on the same device -- from several host threads or on several caller streams --
 * are safe (each call enqueues under a per-device lock) but run one after the other on the GPU, each call's
 * uploads waiting for the previous call's work on those streams. */
size_t tbn_gemm_fxb_host_workspace_bytes(int64_t M, int64_t K, int64_t N, int32_t mode);
int32_t tbn_gemm_fxb_host(const float* h_a, int64_t M, int64_t K, int64_t lda, const uint32_t* d_neg,
                          const uint32_t* d_pos, int64_t N, const float* d_alpha, float scale,
                          const float* d_bias, float* h_c, int64_t ldc, int32_t mode, uint32_t epilogue,
                          void* d_workspace, size_t workspace_bytes, void* stream);

/* "TBN mode": activations ternarised at (lo, hi) x binary weights, exact integer accumulation,
 * C = float(acc) * scale (then alpha/bias per the epilogue flags).  Bit-equal to
 * tbn::qlinear_matmul_binary (quantized_gemm_neon.cpp:165-243, 380-430) and to the GEMM inside
 * Session::execute_conv/execute_gemm with quantisation on (model.hpp:482-503, 835-837). */
int32_t tbn_gemm_tbn(const float* d_a, int64_t M, int64_t K, int64_t lda, float lo, float hi,
                     const uint32_t* d_neg, int64_t N, const float* d_alpha, float scale,
                     const float* d_bias, float* d_c, int64_t ldc, uint32_t epilogue,
                     void* d_workspace, size_t workspace_bytes, void* stream);

/* ---- float weights (the float layers of the CNN graphs) --------------------------------- */

/* Dense fp32 weights are split once into two bf16 terms, stored K-major per output column:
 * [2][ceil8(N)][ceil128(K)] bf16.  Layouts as for the packers (KN: Gemm B [K,N]; NK: filters [M_out, C*kh*kw]). */
size_t tbn_dense_pack_bytes(int64_t K, int64_t N);
int32_t tbn_dense_pack(const float* d_w, int64_t K, int64_t N, int64_t ldw, int32_t layout, void* d_packed,
                       void* stream);
/* Float x float GEMM  C = alpha * A W + bias  in fp32 accuracy (two bf16 terms on both sides:
 * hi*hi + hi*lo + lo*hi on the tensor cores).  Stands in for tbn::gemm (tbn-runtime/src/operators/gemm.cpp:35-129,
 * 349-360) with transA = transB = 0 and a 1-D C; workspace as tbn_gemm_workspace_bytes(M, K, TBN_MODE_TC_BF16X2). */
int32_t tbn_gemm_f32(const float* d_a, int64_t M, int64_t K, int64_t lda, const void* d_packed_w, int64_t N,
                     float alpha, const float* d_bias, float* d_c, int64_t ldc, uint32_t epilogue,
                     void* d_workspace, size_t workspace_bytes, void* stream);

/* ---- convolution (implicit GEMM) ----------------------------------------------------- */

/* Order of K inside the packed / split conv weights handed to the convolution entry points:
 *   REFERENCE  k = (c*kh + i)*kw + j, the reference's im2col order (filters [M_out, C, kh, kw] packed as they
 *              are with TBN_LAYOUT_NK).  Works for every geometry; the activation operand is gathered
 *              element by element from the NCHW input.
 *   TAP_MAJOR  k = (i*kw + j)*C + c (filters first reordered with tbn_permute_filters).  Needs C % 64 == 0.
 *              A pre-pass writes a channels-last bf16 copy of the input (same size as the input, not an
 *              im2col matrix) and the kernel copies whole 64-channel runs with 16-byte asynchronous copies:
 *              several times faster. */
#define TBN_CONV_WEIGHTS_REFERENCE 0
#define TBN_CONV_WEIGHTS_TAP_MAJOR 1

/* [M, C, taps] fp32 -> [M, taps, C] fp32 (taps = kh*kw). */
int32_t tbn_permute_filters(const float* d_w, int64_t M, int64_t C, int64_t taps, float* d_out, void* stream);

/* Bytes of scratch the convolution entry points need (tap table or channels-last copy, partial-sum tiles,
 * and the bf16 expansion of the packed filters: ceil128(C*kh*kw) * ceil8(M_out) * 2 bytes). */
size_t tbn_conv2d_workspace_bytes(int64_t N, int64_t C, int64_t H, int64_t W, int64_t M_out, int64_t kh, int64_t kw,
                                  int32_t weight_order);

/* Float x binary / float x ternary Conv2D, NCHW fp32 in and out:
 *     y[n,m,oh,ow] = (sum_{c,i,j} x[n,c,oh*sh-ph+i*dh, ow*sw-pw+j*dw] * w[m,c,i,j]) * alpha[m] * scale
 *                    + bias[m] (+ residual[n,m,oh,ow]) (then optional ReLU)
 * with w = +-1 (0) from the packed planes of the weights [M_out, C*kh*kw] (TBN_LAYOUT_NK); taps
 * outside the image contribute zero; output size (in + 2p - d(k-1) - 1)/s + 1.  Equals tbn::conv2d
 * (tbn-runtime/src/operators/conv2d.cpp:78-192) on the dequantised weights alpha*sign(w); replaces
 * im2col + transpose + GEMM + reorder + bias of tbn::conv2d_binary / conv2d_binary_with_scales
 * (conv2d.cpp:220-369, 420-507).  The im2col matrix is not materialised.
 *   mode: TBN_MODE_AUTO (two bf16 terms), TBN_MODE_TC_BF16X2 or TBN_MODE_TC_BF16X1.
 *   d_residual: nullable; read when TBN_EPI_ADD_RESIDUAL is set (same shape as y). */
int32_t tbn_conv2d_fxb(const float* d_x, int64_t N, int64_t C, int64_t H, int64_t W, const uint32_t* d_neg,
                       const uint32_t* d_pos, int64_t M_out, int64_t kh, int64_t kw, int32_t sh, int32_t sw,
                       int32_t ph, int32_t pw, int32_t dh, int32_t dw, const float* d_alpha, float scale,
                       const float* d_bias, const float* d_residual, float* d_y, int32_t mode,
                       uint32_t epilogue, int32_t weight_order, void* d_workspace, size_t workspace_bytes,
                       void* stream);

/* Chained forms of tbn_conv2d_fxb / tbn_conv2d_f32 for layer sequences (no reference counterpart: the reference
 * keeps every activation as NCHW fp32).  d_x_cl, when not null, is the input already in the channels-last form
 * bf16 [2 terms][N][H][W][C] (hi = rn(x), lo = rn(x - hi)) that the patch-mode kernel reads: the pre-pass is skipped
 * and d_x may be null (needs C % 64 == 0 and tap-major filters).  d_y_cl, when not null, receives the output in that
 * same form [2][N][OH][OW][M_out] from the epilogue, in addition to d_y or — with d_y null — instead of it.  Feeding
 * d_y_cl of one call as d_x_cl of the next gives bit-identical results to passing the fp32 tensors. */
int32_t tbn_conv2d_fxb_chain(const float* d_x, const void* d_x_cl, int64_t N, int64_t C, int64_t H, int64_t W,
                             const uint32_t* d_neg, const uint32_t* d_pos, int64_t M_out, int64_t kh, int64_t kw,
                             int32_t sh, int32_t sw, int32_t ph, int32_t pw, int32_t dh, int32_t dw,
                             const float* d_alpha, float scale, const float* d_bias, const float* d_residual,
                             float* d_y, void* d_y_cl, int32_t mode, uint32_t epilogue, int32_t weight_order,
                             void* d_workspace, size_t workspace_bytes, void* stream);
int32_t tbn_conv2d_f32_chain(const float* d_x, const void* d_x_cl, int64_t N, int64_t C, int64_t H, int64_t W,
                             const void* d_packed_w, int64_t M_out, int64_t kh, int64_t kw, int32_t sh, int32_t sw,
                             int32_t ph, int32_t pw, int32_t dh, int32_t dw, const float* d_bias,
                             const float* d_residual, float* d_y, void* d_y_cl, uint32_t epilogue,
                             int32_t weight_order, void* d_workspace, size_t workspace_bytes, void* stream);

/* "TBN mode" Conv2D: activations ternarised at (lo, hi) while they are gathered, exact integer
 * accumulation.  With alpha, bias and TBN_EPI_BIAS_BEFORE_ALPHA it is bit-equal to the cached fast
 * path of Session::execute_conv (tbn/runtime/model.hpp:375-559: im2col_ternary_packed,
 * conv2d.cpp:511-601, + GemmEngine::compute + reorder + bias + per-channel scale). */
int32_t tbn_conv2d_tbn(const float* d_x, int64_t N, int64_t C, int64_t H, int64_t W, float lo, float hi,
                       const uint32_t* d_neg, int64_t M_out, int64_t kh, int64_t kw, int32_t sh, int32_t sw,
                       int32_t ph, int32_t pw, int32_t dh, int32_t dw, const float* d_alpha, float scale,
                       const float* d_bias, float* d_y, uint32_t epilogue, int32_t weight_order,
                       void* d_workspace, size_t workspace_bytes, void* stream);

/* Float-filter Conv2D (stem and 1x1 shortcut convolutions): stands in for tbn::conv2d
 * (tbn-runtime/src/operators/conv2d.cpp:78-192); filters from tbn_dense_pack (TBN_LAYOUT_NK). */
int32_t tbn_conv2d_f32(const float* d_x, int64_t N, int64_t C, int64_t H, int64_t W, const void* d_packed_w,
                       int64_t M_out, int64_t kh, int64_t kw, int32_t sh, int32_t sw, int32_t ph, int32_t pw,
                       int32_t dh, int32_t dw, const float* d_bias, const float* d_residual, float* d_y,
                       uint32_t epilogue, int32_t weight_order, void* d_workspace, size_t workspace_bytes,
                       void* stream);

/* ---- whole-network kernel ------------------------------------------------------------------------------- */

/* The LeNet-shaped binary CNN in ONE launch, float x binary mode: x [batch, 1, 28, 28] -> Conv 1 -> c1 5x5 + bias,
 * ReLU, MaxPool 2x2, Conv c1 -> c2 5x5 + bias, ReLU, MaxPool 2x2, Flatten, Gemm c2*16 -> classes + bias, every layer
 * y = (sum +-x) * alpha + bias.  Stands in for the node-by-node execution of that graph by the reference Session
 * (tbn/runtime/model.hpp:190-228 with execute_conv / execute_relu / execute_maxpool / execute_gemm); one image and all
 * its intermediates stay in shared memory, only the image is read and the logits written.
 *   d_w1 / d_w2: packed filters from tbn_quant_pack_binary(TBN_LAYOUT_NK) of [c1, 25] and [c2, c1*25] (reference tap
 *   order); d_wf: packed Gemm weights from tbn_quant_pack_binary(TBN_LAYOUT_KN) of [c2*16, classes];
 *   alphas / biases: nullable fp32 per output channel.  Built for c1 = 6, c2 = 16 (TBN_NOT_IMPLEMENTED otherwise),
 *   1 <= classes <= 64. */
int32_t tbn_lenet_fused_fxb(const float* d_x, int64_t batch, int32_t c1, int32_t c2, int32_t classes, const uint32_t* d_w1,
                            const float* d_alpha1, const float* d_bias1, const uint32_t* d_w2, const float* d_alpha2,
                            const float* d_bias2, const uint32_t* d_wf, const float* d_alphaf, const float* d_biasf, float* d_y,
                            void* stream);

/* ---- glue operators of the CNN graphs (device resident, fp32) --------------------------- */

/* y = max(0, x)   (Session::execute_relu, model.hpp:1166-1169) */
int32_t tbn_relu(const float* d_x, int64_t n, float* d_y, void* stream);
/* y[i] = a[i] + b[(i / inner) % b_n] (+ ReLU): same-shape add (b_n == a_n), per-channel [C] over
 * [N,C,H,W] (inner = H*W) and row broadcast [N] over [M,N] (inner = 1)
 * (Session::execute_add, model.hpp:921-1036). */
int32_t tbn_add(const float* d_a, int64_t a_n, const float* d_b, int64_t b_n, int64_t inner, int32_t relu,
                float* d_y, void* stream);
/* kind 0: tbn::maxpool2d, kind 1: tbn::avgpool2d (tbn-runtime/src/operators/pooling.cpp:10-148). */
int32_t tbn_pool2d(int32_t kind, const float* d_x, int64_t N, int64_t C, int64_t H, int64_t W, int32_t kh,
                   int32_t kw, int32_t sh, int32_t sw, int32_t ph, int32_t pw, int32_t ceil_mode,
                   int32_t count_include_pad, float* d_y, void* stream);
/* tbn::global_avgpool2d (pooling.cpp:184-216): [N,C,H,W] -> [N,C,1,1]. */
int32_t tbn_global_avgpool2d(const float* d_x, int64_t N, int64_t C, int64_t H, int64_t W, float* d_y,
                             void* stream);

/* tbn::global_maxpool2d (pooling.cpp:150-181): [N,C,H,W] -> [N,C,1,1]; a NaN never replaces the maximum. */
int32_t tbn_global_maxpool2d(const float* d_x, int64_t N, int64_t C, int64_t H, int64_t W, float* d_y,
                             void* stream);
/* Session::execute_greater / execute_less / execute_sub (model.hpp:1176-1316): y[i] = x[i] > rhs[i % rhs_n] ? 1 : 0,
 * y[i] = x[i] < rhs[...] ? 1 : 0, y[i] = x[i] - rhs[...]; float 0/1 results as in the reference, which treats
 * the following Cast as a pass-through. */
#define TBN_ELT_GREATER 0
#define TBN_ELT_LESS 1
#define TBN_ELT_SUB 2
int32_t tbn_binary_elementwise(int32_t op, const float* d_x, int64_t n, const float* d_rhs, int64_t rhs_n,
                               float* d_y, void* stream);
/* y[cols][rows] = x[rows][cols]^T: the transA / transB forms of tbn::gemm (gemm.cpp:349-360) are materialised
 * on the device (weights once per tensor, activations per call). */
int32_t tbn_transpose2d(const float* d_x, int64_t rows, int64_t cols, float* d_y, void* stream);

/* ---- multi-GPU helper -------------------------------------------------------------- */

/* Column-sharded GEMM across G GPUs: rank g computes C[:, g*Nc:(g+1)*Nc] as a contiguous
 * [M, Nc] slab; after one all-gather the slabs sit as d_slabs[G][M][Nc].  This kernel
 * interleaves them into the row-major d_c[M][G*Nc] (row stride ldc).  (New: the reference is
 * single-device and has no counterpart.) */
int32_t tbn_gather_cols_permute(const float* d_slabs, int64_t G, int64_t M, int64_t Nc, float* d_c,
                                int64_t ldc, void* stream);

/* Sharing a result matrix between the processes of one box (one process per GPU), for tbn_gemm_fxb_multi: the owner
 * exports a 64-byte handle of a buffer obtained from tbn_cuda_malloc and sends it to the other ranks by any host
 * channel; they open it and receive a pointer, valid in their own process, through which their GPU writes the
 * owner's memory over NVLink (peer access is enabled on first use).  Close every opened pointer before the owner
 * frees the buffer.  (New: the reference is single-device.) */
#define TBN_IPC_HANDLE_BYTES 64
int32_t tbn_ipc_export(void* d_ptr, void* handle64);
int32_t tbn_ipc_open(const void* handle64, void** d_ptr);
int32_t tbn_ipc_close(void* d_ptr);

#ifdef __cplusplus
}
#endif
#endif /* TBN_CUDA_H */
