// Float x {binary, ternary} GEMM for sm_100a.
//
//   C[m,n] = (sum_k A[m,k] * w[k,n]) * alpha[n] * scale + bias[n]
//
// with w in {-1,+1} (binary; one packed plane, bit set <=> -1) or {-1,0,+1} (ternary; two
// planes).  Stands in for the reference's CPU GEMM engine on this path
// (GeMM/05-final/GeMM.cpp:159-363 driven by tbn-runtime/src/operators/quantized_gemm_neon.cpp:165-350)
// and computes the product the reference defines in qlinear_matmul_binary_naive
// (quantized_gemm_neon.cpp:63-90).
//
// Three kernels:
//   split_activations_kernel  fp32 A -> NPASS bf16 terms (hi [, mid] [, lo]) whose sum is A
//                             (exactly for 3 terms), zero padded to [ceil128(M), ceil128(K)];
//                             or -- "TBN mode" -- A ternarised at (lo, hi) to exact -1/0/+1.
//   gemm_tc_kernel            persistent, warp-specialised tcgen05 kernel:
//                               warp 0      TMA producer: activation tiles (128 x 64 bf16, SWIZZLE_128B)
//                               warp 1      MMA issuer: tcgen05.mma kind::f16 into a double-buffered
//                                           fp32 accumulator in tensor memory
//                               warp 0 also streams the packed weight words (16 bytes = 128 k per column)
//                                           into a small shared-memory ring with TMA
//                               warps 2-9   weight transform: packed words smem -> registers -> +-1/0 bf16
//                                           written straight into the swizzled K-major operand tile
//                               warps 10-13 epilogue: tcgen05.ld, alpha/scale/bias/ReLU, store
//                             The weight tile is unpacked once per k-block and reused by all passes.
//                             The tensor cores add into the fp32 accumulator with truncation, an error
//                             that grows linearly with the number of accumulation steps; long K is
//                             therefore cut into segments that each start a fresh accumulator, and the
//                             epilogue adds the segments in fp32 (round to nearest) through a per-CTA
//                             scratch tile that stays resident in L2.
//   gemm_simt_kernel          CUDA-core add/subtract-by-sign, fp32, k ascending (bit-equal to the
//                             naive reference loop); used for tiny problems and as a cross-check.
#include <atomic>
#include "gemm_pair.cuh"
#include "gemm_tc.cuh"
#include "plan.cuh"

namespace tbn_cuda {
namespace {

// =====================================================================================
// Activation split
// =====================================================================================

// One thread converts 8 consecutive k of one row and writes one 16-byte vector per pass.
// F16: one fp16 term of a * 2^e instead of bf16 terms, e from *amax_bits (see f16_scale_exponent).
template <int NPASS, bool TERNARISE, bool F16 = false>
__global__ void __launch_bounds__(256) split_activations_kernel(const float* __restrict__ a, int64_t M, int64_t K,
                                                                int64_t lda, int64_t M_pad, int64_t K_pad,
                                                                __nv_bfloat16* __restrict__ out, float lo, float hi,
                                                                int vec_ok, const uint32_t* __restrict__ amax_bits = nullptr) {
    static_assert(!F16 || (NPASS == 1 && !TERNARISE), "the fp16 mode has one term");
    const float mul = F16 ? f16_scale_mul(__ldg(amax_bits)) : 1.0f;
    const int64_t k8_per_row = K_pad / 8;
    const int64_t total = M_pad * k8_per_row;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total; idx += stride) {
        const int64_t m = idx / k8_per_row;
        const int64_t k = (idx - m * k8_per_row) * 8;
        float v[8];
        if (m < M && vec_ok && k + 8 <= K) {
            const float4 x0 = __ldg(reinterpret_cast<const float4*>(a + m * lda + k));
            const float4 x1 = __ldg(reinterpret_cast<const float4*>(a + m * lda + k + 4));
            v[0] = x0.x; v[1] = x0.y; v[2] = x0.z; v[3] = x0.w;
            v[4] = x1.x; v[5] = x1.y; v[6] = x1.z; v[7] = x1.w;
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = (m < M && k + i < K) ? __ldg(a + m * lda + k + i) : 0.0f;
        }
        uint32_t packed[NPASS][4];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            uint16_t term[NPASS];
            if (F16) term[0] = __half_as_ushort(__float2half_rn(__fmul_rn(v[i], mul)));
            else split_terms<NPASS, TERNARISE>(v[i], lo, hi, term);
#pragma unroll
            for (int p = 0; p < NPASS; ++p) {
                if (i & 1) packed[p][i >> 1] |= static_cast<uint32_t>(term[p]) << 16;
                else packed[p][i >> 1] = term[p];
            }
        }
#pragma unroll
        for (int p = 0; p < NPASS; ++p) {
            uint4* dst = reinterpret_cast<uint4*>(out + (static_cast<int64_t>(p) * M_pad + m) * K_pad + k);
            *dst = make_uint4(packed[p][0], packed[p][1], packed[p][2], packed[p][3]);
        }
    }
}

// Dense weights stored [K, N] (Gemm B, transB = 0): two bf16 terms of W^T, i.e. out[q][n][k], so that the
// kernel finds K-major rows per output column.  Lanes run along n (coalesced reads); one thread handles
// 8 consecutive k of one column and writes one 16-byte vector per term.  One-time weight preparation.
__global__ void __launch_bounds__(256) split_dense_kn_kernel(const float* __restrict__ w, int64_t K, int64_t N, int64_t ldw,
                                                             int64_t N_pad, int64_t K_pad, __nv_bfloat16* __restrict__ out) {
    const int64_t k8_total = K_pad / 8;
    const int64_t total = N_pad * k8_total;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total; idx += stride) {
        const int64_t n = idx % N_pad;
        const int64_t k = (idx / N_pad) * 8;
        uint32_t packed[2][4];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float v = (n < N && k + i < K) ? __ldg(w + (k + i) * ldw + n) : 0.0f;
            uint16_t term[2];
            split_terms<2, false>(v, 0.f, 0.f, term);
#pragma unroll
            for (int q = 0; q < 2; ++q) {
                if (i & 1) packed[q][i >> 1] |= static_cast<uint32_t>(term[q]) << 16;
                else packed[q][i >> 1] = term[q];
            }
        }
#pragma unroll
        for (int q = 0; q < 2; ++q)
            *reinterpret_cast<uint4*>(out + (static_cast<int64_t>(q) * N_pad + n) * K_pad + k) =
                make_uint4(packed[q][0], packed[q][1], packed[q][2], packed[q][3]);
    }
}

// =====================================================================================
// CUDA-core kernel: add / subtract by sign, k ascending
// =====================================================================================

constexpr int kSimtBM = 32, kSimtBN = 64;

template <bool TERNARY>
__global__ void __launch_bounds__(256) gemm_simt_kernel(const float* __restrict__ a, int M, int K, int64_t lda,
                                                        const uint32_t* __restrict__ neg,
                                                        const uint32_t* __restrict__ pos, int64_t KW, int64_t N_pad,
                                                        int N, Epilogue ep, float* __restrict__ c, int64_t ldc,
                                                        int ternarise_act, float act_lo, float act_hi) {
    __shared__ float As[kSimtBM][32];
    __shared__ uint32_t Bn[kSimtBN], Bp[kSimtBN];
    const int tx = threadIdx.x & 63, ty = threadIdx.x >> 6;
    const int m0 = blockIdx.y * kSimtBM, n0 = blockIdx.x * kSimtBN;
    float acc[8];
#pragma unroll
    for (int r = 0; r < 8; ++r) acc[r] = 0.0f;
    const int k_words = (K + 31) / 32;
    for (int kw = 0; kw < k_words; ++kw) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int idx = threadIdx.x + i * 256;
            const int r = idx >> 5, kk = idx & 31;
            const int m = m0 + r, k = kw * 32 + kk;
            float v = (m < M && k < K) ? a[static_cast<int64_t>(m) * lda + k] : 0.0f;
            if (ternarise_act) v = v < act_lo ? -1.0f : (v > act_hi ? 1.0f : 0.0f);
            As[r][kk] = v;
        }
        if (threadIdx.x < kSimtBN) {
            const int64_t n = n0 + threadIdx.x;
            Bn[threadIdx.x] = n < N_pad ? neg[n * KW + kw] : 0u;
            if (TERNARY) Bp[threadIdx.x] = n < N_pad ? pos[n * KW + kw] : 0u;
        }
        __syncthreads();
        const uint32_t wn = Bn[tx];
        const uint32_t wp = TERNARY ? Bp[tx] : 0u;
#pragma unroll 8
        for (int kk = 0; kk < 32; ++kk) {
            const uint32_t sgn = ((wn >> kk) & 1u) << 31;
            const bool nz = !TERNARY || (((wn | wp) >> kk) & 1u);
#pragma unroll
            for (int r = 0; r < 8; ++r) {
                const float x = __uint_as_float(__float_as_uint(As[ty * 8 + r][kk]) ^ sgn);
                acc[r] = __fadd_rn(acc[r], nz ? x : 0.0f);
            }
        }
        __syncthreads();
    }
    const int n = n0 + tx;
    if (n < N) {
        const float al = ep.alpha ? ep.alpha[n] : 1.0f;
        const float bi = ep.bias ? ep.bias[n] : 0.0f;
#pragma unroll
        for (int r = 0; r < 8; ++r) {
            const int m = m0 + ty * 8 + r;
            if (m < M) c[static_cast<int64_t>(m) * ldc + n] = apply_epilogue(acc[r], al, bi, ep.scale, ep.flags & ~TBN_EPI_ADD_RESIDUAL, 0.0f);
        }
    }
}

// =====================================================================================
// Host side
// =====================================================================================

int npass_of(int mode) {
    switch (mode) {
        case TBN_MODE_TC_FP16X1:
        case TBN_MODE_TC_BF16X1: return 1;
        case TBN_MODE_TC_BF16X2: return 2;
        case TBN_MODE_TC_BF16X3: return 3;
        default: return 0;
    }
}


template <int NPASS, bool TERN_ACT>
int32_t launch_split(const float* d_a, int64_t M, int64_t K, int64_t lda, int64_t M_pad, int64_t K_pad,
                     __nv_bfloat16* out, float lo, float hi, cudaStream_t st) {
    const int64_t total = M_pad * (K_pad / 8);
    const int64_t want = (total + 255) / 256;
    const int64_t cap = static_cast<int64_t>(sm_count()) * 16;
    const int grid = static_cast<int>(std::max<int64_t>(1, std::min(want, cap)));
    const int vec_ok = (lda % 4 == 0) && (reinterpret_cast<uintptr_t>(d_a) % 16 == 0);
    profile_begin(kProfSplit, st);
    split_activations_kernel<NPASS, TERN_ACT><<<grid, 256, 0, st>>>(d_a, M, K, lda, M_pad, K_pad, out, lo, hi, vec_ok);
    profile_end(kProfSplit, st);
    return launched("split_activations_kernel");
}

// fp16 mode pre-pass: max |a| of the call into *slot, then the scaled one-term split.
int32_t launch_split_f16(const float* d_a, int64_t M, int64_t K, int64_t lda, int64_t M_pad, int64_t K_pad,
                         __nv_bfloat16* out, uint32_t* slot, cudaStream_t st) {
    TBN_CUDA_TRY(cudaMemsetAsync(slot, 0, sizeof(uint32_t), st));
    const int vec_ok = (lda % 4 == 0) && (K % 4 == 0) && (reinterpret_cast<uintptr_t>(d_a) % 16 == 0);
    const int64_t cap = static_cast<int64_t>(sm_count()) * 16;
    const int64_t units = vec_ok ? M * (K / 4) : M * K;
    const int grid_max = static_cast<int>(std::max<int64_t>(1, std::min((units + 255) / 256, cap)));
    profile_begin(kProfSplit, st);
    absmax_kernel<<<grid_max, 256, 0, st>>>(d_a, M, K, lda, vec_ok, slot);
    int32_t rc = launched("absmax_kernel");
    if (rc) return rc;
    const int64_t total = M_pad * (K_pad / 8);
    const int grid = static_cast<int>(std::max<int64_t>(1, std::min((total + 255) / 256, cap)));
    const int vec8 = (lda % 4 == 0) && (reinterpret_cast<uintptr_t>(d_a) % 16 == 0);
    split_activations_kernel<1, false, true><<<grid, 256, 0, st>>>(d_a, M, K, lda, M_pad, K_pad, out, 0.f, 0.f, vec8, slot);
    profile_end(kProfSplit, st);
    return launched("split_activations_kernel<fp16>");
}

std::atomic<int> g_fused_split{1};
// 0 never, 1 as the per-shape plan says (by default: when the weights have a single column tile), 2 always.
bool fused_split_wanted(const GemmPlan& plan) {
    const int v = g_fused_split.load(std::memory_order_relaxed);
    return v == 2 || (v == 1 && plan.fused_split != 0);
}

// Tensor-core path: split (or ternarise) A into the workspace, then the tcgen05 kernel.
int32_t gemm_tensor_core(const float* d_a, int64_t M, int64_t K, int64_t lda, bool ternarise_act, float act_lo,
                         float act_hi, int npass, const uint32_t* d_neg, const uint32_t* d_pos, int64_t N,
                         const Epilogue& ep, float* d_c, int64_t ldc, void* d_ws, size_t ws_bytes, cudaStream_t st,
                         float* const* outs = nullptr, int num_out = 0, const void* dense_w = nullptr, bool f16 = false) {
    const int64_t M_pad = round_up(M, tc::BM), K_pad = round_up(K, 128), N_pad = round_up(N, 8);
    const size_t split_bytes = static_cast<size_t>(npass) * M_pad * K_pad * sizeof(__nv_bfloat16);
    // fp16 mode: a 256-byte slot after the partial-sum tiles holds max |a| of the call.
    const size_t need = split_bytes + scratch_bytes() + (f16 ? 256 : 0);
    uint32_t* amax_slot = f16 ? reinterpret_cast<uint32_t*>(static_cast<uint8_t*>(d_ws) + split_bytes + scratch_bytes()) : nullptr;
    TBN_REQUIRE(d_ws && ws_bytes >= need, TBN_INVALID_ARGUMENT,
                "gemm: workspace too small (see tbn_gemm_workspace_bytes)");
    TBN_REQUIRE(reinterpret_cast<uintptr_t>(d_ws) % 128 == 0, TBN_INVALID_ARGUMENT,
                "gemm: workspace must be 128-byte aligned");
    TBN_REQUIRE(M_pad / tc::BM <= 0x7fffff && (M_pad / tc::BM) * ((N + 63) / 64) <= 0x7fffffffLL, TBN_INVALID_SHAPE,
                "gemm: too many tiles");
    EncodeTiledFn encode = encode_tiled_fn();
    TBN_REQUIRE(encode != nullptr, TBN_CUDA_ERROR, "cuTensorMapEncodeTiled is not available from the driver");
    __nv_bfloat16* split = static_cast<__nv_bfloat16*>(d_ws);

    // Two-term products whose A rows can be read as float4 may skip the split pass: the GEMM's build warps read
    // the fp32 rows and split them in registers (same arithmetic, bit-identical operands) -- once per column
    // tile of the weights, so by default only when there is a single one.
    const GemmPlan plan = gemm_plan(M, N, K);
    const bool fused_split = !f16 && num_out == 0 && fused_split_wanted(plan) && !ternarise_act && npass == 2 && !dense_w && K % 4 == 0 &&
                             lda % 4 == 0 && reinterpret_cast<uintptr_t>(d_a) % 16 == 0;
    int32_t rc = TBN_SUCCESS;
    if (fused_split) {}
    else if (f16) rc = launch_split_f16(d_a, M, K, lda, M_pad, K_pad, split, amax_slot, st);
    else if (ternarise_act) rc = launch_split<1, true>(d_a, M, K, lda, M_pad, K_pad, split, act_lo, act_hi, st);
    else if (npass == 1) rc = launch_split<1, false>(d_a, M, K, lda, M_pad, K_pad, split, 0.f, 0.f, st);
    else if (npass == 2) rc = launch_split<2, false>(d_a, M, K, lda, M_pad, K_pad, split, 0.f, 0.f, st);
    else rc = launch_split<3, false>(d_a, M, K, lda, M_pad, K_pad, split, 0.f, 0.f, st);
    if (rc) return rc;

    TensorMaps maps;
    CUtensorMap& tmap = maps.a;
    const cuuint64_t gdim[3] = {static_cast<cuuint64_t>(K_pad), static_cast<cuuint64_t>(M_pad),
                                static_cast<cuuint64_t>(npass)};
    const cuuint64_t gstride[2] = {static_cast<cuuint64_t>(K_pad) * 2, static_cast<cuuint64_t>(M_pad) * K_pad * 2};
    const cuuint32_t box[3] = {tc::BK, tc::BM, 1};
    const cuuint32_t estr[3] = {1, 1, 1};
    const CUresult cr = encode(&tmap, f16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, split, gdim, gstride, box, estr,
                               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    TBN_REQUIRE(cr == CUDA_SUCCESS, TBN_CUDA_ERROR,
                "cuTensorMapEncodeTiled failed with CUresult " + std::to_string(static_cast<int>(cr)));

    // CTA pairs (gemm_pair.cuh): the plan's choice for large products; 256 x 256 tiles, each CTA holding 128 columns.
    const bool use_pair = plan.kernel == 2 && !fused_split && !dense_w && num_out == 0;
    const int bn = use_pair ? pair::BH : plan.bn;  // rows of the packed-word box
    if (dense_w) {
        TBN_REQUIRE(reinterpret_cast<uintptr_t>(dense_w) % 16 == 0, TBN_INVALID_ARGUMENT,
                    "gemm: split dense weights must be 16-byte aligned");
        rc = make_split_map(encode, dense_w, K_pad, N_pad, 2, bn, &maps.neg);
        if (rc) return rc;
        maps.pos = maps.neg;
    } else {
        TBN_REQUIRE(reinterpret_cast<uintptr_t>(d_neg) % 16 == 0 && (!d_pos || reinterpret_cast<uintptr_t>(d_pos) % 16 == 0),
                    TBN_INVALID_ARGUMENT, "gemm: packed weight planes must be 16-byte aligned");
        const int wpr = use_pair ? 4 : gemm_words_per_row(d_pos != nullptr, num_out > 0);
        rc = make_word_map(encode, d_neg, K_pad / 32, N_pad, bn, &maps.neg, wpr);
        if (rc) return rc;
        rc = make_word_map(encode, d_pos ? d_pos : d_neg, K_pad / 32, N_pad, bn, &maps.pos, wpr);
        if (rc) return rc;
    }
    tc::Params p = {};
    p.M = static_cast<int>(M);
    p.N = static_cast<int>(N);
    p.num_kb = static_cast<int>((K + tc::BK - 1) / tc::BK);  // k-blocks that hold real k; the operands are zero beyond K
    p.tiles_m = static_cast<int>(M_pad / tc::BM);
    p.tiles_n = static_cast<int>((N + bn - 1) / bn);
    p.group_m = plan.group_m;
    p.c = d_c;
    p.ldc = ldc;
    p.ep = ep;
    p.err_word = device_error_word();
    p.c_vec_ok = (ldc % 4 == 0) && (reinterpret_cast<uintptr_t>(d_c) % 16 == 0);
    set_segments(p, npass);
    p.scratch = reinterpret_cast<float4*>(static_cast<uint8_t*>(d_ws) + split_bytes);
    p.num_out = num_out;
    for (int i = 0; i < num_out; ++i) {
        p.out_list[i] = outs[i];
        rc = make_out_map(encode, outs[i], M, N, ldc, &maps.out.m[i]);
        if (rc) return rc;
    }
    p.a_rows = d_a;
    p.lda = lda;
    p.K = static_cast<int>(K);
    p.f16 = f16 ? 1 : 0;
    p.amax_bits = amax_slot;
    if (use_pair) {
        p.tiles_m = static_cast<int>((M_pad / tc::BM + 1) / 2);
        p.tiles_n = static_cast<int>((N + pair::BN - 1) / pair::BN);
        const bool tern = d_pos != nullptr;
        if (npass == 1) return tern ? pair::launch<1, true>(maps, p, st) : pair::launch<1, false>(maps, p, st);
        if (npass == 2) return tern ? pair::launch<2, true>(maps, p, st) : pair::launch<2, false>(maps, p, st);
        return tern ? pair::launch<3, true>(maps, p, st) : pair::launch<3, false>(maps, p, st);
    }
    if (fused_split)
        return d_pos ? dispatch_bn<2, true, 3, false>(bn, maps, p, st) : dispatch_bn<2, false, 3, false>(bn, maps, p, st);
    if (dense_w) {
        set_segments(p, 3);  // three MMA passes per k-block
        return dispatch_bn<2, false, 0, false, 1>(bn, maps, p, st);
    }
    const bool ternary_w = d_pos != nullptr;
    if (num_out > 0) {  // multi-destination epilogue
        if (npass == 1)
            return ternary_w ? dispatch_bn<1, true, 0, false, 0, true>(bn, maps, p, st)
                             : dispatch_bn<1, false, 0, false, 0, true>(bn, maps, p, st);
        if (npass == 2)
            return ternary_w ? dispatch_bn<2, true, 0, false, 0, true>(bn, maps, p, st)
                             : dispatch_bn<2, false, 0, false, 0, true>(bn, maps, p, st);
        return ternary_w ? dispatch_bn<3, true, 0, false, 0, true>(bn, maps, p, st)
                         : dispatch_bn<3, false, 0, false, 0, true>(bn, maps, p, st);
    }
    if (npass == 1)
        return ternary_w ? dispatch_bn<1, true, 0, false>(bn, maps, p, st)
                         : dispatch_bn<1, false, 0, false>(bn, maps, p, st);
    if (npass == 2)
        return ternary_w ? dispatch_bn<2, true, 0, false>(bn, maps, p, st)
                         : dispatch_bn<2, false, 0, false>(bn, maps, p, st);
    return ternary_w ? dispatch_bn<3, true, 0, false>(bn, maps, p, st)
                     : dispatch_bn<3, false, 0, false>(bn, maps, p, st);
}

int32_t gemm_simt(const float* d_a, int64_t M, int64_t K, int64_t lda, bool ternarise_act, float act_lo, float act_hi,
                  const uint32_t* d_neg, const uint32_t* d_pos, int64_t N, const Epilogue& ep, float* d_c,
                  int64_t ldc, cudaStream_t st) {
    const int64_t K_pad = round_up(K, 128), N_pad = round_up(N, 8);
    dim3 grid(static_cast<unsigned>((N + kSimtBN - 1) / kSimtBN), static_cast<unsigned>((M + kSimtBM - 1) / kSimtBM));
    TBN_REQUIRE(grid.y <= 65535, TBN_INVALID_SHAPE, "gemm (CUDA-core path): M too large; use a tensor-core mode");
    if (d_pos)
        gemm_simt_kernel<true><<<grid, 256, 0, st>>>(d_a, static_cast<int>(M), static_cast<int>(K), lda, d_neg, d_pos,
                                                     K_pad / 32, N_pad, static_cast<int>(N), ep, d_c, ldc,
                                                     ternarise_act, act_lo, act_hi);
    else
        gemm_simt_kernel<false><<<grid, 256, 0, st>>>(d_a, static_cast<int>(M), static_cast<int>(K), lda, d_neg,
                                                      nullptr, K_pad / 32, N_pad, static_cast<int>(N), ep, d_c, ldc,
                                                      ternarise_act, act_lo, act_hi);
    return launched("gemm_simt_kernel");
}

int32_t check_gemm_args(const float* d_a, int64_t M, int64_t K, int64_t lda, const uint32_t* d_neg, int64_t N,
                        float* d_c, int64_t ldc) {
    TBN_REQUIRE(M > 0 && N > 0 && K > 0, TBN_INVALID_SHAPE, "gemm: M, N and K must be positive");
    TBN_REQUIRE(M < (1LL << 31) && N < (1LL << 31) && K < (1LL << 31), TBN_INVALID_SHAPE, "gemm: dimension too large");
    TBN_REQUIRE(d_a && d_neg && d_c, TBN_INVALID_ARGUMENT, "gemm: null pointer");
    TBN_REQUIRE(lda >= K && ldc >= N, TBN_INVALID_ARGUMENT, "gemm: leading dimension smaller than the row length");
    TBN_REQUIRE(device_error_word() != nullptr, TBN_RUNTIME_ERROR, "tbn_cuda_init was not called on this device");
    return TBN_SUCCESS;
}

// Per-shape choice between the CUDA-core and the tensor-core kernel: the plan table (plan.cuh), measured with CUDA
// events on a B200; classes without an entry use the rule "CUDA cores up to M*N*K = 2^24" (the two kernels meet
// around 256^3, where both are launch bound; above it the tensor-core path wins, also for a handful of rows).
bool prefer_simt(int64_t M, int64_t N, int64_t K) { return gemm_plan(M, N, K).kernel == 1 && M <= 65535LL * kSimtBM; }

}  // namespace
}  // namespace tbn_cuda

using namespace tbn_cuda;

extern "C" {

int32_t tbn_cuda_set_fused_split(int32_t value) {
    TBN_REQUIRE(value >= 0 && value <= 2, TBN_INVALID_ARGUMENT, "tbn_cuda_set_fused_split: value must be 0, 1 or 2");
    g_fused_split.store(value, std::memory_order_relaxed);
    return TBN_SUCCESS;
}

size_t tbn_gemm_workspace_bytes(int64_t M, int64_t K, int32_t mode) {
    if (M <= 0 || K <= 0) return 0;
    int np = npass_of(mode);
    if (mode == TBN_MODE_SIMT) return 0;
    if (np == 0) np = 2;  // AUTO resolves to at most the two-term split
    // Split activations + the per-SM partial-sum tiles (sized for the largest SM count in use).
    return static_cast<size_t>(np) * round_up(M, tc::BM) * round_up(K, 128) * sizeof(__nv_bfloat16) +
           static_cast<size_t>(std::max(sm_count(), 160)) * tc::BM * 256 * sizeof(float) + 256;
}

int32_t tbn_gemm_fxb(const float* d_a, int64_t M, int64_t K, int64_t lda, const uint32_t* d_neg,
                     const uint32_t* d_pos, int64_t N, const float* d_alpha, float scale, const float* d_bias,
                     float* d_c, int64_t ldc, int32_t mode, uint32_t epilogue, void* d_workspace,
                     size_t workspace_bytes, void* stream) {
    int32_t rc = check_gemm_args(d_a, M, K, lda, d_neg, N, d_c, ldc);
    if (rc) return rc;
    TBN_REQUIRE(mode >= TBN_MODE_AUTO && mode <= TBN_MODE_TC_FP16X1, TBN_INVALID_ARGUMENT, "tbn_gemm_fxb: unknown mode");
    const Epilogue ep{d_alpha, d_bias, nullptr, scale, epilogue & ~TBN_EPI_ADD_RESIDUAL};
    if (mode == TBN_MODE_AUTO) mode = prefer_simt(M, N, K) ? TBN_MODE_SIMT : TBN_MODE_TC_BF16X2;
    if (mode == TBN_MODE_SIMT)
        return gemm_simt(d_a, M, K, lda, false, 0.f, 0.f, d_neg, d_pos, N, ep, d_c, ldc, as_stream(stream));
    return gemm_tensor_core(d_a, M, K, lda, false, 0.f, 0.f, npass_of(mode), d_neg, d_pos, N, ep, d_c, ldc, d_workspace,
                            workspace_bytes, as_stream(stream), nullptr, 0, nullptr, mode == TBN_MODE_TC_FP16X1);
}

size_t tbn_dense_pack_bytes(int64_t K, int64_t N) {
    if (K <= 0 || N <= 0) return 0;
    return static_cast<size_t>(2) * round_up(N, 8) * round_up(K, 128) * sizeof(__nv_bfloat16);
}

int32_t tbn_dense_pack(const float* d_w, int64_t K, int64_t N, int64_t ldw, int32_t layout, void* d_packed, void* stream) {
    TBN_REQUIRE(K > 0 && N > 0, TBN_INVALID_SHAPE, "tbn_dense_pack: K and N must be positive");
    TBN_REQUIRE(d_w && d_packed && reinterpret_cast<uintptr_t>(d_packed) % 16 == 0, TBN_INVALID_ARGUMENT,
                "tbn_dense_pack: null or misaligned pointer");
    TBN_REQUIRE(layout == TBN_LAYOUT_KN || layout == TBN_LAYOUT_NK, TBN_INVALID_ARGUMENT, "tbn_dense_pack: bad layout");
    TBN_REQUIRE(ldw >= (layout == TBN_LAYOUT_KN ? N : K), TBN_INVALID_ARGUMENT, "tbn_dense_pack: ldw too small");
    const int64_t K_pad = round_up(K, 128), N_pad = round_up(N, 8);
    __nv_bfloat16* out = static_cast<__nv_bfloat16*>(d_packed);
    if (layout == TBN_LAYOUT_NK)  // rows of W are the output columns: the activation split does the job
        return launch_split<2, false>(d_w, N, K, ldw, N_pad, K_pad, out, 0.f, 0.f, as_stream(stream));
    const int64_t total = N_pad * (K_pad / 8);
    const int grid = static_cast<int>(std::max<int64_t>(1, std::min((total + 255) / 256, static_cast<int64_t>(sm_count()) * 16)));
    split_dense_kn_kernel<<<grid, 256, 0, as_stream(stream)>>>(d_w, K, N, ldw, N_pad, K_pad, out);
    return launched("split_dense_kn_kernel");
}

int32_t tbn_gemm_f32(const float* d_a, int64_t M, int64_t K, int64_t lda, const void* d_packed_w, int64_t N, float alpha,
                     const float* d_bias, float* d_c, int64_t ldc, uint32_t epilogue, void* d_workspace,
                     size_t workspace_bytes, void* stream) {
    TBN_REQUIRE(d_packed_w != nullptr, TBN_INVALID_ARGUMENT, "tbn_gemm_f32: null weights");
    int32_t rc = check_gemm_args(d_a, M, K, lda, reinterpret_cast<const uint32_t*>(d_packed_w), N, d_c, ldc);
    if (rc) return rc;
    const Epilogue ep{nullptr, d_bias, nullptr, alpha, epilogue & ~TBN_EPI_ADD_RESIDUAL};
    return gemm_tensor_core(d_a, M, K, lda, false, 0.f, 0.f, 2, nullptr, nullptr, N, ep, d_c, ldc, d_workspace,
                            workspace_bytes, as_stream(stream), nullptr, 0, d_packed_w);
}

int32_t tbn_gemm_fxb_multi(const float* d_a, int64_t M, int64_t K, int64_t lda, const uint32_t* d_neg,
                           const uint32_t* d_pos, int64_t N, const float* d_alpha, float scale, const float* d_bias,
                           float* const* d_c_list, int32_t num_out, int64_t ldc, int32_t mode, uint32_t epilogue,
                           void* d_workspace, size_t workspace_bytes, void* stream) {
    TBN_REQUIRE(d_c_list != nullptr && num_out >= 1 && num_out <= tc::kMaxOutputs, TBN_INVALID_ARGUMENT,
                "tbn_gemm_fxb_multi: between 1 and 8 destinations are required");
    for (int i = 0; i < num_out; ++i)
        TBN_REQUIRE(d_c_list[i] != nullptr && reinterpret_cast<uintptr_t>(d_c_list[i]) % 16 == 0, TBN_INVALID_ARGUMENT,
                    "tbn_gemm_fxb_multi: destinations must be non-null and 16-byte aligned");
    TBN_REQUIRE(N % 4 == 0 && ldc % 4 == 0, TBN_INVALID_SHAPE, "tbn_gemm_fxb_multi: N and ldc must be multiples of 4");
    int32_t rc = check_gemm_args(d_a, M, K, lda, d_neg, N, d_c_list[0], ldc);
    if (rc) return rc;
    if (mode == TBN_MODE_AUTO) mode = TBN_MODE_TC_BF16X2;
    TBN_REQUIRE(npass_of(mode) != 0, TBN_INVALID_ARGUMENT, "tbn_gemm_fxb_multi: a tensor-core mode is required");
    const Epilogue ep{d_alpha, d_bias, nullptr, scale, epilogue & ~TBN_EPI_ADD_RESIDUAL};
    return gemm_tensor_core(d_a, M, K, lda, false, 0.f, 0.f, npass_of(mode), d_neg, d_pos, N, ep, d_c_list[0], ldc,
                            d_workspace, workspace_bytes, as_stream(stream), d_c_list, num_out, nullptr,
                            mode == TBN_MODE_TC_FP16X1);
}

int32_t tbn_gemm_tbn(const float* d_a, int64_t M, int64_t K, int64_t lda, float lo, float hi, const uint32_t* d_neg,
                     int64_t N, const float* d_alpha, float scale, const float* d_bias, float* d_c, int64_t ldc,
                     uint32_t epilogue, void* d_workspace, size_t workspace_bytes, void* stream) {
    int32_t rc = check_gemm_args(d_a, M, K, lda, d_neg, N, d_c, ldc);
    if (rc) return rc;
    // Integer-exact on the tensor cores only while every partial sum fits fp32's 24-bit significand.
    TBN_REQUIRE(K < (1 << 24), TBN_INVALID_SHAPE, "tbn_gemm_tbn: K too large for exact accumulation");
    const Epilogue ep{d_alpha, d_bias, nullptr, scale, epilogue & ~TBN_EPI_ADD_RESIDUAL};
    if (prefer_simt(M, N, K) || d_workspace == nullptr)
        return gemm_simt(d_a, M, K, lda, true, lo, hi, d_neg, nullptr, N, ep, d_c, ldc, as_stream(stream));
    return gemm_tensor_core(d_a, M, K, lda, true, lo, hi, 1, d_neg, nullptr, N, ep, d_c, ldc, d_workspace,
                            workspace_bytes, as_stream(stream));
}

}  // extern "C"
