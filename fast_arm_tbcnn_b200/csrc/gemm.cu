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
#include <cuda.h>
#include <cuda_bf16.h>

#include <algorithm>
#include <climits>
#include <cstdint>

#include "common.cuh"
#include "ptx_sm100.cuh"

namespace tbn_cuda {
namespace {

// =====================================================================================
// Activation split
// =====================================================================================

// One thread converts 8 consecutive k of one row and writes one 16-byte vector per pass.
template <int NPASS, bool TERNARISE>
__global__ void __launch_bounds__(256) split_activations_kernel(const float* __restrict__ a, int64_t M, int64_t K,
                                                                int64_t lda, int64_t M_pad, int64_t K_pad,
                                                                __nv_bfloat16* __restrict__ out, float lo, float hi,
                                                                int vec_ok) {
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
            if (TERNARISE) {
                // TernaryMatrix::pack_from_float (GeMM/05-final/GeMM.cpp:99-106): strict compares.
                const float t = v[i] < lo ? -1.0f : (v[i] > hi ? 1.0f : 0.0f);
                term[0] = __bfloat16_as_ushort(__float2bfloat16_rn(t));
            } else {
                float r = v[i];
#pragma unroll
                for (int p = 0; p < NPASS; ++p) {
                    const __nv_bfloat16 h = __float2bfloat16_rn(r);
                    term[p] = __bfloat16_as_ushort(h);
                    // Exact in fp32; a non-finite input leaves its residual terms at zero.
                    r = (p == 0 && !isfinite(r)) ? 0.0f : __fsub_rn(r, __bfloat162float(h));
                }
            }
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

// =====================================================================================
// Weight unpack helpers: 8 packed bits -> 8 bf16 (+1 = 0x3F80, -1 = 0xBF80, 0 = 0x0000)
// =====================================================================================

template <bool TERNARY>
__device__ __forceinline__ uint4 unpack8(uint32_t neg_byte, uint32_t pos_byte) {
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const uint32_t n0 = (neg_byte >> (2 * j)) & 1u, n1 = (neg_byte >> (2 * j + 1)) & 1u;
        if (TERNARY) {
            const uint32_t p0 = (pos_byte >> (2 * j)) & 1u, p1 = (pos_byte >> (2 * j + 1)) & 1u;
            const uint32_t lo16 = ((n0 | p0) * 0x3F80u) | (n0 << 15);
            const uint32_t hi16 = ((n1 | p1) * 0x3F80u) | (n1 << 15);
            o[j] = lo16 | (hi16 << 16);
        } else {
            o[j] = 0x3F803F80u | (n0 << 15) | (n1 << 31);
        }
    }
    return make_uint4(o[0], o[1], o[2], o[3]);
}

// =====================================================================================
// tcgen05 kernel
// =====================================================================================

namespace tc {

constexpr int BM = 128;
constexpr int BK = 64;          // 64 bf16 = 128 bytes = one swizzle row
constexpr int UMMA_K = 16;
constexpr int A_TILE_BYTES = BM * BK * 2;
constexpr int kProducerWarp = 0, kMmaWarp = 1;
constexpr int kTransformThreads = 256, kEpilogueThreads = 128;
constexpr int kThreads = 64 + kTransformThreads + kEpilogueThreads;
constexpr int kGroupM = 8;      // rasterisation: 8 m-tiles share a sweep over n for L2 reuse
constexpr int kWordStages = 2;  // ring of packed-word tiles, each covering 2 k-blocks (128 k)
constexpr int kAuxBarrierBytes = 1024;
constexpr int kSmemLimit = 232448;  // 227 KB opt-in maximum per CTA

template <int BN, int NPASS, bool TERNARY = false>
struct Cfg {
    static constexpr int B_TILE_BYTES = BN * BK * 2;
    static constexpr int STAGE_BYTES = B_TILE_BYTES + NPASS * A_TILE_BYTES;
    static constexpr int WORD_TILE_BYTES = BN * 16 * (TERNARY ? 2 : 1);  // 4 words per column and plane
    // barriers + alpha/bias staging (x2 buffers) + packed-word ring
    static constexpr int AUX_BYTES = kAuxBarrierBytes + 4 * BN * 4 + kWordStages * WORD_TILE_BYTES;
    static constexpr int RAW_STAGES = (kSmemLimit - 1024 - AUX_BYTES) / STAGE_BYTES;
    static constexpr int STAGES = RAW_STAGES > 6 ? 6 : RAW_STAGES;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + AUX_BYTES + 1024;  // + alignment slack
    static constexpr int TMEM_COLS = 2 * BN;
    static_assert(STAGES >= 2, "need at least a double-buffered pipeline");
    static_assert(TMEM_COLS == 128 || TMEM_COLS == 256 || TMEM_COLS == 512, "TMEM columns must be a power of two");
    static_assert(B_TILE_BYTES % 1024 == 0, "operand tiles must stay 1024-byte aligned");
};

struct Params {
    const uint32_t* neg;   // [N_pad][KW]
    const uint32_t* pos;   // [N_pad][KW] or nullptr
    int64_t KW;            // words per column = K_pad / 32
    int64_t N_pad;
    int M, N;
    int num_kb;            // K_pad / 64
    int tiles_m, tiles_n;
    float* c;
    int64_t ldc;
    Epilogue ep;
    int* err_word;
    int c_vec_ok;          // rows of C are 16-byte aligned
    int num_seg;           // K segments per tile, each with a fresh accumulator
    int kb_per_seg;        // k-blocks per segment (the last one may be shorter)
    float4* scratch;       // [gridDim.x][BN/4][128] partial sums, used when num_seg > 1
};

// Accumulation steps (k elements x passes) after which a fresh accumulator is started.
constexpr int kMaxAccumSteps = 4096;

__device__ __forceinline__ void tile_coords(int t, int tiles_m, int tiles_n, int& tm, int& tn) {
    const int group_size = kGroupM * tiles_n;
    const int g = t / group_size;
    const int first_m = g * kGroupM;
    const int gm = min(tiles_m - first_m, kGroupM);
    const int r = t - g * group_size;
    tm = first_m + r % gm;
    tn = r / gm;
}

template <int BN, int NPASS, bool TERNARY>
__global__ void __launch_bounds__(kThreads, 1) gemm_tc_kernel(const __grid_constant__ CUtensorMap tmap_a,
                                                              const __grid_constant__ CUtensorMap tmap_neg,
                                                              const __grid_constant__ CUtensorMap tmap_pos,
                                                              const Params p) {
    using C = Cfg<BN, NPASS, TERNARY>;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = ptx::smem_u32(smem_raw);
    const uint32_t base = (raw_addr + 1023u) & ~1023u;
    uint8_t* base_ptr = smem_raw + (base - raw_addr);

    const uint32_t aux = base + C::STAGES * C::STAGE_BYTES;
    const uint32_t bar_full_a = aux;                       // STAGES x 8 B
    const uint32_t bar_full_b = aux + 8 * C::STAGES;
    const uint32_t bar_empty = aux + 16 * C::STAGES;
    const uint32_t bar_tmem_full = aux + 24 * C::STAGES;   // 2 x 8 B
    const uint32_t bar_tmem_empty = bar_tmem_full + 16;    // 2 x 8 B
    const uint32_t bar_full_w = bar_tmem_empty + 16;       // kWordStages x 8 B
    const uint32_t bar_empty_w = bar_full_w + 8 * kWordStages;
    const uint32_t tmem_slot = bar_empty_w + 8 * kWordStages;  // 4 B
    uint8_t* aux_ptr = base_ptr + C::STAGES * C::STAGE_BYTES;
    volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(aux_ptr + (tmem_slot - aux));
    float* alpha_s = reinterpret_cast<float*>(aux_ptr + kAuxBarrierBytes);  // [2][BN]
    float* bias_s = alpha_s + 2 * BN;                                       // [2][BN]
    const uint32_t word_ring = aux + kAuxBarrierBytes + 4 * BN * 4;         // [kWordStages][planes][BN][4 words]

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int total_tiles = p.tiles_m * p.tiles_n;

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::STAGES; ++s) {
            ptx::mbar_init(bar_full_a + 8 * s, 1);
            ptx::mbar_init(bar_full_b + 8 * s, kTransformThreads);
            ptx::mbar_init(bar_empty + 8 * s, 1);
        }
        for (int b = 0; b < 2; ++b) {
            ptx::mbar_init(bar_tmem_full + 8 * b, 1);
            ptx::mbar_init(bar_tmem_empty + 8 * b, kEpilogueThreads);
        }
        for (int w = 0; w < kWordStages; ++w) {
            ptx::mbar_init(bar_full_w + 8 * w, 1);
            ptx::mbar_init(bar_empty_w + 8 * w, kTransformThreads);
        }
        ptx::fence_barrier_init();
        ptx::prefetch_tensormap(&tmap_a);
        ptx::prefetch_tensormap(&tmap_neg);
        if (TERNARY) ptx::prefetch_tensormap(&tmap_pos);
    }
    if (warp == kMmaWarp) {
        ptx::tmem_alloc(tmem_slot, C::TMEM_COLS);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot_ptr;

    if (warp == kProducerWarp) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            int stage = 0, wstage = 0;
            uint32_t phase = 0, wphase = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
                int tm, tn;
                tile_coords(t, p.tiles_m, p.tiles_n, tm, tn);
                for (int kb = 0; kb < p.num_kb; ++kb) {
                    if ((kb & 1) == 0) {
                        // Packed words of k-blocks kb and kb+1 for the BN columns of this tile
                        // (rows past the end of the plane are zero-filled by TMA).
                        if (!ptx::mbar_wait(bar_empty_w + 8 * wstage, wphase ^ 1u, p.err_word, kErrWaitEmpty)) {
                            ok = false;
                            break;
                        }
                        const uint32_t wbar = bar_full_w + 8 * wstage;
                        const uint32_t wdst = word_ring + wstage * C::WORD_TILE_BYTES;
                        ptx::mbar_arrive_expect_tx(wbar, C::WORD_TILE_BYTES);
                        ptx::tma_load_2d(wdst, &tmap_neg, kb * 2, tn * BN, wbar);
                        if (TERNARY) ptx::tma_load_2d(wdst + BN * 16, &tmap_pos, kb * 2, tn * BN, wbar);
                        if (++wstage == kWordStages) {
                            wstage = 0;
                            wphase ^= 1u;
                        }
                    }
                    if (!ptx::mbar_wait(bar_empty + 8 * stage, phase ^ 1u, p.err_word, kErrWaitEmpty)) {
                        ok = false;
                        break;
                    }
                    const uint32_t bar = bar_full_a + 8 * stage;
                    ptx::mbar_arrive_expect_tx(bar, NPASS * A_TILE_BYTES);
                    const uint32_t a_dst = base + stage * C::STAGE_BYTES + C::B_TILE_BYTES;
#pragma unroll
                    for (int q = 0; q < NPASS; ++q)
                        ptx::tma_load_3d(a_dst + q * A_TILE_BYTES, &tmap_a, kb * BK, tm * BM, q, bar);
                    if (++stage == C::STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
        }
    } else if (warp == kMmaWarp) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = ptx::umma_idesc_bf16_f32(BM, BN);
            int stage = 0;
            uint32_t phase = 0;
            int iter = 0;  // counts (tile, segment) units; each uses one accumulator buffer
            bool ok = true;
            for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
                for (int seg = 0; seg < p.num_seg && ok; ++seg, ++iter) {
                    const int buf = iter & 1;
                    const uint32_t acc_parity = static_cast<uint32_t>((iter >> 1) & 1);
                    if (!ptx::mbar_wait(bar_tmem_empty + 8 * buf, acc_parity ^ 1u, p.err_word, kErrWaitTmemEmpty)) {
                        ok = false;
                        break;
                    }
                    ptx::tc_fence_after_sync();
                    const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(buf * BN);
                    const int kb_begin = seg * p.kb_per_seg;
                    const int kb_end = min(p.num_kb, kb_begin + p.kb_per_seg);
                    for (int kb = kb_begin; kb < kb_end; ++kb) {
                        if (!ptx::mbar_wait(bar_full_a + 8 * stage, phase, p.err_word, kErrWaitFullA) ||
                            !ptx::mbar_wait(bar_full_b + 8 * stage, phase, p.err_word, kErrWaitFullB)) {
                            ok = false;
                            break;
                        }
                        ptx::tc_fence_after_sync();
                        const uint32_t b_addr = base + stage * C::STAGE_BYTES;
                        const uint32_t a_addr = b_addr + C::B_TILE_BYTES;
#pragma unroll
                        for (int q = 0; q < NPASS; ++q) {
#pragma unroll
                            for (int k4 = 0; k4 < BK / UMMA_K; ++k4) {
                                const uint64_t a_desc =
                                    ptx::umma_desc_k_sw128(a_addr + q * A_TILE_BYTES + k4 * UMMA_K * 2);
                                const uint64_t b_desc = ptx::umma_desc_k_sw128(b_addr + k4 * UMMA_K * 2);
                                ptx::umma_bf16(d_tmem, a_desc, b_desc, idesc, (kb != kb_begin || q != 0 || k4 != 0) ? 1u : 0u);
                            }
                        }
                        ptx::umma_commit(bar_empty + 8 * stage);  // smem stage free once these MMAs retire
                        if (++stage == C::STAGES) {
                            stage = 0;
                            phase ^= 1u;
                        }
                    }
                    if (ok) ptx::umma_commit(bar_tmem_full + 8 * buf);  // this segment's accumulator is complete
                }
            }
        }
    } else if (warp < 2 + kTransformThreads / 32) {
        // ------------------------------------------------------------ weight transform
        static_assert(BN <= kTransformThreads, "one transform thread per weight column of the tile");
        const int r = threadIdx.x - 64;  // weight column (row of the K-major operand tile) of this thread
        int stage = 0, wstage = 0;
        uint32_t phase = 0, wphase = 0;
        bool ok = true;
        uint4 wn = make_uint4(0u, 0u, 0u, 0u), wp = make_uint4(0u, 0u, 0u, 0u);
        for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
            for (int kb = 0; kb < p.num_kb; ++kb) {
                if ((kb & 1) == 0) {
                    // Words of this and the next k-block: shared memory -> registers, then free the slot.
                    if (!ptx::mbar_wait(bar_full_w + 8 * wstage, wphase, p.err_word, kErrWaitFullB)) {
                        ok = false;
                        break;
                    }
                    if (r < BN) {
                        const uint32_t wt = word_ring + wstage * C::WORD_TILE_BYTES + r * 16;
                        wn = ptx::ld_shared_v4(wt);
                        if (TERNARY) wp = ptx::ld_shared_v4(wt + BN * 16);
                    }
                    // The slot may be refilled by TMA as soon as this arrive lands, so the loads above
                    // must have returned their data first: the arrive is made to depend on them.
                    ptx::mbar_arrive_after(bar_empty_w + 8 * wstage, wn.x ^ wn.w ^ wp.x ^ wp.w);
                    if (++wstage == kWordStages) {
                        wstage = 0;
                        wphase ^= 1u;
                    }
                }
                if (!ptx::mbar_wait(bar_empty + 8 * stage, phase ^ 1u, p.err_word, kErrWaitEmpty)) {
                    ok = false;
                    break;
                }
                if (r < BN) {
                    uint8_t* row = base_ptr + stage * C::STAGE_BYTES + r * 128;
                    const uint32_t nw[2] = {(kb & 1) ? wn.z : wn.x, (kb & 1) ? wn.w : wn.y};
                    const uint32_t pw[2] = {(kb & 1) ? wp.z : wp.x, (kb & 1) ? wp.w : wp.y};
#pragma unroll
                    for (int c = 0; c < 8; ++c) {
                        const uint32_t nb = (nw[c >> 2] >> (8 * (c & 3))) & 0xffu;
                        const uint32_t pb = (pw[c >> 2] >> (8 * (c & 3))) & 0xffu;
                        // 16-byte chunk c of row r lands at chunk (c ^ (r & 7)): the 128-byte swizzle.
                        *reinterpret_cast<uint4*>(row + ((c ^ (r & 7)) << 4)) = unpack8<TERNARY>(nb, pb);
                    }
                }
                ptx::fence_proxy_async_smem();
                ptx::mbar_arrive(bar_full_b + 8 * stage);
                if (++stage == C::STAGES) {
                    stage = 0;
                    phase ^= 1u;
                }
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue
        const int e = threadIdx.x - (64 + kTransformThreads);
        const int quarter = warp & 3;  // TMEM lane quarter this warp may read
        float4* scratch = p.scratch + static_cast<int64_t>(blockIdx.x) * (BN / 4) * kEpilogueThreads + e;
        int iter = 0;
        int tile_iter = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, ++tile_iter) {
            int tm, tn;
            tile_coords(t, p.tiles_m, p.tiles_n, tm, tn);
            const int sbuf = tile_iter & 1;
            const int64_t n0 = static_cast<int64_t>(tn) * BN;
            for (int j = e; j < BN; j += kEpilogueThreads) {
                const int64_t n = n0 + j;
                alpha_s[sbuf * BN + j] = (p.ep.alpha && n < p.N) ? __ldg(p.ep.alpha + n) : 1.0f;
                bias_s[sbuf * BN + j] = (p.ep.bias && n < p.N) ? __ldg(p.ep.bias + n) : 0.0f;
            }
            ptx::named_barrier_sync(1, kEpilogueThreads);
            const int64_t m = static_cast<int64_t>(tm) * BM + quarter * 32 + lane;
            float* c_row = p.c + m * p.ldc;
            for (int seg = 0; seg < p.num_seg && ok; ++seg, ++iter) {
                const int buf = iter & 1;
                if (!ptx::mbar_wait(bar_tmem_full + 8 * buf, static_cast<uint32_t>((iter >> 1) & 1), p.err_word,
                                    kErrWaitTmemFull)) {
                    ok = false;
                    break;
                }
                ptx::tc_fence_after_sync();
                const bool first = seg == 0, last = seg == p.num_seg - 1;
#pragma unroll 1
                for (int c = 0; c < BN / 32; ++c) {
                    uint32_t r[32];
                    ptx::tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                                           static_cast<uint32_t>(buf * BN + c * 32), r);
                    ptx::tmem_ld_wait();
                    float v[32];
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
                    if (!first) {
                        // Add the earlier segments (fp32, round to nearest).  Slot layout
                        // [column group][thread] keeps each warp access contiguous.
#pragma unroll
                        for (int j4 = 0; j4 < 8; ++j4) {
                            const float4 s4 = __ldcg(scratch + (c * 8 + j4) * kEpilogueThreads);
                            v[4 * j4 + 0] = __fadd_rn(v[4 * j4 + 0], s4.x);
                            v[4 * j4 + 1] = __fadd_rn(v[4 * j4 + 1], s4.y);
                            v[4 * j4 + 2] = __fadd_rn(v[4 * j4 + 2], s4.z);
                            v[4 * j4 + 3] = __fadd_rn(v[4 * j4 + 3], s4.w);
                        }
                    }
                    if (!last) {
#pragma unroll
                        for (int j4 = 0; j4 < 8; ++j4)
                            __stcg(scratch + (c * 8 + j4) * kEpilogueThreads,
                                   make_float4(v[4 * j4], v[4 * j4 + 1], v[4 * j4 + 2], v[4 * j4 + 3]));
                    } else if (m < p.M) {
                        const int64_t nc = n0 + c * 32;
                        const float* as = alpha_s + sbuf * BN + c * 32;
                        const float* bs = bias_s + sbuf * BN + c * 32;
                        if (p.c_vec_ok && nc + 32 <= p.N) {
#pragma unroll
                            for (int j = 0; j < 32; j += 4) {
                                float4 o;
                                o.x = apply_epilogue(v[j + 0], as[j + 0], bs[j + 0], p.ep.scale, p.ep.flags);
                                o.y = apply_epilogue(v[j + 1], as[j + 1], bs[j + 1], p.ep.scale, p.ep.flags);
                                o.z = apply_epilogue(v[j + 2], as[j + 2], bs[j + 2], p.ep.scale, p.ep.flags);
                                o.w = apply_epilogue(v[j + 3], as[j + 3], bs[j + 3], p.ep.scale, p.ep.flags);
                                *reinterpret_cast<float4*>(c_row + nc + j) = o;
                            }
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; ++j) {
                                if (nc + j < p.N)
                                    c_row[nc + j] = apply_epilogue(v[j], as[j], bs[j], p.ep.scale, p.ep.flags);
                            }
                        }
                    }
                }
                ptx::tc_fence_before_sync();
                ptx::mbar_arrive(bar_tmem_empty + 8 * buf);
            }
        }
    }

    // ------------------------------------------------------------ teardown
    __syncwarp();
    ptx::tc_fence_before_sync();
    __syncthreads();
    if (warp == kMmaWarp) {
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc(tmem_base, C::TMEM_COLS);
    }
}

}  // namespace tc

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
            if (m < M) c[static_cast<int64_t>(m) * ldc + n] = apply_epilogue(acc[r], al, bi, ep.scale, ep.flags);
        }
    }
}

// =====================================================================================
// Host side
// =====================================================================================

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = [] {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess) {
            cudaGetLastError();
            sym = nullptr;
        }
        return reinterpret_cast<EncodeTiledFn>(sym);
    }();
    return fn;
}

int npass_of(int mode) {
    switch (mode) {
        case TBN_MODE_TC_BF16X1: return 1;
        case TBN_MODE_TC_BF16X2: return 2;
        case TBN_MODE_TC_BF16X3: return 3;
        default: return 0;
    }
}

int pick_bn(int64_t N) {
    // Largest tile whose padding waste stays within ~12 % of the best candidate.
    const int cand[3] = {256, 128, 64};
    int64_t best = INT64_MAX;
    for (int bn : cand) best = std::min<int64_t>(best, round_up(N, bn));
    for (int bn : cand)
        if (round_up(N, bn) * 8 <= best * 9) return bn;
    return 64;
}

// Per-CTA partial-sum tiles of the segmented accumulation: one 128 x 256 fp32 tile per SM.
size_t scratch_bytes() { return static_cast<size_t>(std::max(sm_count(), 1)) * tc::BM * 256 * sizeof(float); }

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

struct TensorMaps {
    CUtensorMap a, neg, pos;
};

// Packed-word plane [N_pad][KW] uint32 -> box of 4 words (128 k) x BN columns, no swizzle.
int32_t make_word_map(EncodeTiledFn encode, const uint32_t* words, int64_t KW, int64_t N_pad, int bn, CUtensorMap* out) {
    const cuuint64_t gdim[2] = {static_cast<cuuint64_t>(KW), static_cast<cuuint64_t>(N_pad)};
    const cuuint64_t gstride[1] = {static_cast<cuuint64_t>(KW) * 4};
    const cuuint32_t box[2] = {4, static_cast<cuuint32_t>(bn)};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult cr = encode(out, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<uint32_t*>(words), gdim, gstride, box,
                               estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                               CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    TBN_REQUIRE(cr == CUDA_SUCCESS, TBN_CUDA_ERROR,
                "cuTensorMapEncodeTiled (packed words) failed with CUresult " + std::to_string(static_cast<int>(cr)));
    return TBN_SUCCESS;
}

template <int BN, int NPASS, bool TERNARY>
int32_t launch_tc(const TensorMaps& maps, const tc::Params& p, cudaStream_t st) {
    using C = tc::Cfg<BN, NPASS, TERNARY>;
    auto kernel = tc::gemm_tc_kernel<BN, NPASS, TERNARY>;
    TBN_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES));
    const int total = p.tiles_m * p.tiles_n;
    const int grid = std::max(1, std::min(total, sm_count()));
    profile_begin(kProfGemm, st);
    kernel<<<grid, tc::kThreads, C::SMEM_BYTES, st>>>(maps.a, maps.neg, maps.pos, p);
    profile_end(kProfGemm, st);
    return launched("gemm_tc_kernel");
}

template <int NPASS, bool TERNARY>
int32_t dispatch_bn(int bn, const TensorMaps& maps, const tc::Params& p, cudaStream_t st) {
    switch (bn) {
        case 256: return launch_tc<256, NPASS, TERNARY>(maps, p, st);
        case 128: return launch_tc<128, NPASS, TERNARY>(maps, p, st);
        default: return launch_tc<64, NPASS, TERNARY>(maps, p, st);
    }
}

// Tensor-core path: split (or ternarise) A into the workspace, then the tcgen05 kernel.
int32_t gemm_tensor_core(const float* d_a, int64_t M, int64_t K, int64_t lda, bool ternarise_act, float act_lo,
                         float act_hi, int npass, const uint32_t* d_neg, const uint32_t* d_pos, int64_t N,
                         const Epilogue& ep, float* d_c, int64_t ldc, void* d_ws, size_t ws_bytes, cudaStream_t st) {
    const int64_t M_pad = round_up(M, tc::BM), K_pad = round_up(K, 128), N_pad = round_up(N, 8);
    const size_t split_bytes = static_cast<size_t>(npass) * M_pad * K_pad * sizeof(__nv_bfloat16);
    const size_t need = split_bytes + scratch_bytes();
    TBN_REQUIRE(d_ws && ws_bytes >= need, TBN_INVALID_ARGUMENT,
                "gemm: workspace too small (see tbn_gemm_workspace_bytes)");
    TBN_REQUIRE(reinterpret_cast<uintptr_t>(d_ws) % 128 == 0, TBN_INVALID_ARGUMENT,
                "gemm: workspace must be 128-byte aligned");
    TBN_REQUIRE(M_pad / tc::BM <= 0x7fffff && (M_pad / tc::BM) * ((N + 63) / 64) <= 0x7fffffffLL, TBN_INVALID_SHAPE,
                "gemm: too many tiles");
    EncodeTiledFn encode = encode_tiled_fn();
    TBN_REQUIRE(encode != nullptr, TBN_CUDA_ERROR, "cuTensorMapEncodeTiled is not available from the driver");
    __nv_bfloat16* split = static_cast<__nv_bfloat16*>(d_ws);

    int32_t rc;
    if (ternarise_act) rc = launch_split<1, true>(d_a, M, K, lda, M_pad, K_pad, split, act_lo, act_hi, st);
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
    const CUresult cr = encode(&tmap, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, split, gdim, gstride, box, estr,
                               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    TBN_REQUIRE(cr == CUDA_SUCCESS, TBN_CUDA_ERROR,
                "cuTensorMapEncodeTiled failed with CUresult " + std::to_string(static_cast<int>(cr)));

    const int bn = pick_bn(N);
    TBN_REQUIRE(reinterpret_cast<uintptr_t>(d_neg) % 16 == 0 && (!d_pos || reinterpret_cast<uintptr_t>(d_pos) % 16 == 0),
                TBN_INVALID_ARGUMENT, "gemm: packed weight planes must be 16-byte aligned");
    rc = make_word_map(encode, d_neg, K_pad / 32, N_pad, bn, &maps.neg);
    if (rc) return rc;
    rc = make_word_map(encode, d_pos ? d_pos : d_neg, K_pad / 32, N_pad, bn, &maps.pos);
    if (rc) return rc;
    tc::Params p;
    p.neg = d_neg;
    p.pos = d_pos;
    p.KW = K_pad / 32;
    p.N_pad = N_pad;
    p.M = static_cast<int>(M);
    p.N = static_cast<int>(N);
    p.num_kb = static_cast<int>(K_pad / tc::BK);
    p.tiles_m = static_cast<int>(M_pad / tc::BM);
    p.tiles_n = static_cast<int>((N + bn - 1) / bn);
    p.c = d_c;
    p.ldc = ldc;
    p.ep = ep;
    p.err_word = device_error_word();
    p.c_vec_ok = (ldc % 4 == 0) && (reinterpret_cast<uintptr_t>(d_c) % 16 == 0);
    // Fresh accumulator every kMaxAccumSteps accumulation steps (see the header comment).
    const int max_kb = std::max(1, tc::kMaxAccumSteps / (npass * tc::BK));
    p.num_seg = (p.num_kb + max_kb - 1) / max_kb;
    p.kb_per_seg = (p.num_kb + p.num_seg - 1) / p.num_seg;
    p.scratch = reinterpret_cast<float4*>(static_cast<uint8_t*>(d_ws) + split_bytes);
    const bool ternary_w = d_pos != nullptr;
    if (npass == 1) return ternary_w ? dispatch_bn<1, true>(bn, maps, p, st) : dispatch_bn<1, false>(bn, maps, p, st);
    if (npass == 2) return ternary_w ? dispatch_bn<2, true>(bn, maps, p, st) : dispatch_bn<2, false>(bn, maps, p, st);
    return ternary_w ? dispatch_bn<3, true>(bn, maps, p, st) : dispatch_bn<3, false>(bn, maps, p, st);
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

// Problems this small finish sooner on the CUDA cores than the split + tensor pipeline sets up.
bool prefer_simt(int64_t M, int64_t N, int64_t K) { return M <= 8 || M * N * K <= (1LL << 21); }

}  // namespace
}  // namespace tbn_cuda

using namespace tbn_cuda;

extern "C" {

size_t tbn_gemm_workspace_bytes(int64_t M, int64_t K, int32_t mode) {
    if (M <= 0 || K <= 0) return 0;
    int np = npass_of(mode);
    if (mode == TBN_MODE_SIMT) return 0;
    if (np == 0) np = 2;  // AUTO resolves to at most the two-term split
    // Split activations + the per-SM partial-sum tiles (sized for the largest SM count in use).
    return static_cast<size_t>(np) * round_up(M, tc::BM) * round_up(K, 128) * sizeof(__nv_bfloat16) +
           static_cast<size_t>(std::max(sm_count(), 160)) * tc::BM * 256 * sizeof(float);
}

int32_t tbn_gemm_fxb(const float* d_a, int64_t M, int64_t K, int64_t lda, const uint32_t* d_neg,
                     const uint32_t* d_pos, int64_t N, const float* d_alpha, float scale, const float* d_bias,
                     float* d_c, int64_t ldc, int32_t mode, uint32_t epilogue, void* d_workspace,
                     size_t workspace_bytes, void* stream) {
    int32_t rc = check_gemm_args(d_a, M, K, lda, d_neg, N, d_c, ldc);
    if (rc) return rc;
    TBN_REQUIRE(mode >= TBN_MODE_AUTO && mode <= TBN_MODE_SIMT, TBN_INVALID_ARGUMENT, "tbn_gemm_fxb: unknown mode");
    const Epilogue ep{d_alpha, d_bias, scale, epilogue};
    if (mode == TBN_MODE_AUTO) mode = prefer_simt(M, N, K) ? TBN_MODE_SIMT : TBN_MODE_TC_BF16X2;
    if (mode == TBN_MODE_SIMT)
        return gemm_simt(d_a, M, K, lda, false, 0.f, 0.f, d_neg, d_pos, N, ep, d_c, ldc, as_stream(stream));
    return gemm_tensor_core(d_a, M, K, lda, false, 0.f, 0.f, npass_of(mode), d_neg, d_pos, N, ep, d_c, ldc, d_workspace,
                            workspace_bytes, as_stream(stream));
}

int32_t tbn_gemm_tbn(const float* d_a, int64_t M, int64_t K, int64_t lda, float lo, float hi, const uint32_t* d_neg,
                     int64_t N, const float* d_alpha, float scale, const float* d_bias, float* d_c, int64_t ldc,
                     uint32_t epilogue, void* d_workspace, size_t workspace_bytes, void* stream) {
    int32_t rc = check_gemm_args(d_a, M, K, lda, d_neg, N, d_c, ldc);
    if (rc) return rc;
    // Integer-exact on the tensor cores only while every partial sum fits fp32's 24-bit significand.
    TBN_REQUIRE(K < (1 << 24), TBN_INVALID_SHAPE, "tbn_gemm_tbn: K too large for exact accumulation");
    const Epilogue ep{d_alpha, d_bias, scale, epilogue};
    if (prefer_simt(M, N, K) || d_workspace == nullptr)
        return gemm_simt(d_a, M, K, lda, true, lo, hi, d_neg, nullptr, N, ep, d_c, ldc, as_stream(stream));
    return gemm_tensor_core(d_a, M, K, lda, true, lo, hi, 1, d_neg, nullptr, N, ep, d_c, ldc, d_workspace,
                            workspace_bytes, as_stream(stream));
}

}  // extern "C"
