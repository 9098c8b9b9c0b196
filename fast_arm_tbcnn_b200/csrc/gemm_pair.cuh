// The float x {binary, ternary} GEMM on CTA PAIRS: tcgen05.mma.cta_group::2, one 256 x 256 output tile per pair.
//
// Why: in the one-CTA kernel (gemm_tc.cuh) every SM unpacks and reads the whole 256-column weight tile; the operand
// reads of the MMAs, the build warps' stores and the TMA writes together come to about 120 bytes per cycle of shared
// memory, and the tensor pipe waits for operands a quarter of the time.  With a pair, the two CTAs of a cluster hold
// 128 activation rows each (their own m-tile) and HALF of the weight tile each (128 columns): one instruction issued
// by the leader CTA multiplies 256 x 256 x 16, the hardware reading A and B halves from both CTAs' shared memory at
// the same offsets and writing each CTA's 128 accumulator rows into its own tensor memory.  Per CTA and k-block that is
// half the unpacking and half the weight-operand traffic for the same arithmetic, and a fourth pipeline stage fits.
//
// Roles per CTA (448 threads, as in gemm_tc_kernel): warp 0 TMA producer (its own activation rows, its own 128 columns
// of packed words), warps 2-9 unpack words to +-1/0, warps 10-13 epilogue.  Warp 1: in the LEADER (cluster rank 0) it
// issues the MMAs; in the other CTA it only reports, per stage, that this CTA's operands are in place (a remote
// mbarrier arrive on the leader's `peer_ready` barrier).  Completion of the MMAs is signalled to BOTH CTAs with
// tcgen05.commit ... multicast::cluster (shared-memory stage free; accumulator ready); the peer's epilogue threads
// release an accumulator with remote arrives on the leader's barrier.  No TMA load carries a multicast qualifier.
// Every mbarrier wait is bounded as everywhere in this library; both CTAs always reach the closing cluster barrier.
//
// Measured on B200 (74 resident pairs, four stages): bit-identical to the one-CTA kernel on every test shape, and
// 7-20 % SLOWER (16384^3: 13.1 ms against 12.2 ms; 8192^3: 1.69 against 1.39-1.47 ms).  With one, two or three
// activation terms the pair's time per k-block is 1690 / 1890 / 2290 cycles against 1270 / 1500 / 2150 for one CTA: a
// fixed cost per k-block that the MMAs do not explain -- the cross-CTA chain (commit to both CTAs, refill, the other
// CTA's report, the leader's cluster-scope wait) is longer than four stages hide.  The per-shape plan therefore never
// selects it by itself (kernel code 2 in tbn_gemm_plan_override and in the tuner's sweep); it stays as the measured
// alternative the winner is chosen against.
#pragma once

#include "gemm_tc.cuh"

namespace tbn_cuda {
namespace {
namespace pair {

constexpr int BN = 256;            // columns of the pair's tile
constexpr int BH = 128;            // columns unpacked and held by each CTA
constexpr int kThreads = tc::kThreads;
constexpr int kBuildThreads = tc::kBuildThreads, kEpilogueThreads = tc::kEpilogueThreads;
constexpr int kWordStages = 2;
constexpr int kMaxStages = 6;

template <int NPASS, bool TERNARY>
struct Cfg {
    static constexpr int B_BYTES = BH * tc::BK * 2;                       // 16 KB: this CTA's half of the weight tile
    static constexpr int STAGE_BYTES = B_BYTES + NPASS * tc::A_TILE_BYTES;
    static constexpr int WORD_TILE_BYTES = BH * 16 * (TERNARY ? 2 : 1);
    static constexpr int AUX_BYTES = 1024 + 4 * BN * 4 + kWordStages * WORD_TILE_BYTES;
    static constexpr int RAW_STAGES = (tc::kSmemLimit - 1024 - AUX_BYTES) / STAGE_BYTES;
    static constexpr int STAGES = RAW_STAGES > kMaxStages ? kMaxStages : RAW_STAGES;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + AUX_BYTES + 1024;
    static constexpr int TMEM_COLS = 2 * BN;
    static_assert(STAGES >= 2, "need at least a double-buffered pipeline");
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Address of the same shared-memory location in another CTA of the cluster.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local_addr, uint32_t cta) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(cta));
    return r;
}
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster_scope(uint32_t bar) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait on a barrier that the other CTA of the pair arrives on.
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity, int* err_word, int code) {
    if (mbar_try_wait_cluster(bar, parity)) return true;
    uint64_t t0 = 0;
    uint32_t spins = 0;
    while (!mbar_try_wait_cluster(bar, parity)) {
        if ((++spins & 0x3ffu) == 0) {
            if (*reinterpret_cast<volatile int*>(err_word) != 0) return false;
            const uint64_t limit = *reinterpret_cast<volatile uint64_t*>(err_word + ptx::kWaitLimitWordOffset);
            const uint64_t now = ptx::globaltimer_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > limit) {
                atomicCAS(err_word, 0, code);
                return false;
            }
        }
    }
    return true;
}
__device__ __forceinline__ void tmem_alloc2(uint32_t dst_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish2() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// D[tmem of both CTAs] (+)= A[256 rows: 128 per CTA] * B[256 columns: 128 per CTA]; issued by ONE thread of the leader.
__device__ __forceinline__ void umma2(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Arrive on the barrier at this offset in BOTH CTAs once all MMAs issued so far have completed.
__device__ __forceinline__ void umma_commit_both(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
                 "h"(static_cast<uint16_t>(3))
                 : "memory");
}

// Params: tc::Params with tiles_m = number of 256-row pair tiles.  tmap_a: split activations [terms][M_pad][K_pad], box
// 64 x 128; tmap_neg / tmap_pos: packed word planes, box 4 words x 128 columns.
template <int NPASS, bool TERNARY>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
    gemm_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_neg,
                     const __grid_constant__ CUtensorMap tmap_pos, const tc::Params p) {
    using C = Cfg<NPASS, TERNARY>;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = ptx::smem_u32(smem_raw);
    const uint32_t base = (raw_addr + 1023u) & ~1023u;
    uint8_t* base_ptr = smem_raw + (base - raw_addr);
    const uint32_t aux = base + C::STAGES * C::STAGE_BYTES;
    const uint32_t bar_full_a = aux;                        // TMA: this CTA's activation tiles
    const uint32_t bar_full_b = aux + 8 * kMaxStages;       // build warps: this CTA's half of the weight tile
    const uint32_t bar_empty = aux + 16 * kMaxStages;       // MMAs of the stage retired (signalled in both CTAs)
    const uint32_t bar_peer_ready = aux + 24 * kMaxStages;  // leader only: the other CTA's operands are in place
    const uint32_t bar_tmem_full = aux + 32 * kMaxStages;   // 2 x 8 B, signalled in both CTAs
    const uint32_t bar_tmem_empty = bar_tmem_full + 16;     // 2 x 8 B, leader only: both CTAs' epilogues have drained
    const uint32_t bar_full_w = bar_tmem_empty + 16;
    const uint32_t bar_empty_w = bar_full_w + 8 * kWordStages;
    const uint32_t tmem_slot = bar_empty_w + 8 * kWordStages;
    uint8_t* aux_ptr = base_ptr + C::STAGES * C::STAGE_BYTES;
    volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(aux_ptr + (tmem_slot - aux));
    float* alpha_s = reinterpret_cast<float*>(aux_ptr + 1024);  // [2][BN]
    float* bias_s = alpha_s + 2 * BN;                           // [2][BN]
    const uint32_t word_ring = aux + 1024 + 4 * BN * 4;         // [kWordStages][planes][BH][4 words]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const bool leader = rank == 0;
    const int pair_id = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
    const int total_tiles = p.tiles_m * p.tiles_n;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kMaxStages; ++s) {
            ptx::mbar_init(bar_full_a + 8 * s, 1);
            ptx::mbar_init(bar_full_b + 8 * s, kBuildThreads);
            ptx::mbar_init(bar_empty + 8 * s, 1);
            ptx::mbar_init(bar_peer_ready + 8 * s, 1);
        }
        for (int b = 0; b < 2; ++b) {
            ptx::mbar_init(bar_tmem_full + 8 * b, 1);
            ptx::mbar_init(bar_tmem_empty + 8 * b, 2 * kEpilogueThreads);
        }
        for (int w = 0; w < kWordStages; ++w) {
            ptx::mbar_init(bar_full_w + 8 * w, 1);
            ptx::mbar_init(bar_empty_w + 8 * w, kBuildThreads);
        }
        ptx::fence_barrier_init();
        ptx::prefetch_tensormap(&tmap_a);
        ptx::prefetch_tensormap(&tmap_neg);
        if (TERNARY) ptx::prefetch_tensormap(&tmap_pos);
    }
    if (warp == tc::kMmaWarp) {
        tmem_alloc2(tmem_slot, C::TMEM_COLS);
        tmem_relinquish2();
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();   // both CTAs' barriers are initialised before anyone signals across the pair
    ptx::tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot_ptr;

    if (warp == tc::kProducerWarp) {
        // ------------------------------------------------------------ TMA producer (own rows, own columns)
        if (lane == 0) {
            int stage = 0, wstage = 0;
            uint32_t phase = 0, wphase = 0;
            bool ok = true;
            for (int t = pair_id; t < total_tiles && ok; t += num_pairs) {
                int tm, tn;
                tc::tile_coords(t, p.tiles_m, p.tiles_n, p.group_m, tm, tn);
                const int row0 = (tm * 2 + static_cast<int>(rank)) * tc::BM;
                const int col0 = tn * BN + static_cast<int>(rank) * BH;
                for (int kb = 0; kb < p.num_kb; ++kb) {
                    if ((kb & 1) == 0) {
                        if (!ptx::mbar_wait(bar_empty_w + 8 * wstage, wphase ^ 1u, p.err_word, kErrWaitEmpty)) {
                            ok = false;
                            break;
                        }
                        const uint32_t wbar = bar_full_w + 8 * wstage;
                        const uint32_t wdst = word_ring + wstage * C::WORD_TILE_BYTES;
                        ptx::mbar_arrive_expect_tx(wbar, C::WORD_TILE_BYTES);
                        ptx::tma_load_2d(wdst, &tmap_neg, kb * 2, col0, wbar);
                        if (TERNARY) ptx::tma_load_2d(wdst + BH * 16, &tmap_pos, kb * 2, col0, wbar);
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
                    ptx::mbar_arrive_expect_tx(bar, NPASS * tc::A_TILE_BYTES);
                    const uint32_t a_dst = base + stage * C::STAGE_BYTES + C::B_BYTES;
#pragma unroll
                    for (int q = 0; q < NPASS; ++q) ptx::tma_load_3d(a_dst + q * tc::A_TILE_BYTES, &tmap_a, kb * tc::BK, row0, q, bar);
                    if (++stage == C::STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
        }
    } else if (warp == tc::kMmaWarp) {
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            if (leader) {
                // ------------------------------------------------------------ MMA issuer (leader CTA)
                const uint32_t idesc = p.f16 ? ptx::umma_idesc_f16_f32(2 * tc::BM, BN) : ptx::umma_idesc_bf16_f32(2 * tc::BM, BN);
                int iter = 0;
                for (int t = pair_id; t < total_tiles && ok; t += num_pairs) {
                    for (int seg = 0; seg < p.num_seg && ok; ++seg, ++iter) {
                        const int buf = iter & 1;
                        if (!mbar_wait_cluster(bar_tmem_empty + 8 * buf, static_cast<uint32_t>((iter >> 1) & 1) ^ 1u, p.err_word,
                                               kErrWaitTmemEmpty)) {
                            ok = false;
                            break;
                        }
                        ptx::tc_fence_after_sync();
                        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(buf * BN);
                        const int kb_begin = seg * p.kb_per_seg;
                        const int kb_end = min(p.num_kb, kb_begin + p.kb_per_seg);
                        for (int kb = kb_begin; kb < kb_end; ++kb) {
                            if (!ptx::mbar_wait(bar_full_a + 8 * stage, phase, p.err_word, kErrWaitFullA) ||
                                !ptx::mbar_wait(bar_full_b + 8 * stage, phase, p.err_word, kErrWaitFullB) ||
                                !mbar_wait_cluster(bar_peer_ready + 8 * stage, phase, p.err_word, kErrWaitFullB)) {
                                ok = false;
                                break;
                            }
                            ptx::tc_fence_after_sync();
                            const uint32_t b_addr = base + stage * C::STAGE_BYTES;
                            const uint32_t a_addr = b_addr + C::B_BYTES;
#pragma unroll
                            for (int q = 0; q < NPASS; ++q) {
#pragma unroll
                                for (int k4 = 0; k4 < tc::BK / tc::UMMA_K; ++k4) {
                                    const uint64_t a_desc = ptx::umma_desc_k_sw128(a_addr + q * tc::A_TILE_BYTES + k4 * tc::UMMA_K * 2);
                                    const uint64_t b_desc = ptx::umma_desc_k_sw128(b_addr + k4 * tc::UMMA_K * 2);
                                    umma2(d_tmem, a_desc, b_desc, idesc, (kb != kb_begin || q != 0 || k4 != 0) ? 1u : 0u);
                                }
                            }
                            umma_commit_both(bar_empty + 8 * stage);
                            if (++stage == C::STAGES) {
                                stage = 0;
                                phase ^= 1u;
                            }
                        }
                        if (ok) umma_commit_both(bar_tmem_full + 8 * buf);
                    }
                }
            } else {
                // ------------------------------------------------------------ the other CTA: report its operands, stage by stage
                const uint32_t remote_ready = map_to_cta(bar_peer_ready, 0);
                for (int t = pair_id; t < total_tiles && ok; t += num_pairs) {
                    for (int kb = 0; kb < p.num_kb; ++kb) {
                        if (!ptx::mbar_wait(bar_full_a + 8 * stage, phase, p.err_word, kErrWaitFullA) ||
                            !ptx::mbar_wait(bar_full_b + 8 * stage, phase, p.err_word, kErrWaitFullB)) {
                            ok = false;
                            break;
                        }
                        mbar_arrive_remote(remote_ready + 8 * stage);
                        if (++stage == C::STAGES) {
                            stage = 0;
                            phase ^= 1u;
                        }
                    }
                }
            }
        }
    } else if (warp < 2 + kBuildThreads / 32) {
        // ------------------------------------------------------------ operand build: this CTA's 128 columns
        const int r = threadIdx.x - 64;
        const int col = r & (BH - 1);  // weight column (row of the K-major tile)
        const int half = r >> 7;       // which 32 of the k-block's 64 k this thread unpacks (one packed word)
        const uint32_t one16 = p.f16 ? kOneF16 : kOneBf16;
        int stage = 0, wstage = 0;
        uint32_t phase = 0, wphase = 0;
        bool ok = true;
        uint32_t wn0 = 0u, wn1 = 0u, wp0 = 0u, wp1 = 0u;  // this thread's word of the even and of the odd k-block
        for (int t = pair_id; t < total_tiles && ok; t += num_pairs) {
            for (int kb = 0; kb < p.num_kb; ++kb) {
                if ((kb & 1) == 0) {
                    if (!ptx::mbar_wait(bar_full_w + 8 * wstage, wphase, p.err_word, kErrWaitFullB)) {
                        ok = false;
                        break;
                    }
                    const uint32_t wt = word_ring + wstage * C::WORD_TILE_BYTES + col * 16 + half * 4;
                    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(wn0) : "r"(wt) : "memory");
                    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(wn1) : "r"(wt + 8) : "memory");
                    if (TERNARY) {
                        asm volatile("ld.shared.u32 %0, [%1];" : "=r"(wp0) : "r"(wt + BH * 16) : "memory");
                        asm volatile("ld.shared.u32 %0, [%1];" : "=r"(wp1) : "r"(wt + BH * 16 + 8) : "memory");
                    }
                    ptx::mbar_arrive_after(bar_empty_w + 8 * wstage, wn0 ^ wn1 ^ wp0 ^ wp1);
                    if (++wstage == kWordStages) {
                        wstage = 0;
                        wphase ^= 1u;
                    }
                }
                if (!ptx::mbar_wait(bar_empty + 8 * stage, phase ^ 1u, p.err_word, kErrWaitEmpty)) {
                    ok = false;
                    break;
                }
                uint8_t* row = base_ptr + stage * C::STAGE_BYTES + col * 128;
                const uint32_t nw = (kb & 1) ? wn1 : wn0, pw = (kb & 1) ? wp1 : wp0;
#pragma unroll
                for (int c4 = 0; c4 < 4; ++c4) {
                    const int c = half * 4 + c4;  // 16-byte chunk of the row: k [8c, 8c + 8)
                    const uint32_t nb = (nw >> (8 * c4)) & 0xffu, pb = (pw >> (8 * c4)) & 0xffu;
                    *reinterpret_cast<uint4*>(row + ((c ^ (col & 7)) << 4)) = unpack8<TERNARY>(nb, pb, one16);
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
        // ------------------------------------------------------------ epilogue: this CTA's 128 rows x 256 columns
        const int e = threadIdx.x - (64 + kBuildThreads);
        const int quarter = warp & 3;
        float4* scratch = p.scratch + static_cast<int64_t>(blockIdx.x) * (BN / 4) * kEpilogueThreads + quarter * 32 + lane;
        const uint32_t empty_local = bar_tmem_empty;
        const uint32_t empty_remote = leader ? 0u : map_to_cta(bar_tmem_empty, 0);
        const float ep_scale = p.amax_bits ? __fmul_rn(p.ep.scale, f16_scale_inv(__ldg(p.amax_bits))) : p.ep.scale;
        int iter = 0, tile_iter = 0;
        bool ok = true;
        for (int t = pair_id; t < total_tiles && ok; t += num_pairs, ++tile_iter) {
            int tm, tn;
            tc::tile_coords(t, p.tiles_m, p.tiles_n, p.group_m, tm, tn);
            const int sbuf = tile_iter & 1;
            const int64_t n0 = static_cast<int64_t>(tn) * BN;
            for (int j = e; j < BN; j += kEpilogueThreads) {
                const int64_t n = n0 + j;
                alpha_s[sbuf * BN + j] = (p.ep.alpha && n < p.N) ? __ldg(p.ep.alpha + n) : 1.0f;
                bias_s[sbuf * BN + j] = (p.ep.bias && n < p.N) ? __ldg(p.ep.bias + n) : 0.0f;
            }
            ptx::named_barrier_sync(1, kEpilogueThreads);
            const int64_t m = (static_cast<int64_t>(tm) * 2 + rank) * tc::BM + quarter * 32 + lane;
            const bool row_ok = m < p.M;
            float* c_row = p.c + m * p.ldc;
            for (int seg = 0; seg < p.num_seg && ok; ++seg, ++iter) {
                const int buf = iter & 1;
                if (!ptx::mbar_wait(bar_tmem_full + 8 * buf, static_cast<uint32_t>((iter >> 1) & 1), p.err_word, kErrWaitTmemFull)) {
                    ok = false;
                    break;
                }
                ptx::tc_fence_after_sync();
                const bool first = seg == 0, last = seg == p.num_seg - 1;
#pragma unroll 1
                for (int c = 0; c < BN / 32; ++c) {
                    if (n0 + c * 32 >= p.N) break;
                    uint32_t r[32];
                    ptx::tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(buf * BN + c * 32), r);
                    ptx::tmem_ld_wait();
                    float v[32];
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
                    if (!first) {
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
                            __stcg(scratch + (c * 8 + j4) * kEpilogueThreads, make_float4(v[4 * j4], v[4 * j4 + 1], v[4 * j4 + 2], v[4 * j4 + 3]));
                    } else if (row_ok) {
                        const int64_t nc = n0 + c * 32;
                        const float* as = alpha_s + sbuf * BN + c * 32;
                        const float* bs = bias_s + sbuf * BN + c * 32;
                        if (p.c_vec_ok && nc + 32 <= p.N) {
#pragma unroll
                            for (int j = 0; j < 32; j += 4) {
                                float4 o;
                                o.x = apply_epilogue(v[j + 0], as[j + 0], bs[j + 0], ep_scale, p.ep.flags, 0.0f);
                                o.y = apply_epilogue(v[j + 1], as[j + 1], bs[j + 1], ep_scale, p.ep.flags, 0.0f);
                                o.z = apply_epilogue(v[j + 2], as[j + 2], bs[j + 2], ep_scale, p.ep.flags, 0.0f);
                                o.w = apply_epilogue(v[j + 3], as[j + 3], bs[j + 3], ep_scale, p.ep.flags, 0.0f);
                                *reinterpret_cast<float4*>(c_row + nc + j) = o;
                            }
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; ++j)
                                if (nc + j < p.N) c_row[nc + j] = apply_epilogue(v[j], as[j], bs[j], ep_scale, p.ep.flags, 0.0f);
                        }
                    }
                }
                ptx::tc_fence_before_sync();
                if (leader) mbar_arrive_cluster_scope(empty_local + 8 * buf);
                else mbar_arrive_remote(empty_remote + 8 * buf);
            }
        }
    }

    // ------------------------------------------------------------ teardown: nobody leaves while the pair may still signal it
    ptx::tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();
    if (warp == tc::kMmaWarp) {
        ptx::tc_fence_after_sync();
        tmem_dealloc2(tmem_base, C::TMEM_COLS);
    }
}

// Number of CTAs to launch: two per cluster that can be resident at once (a cluster needs two free SMs of one GPC).
template <int NPASS, bool TERNARY>
int32_t launch(const TensorMaps& maps, const tc::Params& p, cudaStream_t st) {
    using C = Cfg<NPASS, TERNARY>;
    auto kernel = gemm_pair_kernel<NPASS, TERNARY>;
    TBN_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES));
    static int max_clusters = 0;  // per instantiation; the same on every B200 of a box
    if (max_clusters == 0) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(static_cast<unsigned>(std::max(sm_count(), 2) / 2 * 2));
        cfg.blockDim = dim3(kThreads);
        cfg.dynamicSmemBytes = C::SMEM_BYTES;
        cudaLaunchAttribute attr;
        attr.id = cudaLaunchAttributeClusterDimension;
        attr.val.clusterDim.x = 2;
        attr.val.clusterDim.y = 1;
        attr.val.clusterDim.z = 1;
        cfg.attrs = &attr;
        cfg.numAttrs = 1;
        int n = 0;
        TBN_CUDA_TRY(cudaOccupancyMaxActiveClusters(&n, kernel, &cfg));
        TBN_REQUIRE(n >= 1, TBN_RUNTIME_ERROR, "gemm (CTA pairs): no cluster of two CTAs fits on this device");
        max_clusters = n;
    }
    const int total = p.tiles_m * p.tiles_n;
    const int pairs = std::max(1, std::min(total, max_clusters));
    tc::Params q = p;
    if (q.group_m < 1) q.group_m = tc::kDefaultGroupM;
    profile_begin(kProfGemm, st);
    kernel<<<2 * pairs, kThreads, C::SMEM_BYTES, st>>>(maps.a, maps.neg, maps.pos, q);
    profile_end(kProfGemm, st);
    return launched("gemm_pair_kernel");
}

}  // namespace pair
}  // namespace
}  // namespace tbn_cuda
