// Stride-1 convolutions with up to three filter columns, lowered onto tcgen05 with the filter taps of one filter
// row served from ONE shared-memory copy of the input rows ("row mode").
//
// Why: the patch-mode kernel (gemm_tc.cuh, AMODE 4) loads one activation box per filter tap and one weight tile
// per k-block.  Measured on B200, a TMA box arrives at about one 128-byte row per 3-4 cycles per SM, which for
// the 64- and 128-channel layers is 2-4 times longer than the MMAs on those operands take: the convolutions are
// bound by the number of 128-byte rows the TMA unit has to move, not by the tensor pipe, L2 or HBM.  Two changes
// cut the rows per FLOP:
//   * an m-tile is `pbh` output rows of one image, each padded to `pitch` = ceil8(OW + kw - 1) GEMM rows; the
//     activation box of filter row ti and 64 channels is loaded once (`pitch` pixels x `pbh` rows, halo included,
//     zero-filled outside the image by the TMA unit) and the kw taps of that filter row are kw MMA operand windows
//     of that one copy, each shifted by one pixel = one 128-byte row (a shared-memory descriptor may start at any
//     128-byte row of a SWIZZLE_128B tile: the swizzle is a function of the address bits);  rows of the tile whose
//     pixel index within the pitch is >= OW compute garbage that is never stored;
//   * RESIDENT: when all filters fit (N <= BN and K_pad * BN * 2 bytes beside two activation stages), the expanded
//     +-1 filters are loaded into shared memory once per CTA and stay there for all its tiles.
//   * WIDE (BN = 64, three filter columns, resident filters): what a tcgen05.mma costs at these widths is mostly the
//     fetch of its operands (measured: about 100 cycles at N = 64 against 32 of arithmetic), and the three taps of a
//     filter row read the same activation rows.  So the three filter-column tiles of a filter row (kept one behind
//     the other in shared memory) are ONE operand of 192 rows, multiplied with the UNSHIFTED activation window:
//     E[r][tj] = A[r] . W[ti][tj] for all three tj at once, a third of the instructions, each fetching the
//     activations once instead of three times.  The shift moves into the epilogue: out[r] = E[r][0] + E[r+1][1] +
//     E[r+2][2], rows r+1 and r+2 coming from the neighbouring lanes by shuffle.  So that no row is ever needed from
//     another warp (a shared-memory exchange plus a barrier per chunk cost more than the instructions saved:
//     0.35 ms against 0.23 ms without it), the tile is laid out by TMEM lane quarters: each 32-row quarter is a box
//     of its own -- 32 consecutive input pixels of one image row, the first at output column 30 k - pad -- and
//     yields 30 output pixels; `qpr` = ceil(OW / 30) quarters cover an output row, 4 / qpr rows make a tile.
//     (64x56x56 -> 64 at batch 512: 0.23 ms against 0.38 ms with one instruction per tap.)
// Everything else follows gemm_tc_kernel: one persistent 448-thread CTA per SM, warp 0 issues TMA, warp 1 issues
// tcgen05.mma into a double-buffered TMEM accumulator, twelve warps drain it (alpha / bias / residual / ReLU, NCHW
// fp32 and / or channels-last bf16 terms).  One accumulation segment only (K x terms <= 4096); every wait is bounded.
#pragma once

#include "gemm_tc.cuh"

namespace tbn_cuda {
namespace {
namespace rows {

constexpr int kMaxTaps = 3;         // filter columns served from one activation box
constexpr int kMaxStages = 6;
constexpr int kThreads = 448;       // producer warp, MMA warp, twelve epilogue warps
constexpr int kEpiGroups = 3;       // epilogue warps work in groups of four (one warp per TMEM lane quarter) ...
constexpr int kGroupThreads = 128;  // ... and each group drains a whole tile of its own
constexpr int kAccBufs = 4;         // accumulators in tensor memory: MMAs run up to four tiles ahead of the drain

struct Params {
    int N;                 // output channels
    int C, cblocks;        // input channels, C / 64
    int kh, kw, dh;        // filter rows, filter columns (<= 3), row dilation
    int ph, pw;            // pads
    int H, W, OH, OW;
    int pitch, pbh;        // GEMM rows per output row (multiple of 8), output rows per tile (pitch * pbh <= 128)
    int qpr;               // WIDE: quarters (boxes of 32 pixels, 30 outputs each) per output row; pbh = 4 / qpr
    int tiles_per_image;   // ceil(OH / pbh)
    // stack != 0: the output rows of all `images` form one sequence s = img * OH + oh and a tile is pbh consecutive
    // rows of it, whatever images they come from (no half-empty last tile per image).  The rows from one image are
    // one TMA box; its height belongs to the tensor map: heights below the largest travel in RowMaps.  (WIDE tiles
    // are built from per-row boxes anyway and need no extra maps.)
    int stack, images, max_h;
    int tiles_m, tiles_n;  // images * tiles_per_image, ceil(N / BN)
    int a_box_bytes;       // bytes one activation box delivers, all terms together
    int nstages;           // pipeline depth (2 .. kMaxStages), chosen by the host from the shared memory left
    int n_btiles;          // RESIDENT: kh * kw * cblocks weight tiles of BN x 64
    int f16;               // operands are fp16 (one-pass mode), see gemm_tc.cuh
    const uint32_t* amax_bits;
    float* y;              // NCHW fp32 result or null
    __nv_bfloat16* y_cl;   // channels-last bf16 terms [2][pixel][N] or null
    int64_t y_cl_term_stride;
    Epilogue ep;
    int* err_word;
};

constexpr int kQuarterOutputs = 30;  // WIDE: output pixels of a 32-row quarter (rows 30 and 31 only feed the shifts)

struct RowMaps {
    CUtensorMap m[8];  // activation maps with box heights 1 .. 8 (stacked tiles)
};

template <int BN, int NPASS, bool RESIDENT, bool WIDE = false>
struct Cfg {
    static constexpr int B_TILE_BYTES = BN * tc::BK * 2;
    static constexpr int A_BYTES = NPASS * tc::A_TILE_BYTES;
    static constexpr int STAGE_BYTES = A_BYTES + (RESIDENT ? 0 : kMaxTaps * B_TILE_BYTES);
    static constexpr int AUX_BYTES = 1024 + 2 * kEpiGroups * BN * 4;  // barriers + alpha / bias staging per epilogue group
    static constexpr int ACC_COLS = WIDE ? kMaxTaps * BN : BN;  // columns of one accumulator
    static constexpr int ACC_BUFS = WIDE ? 2 : kAccBufs;
    static constexpr int TMEM_COLS = WIDE ? 512 : kAccBufs * BN;
    static_assert(BN == 64 || BN == 128, "row mode keeps the column tile at 64 or 128");
    static_assert(!WIDE || (BN == 64 && RESIDENT), "one instruction for three filter columns: 192 columns, resident filters");
    static_assert(ACC_BUFS * ACC_COLS <= TMEM_COLS, "accumulators must fit the allocation");
};

// Shared memory a launch needs: alignment slack + resident filters + stages + aux.
template <int BN, int NPASS, bool RESIDENT, bool WIDE = false>
inline int smem_bytes(int nstages, int n_btiles) {
    using C = Cfg<BN, NPASS, RESIDENT, WIDE>;
    return 1024 + (RESIDENT ? n_btiles * C::B_TILE_BYTES : 0) + nstages * C::STAGE_BYTES + C::AUX_BYTES;
}

template <int BN, int NPASS, bool RESIDENT, bool WIDE = false>
__global__ void __launch_bounds__(kThreads, 1) conv_rows_kernel(const __grid_constant__ CUtensorMap tmap_x,
                                                                const __grid_constant__ CUtensorMap tmap_w,
                                                                const __grid_constant__ RowMaps row_maps, const Params p) {
    using C = Cfg<BN, NPASS, RESIDENT, WIDE>;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = ptx::smem_u32(smem_raw);
    const uint32_t base = (raw_addr + 1023u) & ~1023u;
    uint8_t* base_ptr = smem_raw + (base - raw_addr);
    const uint32_t resident = base;                                                    // [n_btiles][BN][128 B]
    const uint32_t stages = base + (RESIDENT ? p.n_btiles * C::B_TILE_BYTES : 0);      // [nstages][STAGE_BYTES]
    const uint32_t aux = stages + p.nstages * C::STAGE_BYTES;
    const uint32_t bar_full = aux, bar_empty = aux + 8 * kMaxStages;
    const uint32_t bar_tmem_full = aux + 16 * kMaxStages, bar_tmem_empty = bar_tmem_full + 8 * kAccBufs;
    const uint32_t bar_resident = bar_tmem_empty + 8 * kAccBufs;
    const uint32_t tmem_slot = bar_resident + 8;
    uint8_t* aux_ptr = base_ptr + (aux - base);
    volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(aux_ptr + (tmem_slot - aux));
    float* alpha_s = reinterpret_cast<float*>(aux_ptr + 1024);  // [kEpiGroups][BN]
    float* bias_s = alpha_s + kEpiGroups * BN;                  // [kEpiGroups][BN]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int total_tiles = p.tiles_m * p.tiles_n;
    const int kb_per_tile = p.kh * p.cblocks;  // one pipeline stage per (filter row, 64-channel block)

    if (threadIdx.x == 0) {
        for (int s = 0; s < kMaxStages; ++s) {
            ptx::mbar_init(bar_full + 8 * s, 1);
            ptx::mbar_init(bar_empty + 8 * s, 1);
        }
        for (int b = 0; b < kAccBufs; ++b) {
            ptx::mbar_init(bar_tmem_full + 8 * b, 1);
            ptx::mbar_init(bar_tmem_empty + 8 * b, WIDE ? 2 * kGroupThreads : kGroupThreads);  // WIDE: one group per 32-column chunk
        }
        ptx::mbar_init(bar_resident, 1);
        ptx::fence_barrier_init();
        ptx::prefetch_tensormap(&tmap_x);
        ptx::prefetch_tensormap(&tmap_w);
    }
    if (warp == 1) {
        ptx::tmem_alloc(tmem_slot, C::TMEM_COLS);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot_ptr;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            if (RESIDENT) {
                // All filters of this CTA's column tile (tiles_n == 1: columns [0, BN)), once.
                ptx::mbar_arrive_expect_tx(bar_resident, static_cast<uint32_t>(p.n_btiles) * C::B_TILE_BYTES);
                for (int kt = 0; kt < p.n_btiles; ++kt) {
                    // k-block kt = (tap, channel block).  WIDE keeps the kw tiles of one filter row and channel block
                    // one behind the other: slot ((ti * cblocks + cb) * kw + tj).
                    int slot = kt;
                    if (WIDE) {
                        const int tap = kt / p.cblocks, cb = kt - tap * p.cblocks;
                        const int ti = tap / p.kw, tj = tap - ti * p.kw;
                        slot = (ti * p.cblocks + cb) * p.kw + tj;
                    }
                    ptx::tma_load_3d(resident + slot * C::B_TILE_BYTES, &tmap_w, kt * tc::BK, 0, 0, bar_resident);
                }
            }
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
                const int tm = t % p.tiles_m, tn = t / p.tiles_m;
                int img, oh0;  // first output row of the tile
                if (p.stack) {
                    img = (tm * p.pbh) / p.OH;
                    oh0 = tm * p.pbh - img * p.OH;
                } else {
                    img = tm / p.tiles_per_image;
                    oh0 = (tm - img * p.tiles_per_image) * p.pbh;
                }
                for (int ti = 0; ti < p.kh && ok; ++ti) {
                    for (int cb = 0; cb < p.cblocks; ++cb) {
                        if (!ptx::mbar_wait(bar_empty + 8 * stage, phase ^ 1u, p.err_word, kErrWaitEmpty)) {
                            ok = false;
                            break;
                        }
                        const uint32_t bar = bar_full + 8 * stage;
                        ptx::mbar_arrive_expect_tx(bar, static_cast<uint32_t>(p.a_box_bytes) +
                                                            (RESIDENT ? 0u : static_cast<uint32_t>(p.kw) * C::B_TILE_BYTES));
                        const uint32_t a_dst = stages + stage * C::STAGE_BYTES;
                        // Input pixels (x, y) = (-pw .. -pw + pitch - 1, oh0 - ph + ti*dh .. + pbh - 1), channels [64 cb, +64):
                        // tile row bh * pitch + bw holds pixel (bw - pw, oh0 + bh - ph + ti*dh); outside the image: zeros.
                        if constexpr (WIDE) {
                            // One box of 32 pixels per lane quarter: quarter qq holds output row oh0 + qq / qpr, output
                            // columns 30 (qq % qpr) .. + 29 (and the two pixels to their right for the shifted taps).
                            for (int qq = 0; qq < 4; ++qq) {
                                const int x = (qq % p.qpr) * kQuarterOutputs - p.pw;
                                int oh = oh0 + qq / p.qpr, im = img;
                                if (p.stack && oh >= p.OH) {  // the tile runs on into the next image(s)
                                    im += oh / p.OH;
                                    oh %= p.OH;
                                }
                                const int y = oh - p.ph + ti * p.dh;
#pragma unroll
                                for (int q = 0; q < NPASS; ++q)
                                    ptx::tma_load_5d(a_dst + q * tc::A_TILE_BYTES + qq * 32 * 128, &tmap_x, cb * tc::BK, x, y, im, q, bar);
                            }
                        } else if (p.stack) {
                            // One box per image the tile's rows come from (rows past the last image: zeros).
                            int im = img, oh = oh0, done = 0;
                            while (done < p.pbh) {
                                const int h = min(p.pbh - done, p.OH - oh);
                                const CUtensorMap* map = h == p.max_h ? &tmap_x : &row_maps.m[h - 1];
#pragma unroll
                                for (int q = 0; q < NPASS; ++q)
                                    ptx::tma_load_5d(a_dst + q * tc::A_TILE_BYTES + done * p.pitch * 128, map, cb * tc::BK, -p.pw,
                                                     oh - p.ph + ti * p.dh, im, q, bar);
                                done += h;
                                oh = 0;
                                ++im;
                            }
                        } else {
#pragma unroll
                            for (int q = 0; q < NPASS; ++q)
                                ptx::tma_load_5d(a_dst + q * tc::A_TILE_BYTES, &tmap_x, cb * tc::BK, -p.pw, oh0 - p.ph + ti * p.dh, img, q, bar);
                        }
                        if (!RESIDENT) {
                            const uint32_t b_dst = a_dst + C::A_BYTES;
                            for (int tj = 0; tj < p.kw; ++tj)
                                ptx::tma_load_3d(b_dst + tj * C::B_TILE_BYTES, &tmap_w, ((ti * p.kw + tj) * p.cblocks + cb) * tc::BK,
                                                 tn * BN, 0, bar);
                        }
                        if (++stage == p.nstages) {
                            stage = 0;
                            phase ^= 1u;
                        }
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            const uint32_t idesc = p.f16 ? ptx::umma_idesc_f16_f32(tc::BM, BN) : ptx::umma_idesc_bf16_f32(tc::BM, BN);
            int stage = 0, iter = 0;
            uint32_t phase = 0;
            bool ok = true;
            if (RESIDENT) ok = ptx::mbar_wait(bar_resident, 0, p.err_word, kErrWaitFullB);
            for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, ++iter) {
                const int buf = iter % C::ACC_BUFS;
                if (!ptx::mbar_wait(bar_tmem_empty + 8 * buf, static_cast<uint32_t>((iter / C::ACC_BUFS) & 1) ^ 1u, p.err_word,
                                    kErrWaitTmemEmpty)) {
                    ok = false;
                    break;
                }
                ptx::tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(buf * C::ACC_COLS);
                uint32_t accumulate = 0;
                for (int ti = 0; ti < p.kh && ok; ++ti) {
                    for (int cb = 0; cb < p.cblocks; ++cb) {
                        if (!ptx::mbar_wait(bar_full + 8 * stage, phase, p.err_word, kErrWaitFullA)) {
                            ok = false;
                            break;
                        }
                        ptx::tc_fence_after_sync();
                        const uint32_t a_addr = stages + stage * C::STAGE_BYTES;
                        if constexpr (WIDE) {
                            // All three filter columns of filter row ti at once: the unshifted window against 3 BN weight rows.
                            const uint32_t idesc_wide = p.f16 ? ptx::umma_idesc_f16_f32(tc::BM, kMaxTaps * BN)
                                                              : ptx::umma_idesc_bf16_f32(tc::BM, kMaxTaps * BN);
                            const uint32_t b_addr = resident + ((ti * p.cblocks + cb) * kMaxTaps) * C::B_TILE_BYTES;
#pragma unroll
                            for (int q = 0; q < NPASS; ++q) {
#pragma unroll
                                for (int k4 = 0; k4 < tc::BK / tc::UMMA_K; ++k4) {
                                    const uint64_t a_desc = ptx::umma_desc_k_sw128(a_addr + q * tc::A_TILE_BYTES + k4 * tc::UMMA_K * 2);
                                    const uint64_t b_desc = ptx::umma_desc_k_sw128(b_addr + k4 * tc::UMMA_K * 2);
                                    ptx::umma_bf16(d_tmem, a_desc, b_desc, idesc_wide, accumulate);
                                    accumulate = 1u;
                                }
                            }
                        }
                        for (int tj = 0; tj < (WIDE ? 0 : p.kw); ++tj) {
                            // Filter column tj: the same rows one pixel (one 128-byte row) further on.
                            const uint32_t b_addr = RESIDENT ? resident + ((ti * p.kw + tj) * p.cblocks + cb) * C::B_TILE_BYTES
                                                             : a_addr + C::A_BYTES + tj * C::B_TILE_BYTES;
#pragma unroll
                            for (int q = 0; q < NPASS; ++q) {
#pragma unroll
                                for (int k4 = 0; k4 < tc::BK / tc::UMMA_K; ++k4) {
                                    const uint64_t a_desc =
                                        ptx::umma_desc_k_sw128(a_addr + q * tc::A_TILE_BYTES + tj * 128 + k4 * tc::UMMA_K * 2);
                                    const uint64_t b_desc = ptx::umma_desc_k_sw128(b_addr + k4 * tc::UMMA_K * 2);
                                    ptx::umma_bf16(d_tmem, a_desc, b_desc, idesc, accumulate);
                                    accumulate = 1u;
                                }
                            }
                        }
                        ptx::umma_commit(bar_empty + 8 * stage);
                        if (++stage == p.nstages) {
                            stage = 0;
                            phase ^= 1u;
                        }
                    }
                }
                if (ok) ptx::umma_commit(bar_tmem_full + 8 * buf);
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue
        // Twelve warps in three groups of four (one warp per TMEM lane quarter).  Draining a tile is a chain of
        // latencies (accumulator ready -> tcgen05.ld -> arithmetic -> stores) of a few microseconds, longer than the
        // MMAs of a short-K tile take; so each group drains every third tile on its own and the chains of three
        // tiles overlap, with four accumulators in tensor memory between the MMA issuer and the groups.
        const int quarter = warp & 3;
        const int group = (warp - 2) >> 2;
        const int e = threadIdx.x - 64 - group * kGroupThreads;  // index inside the group, 0..127 (warps 2-5, 6-9, 10-13)
        float* as_g = alpha_s + group * BN;
        float* bs_g = bias_s + group * BN;
        int staged_tn = -1;
        const float ep_scale = p.amax_bits ? __fmul_rn(p.ep.scale, f16_scale_inv(__ldg(p.amax_bits))) : p.ep.scale;
        const int64_t hw = static_cast<int64_t>(p.OH) * p.OW;
        const bool add_res = (p.ep.flags & TBN_EPI_ADD_RESIDUAL) != 0;
        const bool bias_first = (p.ep.flags & TBN_EPI_BIAS_BEFORE_ALPHA) != 0;
        int iter = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, ++iter) {
            // A group drains every third tile -- or, WIDE, every third 32-column chunk: chunk (iter, c) is job 2 iter + c.
            if (!WIDE && iter % kEpiGroups != group) continue;
            const int tm = t % p.tiles_m, tn = t / p.tiles_m;
            const int buf = iter % C::ACC_BUFS;
            const int n0 = tn * BN;
            if (tn != staged_tn) {  // per-channel scale and bias of this column tile: reloaded only when it changes
                ptx::named_barrier_sync(1 + group, kGroupThreads);  // everyone has finished reading the old values
                for (int j = e; j < BN; j += kGroupThreads) {
                    const int n = n0 + j;
                    as_g[j] = (p.ep.alpha && n < p.N) ? __ldg(p.ep.alpha + n) : 1.0f;
                    bs_g[j] = (p.ep.bias && n < p.N) ? __ldg(p.ep.bias + n) : 0.0f;
                }
                ptx::named_barrier_sync(1 + group, kGroupThreads);
                staged_tn = tn;
            }
            const int row = quarter * 32 + lane;
            const int bh = WIDE ? quarter / p.qpr : row / p.pitch;
            const int bw = WIDE ? (quarter % p.qpr) * kQuarterOutputs + lane : row - bh * p.pitch;
            int img, oh;
            if (p.stack) {
                const int srow = tm * p.pbh + bh;  // row of the sequence img * OH + oh
                img = srow / p.OH;
                oh = srow - img * p.OH;
            } else {
                img = tm / p.tiles_per_image;
                oh = (tm - img * p.tiles_per_image) * p.pbh + bh;
            }
            const bool row_ok = bh < p.pbh && bw < p.OW && oh < p.OH && img < p.images && (!WIDE || lane < kQuarterOutputs);
            const int64_t pix = static_cast<int64_t>(oh) * p.OW + bw;          // pixel inside the image
            const int64_t out_base = static_cast<int64_t>(img) * p.N * hw + pix;  // + n * hw
            const int64_t cl_row = static_cast<int64_t>(img) * hw + pix;
            if (!WIDE) {
                if (!ptx::mbar_wait(bar_tmem_full + 8 * buf, static_cast<uint32_t>((iter / C::ACC_BUFS) & 1), p.err_word, kErrWaitTmemFull)) {
                    ok = false;
                    break;
                }
                ptx::tc_fence_after_sync();
            }
#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
                const int nc = n0 + c * 32;
                if (!WIDE && nc >= p.N) break;
                if (WIDE && (iter * (BN / 32) + c) % kEpiGroups != group) continue;
                uint32_t r[32];
                const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(buf * C::ACC_COLS + c * 32);
                float rv[32];  // WIDE: the residual values of this chunk, requested before the accumulator is waited for
                if constexpr (WIDE) {
                    // out[row] = E[row][0] + E[row + 1][1] + E[row + 2][2]; this thread holds row = 32 quarter + lane.
                    // The residual loads go out first: their latency (the top stall of this epilogue) then runs
                    // beside the wait for the accumulator and the tensor-memory loads.
                    if (add_res) {
                        const float* rp = p.ep.residual + out_base + static_cast<int64_t>(nc) * hw;
#pragma unroll
                        for (int j = 0; j < 32; ++j) rv[j] = row_ok ? __ldg(rp + j * hw) : 0.0f;
                    }
                    if (!ptx::mbar_wait(bar_tmem_full + 8 * buf, static_cast<uint32_t>((iter / C::ACC_BUFS) & 1), p.err_word, kErrWaitTmemFull)) {
                        ok = false;
                        break;
                    }
                    ptx::tc_fence_after_sync();
                    // Two halves of 16 columns, so that three tensor-memory operands and the residual fit the registers.
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        uint32_t e0[16], e1[16], e2[16];
                        ptx::tmem_ld_32x16(t_addr + h * 16, e0);
                        ptx::tmem_ld_32x16(t_addr + BN + h * 16, e1);
                        ptx::tmem_ld_32x16(t_addr + 2 * BN + h * 16, e2);
                        ptx::tmem_ld_wait();
                        if (h == 1) {
                            // The chunk is in registers: hand the accumulator back now (the other chunk's group does the
                            // same), so that the next tile's MMAs do not wait for the arithmetic and the stores below.
                            ptx::tc_fence_before_sync();
                            ptx::mbar_arrive(bar_tmem_empty + 8 * buf);
                        }
                        // Rows + 1 and + 2 sit in the next lanes of this warp (lanes 30 and 31 hold no output).
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            const float s1 = __shfl_down_sync(0xffffffffu, __uint_as_float(e1[j]), 1);
                            const float s2 = __shfl_down_sync(0xffffffffu, __uint_as_float(e2[j]), 2);
                            r[h * 16 + j] = __float_as_uint(__fadd_rn(__fadd_rn(__uint_as_float(e0[j]), s1), s2));
                        }
                    }
                } else {
                    ptx::tmem_ld_32x32(t_addr, r);
                    ptx::tmem_ld_wait();
                }
                if (!row_ok) continue;
                const float* as = as_g + c * 32;
                const float* bs = bs_g + c * 32;
                float o[32];
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    const float v = __uint_as_float(r[j]);
                    o[j] = bias_first ? __fmul_rn(__fadd_rn(__fmul_rn(v, ep_scale), bs[j]), as[j])
                                      : __fadd_rn(__fmul_rn(__fmul_rn(v, as[j]), ep_scale), bs[j]);
                }
                const int ncols = min(32, p.N - nc);
                const int64_t first = out_base + static_cast<int64_t>(nc) * hw;
                if (add_res) {
                    if constexpr (!WIDE) {
                        const float* rp = p.ep.residual + first;
#pragma unroll
                        for (int j = 0; j < 32; ++j) rv[j] = j < ncols ? __ldg(rp + j * hw) : 0.0f;
                    }
#pragma unroll
                    for (int j = 0; j < 32; ++j) o[j] = __fadd_rn(o[j], rv[j]);
                }
                if (p.ep.flags & TBN_EPI_RELU) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) o[j] = fmaxf(o[j], 0.0f);
                }
                if (p.y_cl != nullptr) {
                    __nv_bfloat16* cl = p.y_cl + cl_row * p.N + nc;
                    if (ncols == 32 && (p.N & 7) == 0) {
#pragma unroll
                        for (int g8 = 0; g8 < 4; ++g8) {
                            uint32_t hi[4], lo[4];
#pragma unroll
                            for (int k = 0; k < 4; ++k) split_pair_terms(o[g8 * 8 + 2 * k], o[g8 * 8 + 2 * k + 1], hi[k], lo[k]);
                            *reinterpret_cast<uint4*>(cl + g8 * 8) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
                            *reinterpret_cast<uint4*>(cl + p.y_cl_term_stride + g8 * 8) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            if (j < ncols) {
                                uint16_t term[2];
                                split_terms<2, false>(o[j], 0.f, 0.f, term);
                                cl[j] = __ushort_as_bfloat16(term[0]);
                                cl[p.y_cl_term_stride + j] = __ushort_as_bfloat16(term[1]);
                            }
                        }
                    }
                }
                if (p.y != nullptr) {
                    float* dst = p.y + first;
                    if (ncols == 32) {
#pragma unroll
                        for (int j = 0; j < 32; ++j) dst[j * hw] = o[j];
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            if (j < ncols) dst[j * hw] = o[j];
                    }
                }
            }
            if (!WIDE) {
                ptx::tc_fence_before_sync();
                ptx::mbar_arrive(bar_tmem_empty + 8 * buf);
            }
        }
    }

    ptx::tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc(tmem_base, C::TMEM_COLS);
    }
}

template <int BN, int NPASS, bool RESIDENT, bool WIDE = false>
int32_t launch(const CUtensorMap& tmap_x, const CUtensorMap& tmap_w, const Params& p, cudaStream_t st,
               const RowMaps* row_maps = nullptr) {
    static const RowMaps no_maps = {};
    auto kernel = conv_rows_kernel<BN, NPASS, RESIDENT, WIDE>;
    const int smem = smem_bytes<BN, NPASS, RESIDENT, WIDE>(p.nstages, p.n_btiles);
    TBN_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    const int total = p.tiles_m * p.tiles_n;
    const int grid = std::max(1, std::min(total, sm_count()));
    profile_begin(kProfGemm, st);
    kernel<<<grid, kThreads, smem, st>>>(tmap_x, tmap_w, row_maps ? *row_maps : no_maps, p);
    profile_end(kProfGemm, st);
    return launched("conv_rows_kernel");
}

// Pipeline depth that fits beside the resident filters (0: does not fit with at least two stages).
template <int BN, int NPASS, bool RESIDENT, bool WIDE = false>
inline int stages_that_fit(int n_btiles) {
    using C = Cfg<BN, NPASS, RESIDENT, WIDE>;
    const int left = tc::kSmemLimit - 1024 - C::AUX_BYTES - (RESIDENT ? n_btiles * C::B_TILE_BYTES : 0);
    const int s = left / C::STAGE_BYTES;
    return s < 2 ? 0 : (s > kMaxStages ? kMaxStages : s);
}

}  // namespace rows
}  // namespace
}  // namespace tbn_cuda
