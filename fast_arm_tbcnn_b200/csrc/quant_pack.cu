// Weight quantise-and-pack kernels (HBM-bound, one read of the fp32 weights).
//
// Replaces, in one pass: tbn::quantize_to_binary / quantize_to_ternary
// (tbn-runtime/src/operators/quantized_gemm_neon.cpp:544-597), the +1 padding and
// BinaryMatrix::pack (quantized_gemm_neon.cpp:199-214, GeMM/05-final/GeMM.cpp:114-151),
// the Session's transposed conv-weight packing (tbn/runtime/model.hpp:464-477) and the
// TernaryPackedWeights::set_weight loop (tbn/memory/packed_weights.hpp:53-71).
//
// Packed layout (all planes): uint32 word[n * (K_pad/32) + k/32], bit (k % 32);
// K_pad = ceil128(K), N_pad = ceil8(N); padding bits are 0.
// Comparisons are IEEE (no flush-to-zero on the compare, NaN compares false).
#include <algorithm>
#include <cstdlib>
#include <mutex>
#include <string>

#include "common.cuh"
#include "ptx_sm100.cuh"

namespace tbn_cuda {
namespace {

constexpr int kChunkK = 128;  // k rows per partial sum / per uint4 of packed words

// +1/-1/0 decision of one weight.  Returns bit0 = "negative plane", bit1 = "positive plane".
// Binary: the negative-plane bit is what the reference packs (bit set <=> -1).
template <bool TERNARY>
__device__ __forceinline__ uint32_t classify(float w, float lo_or_thr, float hi, int ge) {
    if (TERNARY) {
        const uint32_t neg = w < lo_or_thr ? 1u : 0u;
        const uint32_t pos = (!neg && w > hi) ? 2u : 0u;
        return neg | pos;
    }
    const bool plus = ge ? (w >= lo_or_thr) : (w > lo_or_thr);
    return plus ? 0u : 1u;
}

// Layout KN: W[k*ldw + n].  One warp packs a 128(k) x 32(n) tile: lane = column, rows read
// coalesced (128 B per row), 4 words per plane written as one uint4 per lane.
template <bool TERNARY>
__global__ void __launch_bounds__(128) pack_kn_kernel(const float* __restrict__ w, int64_t K, int64_t N,
                                                      int64_t ldw, float lo, float hi, int ge,
                                                      uint32_t* __restrict__ neg_words,
                                                      uint32_t* __restrict__ pos_words, int64_t KW,
                                                      int64_t N_pad, float* __restrict__ part_sum,
                                                      float* __restrict__ part_cnt) {
    const int lane = threadIdx.x & 31;
    const int64_t chunk = static_cast<int64_t>(blockIdx.y) * 4 + (threadIdx.x >> 5);
    const int64_t n = static_cast<int64_t>(blockIdx.x) * 32 + lane;
    if (chunk * kChunkK >= KW * 32 || n >= N_pad) return;
    const int64_t k0 = chunk * kChunkK;
    uint32_t negw[4] = {0, 0, 0, 0}, posw[4] = {0, 0, 0, 0};
    float sum = 0.0f, cnt = 0.0f;
    if (n < N) {
#pragma unroll
        for (int wi = 0; wi < 4; ++wi) {
            float v[32];
#pragma unroll
            for (int r = 0; r < 32; ++r) {
                const int64_t k = k0 + wi * 32 + r;
                v[r] = (k < K) ? __ldg(w + k * ldw + n) : __int_as_float(0x7fc00000);
            }
#pragma unroll
            for (int r = 0; r < 32; ++r) {
                const int64_t k = k0 + wi * 32 + r;
                if (k < K) {
                    const uint32_t c = classify<TERNARY>(v[r], lo, hi, ge);
                    negw[wi] |= (c & 1u) << r;
                    if (TERNARY) {
                        posw[wi] |= (c >> 1) << r;
                        if (c) {
                            sum += fabsf(v[r]);
                            cnt += 1.0f;
                        }
                    } else {
                        sum += fabsf(v[r]);
                    }
                }
            }
        }
    }
    const int64_t widx = n * KW + chunk * 4;
    *reinterpret_cast<uint4*>(neg_words + widx) = make_uint4(negw[0], negw[1], negw[2], negw[3]);
    if (TERNARY) *reinterpret_cast<uint4*>(pos_words + widx) = make_uint4(posw[0], posw[1], posw[2], posw[3]);
    if (part_sum && n < N) {
        part_sum[chunk * N + n] = sum;
        if (TERNARY) part_cnt[chunk * N + n] = cnt;
    }
}

// Layout KN, wide variant (rows 16-byte aligned, N % 4 == 0): each lane owns FOUR adjacent columns and reads
// them as one float4, so a warp reads 512 contiguous bytes per weight row -- wide enough for DRAM to run
// near its streaming rate -- and packs a 128(k) x 128(n) tile.
template <bool TERNARY>
__global__ void __launch_bounds__(128) pack_kn_vec4_kernel(const float* __restrict__ w, int64_t K, int64_t N,
                                                           int64_t ldw, float lo, float hi, int ge,
                                                           uint32_t* __restrict__ neg_words,
                                                           uint32_t* __restrict__ pos_words, int64_t KW,
                                                           int64_t N_pad, float* __restrict__ part_sum,
                                                           float* __restrict__ part_cnt) {
    const int lane = threadIdx.x & 31;
    const int64_t chunk = static_cast<int64_t>(blockIdx.y) * 4 + (threadIdx.x >> 5);
    const int64_t n = static_cast<int64_t>(blockIdx.x) * 128 + lane * 4;
    if (chunk * kChunkK >= KW * 32 || n >= N_pad) return;
    const int64_t k0 = chunk * kChunkK;
    uint32_t negw[4][4], posw[4][4];
    float sum[4] = {0.f, 0.f, 0.f, 0.f}, cnt[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int wi = 0; wi < 4; ++wi) negw[j][wi] = posw[j][wi] = 0u;
    if (n < N) {
#pragma unroll
        for (int wi = 0; wi < 4; ++wi) {
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                float4 v[16];
#pragma unroll
                for (int r = 0; r < 16; ++r) {
                    const int64_t k = k0 + wi * 32 + half * 16 + r;
                    v[r] = (k < K) ? __ldg(reinterpret_cast<const float4*>(w + k * ldw + n))
                                   : make_float4(0.f, 0.f, 0.f, 0.f);
                }
#pragma unroll
                for (int r = 0; r < 16; ++r) {
                    const int64_t k = k0 + wi * 32 + half * 16 + r;
                    if (k < K) {
                        const float e[4] = {v[r].x, v[r].y, v[r].z, v[r].w};
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const uint32_t c = classify<TERNARY>(e[j], lo, hi, ge);
                            negw[j][wi] |= (c & 1u) << (half * 16 + r);
                            if (TERNARY) {
                                posw[j][wi] |= (c >> 1) << (half * 16 + r);
                                if (c) {
                                    sum[j] += fabsf(e[j]);
                                    cnt[j] += 1.0f;
                                }
                            } else {
                                sum[j] += fabsf(e[j]);
                            }
                        }
                    }
                }
            }
        }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        if (n + j >= N_pad) break;
        const int64_t widx = (n + j) * KW + chunk * 4;
        *reinterpret_cast<uint4*>(neg_words + widx) = make_uint4(negw[j][0], negw[j][1], negw[j][2], negw[j][3]);
        if (TERNARY) *reinterpret_cast<uint4*>(pos_words + widx) = make_uint4(posw[j][0], posw[j][1], posw[j][2], posw[j][3]);
    }
    if (part_sum && n < N) {
        *reinterpret_cast<float4*>(part_sum + chunk * N + n) = make_float4(sum[0], sum[1], sum[2], sum[3]);
        if (TERNARY) *reinterpret_cast<float4*>(part_cnt + chunk * N + n) = make_float4(cnt[0], cnt[1], cnt[2], cnt[3]);
    }
}

// Layout KN, streaming variant for large matrices: persistent CTAs (one per SM), a producer warp that keeps a
// ring of TMA tiles in flight and sixteen consumer warps that classify from shared memory.
//   job   = 128 (k) x 512 (n) block of W: four tiles of 32 rows x 512 columns, each row 2 KB contiguous in HBM;
//   tile  = two TMA boxes of 32 x 256 fp32 (32 KB each); kPackStages tiles in flight per SM;
//   thread t owns column t of the job: conflict-free shared-memory reads (lane = bank), one word per tile and
//   plane, one uint4 (128 k) per column and plane at the end of the job.
// Jobs are numbered strip-fastest, so CTAs running at the same time read neighbouring 2 KB pieces of the same
// rows.  The partial |w| sums per 128-row chunk are accumulated in the same order as in the other kernels.
constexpr int kPackStages = 3;
constexpr int kPackBoxCols = 256;
constexpr int kPackTileBytes = 64 * 1024;
constexpr int kPackConsumers = 512;  // one per column (CPT = 1) or per pair of columns 512 apart (CPT = 2) of a job
constexpr int kPackSmemBytes = kPackStages * kPackTileBytes + 1024 + 256;

// CPT = columns per consumer thread.  The job is 128 (k) x 512 CPT (n); a tile is 32 / CPT rows of it (64 KB either
// way): CPT = 2 halves the rows per tile and doubles their length, so that every row piece read from HBM is 4 KB
// contiguous instead of 2 KB.
template <bool TERNARY, int CPT>
__global__ void __launch_bounds__(kPackConsumers + 32, 1)
pack_kn_tma_kernel(const __grid_constant__ CUtensorMap tmap_w, int64_t K, int64_t N, float lo, float hi, int ge,
                   uint32_t* __restrict__ neg_words, uint32_t* __restrict__ pos_words, int64_t KW, int64_t N_pad,
                   float* __restrict__ part_sum, float* __restrict__ part_cnt, int64_t strips, int64_t jobs,
                   int* err_word) {
    constexpr int kTileRows = 32 / CPT, kBoxes = 2 * CPT, kBoxBytes = kTileRows * kPackBoxCols * 4;
    constexpr int kJobCols = 512 * CPT, kTilesPerJob = kChunkK / kTileRows;
    static_assert(kBoxes * kBoxBytes == kPackTileBytes, "a tile is 64 KB");
    extern __shared__ uint8_t pack_smem_raw[];
    const uint32_t raw_addr = ptx::smem_u32(pack_smem_raw);
    const uint32_t base = (raw_addr + 1023u) & ~1023u;
    const float* tiles = reinterpret_cast<const float*>(pack_smem_raw + (base - raw_addr));
    const uint32_t bar_full = base + kPackStages * kPackTileBytes;
    const uint32_t bar_empty = bar_full + 8 * kPackStages;
    if (threadIdx.x == 0) {
        for (int s = 0; s < kPackStages; ++s) {
            ptx::mbar_init(bar_full + 8 * s, 1);
            ptx::mbar_init(bar_empty + 8 * s, kPackConsumers);
        }
        ptx::fence_barrier_init();
        ptx::prefetch_tensormap(&tmap_w);
    }
    // Lets the blocks of alpha_finalize_kernel (launched next in the stream) take their places now; they wait for
    // this whole grid to complete before they read anything.
    asm volatile("griddepcontrol.launch_dependents;");
    __syncthreads();

    if (threadIdx.x >= kPackConsumers) {
        // ---------------------------------------------------------------- producer warp (one lane)
        if (threadIdx.x == kPackConsumers) {
            int stage = 0;
            uint32_t phase = 0;
            for (int64_t job = blockIdx.x; job < jobs; job += gridDim.x) {
                const int64_t strip = job % strips, chunk = job / strips;
                bool ok = true;
                for (int sub = 0; sub < kTilesPerJob && ok; ++sub) {
                    if (!ptx::mbar_wait(bar_empty + 8 * stage, phase ^ 1u, err_word, kErrPackWaitEmpty)) {
                        ok = false;
                        break;
                    }
                    const uint32_t bar = bar_full + 8 * stage;
                    const uint32_t dst = base + stage * kPackTileBytes;
                    const int x = static_cast<int>(strip * kJobCols);
                    const int y = static_cast<int>(chunk * kChunkK + sub * kTileRows);
                    ptx::mbar_arrive_expect_tx(bar, kPackTileBytes);
#pragma unroll
                    for (int b = 0; b < kBoxes; ++b)   // out-of-range parts arrive as zeros
                        ptx::tma_load_2d(dst + b * kBoxBytes, &tmap_w, x + b * kPackBoxCols, y, bar);
                    if (++stage == kPackStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (!ok) break;
            }
        }
        return;
    }

    // -------------------------------------------------------------------- consumers
    const int t = threadIdx.x;
    // Column i of this thread is job column t + 512 i: box (t >> 8) + 2 i, column t & 255 inside the box.
    const int tile_off = (t >> 8) * (kBoxBytes / 4) + (t & 255);
    int stage = 0;
    uint32_t phase = 0;
    for (int64_t job = blockIdx.x; job < jobs; job += gridDim.x) {
        const int64_t strip = job % strips, chunk = job / strips;
        uint32_t negw[CPT][4], posw[CPT][4];
        float sum[CPT], cnt[CPT];
#pragma unroll
        for (int i = 0; i < CPT; ++i) sum[i] = cnt[i] = 0.f;
        uint32_t nb[CPT], pb[CPT];
#pragma unroll
        for (int sub = 0; sub < kTilesPerJob; ++sub) {
            if (!ptx::mbar_wait(bar_full + 8 * stage, phase, err_word, kErrPackWaitFull)) return;
            const float* tile = tiles + stage * (kPackTileBytes / 4) + tile_off;
            const int64_t k0 = chunk * kChunkK + sub * kTileRows;
            const int rows = static_cast<int>(min(static_cast<int64_t>(kTileRows), K - k0));  // <= 0 past the end
            if (sub % CPT == 0) {
#pragma unroll
                for (int i = 0; i < CPT; ++i) nb[i] = pb[i] = 0u;
            }
            const int bit0 = (sub % CPT) * kTileRows;
#pragma unroll
            for (int r = 0; r < kTileRows; ++r) {
#pragma unroll
                for (int i = 0; i < CPT; ++i) {
                    const float e = tile[2 * i * (kBoxBytes / 4) + r * kPackBoxCols];
                    if (r < rows) {
                        const uint32_t c = classify<TERNARY>(e, lo, hi, ge);
                        nb[i] |= (c & 1u) << (bit0 + r);
                        if (TERNARY) {
                            pb[i] |= (c >> 1) << (bit0 + r);
                            if (c) {
                                sum[i] += fabsf(e);
                                cnt[i] += 1.0f;
                            }
                        } else {
                            sum[i] += fabsf(e);
                        }
                    }
                }
            }
            // The stage goes back to the producer only after every value read above has arrived in registers:
            // the arrive is made to depend on them.
            uint32_t dep = 0u;
#pragma unroll
            for (int i = 0; i < CPT; ++i) dep ^= nb[i] ^ pb[i] ^ __float_as_uint(sum[i]);
            ptx::mbar_arrive_after(bar_empty + 8 * stage, dep);
            if (++stage == kPackStages) {
                stage = 0;
                phase ^= 1u;
            }
            if (sub % CPT == CPT - 1) {
#pragma unroll
                for (int i = 0; i < CPT; ++i) {
                    negw[i][sub / CPT] = nb[i];
                    posw[i][sub / CPT] = pb[i];
                }
            }
        }
#pragma unroll
        for (int i = 0; i < CPT; ++i) {
            const int64_t n = strip * kJobCols + t + 512 * i;
            if (n >= N_pad) continue;
            const bool real = n < N;  // columns N .. N_pad-1 are padding: all bits 0
            const int64_t widx = n * KW + chunk * 4;
            *reinterpret_cast<uint4*>(neg_words + widx) =
                real ? make_uint4(negw[i][0], negw[i][1], negw[i][2], negw[i][3]) : make_uint4(0u, 0u, 0u, 0u);
            if (TERNARY)
                *reinterpret_cast<uint4*>(pos_words + widx) =
                    real ? make_uint4(posw[i][0], posw[i][1], posw[i][2], posw[i][3]) : make_uint4(0u, 0u, 0u, 0u);
            if (part_sum && real) {
                part_sum[chunk * N + n] = sum[i];
                if (TERNARY) part_cnt[chunk * N + n] = cnt[i];
            }
        }
    }
}

// Layout NK: W[n*ldw + k] (k contiguous).  One warp packs one 128-k chunk of one column:
// four coalesced 128 B reads, four ballots.
template <bool TERNARY>
__global__ void __launch_bounds__(128) pack_nk_kernel(const float* __restrict__ w, int64_t K, int64_t N,
                                                      int64_t ldw, float lo, float hi, int ge,
                                                      uint32_t* __restrict__ neg_words,
                                                      uint32_t* __restrict__ pos_words, int64_t KW,
                                                      int64_t N_pad, float* __restrict__ part_sum,
                                                      float* __restrict__ part_cnt) {
    const int lane = threadIdx.x & 31;
    const int64_t chunk = static_cast<int64_t>(blockIdx.y) * 4 + (threadIdx.x >> 5);
    const int64_t n = blockIdx.x;
    if (chunk * kChunkK >= KW * 32) return;
    const int64_t k0 = chunk * kChunkK;
    float v[4];
#pragma unroll
    for (int wi = 0; wi < 4; ++wi) {
        const int64_t k = k0 + wi * 32 + lane;
        v[wi] = (n < N && k < K) ? __ldg(w + n * ldw + k) : __int_as_float(0x7fc00000);
    }
    uint32_t negw[4], posw[4];
    float sum = 0.0f, cnt = 0.0f;
#pragma unroll
    for (int wi = 0; wi < 4; ++wi) {
        const int64_t k = k0 + wi * 32 + lane;
        const bool valid = n < N && k < K;
        const uint32_t c = valid ? classify<TERNARY>(v[wi], lo, hi, ge) : 0u;
        negw[wi] = __ballot_sync(0xffffffffu, c & 1u);
        posw[wi] = TERNARY ? __ballot_sync(0xffffffffu, c & 2u) : 0u;
        if (valid && (!TERNARY || c)) {
            sum += fabsf(v[wi]);
            cnt += 1.0f;
        }
    }
    // Deterministic in-warp tree reduction of the partial |w| sum.
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        sum += __shfl_down_sync(0xffffffffu, sum, off);
        cnt += __shfl_down_sync(0xffffffffu, cnt, off);
    }
    if (lane == 0) {
        const int64_t widx = n * KW + chunk * 4;
        *reinterpret_cast<uint4*>(neg_words + widx) = make_uint4(negw[0], negw[1], negw[2], negw[3]);
        if (TERNARY) *reinterpret_cast<uint4*>(pos_words + widx) = make_uint4(posw[0], posw[1], posw[2], posw[3]);
        if (part_sum && n < N) {
            part_sum[chunk * N + n] = sum;
            if (TERNARY) part_cnt[chunk * N + n] = cnt;
        }
    }
}

// alpha[n] = (sum over chunks, in chunk order) / (K or number of non-zero weights).
// Launched with programmatic stream serialisation: its blocks may become resident while the pack kernel before it in
// the stream still runs (the streaming pack kernel releases them at its start) and wait here until that grid has
// completed and its partial sums are visible, which takes the launch latency off the critical path.
// A block owns 32 columns.  Its sixteen warps fetch 128 chunks' partial sums at once into shared memory (a serial
// loop over chunks per column is bound by memory latency: one round trip per few chunks), then one warp adds them
// per column in chunk order.
constexpr int kFinalizeCols = 32, kFinalizeWarps = 16, kFinalizeBatch = 128;
__global__ void __launch_bounds__(kFinalizeCols * kFinalizeWarps)
alpha_finalize_kernel(const float* __restrict__ part_sum, const float* __restrict__ part_cnt, int64_t chunks, int64_t N,
                      int64_t K, float* __restrict__ alpha) {
    __shared__ float sum_s[kFinalizeBatch][kFinalizeCols];
    __shared__ float cnt_s[kFinalizeBatch][kFinalizeCols];
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t n = static_cast<int64_t>(blockIdx.x) * kFinalizeCols + lane;
    float s = 0.0f, c = 0.0f;
    for (int64_t c0 = 0; c0 < chunks; c0 += kFinalizeBatch) {
        const int in_batch = static_cast<int>(min(static_cast<int64_t>(kFinalizeBatch), chunks - c0));
#pragma unroll
        for (int u = 0; u < kFinalizeBatch / kFinalizeWarps; ++u) {
            const int i = u * kFinalizeWarps + warp;
            if (i < in_batch && n < N) {
                sum_s[i][lane] = __ldcg(part_sum + (c0 + i) * N + n);
                if (part_cnt) cnt_s[i][lane] = __ldcg(part_cnt + (c0 + i) * N + n);
            }
        }
        __syncthreads();
        if (warp == 0 && n < N) {
            for (int i = 0; i < in_batch; ++i) {
                s += sum_s[i][lane];
                if (part_cnt) c += cnt_s[i][lane];
            }
        }
        __syncthreads();
    }
    if (warp != 0 || n >= N) return;
    if (part_cnt) alpha[n] = c > 0.0f ? __fdiv_rn(s, c) : 0.0f;
    else alpha[n] = __fdiv_rn(s, static_cast<float>(K));
}

// Reference 2-bit codes over the flat row-major [K,N] element order: one thread per uint32.
__global__ void ternary_codes_kernel(const float* __restrict__ w, int64_t K, int64_t N, int64_t ldw, int layout,
                                     float lo, float hi, uint32_t* __restrict__ codes, int64_t n_words) {
    const int64_t j = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (j >= n_words) return;
    const int64_t total = K * N;
    uint32_t word = 0;
#pragma unroll 4
    for (int e = 0; e < 16; ++e) {
        const int64_t i = j * 16 + e;
        if (i >= total) break;
        const int64_t k = i / N, n = i - k * N;
        const float v = layout == TBN_LAYOUT_KN ? __ldg(w + k * ldw + n) : __ldg(w + n * ldw + k);
        const uint32_t code = v < lo ? 0u : (v > hi ? 2u : 1u);
        word |= code << (2 * e);
    }
    codes[j] = word;
}

// alpha[c] = (sum_i |w[c*per + i]|) / per, fp32, summed in memory order by one thread per channel:
// bit-equal to the loop of Session::execute_conv (model.hpp:388-394).
__global__ void channel_abs_mean_seq_kernel(const float* __restrict__ w, int64_t channels, int64_t per,
                                            float* __restrict__ alpha) {
    const int64_t c = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (c >= channels) return;
    const float* row = w + c * per;
    float sum = 0.0f;
    for (int64_t i = 0; i < per; ++i) sum = __fadd_rn(sum, fabsf(row[i]));
    alpha[c] = __fdiv_rn(sum, static_cast<float>(per));
}

__global__ void quantize_binary_kernel(const float* __restrict__ w, int64_t n, float thr, uint8_t* __restrict__ out) {
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride)
        out[i] = w[i] > thr ? 1 : 0;
}

__global__ void quantize_ternary_kernel(const float* __restrict__ w, int64_t n, float lo, float hi,
                                        int8_t* __restrict__ out) {
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
        const float v = w[i];
        out[i] = v < lo ? -1 : (v > hi ? 1 : 0);
    }
}

int grid_for(int64_t n, int block) {
    const int64_t want = (n + block - 1) / block;
    const int64_t cap = static_cast<int64_t>(sm_count() > 0 ? sm_count() : 148) * 16;
    return static_cast<int>(want < 1 ? 1 : (want > cap ? cap : want));
}

template <bool TERNARY>
int32_t quant_pack(const float* d_w, int64_t K, int64_t N, int64_t ldw, int32_t layout, float lo, float hi,
                   int32_t ge, uint32_t* d_neg, uint32_t* d_pos, float* d_alpha, void* d_ws, size_t ws_bytes,
                   cudaStream_t st) {
    TBN_REQUIRE(K > 0 && N > 0, TBN_INVALID_SHAPE, "quant_pack: K and N must be positive");
    TBN_REQUIRE(d_w && d_neg && (!TERNARY || d_pos), TBN_INVALID_ARGUMENT, "quant_pack: null pointer");
    TBN_REQUIRE(layout == TBN_LAYOUT_KN || layout == TBN_LAYOUT_NK, TBN_INVALID_ARGUMENT, "quant_pack: bad layout");
    TBN_REQUIRE(ldw >= (layout == TBN_LAYOUT_KN ? N : K), TBN_INVALID_ARGUMENT, "quant_pack: ldw too small");
    const int64_t K_pad = round_up(K, 128), N_pad = round_up(N, 8), KW = K_pad / 32;
    const int64_t chunks = K_pad / kChunkK;
    TBN_REQUIRE(N_pad <= 0x7fffffffLL && chunks <= 4LL * 65535, TBN_INVALID_SHAPE, "quant_pack: matrix too large");
    float* part_sum = nullptr;
    float* part_cnt = nullptr;
    if (d_alpha) {
        const size_t need = tbn_quant_pack_workspace_bytes(K, N, TERNARY ? 1 : 0);
        TBN_REQUIRE(d_ws && ws_bytes >= need, TBN_INVALID_ARGUMENT, "quant_pack: workspace too small for alpha");
        part_sum = static_cast<float*>(d_ws);
        if (TERNARY) part_cnt = part_sum + chunks * N;
    }
    const unsigned gy = static_cast<unsigned>((chunks + 3) / 4);
    const bool wide = layout == TBN_LAYOUT_KN && N % 4 == 0 && ldw % 4 == 0 && reinterpret_cast<uintptr_t>(d_w) % 16 == 0 &&
                      (!part_sum || reinterpret_cast<uintptr_t>(part_sum) % 16 == 0) && N >= 128;
    // Large matrices stream through TMA; the register kernels keep the small and the unaligned ones.
    const bool stream = wide && K * N >= (1LL << 22) && N < (1LL << 31) && K < (1LL << 31) && device_error_word() != nullptr;
    if (stream) {
        EncodeTiledFn encode = encode_tiled_fn();
        TBN_REQUIRE(encode != nullptr, TBN_CUDA_ERROR, "cuTensorMapEncodeTiled is not available from the driver");
        // Two columns per consumer thread (4 KB row pieces) once a job of 1024 columns fits the matrix at least twice.
        const int cpt = N_pad >= 2048 ? 2 : 1;
        CUtensorMap tmap;
        const cuuint64_t gdim[2] = {static_cast<cuuint64_t>(N), static_cast<cuuint64_t>(K)};
        const cuuint64_t gstride[1] = {static_cast<cuuint64_t>(ldw) * 4};
        const cuuint32_t box[2] = {kPackBoxCols, static_cast<cuuint32_t>(32 / cpt)};
        const cuuint32_t estr[2] = {1, 1};
        const CUresult cr = encode(&tmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(d_w), gdim, gstride, box, estr,
                                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        TBN_REQUIRE(cr == CUDA_SUCCESS, TBN_CUDA_ERROR,
                    "cuTensorMapEncodeTiled failed with CUresult " + std::to_string(static_cast<int>(cr)));
        const int64_t job_cols = 512 * cpt;
        const int64_t strips = (N_pad + job_cols - 1) / job_cols, jobs = strips * chunks;
        auto kernel = cpt == 2 ? pack_kn_tma_kernel<TERNARY, 2> : pack_kn_tma_kernel<TERNARY, 1>;
        TBN_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kPackSmemBytes));
        const int grid = static_cast<int>(std::min<int64_t>(jobs, std::max(sm_count(), 1)));
        kernel<<<grid, kPackConsumers + 32, kPackSmemBytes, st>>>(tmap, K, N, lo, hi, ge, d_neg, d_pos, KW, N_pad, part_sum,
                                                                  part_cnt, strips, jobs, device_error_word());
    } else if (wide) {
        dim3 grid(static_cast<unsigned>((N_pad + 127) / 128), gy);
        pack_kn_vec4_kernel<TERNARY><<<grid, 128, 0, st>>>(d_w, K, N, ldw, lo, hi, ge, d_neg, d_pos, KW, N_pad, part_sum,
                                                           part_cnt);
    } else if (layout == TBN_LAYOUT_KN) {
        dim3 grid(static_cast<unsigned>((N_pad + 31) / 32), gy);
        pack_kn_kernel<TERNARY><<<grid, 128, 0, st>>>(d_w, K, N, ldw, lo, hi, ge, d_neg, d_pos, KW, N_pad, part_sum,
                                                      part_cnt);
    } else {
        dim3 grid(static_cast<unsigned>(N_pad), gy);
        pack_nk_kernel<TERNARY><<<grid, 128, 0, st>>>(d_w, K, N, ldw, lo, hi, ge, d_neg, d_pos, KW, N_pad, part_sum,
                                                      part_cnt);
    }
    int32_t rc = launched(TERNARY ? "pack_kernel<ternary>" : "pack_kernel<binary>");
    if (rc) return rc;
    if (d_alpha) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(static_cast<unsigned>((N + kFinalizeCols - 1) / kFinalizeCols));
        cfg.blockDim = dim3(kFinalizeCols * kFinalizeWarps);
        cfg.stream = st;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        TBN_CUDA_TRY(cudaLaunchKernelEx(&cfg, alpha_finalize_kernel, static_cast<const float*>(part_sum),
                                        static_cast<const float*>(part_cnt), chunks, N, K, d_alpha));
        rc = launched("alpha_finalize_kernel");
    }
    return rc;
}

// ---- scratch of the entry point that allocates nothing --------------------------------
// Lives in the library image: every GPU that loads the library holds these 4 MiB until the
// process exits.  Shared by all calls of tbn_quant_pack_binary_noalloc on a device.
constexpr size_t kNoAllocScratchFloats = size_t(1) << 20;
static __device__ __align__(256) float g_noalloc_scratch[kNoAllocScratchFloats];

constexpr int kNoAllocMaxDevices = 64;
std::mutex g_noalloc_mutex;
float* g_noalloc_ptr[kNoAllocMaxDevices] = {};

// Device address of g_noalloc_scratch on the CURRENT device.  In host code the array's name is
// only a handle for the runtime; the address a kernel can use has to be asked for, once per
// device, with that device current.
int32_t noalloc_scratch_address(float** out) {
    int dev = -1;
    TBN_CUDA_TRY(cudaGetDevice(&dev));
    TBN_REQUIRE(dev >= 0 && dev < kNoAllocMaxDevices, TBN_RUNTIME_ERROR, "device index out of range");
    std::lock_guard<std::mutex> lock(g_noalloc_mutex);
    if (g_noalloc_ptr[dev] == nullptr) {
        float* p = nullptr;
        TBN_CUDA_TRY(cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_noalloc_scratch));
        TBN_REQUIRE(p != nullptr, TBN_CUDA_ERROR, "cudaGetSymbolAddress returned a null scratch address");
        g_noalloc_ptr[dev] = p;
    }
    *out = g_noalloc_ptr[dev];
    return TBN_SUCCESS;
}

}  // namespace
}  // namespace tbn_cuda

using namespace tbn_cuda;

extern "C" {

int32_t tbn_quant_pack_binary_noalloc(const float* d_w, int64_t K, int64_t N, int64_t ldw, int32_t layout, float thr,
                                      int32_t ge, uint32_t* d_words, float* d_alpha, void* stream) {
    TBN_REQUIRE(K > 0 && N > 0, TBN_INVALID_SHAPE, "tbn_quant_pack_binary_noalloc: K and N must be positive");
    TBN_REQUIRE(K < (int64_t(1) << 40) && N < (int64_t(1) << 40), TBN_INVALID_SHAPE,
                "tbn_quant_pack_binary_noalloc: dimension too large");
    // The scratch holds the partial sums of the per-column scale: without d_alpha none is used and any size goes.
    const size_t chunks = static_cast<size_t>(round_up(K, 128) / kChunkK);
    const size_t partials = chunks * static_cast<size_t>(N);  // < 2^80 / 128: no overflow after the check above
    if (d_alpha != nullptr && partials > kNoAllocScratchFloats) {
        return fail(TBN_INVALID_ARGUMENT,
                    "tbn_quant_pack_binary_noalloc: ceil(K/128)*N = " + std::to_string(partials) +
                        " exceeds the built-in scratch of " + std::to_string(kNoAllocScratchFloats) +
                        " partial sums; use tbn_quant_pack_binary with a caller workspace");
    }
    float* scratch = nullptr;
    const int32_t rc = noalloc_scratch_address(&scratch);
    if (rc) return rc;
    // Every partial sum that alpha_finalize_kernel reads is written by the pack kernel of this same
    // call first, so nothing left over from an earlier call is ever read and nothing needs clearing.
    return quant_pack<false>(d_w, K, N, ldw, layout, thr, 0.0f, ge, d_words, nullptr, d_alpha, scratch,
                             kNoAllocScratchFloats * sizeof(float), as_stream(stream));
}

int32_t tbn_channel_abs_mean(const float* d_w, int64_t channels, int64_t per, float* d_alpha, void* stream) {
    TBN_REQUIRE(channels > 0 && per > 0, TBN_INVALID_SHAPE, "tbn_channel_abs_mean: sizes must be positive");
    TBN_REQUIRE(d_w && d_alpha, TBN_INVALID_ARGUMENT, "tbn_channel_abs_mean: null pointer");
    channel_abs_mean_seq_kernel<<<static_cast<unsigned>((channels + 63) / 64), 64, 0, as_stream(stream)>>>(d_w, channels, per,
                                                                                                    d_alpha);
    return launched("channel_abs_mean_seq_kernel");
}

int32_t tbn_quantize_to_binary(const float* d_w, int64_t n, float thr, uint8_t* d_out, void* stream) {
    TBN_REQUIRE(n >= 0, TBN_INVALID_ARGUMENT, "tbn_quantize_to_binary: negative size");
    if (n == 0) return TBN_SUCCESS;
    TBN_REQUIRE(d_w && d_out, TBN_INVALID_ARGUMENT, "tbn_quantize_to_binary: null pointer");
    quantize_binary_kernel<<<grid_for(n, 256), 256, 0, as_stream(stream)>>>(d_w, n, thr, d_out);
    return launched("quantize_binary_kernel");
}

int32_t tbn_quantize_to_ternary(const float* d_w, int64_t n, float lo, float hi, int8_t* d_out, void* stream) {
    TBN_REQUIRE(n >= 0, TBN_INVALID_ARGUMENT, "tbn_quantize_to_ternary: negative size");
    if (n == 0) return TBN_SUCCESS;
    TBN_REQUIRE(d_w && d_out, TBN_INVALID_ARGUMENT, "tbn_quantize_to_ternary: null pointer");
    quantize_ternary_kernel<<<grid_for(n, 256), 256, 0, as_stream(stream)>>>(d_w, n, lo, hi, d_out);
    return launched("quantize_ternary_kernel");
}

size_t tbn_quant_pack_workspace_bytes(int64_t K, int64_t N, int32_t ternary) {
    if (K <= 0 || N <= 0) return 0;
    const int64_t chunks = round_up(K, 128) / kChunkK;
    return static_cast<size_t>(chunks * N) * sizeof(float) * (ternary ? 2 : 1);
}

int32_t tbn_quant_pack_binary(const float* d_w, int64_t K, int64_t N, int64_t ldw, int32_t layout, float thr,
                              int32_t ge, uint32_t* d_words, float* d_alpha, void* d_workspace,
                              size_t workspace_bytes, void* stream) {
    return quant_pack<false>(d_w, K, N, ldw, layout, thr, 0.0f, ge, d_words, nullptr, d_alpha, d_workspace,
                             workspace_bytes, as_stream(stream));
}

int32_t tbn_quant_pack_ternary(const float* d_w, int64_t K, int64_t N, int64_t ldw, int32_t layout, float lo,
                               float hi, uint32_t* d_codes, uint32_t* d_pos, uint32_t* d_neg, float* d_alpha,
                               void* d_workspace, size_t workspace_bytes, void* stream) {
    int32_t rc = quant_pack<true>(d_w, K, N, ldw, layout, lo, hi, 0, d_neg, d_pos, d_alpha, d_workspace,
                                  workspace_bytes, as_stream(stream));
    if (rc || !d_codes) return rc;
    const int64_t n_words = (K * N + 15) / 16;
    ternary_codes_kernel<<<static_cast<unsigned>((n_words + 255) / 256), 256, 0, as_stream(stream)>>>(
        d_w, K, N, ldw, layout, lo, hi, d_codes, n_words);
    return launched("ternary_codes_kernel");
}

}  // extern "C"
