// The tcgen05 GEMM kernel shared by the plain GEMM (gemm.cu) and the implicit-GEMM convolution
// (conv.cu):   D[m, n] = sum_k A[m, k] * w[k, n]   with w in {-1, +1} or {-1, 0, +1} from packed planes.
//
// Persistent, one 448-thread CTA per SM, tile 128 x BN x 64, warp specialised:
//   warp 0      producer: TMA loads of the packed weight words (16 bytes = 128 k per column) into a
//               small ring and -- GEMM mode -- of the pre-split bf16 activation tiles (SWIZZLE_128B)
//   warp 1      MMA issuer: tcgen05.mma.cta_group::1.kind::f16 (M128 x BN x K16) for every activation
//               term against the same unpacked weight tile, fp32 accumulators double-buffered in
//               tensor memory
//   warps 2-9   operand build: packed words smem -> registers -> +-1/0 bf16 written into the swizzled
//               K-major operand tile; -- CONV modes -- also the activation operand (the im2col matrix is
//               never materialised): either gathered element-wise from the NCHW fp32 input, split into
//               bf16 terms (or ternarised) and written to the swizzled tile (any geometry), or -- when the
//               channel count is a multiple of 64 -- copied with 16-byte cp.async from a channels-last
//               bf16 copy of the input that a cheap pre-pass has already split (one filter tap and 64
//               channels per k-block)
//   warps 10-13 epilogue: tcgen05.ld, alpha / scale / bias / residual / ReLU, store (row-major or NCHW)
//
// The tensor cores add into the fp32 accumulator with truncation, an error that grows linearly with the
// number of accumulation steps; long K is therefore cut into segments that each start a fresh
// accumulator, and the epilogue adds the segments in fp32 (round to nearest) through a per-CTA scratch
// tile that stays resident in L2.
//
// Weight source BSRC.  0: packed sign words, unpacked by the build warps (the GEMM).  1: float weights (the
// float x float Gemm / Conv of the CNN graphs) arriving by TMA as two pre-split bf16 terms; the MMA issuer
// forms hi*hi + hi*lo + lo*hi.  2: sign weights already expanded to +-1/0 bf16 (one term) arriving by TMA --
// the convolutions, whose small weight matrices are expanded once per call and stay in L2, so that the
// build warps only gather activations.
//
// Every wait is bounded and reports through the library's device error word.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>
#include <climits>
#include <cstdint>
#include <string>

#include "common.cuh"
#include "ptx_sm100.cuh"

namespace tbn_cuda {
namespace {

// Bit pattern of +1.0 in the 16-bit operand type: bf16 0x3F80, fp16 0x3C00 (-1.0 sets bit 15 in both, 0 is 0).
constexpr uint32_t kOneBf16 = 0x3F80u, kOneF16 = 0x3C00u;

// 8 packed bits -> 8 sixteen-bit values (+1 = one16, -1 = one16 | 0x8000, 0 = 0x0000)
template <bool TERNARY>
__device__ __forceinline__ uint4 unpack8(uint32_t neg_byte, uint32_t pos_byte, uint32_t one16 = kOneBf16) {
    uint32_t o[4];
    const uint32_t one2 = one16 | (one16 << 16);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const uint32_t n0 = (neg_byte >> (2 * j)) & 1u, n1 = (neg_byte >> (2 * j + 1)) & 1u;
        if (TERNARY) {
            const uint32_t p0 = (pos_byte >> (2 * j)) & 1u, p1 = (pos_byte >> (2 * j + 1)) & 1u;
            const uint32_t lo16 = ((n0 | p0) * one16) | (n0 << 15);
            const uint32_t hi16 = ((n1 | p1) * one16) | (n1 << 15);
            o[j] = lo16 | (hi16 << 16);
        } else {
            o[j] = one2 | (n0 << 15) | (n1 << 31);
        }
    }
    return make_uint4(o[0], o[1], o[2], o[3]);
}

// The same with fewer instructions on the integer pipe (the build warps of the GEMM spend their issue slots here; the
// ternary kernel ran 20 % behind the binary one on them).  Four bits become four bytes with one multiply and one mask
// (bit e of a nibble lands at bit 8 e: the partial products of 0x00204081 never meet), a value's code is its byte
// (binary: 0 plus, 1 minus; ternary: 0 zero, 1 plus, 2 minus = pos + 2 neg), and each pair of values is ONE byte
// permute out of two small byte tables -- the high and the low byte of the operand-type constants -- whose selector is
// code * 0x11 + 0x0404 (prmt reads only the low 16 bits of its selector).
//   binary:  lut_hi = {hi(+1), hi(-1)},     lut_lo = {lo(+1), lo(-1)}          (byte 0, 1 of each word)
//   ternary: lut_hi = {0, hi(+1), hi(-1)},  lut_lo = {0, lo(+1), lo(-1)}       (byte 0, 1, 2)
__device__ __forceinline__ uint32_t nibble_to_bytes(uint32_t bits4) { return (bits4 * 0x00204081u) & 0x01010101u; }

template <bool TERNARY>
__device__ __forceinline__ uint4 unpack8_lut(uint32_t neg_byte, uint32_t pos_byte, uint32_t lut_hi, uint32_t lut_lo) {
    uint32_t lo4 = nibble_to_bytes(neg_byte & 0xFu), hi4 = nibble_to_bytes(neg_byte >> 4);  // values 0-3, 4-7
    if (TERNARY) {
        lo4 = nibble_to_bytes(pos_byte & 0xFu) + 2u * lo4;
        hi4 = nibble_to_bytes(pos_byte >> 4) + 2u * hi4;
    }
    return make_uint4(__byte_perm(lut_hi, lut_lo, lo4 * 0x11u + 0x0404u), __byte_perm(lut_hi, lut_lo, (lo4 >> 16) * 0x11u + 0x0404u),
                      __byte_perm(lut_hi, lut_lo, hi4 * 0x11u + 0x0404u), __byte_perm(lut_hi, lut_lo, (hi4 >> 16) * 0x11u + 0x0404u));
}

// The one-pass fp16 mode scales the activations of a call by a power of two so that the largest magnitude lands in
// [2^14, 2^15): nothing overflows fp16 and values down to 2^-28 of the largest stay normal.  `amax_bits` is the
// bit pattern of max |a| (a non-negative float).  mul * inv == 1 exactly; the epilogue multiplies by inv.
__host__ __device__ __forceinline__ uint32_t f16_scale_exponent(uint32_t amax_bits) {
    int mb = 268 - static_cast<int>((amax_bits >> 23) & 0xffu);  // biased exponent of 2^(14 - floor(log2 amax))
    mb = mb < 1 ? 1 : (mb > 253 ? 253 : mb);
    return static_cast<uint32_t>(mb);
}
__device__ __forceinline__ float f16_scale_mul(uint32_t amax_bits) { return __uint_as_float(f16_scale_exponent(amax_bits) << 23); }
__device__ __forceinline__ float f16_scale_inv(uint32_t amax_bits) {
    return __uint_as_float((254u - f16_scale_exponent(amax_bits)) << 23);
}

// fp32 -> NPASS bf16 terms whose sum approximates (NPASS = 3: equals) the input; or its ternarisation.
template <int NPASS, bool TERNARISE>
__device__ __forceinline__ void split_terms(float v, float lo, float hi, uint16_t (&term)[NPASS]) {
    if (TERNARISE) {
        // TernaryMatrix::pack_from_float (GeMM/05-final/GeMM.cpp:99-106): strict compares.
        const float t = v < lo ? -1.0f : (v > hi ? 1.0f : 0.0f);
        term[0] = __bfloat16_as_ushort(__float2bfloat16_rn(t));
#pragma unroll
        for (int q = 1; q < NPASS; ++q) term[q] = 0;
    } else {
        float r = v;
#pragma unroll
        for (int q = 0; q < NPASS; ++q) {
            const __nv_bfloat16 h = __float2bfloat16_rn(r);
            term[q] = __bfloat16_as_ushort(h);
            // Exact in fp32; a non-finite input leaves its residual terms at zero.
            r = (q == 0 && !isfinite(r)) ? 0.0f : __fsub_rn(r, __bfloat162float(h));
        }
    }
}

// Two values at once, two terms each, as the packed words the channels-last form stores: hi = {rn(a), rn(b)},
// lo = {rn(a - hi_a), rn(b - hi_b)}, a in the low half.  Same values as split_terms<2, false> gives one by one (a
// non-finite input leaves its second term at zero); one packed conversion per pair and term instead of two scalar ones.
__device__ __forceinline__ void split_pair_terms(float a, float b, uint32_t& hi, uint32_t& lo) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    hi = *reinterpret_cast<const uint32_t*>(&h);
    const float ra = isfinite(a) ? __fsub_rn(a, __uint_as_float(hi << 16)) : 0.0f;
    const float rb = isfinite(b) ? __fsub_rn(b, __uint_as_float(hi & 0xffff0000u)) : 0.0f;
    const __nv_bfloat162 l = __floats2bfloat162_rn(ra, rb);
    lo = *reinterpret_cast<const uint32_t*>(&l);
}

// max |a| over a strided matrix as the bit pattern of a non-negative float (for those, integer order = float order;
// a NaN has the largest pattern and so wins).  *out must be zero before the launch.
__global__ void __launch_bounds__(256) absmax_kernel(const float* __restrict__ a, int64_t rows, int64_t cols, int64_t ld,
                                                     int vec_ok, uint32_t* __restrict__ out) {
    uint32_t best = 0u;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    if (vec_ok) {
        const int64_t c4 = cols / 4, total = rows * c4;
        for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
            const int64_t r = i / c4, c = (i - r * c4) * 4;
            const float4 v = __ldg(reinterpret_cast<const float4*>(a + r * ld + c));
            best = max(max(best, __float_as_uint(v.x) & 0x7fffffffu), __float_as_uint(v.y) & 0x7fffffffu);
            best = max(max(best, __float_as_uint(v.z) & 0x7fffffffu), __float_as_uint(v.w) & 0x7fffffffu);
        }
    } else {
        const int64_t total = rows * cols;
        for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
            const int64_t r = i / cols;
            best = max(best, __float_as_uint(__ldg(a + r * ld + (i - r * cols))) & 0x7fffffffu);
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) best = max(best, __shfl_xor_sync(0xffffffffu, best, o));
    if ((threadIdx.x & 31) == 0 && best != 0u) atomicMax(out, best);
}

namespace tc {

constexpr int BM = 128;
constexpr int BK = 64;          // 64 bf16 = 128 bytes = one swizzle row
constexpr int UMMA_K = 16;
constexpr int A_TILE_BYTES = BM * BK * 2;
constexpr int kProducerWarp = 0, kMmaWarp = 1;
constexpr int kBuildThreads = 256, kEpilogueThreads = 128;
constexpr int kThreads = 64 + kBuildThreads + kEpilogueThreads;
constexpr int kDefaultGroupM = 4;  // rasterisation: this many m-tiles share a sweep over n for L2 reuse (Params::group_m)
// Ring of packed-word tiles, each covering 2 k-blocks (128 k): 2 slots keep the GEMM fed; the convolutions,
// whose k-blocks are short-lived, run 4 slots ahead.
constexpr int kWordStagesGemm = 2, kWordStagesConv = 4;
constexpr int kAuxBarrierBytes = 1024;
constexpr int kMaxOutputs = 8;           // destinations of the multi-destination epilogue (GPUs of one box)
constexpr int kStageOutBytes = 4 * 4096;  // per epilogue warp: 32 rows x 32 fp32 transposition buffer
constexpr int kSmemLimit = 232448;  // 227 KB opt-in maximum per CTA
// Accumulation steps (k elements x passes) after which a fresh accumulator is started.
constexpr int kMaxAccumSteps = 4096;

// Operand modes that lower a convolution (see AMODE at the kernel).
__host__ __device__ constexpr bool is_conv_mode(int amode) { return amode == 1 || amode == 2 || amode == 4; }

// MULTI: the multi-destination epilogue (column-sharded multi-GPU GEMM) is compiled in, with its staging buffers.
template <int BN, int NPASS, bool TERNARY, int BSRC = 0, bool CONV = false, bool MULTI = false>
struct Cfg {
    static constexpr bool DENSE = BSRC == 1;
    // k-blocks covered by one packed-word tile.  A TMA box is delivered row by row (a row here = the words of one
    // column), so longer rows mean fewer rows per k-block for the TMA unit: 32-byte rows (4 k-blocks) where the
    // shared memory allows it, 16-byte rows (2 k-blocks) with two planes or with the staging buffers of MULTI.
    // (Measured A/B at 16384^3 on one box, binary: 11.74-11.82 ms against 11.67-11.85 ms -- no difference; with TWO
    // planes the 16-byte rows are what binds: 256 activation rows plus 2 x 128 word rows per k-block through a TMA unit
    // that moves a row in 3-4 cycles is longer than the k-block's MMAs, and the ternary 4096 x 4096 x 11008 product ran
    // 20 % slower than the binary one until its word rows were 32 bytes too.)
    static constexpr int WORD_KB = (!MULTI && !CONV && BSRC == 0) ? 4 : 2;
    // Word tiles in flight.  The build warps copy a tile's words to registers as soon as it arrives and hand the slot
    // back at once, so the two 4-k-block planes of the ternary GEMM (16 KB) get along with a single slot -- two
    // would cost a pipeline stage.  (TMA-fed weights use no words.)
    static constexpr int kWordStages = BSRC != 0 ? 1 : (CONV ? kWordStagesConv : ((TERNARY && WORD_KB == 4) ? 1 : kWordStagesGemm));
    static constexpr int B_TILE_BYTES = BN * BK * 2;
    static constexpr int B_TERMS = DENSE ? 2 : 1;  // dense weights: hi and lo bf16 terms
    static constexpr int B_BYTES = B_TERMS * B_TILE_BYTES;
    static constexpr int STAGE_BYTES = B_BYTES + NPASS * A_TILE_BYTES;
    static constexpr int WORD_ROW_BYTES = 8 * WORD_KB;  // two words per k-block and column
    static constexpr int WORD_TILE_BYTES = BN * WORD_ROW_BYTES * (TERNARY ? 2 : 1);
    // barriers + alpha/bias staging (x2 buffers) + packed-word ring (+ epilogue transposition buffers)
    static constexpr int AUX_BYTES = kAuxBarrierBytes + 4 * BN * 4 + kWordStages * WORD_TILE_BYTES + (MULTI ? kStageOutBytes : 0);
    static constexpr int RAW_STAGES = (kSmemLimit - 1024 - AUX_BYTES) / STAGE_BYTES;
    static constexpr int STAGES = RAW_STAGES > 6 ? 6 : RAW_STAGES;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + AUX_BYTES + 1024;  // + alignment slack
    // Dense weights with BN <= 128: one instruction multiplies the high activation term with the high AND the low
    // weight tile (they lie one behind the other in shared memory = one K-major operand of 2 BN rows), so that an
    // accumulator is 2 BN columns wide and the epilogue adds its halves.  Two instructions per k-step instead of three;
    // what an instruction costs at these widths is mostly its operand fetch, and the activation tile is fetched twice
    // instead of three times.
    static constexpr bool DENSE_WIDE = DENSE && BN <= 128;
    static constexpr int ACC_COLS = DENSE_WIDE ? 2 * BN : BN;
    static constexpr int TMEM_COLS = 2 * ACC_COLS;
    static_assert(STAGES >= 2, "need at least a double-buffered pipeline");
    static_assert(TMEM_COLS == 128 || TMEM_COLS == 256 || TMEM_COLS == 512, "TMEM columns must be a power of two");
    static_assert(B_TILE_BYTES % 1024 == 0, "operand tiles must stay 1024-byte aligned");
};

// Geometry of the implicit im2col (CONV mode).  Row m of the GEMM is output pixel
// (img, oh, ow) = (m / (OH*OW), ...); column k is (c, i, j) = the reference's im2col order
// (tbn-runtime/src/operators/conv2d.cpp:484-501).  `table[k]` = {input offset of tap k relative to the
// pixel's window origin, (dy << 16) | (dx & 0xffff)} with dy = i*dilation_h, dx = j*dilation_w;
// entries for k >= K carry dy = 0x7fff so that they always fall outside the image.
struct ConvGeom {
    const float* x;
    const int2* table;
    int C, H, W, OH, OW;
    int sh, sw, ph, pw;
    float act_lo, act_hi;  // thresholds when the activations are ternarised (TBN mode)
    // Channels-last fast path (AMODE 2): xs[term][img][h][w][c] bf16, K ordered tap-major:
    // k = (i*kw + j)*C + c, so k-block kb covers tap kb / cblocks and channels [64*(kb % cblocks), +64).
    const __nv_bfloat16* xs;
    int64_t xs_term_stride;  // elements between the bf16 terms
    int kw, taps, dh, dw, cblocks;
    // Patch mode (AMODE 4): an m-tile is a box of pbi images x pbh output rows x pbw output columns
    // (pbi*pbh*pbw <= 128 GEMM rows, row = (bi*pbh + bh)*pbw + bw); patches_w x patches_h boxes cover one image
    // group.  a_box_bytes: bytes one TMA box delivers (all terms together).
    int pbw, pbh, pbi, patches_w, patches_h, a_box_bytes;
    // Patch mode, stacked rows (stack_rows > 0, pbw = OW): the output rows of all images form one sequence
    // s = img * OH + oh and an m-tile is `stack_rows` consecutive rows of it, whatever images they belong to, so
    // that tiles stay full where an image's pixel count is not a multiple of the tile (14 x 14: 9 rows = 126 of
    // 128 GEMM rows instead of 126 and 70 in turn; 7 x 7: 18 rows of up to four images instead of two whole
    // images).  The rows a tile takes from one image are one TMA box; the box height is a property of the tensor
    // map, so there is one map per height: heights 1 .. 8 in the (otherwise unused) destination maps, the largest
    // height min(stack_rows, OH) <= 9 in the activation map itself.
    int stack_rows, stack_max_h;
};

// Tensor maps of the destinations of the multi-destination epilogue: [N columns][M rows] fp32 with row stride
// ldc, box 32 x 32, 128-byte swizzle.  Rows and columns past the matrix are clipped by the hardware.
struct OutMaps {
    CUtensorMap m[kMaxOutputs];
};

struct Params {
    int M, N;
    int num_kb;            // K_pad / 64
    int tiles_m, tiles_n;
    int group_m;           // rasterisation group (>= 1): m-tiles that share one sweep over the column tiles
    float* c;
    int64_t ldc;           // row-major output: row stride
    int out_nchw;          // 1: output element (m, n) lives at ((img*N + n)*OH*OW + pixel)
    int out_hw;            // OH*OW when out_nchw
    Epilogue ep;
    int* err_word;
    int c_vec_ok;          // row-major output rows are 16-byte aligned
    int num_seg;           // K segments per tile, each with a fresh accumulator
    int kb_per_seg;        // k-blocks per segment (the last one may be shorter)
    float4* scratch;       // [gridDim.x][BN/4][128] partial sums, used when num_seg > 1
    // Multi-destination epilogue (column-sharded multi-GPU GEMM): when num_out > 0 the finished tile is
    // written to every destination (same row stride ldc) -- the local result buffer and the peers' buffers
    // mapped into this GPU's address space -- instead of p.c: each epilogue warp stages its 32 x 32 block in
    // shared memory and one lane issues a tiled TMA store per destination (OutMaps), so that the transfer over
    // NVLink runs asynchronously beside the next block.  out_list keeps the raw pointers (argument checks).
    int num_out;
    float* out_list[kMaxOutputs];
    // Optional second result of a convolution: the output as channels-last bf16 terms [2][pixel][N] (what the
    // next convolution's patch mode reads), written by the epilogue so that no pre-pass is needed in between.
    // p.c may be null when only this form is wanted.
    __nv_bfloat16* out_cl;
    int64_t out_cl_term_stride;
    // One-pass fp16 mode: both operands are fp16 instead of bf16 (same tiles, same swizzle; only the instruction
    // descriptor and the bit pattern of +-1 differ) and the result is multiplied by the inverse of the power-of-two
    // scale the activation pre-pass applied (derived from *amax_bits, the bit pattern of max |a| of this call).
    int f16;
    const uint32_t* amax_bits;
    // AMODE 3: the fp32 activation rows themselves (16-byte aligned, lda % 4 == 0, K % 4 == 0).
    const float* a_rows;
    int64_t lda;
    int K;
    ConvGeom conv;
};

__device__ __forceinline__ void tile_coords(int t, int tiles_m, int tiles_n, int group_m, int& tm, int& tn) {
    const int group_size = group_m * tiles_n;
    const int g = t / group_size;
    const int first_m = g * group_m;
    const int gm = min(tiles_m - first_m, group_m);
    const int r = t - g * group_size;
    tm = first_m + r % gm;
    tn = r / gm;
}

// tmap_a: split activations (GEMM mode).  tmap_neg / tmap_pos: packed word planes; with BSRC 1 or 2 tmap_neg is
// the map of the split weights [2][N_pad][K_pad] instead.
// AMODE: source of the activation operand.  0 = TMA from pre-split [terms][M][K] (plain GEMM);
// 1 = element-wise gather from NCHW fp32 (any convolution geometry); 2 = cp.async from the channels-last
// bf16 copy (convolutions with C % 64 == 0); 3 = the fp32 rows of A read by the build warps and split in
// registers (plain GEMM without the separate split pass; loads run two k-blocks ahead of their use);
// 4 = convolution whose m-tiles are rectangular patches of output pixels, so that the activation operand of one
// filter tap and 64 channels is ONE tiled TMA box of the channels-last copy [term][img][h][w][c] (the hardware
// zero-fills the halo, the tensor map's element strides implement the convolution stride): no thread touches
// the operands.
template <int BN, int NPASS, bool TERNARY, int AMODE, bool TERN_ACT, int BSRC, bool MULTI>
__global__ void __launch_bounds__(kThreads, 1) gemm_tc_kernel(const __grid_constant__ CUtensorMap tmap_a,
                                                              const __grid_constant__ CUtensorMap tmap_neg,
                                                              const __grid_constant__ CUtensorMap tmap_pos,
                                                              const __grid_constant__ OutMaps out_maps, const Params p) {
    constexpr bool CONV = is_conv_mode(AMODE);
    constexpr bool FAST = AMODE == 2;
    constexpr bool ROWS = AMODE == 3;
    constexpr bool PATCH = AMODE == 4;
    constexpr bool BUILT_A = AMODE == 1 || AMODE == 2 || ROWS;  // the build warps write the activation operand
    static_assert(!PATCH || BSRC != 0, "patch-mode convolutions take both operands by TMA");
    constexpr bool DENSE = BSRC == 1;      // two-term float weights
    constexpr bool TMA_B = BSRC != 0;      // the weight tile arrives by TMA instead of being unpacked here
    static_assert(!(ROWS && TMA_B), "TMA-fed weights take their activations by TMA or by the convolution gathers");
    static_assert(BSRC != 2 || !TERNARY, "expanded weights carry their zeros themselves");
    using C = Cfg<BN, NPASS, TERNARY, BSRC, CONV, MULTI>;
    constexpr int kWordStages = C::kWordStages;
    constexpr int WORD_KB = C::WORD_KB;
    static_assert(!MULTI || (AMODE == 0 && BSRC == 0), "the multi-destination epilogue belongs to the plain GEMM");
    static_assert(!DENSE || (NPASS == 2 && !TERNARY && !TERN_ACT), "dense weights use the two-term split on both sides");
    // Which operands arrive by TMA (signalled on full_a) and which are built by the build warps (full_b).
    constexpr bool kTmaOperands = !BUILT_A || TMA_B;
    constexpr bool kBuiltOperands = BUILT_A || !TMA_B;
    // When no operand is built by threads, the eight build warps join the epilogue: three warps per TMEM lane
    // quarter, each taking every third 32-column chunk.
    constexpr bool kWideEpilogue = !kBuiltOperands;
    constexpr int kEpiGroups = kWideEpilogue ? 3 : 1;
    constexpr int kEpiThreads = kEpilogueThreads * kEpiGroups;
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
    float* stage_out = reinterpret_cast<float*>(aux_ptr + kAuxBarrierBytes + 4 * BN * 4 + kWordStages * C::WORD_TILE_BYTES);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int total_tiles = p.tiles_m * p.tiles_n;

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::STAGES; ++s) {
            ptx::mbar_init(bar_full_a + 8 * s, 1);
            ptx::mbar_init(bar_full_b + 8 * s, kBuildThreads);
            ptx::mbar_init(bar_empty + 8 * s, 1);
        }
        for (int b = 0; b < 2; ++b) {
            ptx::mbar_init(bar_tmem_full + 8 * b, 1);
            ptx::mbar_init(bar_tmem_empty + 8 * b, kEpiThreads);
        }
        for (int w = 0; w < kWordStages; ++w) {
            ptx::mbar_init(bar_full_w + 8 * w, 1);
            ptx::mbar_init(bar_empty_w + 8 * w, kBuildThreads);
        }
        ptx::fence_barrier_init();
        if (!BUILT_A) ptx::prefetch_tensormap(&tmap_a);
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
                tile_coords(t, p.tiles_m, p.tiles_n, p.group_m, tm, tn);
                // Patch mode: input coordinates of the patch's first pixel under tap (0, 0), and the tap state.
                int pw0 = 0, ph0 = 0, pimg0 = 0, p_cb = 0, p_ti = 0, p_tj = 0;
                if (PATCH) {
                    const int px = tm % p.conv.patches_w;
                    const int py = (tm / p.conv.patches_w) % p.conv.patches_h;
                    pimg0 = (tm / (p.conv.patches_w * p.conv.patches_h)) * p.conv.pbi;
                    pw0 = px * p.conv.pbw * p.conv.sw - p.conv.pw;
                    ph0 = py * p.conv.pbh * p.conv.sh - p.conv.ph;
                }
                for (int kb = 0; kb < p.num_kb; ++kb) {
                    if (!TMA_B && (kb % WORD_KB) == 0) {
                        // Packed words of k-blocks kb .. kb + WORD_KB - 1 for the BN columns of this tile
                        // (rows past the end of the plane are zero-filled by TMA).
                        if (!ptx::mbar_wait(bar_empty_w + 8 * wstage, wphase ^ 1u, p.err_word, kErrWaitEmpty)) {
                            ok = false;
                            break;
                        }
                        const uint32_t wbar = bar_full_w + 8 * wstage;
                        const uint32_t wdst = word_ring + wstage * C::WORD_TILE_BYTES;
                        ptx::mbar_arrive_expect_tx(wbar, C::WORD_TILE_BYTES);
                        ptx::tma_load_2d(wdst, &tmap_neg, kb * 2, tn * BN, wbar);
                        if (TERNARY) ptx::tma_load_2d(wdst + BN * C::WORD_ROW_BYTES, &tmap_pos, kb * 2, tn * BN, wbar);
                        if (++wstage == kWordStages) {
                            wstage = 0;
                            wphase ^= 1u;
                        }
                    }
                    if (kTmaOperands) {
                        if (!ptx::mbar_wait(bar_empty + 8 * stage, phase ^ 1u, p.err_word, kErrWaitEmpty)) {
                            ok = false;
                            break;
                        }
                        const uint32_t bar = bar_full_a + 8 * stage;
                        ptx::mbar_arrive_expect_tx(bar, (BUILT_A ? 0 : (PATCH ? p.conv.a_box_bytes : NPASS * A_TILE_BYTES)) +
                                                            (TMA_B ? C::B_BYTES : 0));
                        const uint32_t b_dst = base + stage * C::STAGE_BYTES;
                        const uint32_t a_dst = b_dst + C::B_BYTES;
                        if (TMA_B) {
#pragma unroll
                            for (int q = 0; q < C::B_TERMS; ++q)
                                ptx::tma_load_3d(b_dst + q * C::B_TILE_BYTES, &tmap_neg, kb * BK, tn * BN, q, bar);
                        }
                        if (PATCH) {
                            // One box per term: channels [64*cb, +64) of the input pixels under filter tap (ti, tj)
                            // for the whole patch; coordinates outside the image read zeros.
                            const int x = pw0 + p_tj * p.conv.dw, y = ph0 + p_ti * p.conv.dh;
                            const bool tap_valid = p_ti * p.conv.kw + p_tj < p.conv.taps;
                            if (p.conv.stack_rows > 0) {
                                // One box per image the tile's rows come from (rows past the last image: zeros).
                                int img = (tm * p.conv.stack_rows) / p.conv.OH;
                                int oh = tm * p.conv.stack_rows - img * p.conv.OH;
                                int done = 0;
                                while (done < p.conv.stack_rows) {
                                    const int h = min(p.conv.stack_rows - done, p.conv.OH - oh);
                                    const CUtensorMap* map = h == p.conv.stack_max_h ? &tmap_a : &out_maps.m[h - 1];
                                    const int yr = oh * p.conv.sh - p.conv.ph + p_ti * p.conv.dh;
#pragma unroll
                                    for (int q = 0; q < NPASS; ++q)
                                        ptx::tma_load_5d(a_dst + q * A_TILE_BYTES + done * p.conv.OW * 128, map, p_cb * BK,
                                                         tap_valid ? -p.conv.pw + p_tj * p.conv.dw : -(1 << 20), yr, img, q, bar);
                                    done += h;
                                    oh = 0;
                                    ++img;
                                }
                            } else
#pragma unroll
                            for (int q = 0; q < NPASS; ++q)
                                ptx::tma_load_5d(a_dst + q * A_TILE_BYTES, &tmap_a, p_cb * BK, tap_valid ? x : -(1 << 20), y, pimg0, q, bar);
                            if (++p_cb == p.conv.cblocks) {
                                p_cb = 0;
                                if (++p_tj == p.conv.kw) {
                                    p_tj = 0;
                                    ++p_ti;
                                }
                            }
                        } else if (!BUILT_A) {
#pragma unroll
                            for (int q = 0; q < NPASS; ++q)
                                ptx::tma_load_3d(a_dst + q * A_TILE_BYTES, &tmap_a, kb * BK, tm * BM, q, bar);
                        }
                        if (++stage == C::STAGES) {
                            stage = 0;
                            phase ^= 1u;
                        }
                    }
                }
            }
        }
    } else if (warp == kMmaWarp) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            const uint32_t idesc = p.f16 ? ptx::umma_idesc_f16_f32(BM, BN) : ptx::umma_idesc_bf16_f32(BM, BN);
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
                    const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(buf * C::ACC_COLS);
                    const int kb_begin = seg * p.kb_per_seg;
                    const int kb_end = min(p.num_kb, kb_begin + p.kb_per_seg);
                    for (int kb = kb_begin; kb < kb_end; ++kb) {
                        // TMA-delivered operands signal on full_a, operands written by the build warps on full_b.
                        if ((kTmaOperands && !ptx::mbar_wait(bar_full_a + 8 * stage, phase, p.err_word, kErrWaitFullA)) ||
                            (kBuiltOperands && !ptx::mbar_wait(bar_full_b + 8 * stage, phase, p.err_word, kErrWaitFullB))) {
                            ok = false;
                            break;
                        }
                        ptx::tc_fence_after_sync();
                        const uint32_t b_addr = base + stage * C::STAGE_BYTES;
                        const uint32_t a_addr = b_addr + C::B_BYTES;
                        // Binary/ternary weights: every activation term against the one exact weight tile.
                        // Dense weights: hi*hi + hi*lo + lo*hi (the lo*lo term is below fp32 resolution).
                        if constexpr (C::DENSE_WIDE) {
                            const uint32_t idesc_wide = ptx::umma_idesc_bf16_f32(BM, 2 * BN);
#pragma unroll
                            for (int k4 = 0; k4 < BK / UMMA_K; ++k4) {  // hi x [hi ; lo] -> columns [0, 2 BN)
                                const uint64_t a_desc = ptx::umma_desc_k_sw128(a_addr + k4 * UMMA_K * 2);
                                const uint64_t b_desc = ptx::umma_desc_k_sw128(b_addr + k4 * UMMA_K * 2);
                                ptx::umma_bf16(d_tmem, a_desc, b_desc, idesc_wide, (kb != kb_begin || k4 != 0) ? 1u : 0u);
                            }
#pragma unroll
                            for (int k4 = 0; k4 < BK / UMMA_K; ++k4) {  // lo x hi -> columns [0, BN)
                                const uint64_t a_desc = ptx::umma_desc_k_sw128(a_addr + A_TILE_BYTES + k4 * UMMA_K * 2);
                                const uint64_t b_desc = ptx::umma_desc_k_sw128(b_addr + k4 * UMMA_K * 2);
                                ptx::umma_bf16(d_tmem, a_desc, b_desc, idesc, 1u);
                            }
                        }
                        constexpr int kPairs = C::DENSE_WIDE ? 0 : (DENSE ? 3 : NPASS);
#pragma unroll
                        for (int pr = 0; pr < kPairs; ++pr) {
                            const int qa = DENSE ? (pr == 2 ? 1 : 0) : pr;
                            const int qb = DENSE ? (pr == 1 ? 1 : 0) : 0;
#pragma unroll
                            for (int k4 = 0; k4 < BK / UMMA_K; ++k4) {
                                const uint64_t a_desc =
                                    ptx::umma_desc_k_sw128(a_addr + qa * A_TILE_BYTES + k4 * UMMA_K * 2);
                                const uint64_t b_desc =
                                    ptx::umma_desc_k_sw128(b_addr + qb * C::B_TILE_BYTES + k4 * UMMA_K * 2);
                                ptx::umma_bf16(d_tmem, a_desc, b_desc, idesc, (kb != kb_begin || pr != 0 || k4 != 0) ? 1u : 0u);
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
    } else if (!kWideEpilogue && warp < 2 + kBuildThreads / 32) {
        // ------------------------------------------------------------ operand build
        static_assert(BN <= kBuildThreads, "one build thread per weight column of the tile");
        const int r = threadIdx.x - 64;  // weight column (row of the K-major weight tile) of this thread
        const uint32_t one16 = p.f16 ? kOneF16 : kOneBf16;
        // byte tables of unpack8_lut: binary {+1, -1}, ternary {0, +1, -1}
        const uint32_t hi_p = one16 >> 8, hi_m = hi_p | 0x80u, lo_b = one16 & 0xffu;
        const uint32_t lut_hi = TERNARY ? ((hi_p << 8) | (hi_m << 16)) : (hi_p | (hi_m << 8));
        const uint32_t lut_lo = TERNARY ? ((lo_b << 8) | (lo_b << 16)) : (lo_b | (lo_b << 8));
        // CONV mode: this thread also builds activation row (r & 127), 16-byte chunks (r >> 7) + {0, 2, 4, 6}.
        const int a_row = r & (BM - 1);
        const int a_chunk0 = r >> 7;
        int stage = 0, wstage = 0;
        uint32_t phase = 0, wphase = 0;
        bool ok = true;
        uint4 wn = make_uint4(0u, 0u, 0u, 0u), wp = make_uint4(0u, 0u, 0u, 0u), wp2 = make_uint4(0u, 0u, 0u, 0u);
        uint4 wn2 = make_uint4(0u, 0u, 0u, 0u);  // words of the third and fourth k-block of a 4-k-block tile
        // FAST: oldest stage whose copies are in flight and whose arrive is still owed, and how many are owed.
        constexpr int kCopyLag = C::STAGES >= 4 ? 2 : 1;
        int pending_stage = 0, pending_count = 0;
        // ROWS: this thread reads float4 number (r & 15) of the 64-float k-block slice of rows (r >> 4) + 16*j, so
        // that 16 lanes cover one row's 256 bytes.  The loads run two k-blocks ahead of their use, across tile
        // boundaries: pf_a holds the k-block consumed next, pf_b the one after.
        int pf_t = blockIdx.x, pf_kb = 0, pf_tm = 0;
        float4 pf_a[8], pf_b[8];
        auto rows_load = [&](float4 (&dst)[8]) {
            const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
            if (pf_t < total_tiles) {
                if (pf_kb == 0) {
                    int tn_unused;
                    tile_coords(pf_t, p.tiles_m, p.tiles_n, p.group_m, pf_tm, tn_unused);
                }
                const int k0 = pf_kb * BK + (r & 15) * 4;
                const float* src = p.a_rows + (static_cast<int64_t>(pf_tm) * BM + (r >> 4)) * p.lda + k0;
                const int rows_left = p.M - (pf_tm * BM + (r >> 4));
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    dst[j] = (k0 < p.K && 16 * j < rows_left)
                                 ? __ldg(reinterpret_cast<const float4*>(src + static_cast<int64_t>(16 * j) * p.lda))
                                 : zero;
                if (++pf_kb == p.num_kb) {
                    pf_kb = 0;
                    pf_t += gridDim.x;
                }
            } else {
#pragma unroll
                for (int j = 0; j < 8; ++j) dst[j] = zero;
            }
        };
        if (ROWS) {
            rows_load(pf_a);
            rows_load(pf_b);
        }
        for (int t = blockIdx.x; kBuiltOperands && t < total_tiles && ok; t += gridDim.x) {
            int tm, tn;
            tile_coords(t, p.tiles_m, p.tiles_n, p.group_m, tm, tn);
            // Window origin of this thread's output pixel (CONV modes).  Element-wise gather: one pixel per
            // thread (lanes = consecutive pixels).  Channels-last copy: four pixels per thread, rows
            // (r >> 3) + 32*j, and ONE 16-byte chunk r & 7, so that 8 lanes cover one pixel's 128 bytes and a
            // warp reads 512 contiguous bytes.
            int ih0 = 0, iw0 = 0;
            bool row_valid = false;
            const float* xwin = nullptr;
            int f_ih0[4], f_iw0[4];
            int64_t f_base[4];  // element offset of (image, window origin, this thread's 8 channels) in xs
            bool f_valid[4];
            int f_cb = 0, f_ti = 0, f_tj = 0;  // channel block and filter tap of the current k-block
            if (CONV && !FAST) {
                const int64_t m = static_cast<int64_t>(tm) * BM + a_row;
                row_valid = m < p.M;
                const int hw = p.conv.OH * p.conv.OW;
                const int64_t img = m / hw;
                const int pix = static_cast<int>(m - img * hw);
                const int oh = pix / p.conv.OW, ow = pix - oh * p.conv.OW;
                ih0 = oh * p.conv.sh - p.conv.ph;
                iw0 = ow * p.conv.sw - p.conv.pw;
                xwin = p.conv.x + img * p.conv.C * p.conv.H * p.conv.W +
                       static_cast<int64_t>(ih0) * p.conv.W + iw0;
            }
            if (FAST) {
                const int hw = p.conv.OH * p.conv.OW;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int64_t m = static_cast<int64_t>(tm) * BM + (r >> 3) + 32 * j;
                    f_valid[j] = m < p.M;
                    const int64_t img = m / hw;
                    const int pix = static_cast<int>(m - img * hw);
                    const int oh = pix / p.conv.OW, ow = pix - oh * p.conv.OW;
                    f_ih0[j] = oh * p.conv.sh - p.conv.ph;
                    f_iw0[j] = ow * p.conv.sw - p.conv.pw;
                    f_base[j] = (img * p.conv.H * p.conv.W + static_cast<int64_t>(f_ih0[j]) * p.conv.W + f_iw0[j]) * p.conv.C +
                                (r & 7) * 8;
                }
            }
            for (int kb = 0; kb < p.num_kb; ++kb) {
                if (!TMA_B && (kb % WORD_KB) == 0) {
                    // Words of this and the next k-block(s): shared memory -> registers, then free the slot.
                    if (!ptx::mbar_wait(bar_full_w + 8 * wstage, wphase, p.err_word, kErrWaitFullB)) {
                        ok = false;
                        break;
                    }
                    if (r < BN) {
                        const uint32_t wt = word_ring + wstage * C::WORD_TILE_BYTES + r * C::WORD_ROW_BYTES;
                        wn = ptx::ld_shared_v4(wt);
                        if (WORD_KB == 4) wn2 = ptx::ld_shared_v4(wt + 16);
                        if (TERNARY) wp = ptx::ld_shared_v4(wt + BN * C::WORD_ROW_BYTES);
                        if (TERNARY && WORD_KB == 4) wp2 = ptx::ld_shared_v4(wt + BN * C::WORD_ROW_BYTES + 16);
                    }
                    // The slot may be refilled by TMA as soon as this arrive lands, so the loads above
                    // must have returned their data first: the arrive is made to depend on them.
                    ptx::mbar_arrive_after(bar_empty_w + 8 * wstage, wn.x ^ wn.w ^ wp.x ^ wp.w ^ wn2.x ^ wn2.w ^ wp2.x ^ wp2.w);
                    if (++wstage == kWordStages) {
                        wstage = 0;
                        wphase ^= 1u;
                    }
                }
                float av[32];
                if (CONV && !FAST) {
                    // Issue this k-block's 32 gathers before waiting for the stage, so that their latency
                    // overlaps the wait.  Lanes hold consecutive output pixels: coalesced for stride 1.
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        // An 8-element chunk that lies entirely beyond the real K is zero: no table reads, no tests.
                        if (kb * BK + (a_chunk0 + 2 * j) * 8 >= p.K) {
#pragma unroll
                            for (int i = 0; i < 8; ++i) av[j * 8 + i] = 0.0f;
                            continue;
                        }
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const int k = kb * BK + (a_chunk0 + 2 * j) * 8 + i;
                            const int2 e = __ldg(p.conv.table + k);
                            const int ih = ih0 + (e.y >> 16);
                            const int iw = iw0 + static_cast<int>(static_cast<short>(e.y & 0xffff));
                            const bool inside = row_valid && static_cast<unsigned>(ih) < static_cast<unsigned>(p.conv.H) &&
                                                static_cast<unsigned>(iw) < static_cast<unsigned>(p.conv.W);
                            av[j * 8 + i] = inside ? __ldg(xwin + e.x) : 0.0f;
                        }
                    }
                }
                if (!ptx::mbar_wait(bar_empty + 8 * stage, phase ^ 1u, p.err_word, kErrWaitEmpty)) {
                    ok = false;
                    break;
                }
                uint8_t* stage_ptr = base_ptr + stage * C::STAGE_BYTES;
                if (!TMA_B && r < BN) {
                    uint8_t* row = stage_ptr + r * 128;
                    const uint4 wsel = (WORD_KB == 4 && (kb & 2)) ? wn2 : wn;
                    const uint32_t nw[2] = {(kb & 1) ? wsel.z : wsel.x, (kb & 1) ? wsel.w : wsel.y};
                    const uint4 psel = (WORD_KB == 4 && (kb & 2)) ? wp2 : wp;
                    const uint32_t pw[2] = {(kb & 1) ? psel.z : psel.x, (kb & 1) ? psel.w : psel.y};
#pragma unroll
                    for (int c = 0; c < 8; ++c) {
                        const uint32_t nb = (nw[c >> 2] >> (8 * (c & 3))) & 0xffu;
                        const uint32_t pb = (pw[c >> 2] >> (8 * (c & 3))) & 0xffu;
                        // 16-byte chunk c of row r lands at chunk (c ^ (r & 7)): the 128-byte swizzle.
                        *reinterpret_cast<uint4*>(row + ((c ^ (r & 7)) << 4)) = unpack8_lut<TERNARY>(nb, pb, lut_hi, lut_lo);
                    }
                }
                if (FAST) {
                    // One filter tap and 64 channels per k-block: this thread copies its 16-byte chunk (8 channels)
                    // of four pixels per term, or zeros where the tap falls outside the image.
                    // (tap, channel block) advance with kb: no divisions in the loop.
                    const int dy = f_ti * p.conv.dh, dx = f_tj * p.conv.dw;
                    const bool tap_valid = f_ti * p.conv.kw + f_tj < p.conv.taps;
                    const int64_t tap_off = (static_cast<int64_t>(dy) * p.conv.W + dx) * p.conv.C + f_cb * BK;
                    if (++f_cb == p.conv.cblocks) {
                        f_cb = 0;
                        if (++f_tj == p.conv.kw) {
                            f_tj = 0;
                            ++f_ti;
                        }
                    }
                    const uint32_t a_base = base + stage * C::STAGE_BYTES + C::B_BYTES;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const int row = (r >> 3) + 32 * j;
                        const int ih = f_ih0[j] + dy, iw = f_iw0[j] + dx;
                        const bool inside = f_valid[j] && tap_valid &&
                                            static_cast<unsigned>(ih) < static_cast<unsigned>(p.conv.H) &&
                                            static_cast<unsigned>(iw) < static_cast<unsigned>(p.conv.W);
                        const __nv_bfloat16* src = inside ? p.conv.xs + (f_base[j] + tap_off) : p.conv.xs;
                        const uint32_t dst = a_base + row * 128 + (((r & 7) ^ (row & 7)) << 4);
#pragma unroll
                        for (int q = 0; q < NPASS; ++q)
                            ptx::cp_async_16(dst + q * A_TILE_BYTES, src + q * p.conv.xs_term_stride, inside ? 16u : 0u);
                    }
                    ptx::cp_async_commit();
                    // The arrive for a stage is deferred by kCopyLag k-blocks, so that several stages of copies
                    // are in flight and their latency overlaps: wait_group leaves the newest kCopyLag groups
                    // pending, i.e. the group of the stage being released has landed; the writer then fences
                    // and signals.
                    if (pending_count == kCopyLag) {
                        ptx::cp_async_wait<kCopyLag>();
                        ptx::fence_proxy_async_smem();
                        ptx::mbar_arrive(bar_full_b + 8 * pending_stage);
                        if (++pending_stage == C::STAGES) pending_stage = 0;
                    } else {
                        if (pending_count == 0) pending_stage = stage;
                        ++pending_count;
                    }
                    if (++stage == C::STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
                    continue;
                }
                if (ROWS) {
                    uint8_t* a_tile = stage_ptr + C::B_BYTES;
                    const int c16 = (r & 15) >> 1, half = (r & 1) * 8;
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const int row = (r >> 4) + 16 * j;
                        const float f[4] = {pf_a[j].x, pf_a[j].y, pf_a[j].z, pf_a[j].w};
                        uint32_t packed[NPASS][2];
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            uint16_t term[NPASS];
                            split_terms<NPASS, TERN_ACT>(f[i], p.conv.act_lo, p.conv.act_hi, term);
#pragma unroll
                            for (int q = 0; q < NPASS; ++q) {
                                if (i & 1) packed[q][i >> 1] |= static_cast<uint32_t>(term[q]) << 16;
                                else packed[q][i >> 1] = term[q];
                            }
                        }
#pragma unroll
                        for (int q = 0; q < NPASS; ++q)
                            *reinterpret_cast<uint2*>(a_tile + q * A_TILE_BYTES + row * 128 + ((c16 ^ (row & 7)) << 4) + half) =
                                make_uint2(packed[q][0], packed[q][1]);
                    }
#pragma unroll
                    for (int j = 0; j < 8; ++j) pf_a[j] = pf_b[j];
                    rows_load(pf_b);
                }
                if (CONV) {
                    uint8_t* a_tile = stage_ptr + C::B_BYTES + a_row * 128;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        uint32_t packed[NPASS][4];
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            uint16_t term[NPASS];
                            split_terms<NPASS, TERN_ACT>(av[j * 8 + i], p.conv.act_lo, p.conv.act_hi, term);
#pragma unroll
                            for (int q = 0; q < NPASS; ++q) {
                                if (i & 1) packed[q][i >> 1] |= static_cast<uint32_t>(term[q]) << 16;
                                else packed[q][i >> 1] = term[q];
                            }
                        }
                        const int c = a_chunk0 + 2 * j;
#pragma unroll
                        for (int q = 0; q < NPASS; ++q)
                            *reinterpret_cast<uint4*>(a_tile + q * A_TILE_BYTES + ((c ^ (a_row & 7)) << 4)) =
                                make_uint4(packed[q][0], packed[q][1], packed[q][2], packed[q][3]);
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
        if (FAST && ok && pending_count > 0) {  // the deferred arrives of the last stages
            ptx::cp_async_wait<0>();
            ptx::fence_proxy_async_smem();
            for (; pending_count > 0; --pending_count) {
                ptx::mbar_arrive(bar_full_b + 8 * pending_stage);
                if (++pending_stage == C::STAGES) pending_stage = 0;
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue
        const int e = kWideEpilogue ? threadIdx.x - 64 : threadIdx.x - (64 + kBuildThreads);  // index among the epilogue threads
        const int quarter = warp & 3;  // TMEM lane quarter this warp may read
        const int group = kWideEpilogue ? (warp - 2) >> 2 : 0;  // which of the warps sharing this quarter
        // Partial-sum slot of this thread's tile row (the warps of one quarter own the same rows, different chunks).
        float4* scratch = p.scratch + static_cast<int64_t>(blockIdx.x) * (BN / 4) * kEpilogueThreads + quarter * 32 + lane;
        int iter = 0;
        int tile_iter = 0;
        bool ok = true;
        // fp16 mode: undo the power-of-two scale of the activations (exact) together with the caller's scale.
        const float ep_scale = p.amax_bits ? __fmul_rn(p.ep.scale, f16_scale_inv(__ldg(p.amax_bits))) : p.ep.scale;
        for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, ++tile_iter) {
            int tm, tn;
            tile_coords(t, p.tiles_m, p.tiles_n, p.group_m, tm, tn);
            const int sbuf = tile_iter & 1;
            const int64_t n0 = static_cast<int64_t>(tn) * BN;
            for (int j = e; j < BN; j += kEpiThreads) {
                const int64_t n = n0 + j;
                alpha_s[sbuf * BN + j] = (p.ep.alpha && n < p.N) ? __ldg(p.ep.alpha + n) : 1.0f;
                bias_s[sbuf * BN + j] = (p.ep.bias && n < p.N) ? __ldg(p.ep.bias + n) : 0.0f;
            }
            ptx::named_barrier_sync(1, kEpiThreads);
            const int64_t m = static_cast<int64_t>(tm) * BM + quarter * 32 + lane;
            bool row_ok = m < p.M;
            // Output element (m, n) lives at out_base + n * out_cs; cl_row is the pixel index of the row.
            int64_t out_base, out_cs, cl_row = m;
            if (PATCH) {
                // Row of the tile -> (image, output row, output column) inside this tile's patch.
                const int row = quarter * 32 + lane;
                int64_t img;
                int oh, ow;
                if (p.conv.stack_rows > 0) {
                    // Stacked rows: tile row r of this tile is row tm * stack_rows + r of the sequence img * OH + oh.
                    const int r = row / p.conv.OW;
                    const int64_t s = static_cast<int64_t>(tm) * p.conv.stack_rows + r;
                    img = s / p.conv.OH;
                    oh = static_cast<int>(s - img * p.conv.OH);
                    ow = row - r * p.conv.OW;
                    row_ok = r < p.conv.stack_rows && img * p.out_hw < p.M;
                } else {
                    const int bw = row % p.conv.pbw, bh = (row / p.conv.pbw) % p.conv.pbh, bi = row / (p.conv.pbw * p.conv.pbh);
                    const int px = tm % p.conv.patches_w, py = (tm / p.conv.patches_w) % p.conv.patches_h;
                    img = static_cast<int64_t>(tm / (p.conv.patches_w * p.conv.patches_h)) * p.conv.pbi + bi;
                    oh = py * p.conv.pbh + bh;
                    ow = px * p.conv.pbw + bw;
                    row_ok = bi < p.conv.pbi && oh < p.conv.OH && ow < p.conv.OW && img * p.out_hw < p.M;
                }
                out_base = img * p.N * p.out_hw + static_cast<int64_t>(oh) * p.conv.OW + ow;
                out_cs = p.out_hw;
                cl_row = img * p.out_hw + static_cast<int64_t>(oh) * p.conv.OW + ow;
            } else if (p.out_nchw) {
                const int64_t img = m / p.out_hw;
                out_base = img * p.N * p.out_hw + (m - img * p.out_hw);
                out_cs = p.out_hw;
            } else {
                out_base = m * p.ldc;
                out_cs = 1;
            }
            const float* res = p.ep.residual;
            const bool add_res = (p.ep.flags & TBN_EPI_ADD_RESIDUAL) != 0;
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
                for (int c = group; c < BN / 32; c += kEpiGroups) {
                    if (n0 + c * 32 >= p.N) break;  // columns past the matrix: nothing to read, add or store
                    uint32_t r[32];
                    ptx::tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                                           static_cast<uint32_t>(buf * C::ACC_COLS + c * 32), r);
                    float v[32];
                    if constexpr (C::DENSE_WIDE) {
                        uint32_t r2[32];  // the hi x lo products of the same columns
                        ptx::tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                                               static_cast<uint32_t>(buf * C::ACC_COLS + BN + c * 32), r2);
                        ptx::tmem_ld_wait();
#pragma unroll
                        for (int j = 0; j < 32; ++j) v[j] = __fadd_rn(__uint_as_float(r[j]), __uint_as_float(r2[j]));
                    } else {
                        ptx::tmem_ld_wait();
#pragma unroll
                        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
                    }
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
                    } else if (MULTI && p.num_out > 0) {
                        const int64_t nc = n0 + c * 32;
                        const float* as = alpha_s + sbuf * BN + c * 32;
                        const float* bs = bias_s + sbuf * BN + c * 32;
                        float* tbuf = stage_out + (warp & 3) * (kStageOutBytes / 16);  // 32 x 32 floats per warp
                        const int64_t m_warp = static_cast<int64_t>(tm) * BM + quarter * 32;
                        // The previous block's stores must have read the staging buffer before it is rewritten.
                        if (lane == 0) ptx::bulk_wait_group_read<0>();
                        __syncwarp();
                        // lane = row: write this row's 32 columns as 8 float4 at swizzled positions.
#pragma unroll
                        for (int j4 = 0; j4 < 8; ++j4) {
                            const int j = j4 * 4;
                            float4 o;
                            o.x = apply_epilogue(v[j + 0], as[j + 0], bs[j + 0], ep_scale, p.ep.flags, 0.0f);
                            o.y = apply_epilogue(v[j + 1], as[j + 1], bs[j + 1], ep_scale, p.ep.flags, 0.0f);
                            o.z = apply_epilogue(v[j + 2], as[j + 2], bs[j + 2], ep_scale, p.ep.flags, 0.0f);
                            o.w = apply_epilogue(v[j + 3], as[j + 3], bs[j + 3], ep_scale, p.ep.flags, 0.0f);
                            *reinterpret_cast<float4*>(tbuf + lane * 32 + ((j4 ^ (lane & 7)) << 2)) = o;
                        }
                        // Shared memory written by these lanes -> readable by the TMA engine; then one lane sends the
                        // block to every destination.
                        ptx::fence_proxy_async_smem();
                        __syncwarp();
                        if (lane == 0) {
                            const uint32_t src = ptx::smem_u32(tbuf);
#pragma unroll 1
                            for (int d = 0; d < p.num_out; ++d)
                                ptx::tma_store_2d(&out_maps.m[d], src, static_cast<int>(nc), static_cast<int>(m_warp));
                            ptx::bulk_commit_group();
                        }
                    } else if (row_ok) {
                        const int64_t nc = n0 + c * 32;
                        const float* as = alpha_s + sbuf * BN + c * 32;
                        const float* bs = bias_s + sbuf * BN + c * 32;
                        if (p.c_vec_ok && !add_res && nc + 32 <= p.N) {
                            float* c_row = p.c + out_base;
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
                            // Ragged edge, residual add or NCHW: element stores.  In NCHW consecutive lanes
                            // hold consecutive pixels of one channel, so each store is coalesced.  The flags are
                            // uniform: each is tested once per chunk, outside the unrolled element loops, and
                            // the residual loads are all issued before the first one is used.
                            float o[32];
                            const bool bias_first = (p.ep.flags & TBN_EPI_BIAS_BEFORE_ALPHA) != 0;
#pragma unroll
                            for (int j4 = 0; j4 < 8; ++j4) {
                                const float4 a4 = *reinterpret_cast<const float4*>(as + 4 * j4);
                                const float4 b4 = *reinterpret_cast<const float4*>(bs + 4 * j4);
                                const float aj[4] = {a4.x, a4.y, a4.z, a4.w}, bj[4] = {b4.x, b4.y, b4.z, b4.w};
#pragma unroll
                                for (int i = 0; i < 4; ++i) {
                                    const int j = 4 * j4 + i;
                                    o[j] = bias_first ? __fmul_rn(__fadd_rn(__fmul_rn(v[j], ep_scale), bj[i]), aj[i])
                                                      : __fadd_rn(__fmul_rn(__fmul_rn(v[j], aj[i]), ep_scale), bj[i]);
                                }
                            }
                            const int ncols = static_cast<int>(min(static_cast<int64_t>(32), p.N - nc));
                            const int64_t first = out_base + nc * out_cs;
                            if (add_res) {
                                const float* rp = res + first;
                                float rv[32];
#pragma unroll
                                for (int j = 0; j < 32; ++j) rv[j] = j < ncols ? __ldg(rp + j * out_cs) : 0.0f;
#pragma unroll
                                for (int j = 0; j < 32; ++j) o[j] = __fadd_rn(o[j], rv[j]);
                            }
                            if (p.ep.flags & TBN_EPI_RELU) {
#pragma unroll
                                for (int j = 0; j < 32; ++j) o[j] = fmaxf(o[j], 0.0f);
                            }
                            if (p.out_cl != nullptr) {
                                // Channels-last bf16 terms of the same values (hi = rn(o), lo = rn(o - hi)): what the
                                // pre-pass of the next convolution would have computed from the fp32 result.
                                __nv_bfloat16* cl = p.out_cl + cl_row * p.N + nc;
                                if (ncols == 32 && (p.N & 7) == 0) {
#pragma unroll
                                    for (int g8 = 0; g8 < 4; ++g8) {
                                        uint32_t hi[4], lo[4];
#pragma unroll
                                        for (int e = 0; e < 4; ++e) split_pair_terms(o[g8 * 8 + 2 * e], o[g8 * 8 + 2 * e + 1], hi[e], lo[e]);
                                        *reinterpret_cast<uint4*>(cl + g8 * 8) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
                                        *reinterpret_cast<uint4*>(cl + p.out_cl_term_stride + g8 * 8) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
                                    }
                                } else {
#pragma unroll
                                    for (int j = 0; j < 32; ++j) {
                                        if (j < ncols) {
                                            uint16_t term[2];
                                            split_terms<2, false>(o[j], 0.f, 0.f, term);
                                            cl[j] = __ushort_as_bfloat16(term[0]);
                                            cl[p.out_cl_term_stride + j] = __ushort_as_bfloat16(term[1]);
                                        }
                                    }
                                }
                            }
                            if (p.c != nullptr) {
                                float* dst = p.c + first;
                                if (ncols == 32) {
#pragma unroll
                                    for (int j = 0; j < 32; ++j) dst[j * out_cs] = o[j];
                                } else {
#pragma unroll
                                    for (int j = 0; j < 32; ++j)
                                        if (j < ncols) dst[j * out_cs] = o[j];
                                }
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
    ptx::bulk_wait_group<0>();  // stores issued by this thread (multi-destination epilogue) have completed
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
// Host-side helpers shared by the GEMM and convolution entry points
// =====================================================================================

inline int pick_bn(int64_t N) {
    // Largest tile whose padding waste stays within ~12 % of the best candidate.
    const int cand[3] = {256, 128, 64};
    int64_t best = INT64_MAX;
    for (int bn : cand) best = std::min<int64_t>(best, round_up(N, bn));
    for (int bn : cand)
        if (round_up(N, bn) * 8 <= best * 9) return bn;
    return 64;
}

// Per-CTA partial-sum tiles of the segmented accumulation: one 128 x 256 fp32 tile per SM.
inline size_t scratch_bytes() { return static_cast<size_t>(std::max(sm_count(), 1)) * tc::BM * 256 * sizeof(float); }

struct TensorMaps {
    CUtensorMap a, neg, pos;
    tc::OutMaps out = {};
};

// Destination map of the multi-destination epilogue (see tc::OutMaps).
inline int32_t make_out_map(EncodeTiledFn encode, float* base, int64_t M, int64_t N, int64_t ldc, CUtensorMap* out) {
    const cuuint64_t gdim[2] = {static_cast<cuuint64_t>(N), static_cast<cuuint64_t>(M)};
    const cuuint64_t gstride[1] = {static_cast<cuuint64_t>(ldc) * 4};
    const cuuint32_t box[2] = {32, 32};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult cr = encode(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, base, gdim, gstride, box, estr,
                               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                               CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    TBN_REQUIRE(cr == CUDA_SUCCESS, TBN_CUDA_ERROR,
                "cuTensorMapEncodeTiled (destination) failed with CUresult " + std::to_string(static_cast<int>(cr)));
    return TBN_SUCCESS;
}

// Packed-word plane [N_pad][KW] uint32 -> box of 4 words (128 k) x BN columns, no swizzle.
inline int32_t make_word_map(EncodeTiledFn encode, const uint32_t* words, int64_t KW, int64_t N_pad, int bn,
                             CUtensorMap* out, int words_per_row = 4) {
    const cuuint64_t gdim[2] = {static_cast<cuuint64_t>(KW), static_cast<cuuint64_t>(N_pad)};
    const cuuint64_t gstride[1] = {static_cast<cuuint64_t>(KW) * 4};
    const cuuint32_t box[2] = {static_cast<cuuint32_t>(words_per_row), static_cast<cuuint32_t>(bn)};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult cr = encode(out, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<uint32_t*>(words), gdim, gstride, box,
                               estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                               CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    TBN_REQUIRE(cr == CUDA_SUCCESS, TBN_CUDA_ERROR,
                "cuTensorMapEncodeTiled (packed words) failed with CUresult " + std::to_string(static_cast<int>(cr)));
    return TBN_SUCCESS;
}

// Fills the segmentation fields: a fresh accumulator every kMaxAccumSteps accumulation steps.
inline void set_segments(tc::Params& p, int npass) {
    const int max_kb = std::max(1, tc::kMaxAccumSteps / (npass * tc::BK));
    p.num_seg = (p.num_kb + max_kb - 1) / max_kb;
    p.kb_per_seg = (p.num_kb + p.num_seg - 1) / p.num_seg;
}

template <int BN, int NPASS, bool TERNARY, int AMODE, bool TERN_ACT, int BSRC = 0, bool MULTI = false>
int32_t launch_tc(const TensorMaps& maps, const tc::Params& p, cudaStream_t st) {
    using C = tc::Cfg<BN, NPASS, TERNARY, BSRC, tc::is_conv_mode(AMODE), MULTI>;
    auto kernel = tc::gemm_tc_kernel<BN, NPASS, TERNARY, AMODE, TERN_ACT, BSRC, MULTI>;
    TBN_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES));
    const int total = p.tiles_m * p.tiles_n;
    const int grid = std::max(1, std::min(total, sm_count()));
    tc::Params q = p;
    if (q.group_m < 1) q.group_m = tc::kDefaultGroupM;
    profile_begin(kProfGemm, st);
    kernel<<<grid, tc::kThreads, C::SMEM_BYTES, st>>>(maps.a, maps.neg, maps.pos, maps.out, q);
    profile_end(kProfGemm, st);
    return launched(tc::is_conv_mode(AMODE) ? "gemm_tc_kernel<conv>" : "gemm_tc_kernel");
}

template <int NPASS, bool TERNARY, int AMODE, bool TERN_ACT, int BSRC = 0, bool MULTI = false>
int32_t dispatch_bn(int bn, const TensorMaps& maps, const tc::Params& p, cudaStream_t st) {
    switch (bn) {
        case 256: return launch_tc<256, NPASS, TERNARY, AMODE, TERN_ACT, BSRC, MULTI>(maps, p, st);
        case 128: return launch_tc<128, NPASS, TERNARY, AMODE, TERN_ACT, BSRC, MULTI>(maps, p, st);
        default: return launch_tc<64, NPASS, TERNARY, AMODE, TERN_ACT, BSRC, MULTI>(maps, p, st);
    }
}

// Words per row of the packed-word box that the kernel instantiation (plain GEMM, AMODE 0 or 3) expects.
inline int gemm_words_per_row(bool ternary, bool multi) { (void)ternary; return !multi ? 8 : 4; }

// Tensor map over bf16 terms laid out [terms][rows_pad][K_pad] (split activations or split dense weights):
// box = 64 k x `box_rows` rows x 1 term, 128-byte swizzle.
inline int32_t make_split_map(EncodeTiledFn encode, const void* base, int64_t K_pad, int64_t rows_pad, int terms,
                              int box_rows, CUtensorMap* out) {
    const cuuint64_t gdim[3] = {static_cast<cuuint64_t>(K_pad), static_cast<cuuint64_t>(rows_pad),
                                static_cast<cuuint64_t>(terms)};
    const cuuint64_t gstride[2] = {static_cast<cuuint64_t>(K_pad) * 2, static_cast<cuuint64_t>(rows_pad) * K_pad * 2};
    const cuuint32_t box[3] = {tc::BK, static_cast<cuuint32_t>(box_rows), 1};
    const cuuint32_t estr[3] = {1, 1, 1};
    const CUresult cr = encode(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), gdim, gstride, box, estr,
                               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    TBN_REQUIRE(cr == CUDA_SUCCESS, TBN_CUDA_ERROR,
                "cuTensorMapEncodeTiled (bf16 terms) failed with CUresult " + std::to_string(static_cast<int>(cr)));
    return TBN_SUCCESS;
}

}  // namespace
}  // namespace tbn_cuda
