// Conv2D lowered onto the packed-weight GEMM as an IMPLICIT GEMM: the im2col matrix
// (tbn-runtime/src/operators/conv2d.cpp:420-507) is never written; the operand-build warps of
// gemm_tc_kernel gather each 128 x 64 activation tile straight from the NCHW fp32 input, split it
// into bf16 terms (or ternarise it, TBN mode) and write the swizzled shared-memory tile; the epilogue
// stores NCHW with alpha / bias / residual / ReLU applied.  Replaces, on this path,
// tbn::conv2d_binary / conv2d_binary_with_scales (conv2d.cpp:220-369) and the cached fast path of
// Session::execute_conv (tbn/runtime/model.hpp:375-559).  GEMM view: M = N_img*OH*OW output pixels,
// K = C*kh*kw in the reference's (c, i, j) order, N = output channels; the weights are packed from
// [M_out, C*kh*kw] with TBN_LAYOUT_NK, which yields the same words as the Session's transpose + pack.
#include <cstdlib>

#include "conv_rows.cuh"
#include "gemm_tc.cuh"
#include "plan.cuh"

namespace tbn_cuda {
namespace {

// table[k] = {input offset of tap k relative to the window origin, (dy << 16) | dx}; see ConvGeom.
__global__ void conv_tap_table_kernel(int2* __restrict__ table, int K, int K_pad, int H, int W, int kh, int kw, int dh,
                                      int dw) {
    const int k = blockIdx.x * blockDim.x + threadIdx.x;
    if (k >= K_pad) return;
    if (k >= K) {
        table[k] = make_int2(0, 0x7fff << 16);
        return;
    }
    const int c = k / (kh * kw);
    const int rem = k - c * kh * kw;
    const int i = rem / kw, j = rem - i * kw;
    table[k] = make_int2(c * H * W + i * dh * W + j * dw, ((i * dh) << 16) | ((j * dw) & 0xffff));
}

// NCHW fp32 -> channels-last bf16 terms xs[q][n][h][w][c] (or the ternarised activation as one exact term).
// One block transposes a 64-channel x 32-pixel tile of one image through shared memory; pixels are taken along the
// flattened h*W + w index, so that reads are 128 contiguous bytes per channel whatever the image width, and writes
// are 128 bytes per pixel.  HBM bound: 4 B read + 2 NPASS B written per element.
// F16: one fp16 term of x * 2^e, e from *amax_bits (the one-pass fp16 mode, see f16_scale_exponent).
template <int NPASS, bool TERNARISE, bool F16 = false>
__global__ void __launch_bounds__(256) nhwc_split_kernel(const float* __restrict__ x, int C, int HW, int tiles_per_image,
                                                         __nv_bfloat16* __restrict__ xs, int64_t term_stride, float lo,
                                                         float hi, const uint32_t* __restrict__ amax_bits = nullptr) {
    static_assert(!F16 || (NPASS == 1 && !TERNARISE), "the fp16 mode has one term");
    const float mul = F16 ? f16_scale_mul(__ldg(amax_bits)) : 1.0f;
    __shared__ float tile[64][33];
    const int64_t n = blockIdx.x / tiles_per_image;  // grid.x: the only dimension that may exceed 65535
    const int p0 = static_cast<int>(blockIdx.x - n * tiles_per_image) * 32;
    const int c0 = blockIdx.y * 64;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int c = ty + 8 * i;
        tile[c][tx] = (p0 + tx < HW) ? __ldg(x + (n * C + c0 + c) * HW + p0 + tx) : 0.0f;
    }
    __syncthreads();
    const int chunk = threadIdx.x & 7, pp = threadIdx.x >> 3;  // 8 channels of pixel (p0 + pp)
    if (p0 + pp >= HW) return;
    uint32_t packed[NPASS][4];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        uint16_t term[NPASS];
        if (F16) term[0] = __half_as_ushort(__float2half_rn(__fmul_rn(tile[chunk * 8 + e][pp], mul)));
        else split_terms<NPASS, TERNARISE>(tile[chunk * 8 + e][pp], lo, hi, term);
#pragma unroll
        for (int q = 0; q < NPASS; ++q) {
            if (e & 1) packed[q][e >> 1] |= static_cast<uint32_t>(term[q]) << 16;
            else packed[q][e >> 1] = term[q];
        }
    }
    const int64_t off = (n * HW + p0 + pp) * C + c0 + chunk * 8;
#pragma unroll
    for (int q = 0; q < NPASS; ++q)
        *reinterpret_cast<uint4*>(xs + q * term_stride + off) = make_uint4(packed[q][0], packed[q][1], packed[q][2], packed[q][3]);
}

// [M][C][taps] -> [M][taps][C]: filters in tap-major order for the channels-last path.
__global__ void permute_filters_kernel(const float* __restrict__ w, int64_t M, int C, int taps, float* __restrict__ out) {
    const int64_t total = M * C * taps;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
        const int c = static_cast<int>(i % C);
        const int t = static_cast<int>((i / C) % taps);
        const int64_t m = i / (static_cast<int64_t>(C) * taps);
        out[i] = __ldg(w + (m * C + c) * taps + t);
    }
}

// Sign words [N_pad][KW] -> bf16 [N_pad][K_pad] (+1 = 0x3F80, -1 = 0xBF80, ternary zero = 0): the weight operand
// of the convolutions, expanded once per call so that the GEMM kernel takes it by TMA.  One word (32 k, 64 output
// bytes) per thread; a warp writes 2 KB contiguous.
__global__ void expand_words_kernel(const uint32_t* __restrict__ neg, const uint32_t* __restrict__ pos, int64_t words,
                                    uint4* __restrict__ out, uint32_t one16) {
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < words; i += stride) {
        const uint32_t nw = __ldg(neg + i), pw = pos ? __ldg(pos + i) : 0u;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const uint32_t nb = (nw >> (8 * q)) & 0xffu, pb = (pw >> (8 * q)) & 0xffu;
            out[i * 4 + q] = pos ? unpack8<true>(nb, pb, one16) : unpack8<false>(nb, pb, one16);
        }
    }
}

// ---- stride-2 convolutions over very few channels (image stems) ------------------------------------------
// A 2 x 2 space-to-depth of the input turns a stride-2 convolution over C <= 4 channels into a stride-1 one over
// 4C <= 16 channels.  Stored channels-last with 16 bf16 per position, four neighbouring positions are 128
// contiguous bytes: one 64-deep k-block = one row of the folded filter, and its operand for output column ow is
// the window of positions ow .. ow+3.  A tensor map whose position stride (32 bytes) is smaller than its window
// (128 bytes) hands those overlapping windows to the patch-mode kernel as ordinary boxes.
//   T[term][n][Rs][Qs][(pr*2 + pc)*C + c] = x[n][c][2*Rs + pr][2*(Qs - left) + pc]   (0 outside the image / channels)
template <int NPASS, bool TERNARISE>
__global__ void s2d_split_kernel(const float* __restrict__ x, int64_t N, int C, int H, int W, int rows, int Qp, int left,
                                 __nv_bfloat16* __restrict__ t, int64_t term_stride, float lo, float hi) {
    const int64_t total = N * rows * Qp;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    const bool pair_ok = (W & 1) == 0 && (reinterpret_cast<uintptr_t>(x) & 7) == 0;
    for (int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total; idx += stride) {
        int qs, rs;
        int64_t n;
        if (total < (1LL << 31)) {  // 32-bit index arithmetic where it fits
            const unsigned u = static_cast<unsigned>(idx), r = u / static_cast<unsigned>(Qp);
            qs = static_cast<int>(u - r * static_cast<unsigned>(Qp));
            const unsigned img = r / static_cast<unsigned>(rows);
            rs = static_cast<int>(r - img * static_cast<unsigned>(rows));
            n = img;
        } else {
            qs = static_cast<int>(idx % Qp);
            rs = static_cast<int>((idx / Qp) % rows);
            n = idx / (static_cast<int64_t>(Qp) * rows);
        }
        uint32_t packed[NPASS][8];
#pragma unroll
        for (int q = 0; q < NPASS; ++q)
#pragma unroll
            for (int e = 0; e < 8; ++e) packed[q][e] = 0u;
        // The two columns of a position are neighbours in memory: one 8-byte load where the row allows it.
        float in[2][2][4];  // [pr][pc][c]
        const int w0 = 2 * (qs - left);
#pragma unroll
        for (int pr = 0; pr < 2; ++pr)
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                float2 v2 = make_float2(0.f, 0.f);
                const int h = 2 * rs + pr;
                if (c < C && h < H) {
                    const float* src = x + ((n * C + c) * H + h) * static_cast<int64_t>(W) + w0;
                    if (pair_ok && w0 >= 0 && w0 + 1 < W) v2 = __ldg(reinterpret_cast<const float2*>(src));
                    else {
                        if (w0 >= 0 && w0 < W) v2.x = __ldg(src);
                        if (w0 + 1 >= 0 && w0 + 1 < W) v2.y = __ldg(src + 1);
                    }
                }
                in[pr][0][c] = v2.x;
                in[pr][1][c] = v2.y;
            }
#pragma unroll
        for (int sidx = 0; sidx < 16; ++sidx) {
            float v = 0.0f;
#pragma unroll
            for (int pr = 0; pr < 2; ++pr)
#pragma unroll
                for (int pc = 0; pc < 2; ++pc)
#pragma unroll
                    for (int c = 0; c < 4; ++c)
                        if (c < C && (pr * 2 + pc) * C + c == sidx) v = in[pr][pc][c];
            uint16_t term[NPASS];
            split_terms<NPASS, TERNARISE>(v, lo, hi, term);
#pragma unroll
            for (int q = 0; q < NPASS; ++q) packed[q][sidx >> 1] |= static_cast<uint32_t>(term[q]) << (16 * (sidx & 1));
        }
#pragma unroll
        for (int q = 0; q < NPASS; ++q) {
            uint4* dst = reinterpret_cast<uint4*>(t + q * term_stride + idx * 16);
            dst[0] = make_uint4(packed[q][0], packed[q][1], packed[q][2], packed[q][3]);
            dst[1] = make_uint4(packed[q][4], packed[q][5], packed[q][6], packed[q][7]);
        }
    }
}

// Filters [terms][N_pad][K_pad] bf16 in the reference order k = (c*kh + i)*kw + j  ->  folded order
// k' = t*64 + q*16 + (pr*2 + pc)*C + c with i = 2t + pr - eh, j = 2q + pc - ew (zero where no such tap exists).
__global__ void fold_filters_kernel(const __nv_bfloat16* __restrict__ src, int terms, int64_t N_pad, int64_t K_pad, int C,
                                    int kh, int kw, int eh, int ew, int kh2, int64_t K2_pad,
                                    __nv_bfloat16* __restrict__ dst) {
    const int64_t total = static_cast<int64_t>(terms) * N_pad * K2_pad;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total; idx += stride) {
        const int64_t k2 = idx % K2_pad, row = idx / K2_pad;  // row = term * N_pad + n
        const int t = static_cast<int>(k2 / 64), q = static_cast<int>((k2 % 64) / 16), sidx = static_cast<int>(k2 % 16);
        __nv_bfloat16 v = __float2bfloat16_rn(0.0f);
        if (t < kh2 && sidx < 4 * C) {
            const int pr = sidx / (2 * C), pc = (sidx / C) & 1, c = sidx % C;
            const int i = 2 * t + pr - eh, j = 2 * q + pc - ew;
            if (i >= 0 && i < kh && j >= 0 && j < kw) v = src[row * K_pad + (static_cast<int64_t>(c) * kh + i) * kw + j];
        }
        dst[idx] = v;
    }
}

struct ConvArgs {
    const void* dense_w = nullptr;  // split dense weights (float filters) instead of packed planes
    const float* x;
    int64_t N, C, H, W;
    const uint32_t* neg;
    const uint32_t* pos;
    int64_t M_out, kh, kw;
    int32_t sh, sw, ph, pw, dh, dw;
    Epilogue ep;
    float* y;
    void* ws;
    size_t ws_bytes;
    cudaStream_t st;
    int32_t weight_order = 0;  // TBN_CONV_WEIGHTS_*
    const void* x_cl = nullptr;  // input already as channels-last bf16 terms [2][N][H][W][C] (skips the pre-pass)
    void* y_cl = nullptr;        // also / instead write the output as channels-last bf16 terms [2][N][OH][OW][M_out]
    bool f16 = false;            // one-pass fp16 mode (tap-major filters, NCHW fp32 input): see TBN_MODE_TC_FP16X1
};

size_t xs_bytes(int64_t N, int64_t C, int64_t H, int64_t W, int npass) {
    return static_cast<size_t>(round_up(static_cast<int64_t>(npass) * N * H * W * C * 2, 256));
}

size_t table_bytes(int64_t K_pad) { return static_cast<size_t>(round_up(K_pad * static_cast<int64_t>(sizeof(int2)), 256)); }

// Expanded (bf16) copy of the packed filters, after the partial-sum tiles in the workspace.
size_t expanded_bytes(int64_t K_pad, int64_t N_pad) { return static_cast<size_t>(round_up(K_pad * N_pad * 2, 256)); }

// Geometry of the folded (space-to-depth) form of a stride-2 convolution; `ok` says whether it applies.
struct FoldGeom {
    bool ok = false;
    int eh = 0, ew = 0, kh2 = 0, kw2 = 0, rows = 0, Qp = 0, left = 0, top = 0;
    int64_t t_bytes = 0, K2_pad = 0;
};

FoldGeom fold_geometry(int64_t N, int64_t C, int64_t H, int64_t W, int64_t kh, int64_t kw, int sh, int sw, int ph, int pw,
                       int dh, int dw, int64_t OW, int npass) {
    FoldGeom g;
    if (C < 1 || C > 4 || sh != 2 || sw != 2 || dh != 1 || dw != 1 || kh > 64 || kw > 8) return g;
    const int Sh = (ph + 1) / 2 * 2, Sw = (pw + 1) / 2 * 2;  // even shifts >= the pads
    g.eh = Sh - ph;
    g.ew = Sw - pw;
    g.kh2 = (g.eh + static_cast<int>(kh) - 1) / 2 + 1;
    g.kw2 = (g.ew + static_cast<int>(kw) - 1) / 2 + 1;
    if (g.kw2 > 4) return g;
    g.top = Sh / 2;
    g.left = Sw / 2;
    g.rows = static_cast<int>((H + 1) / 2);
    g.Qp = static_cast<int>(std::max<int64_t>(OW + 3, g.left + (W + 1) / 2));  // every window of 4 positions is in storage
    g.t_bytes = round_up(static_cast<int64_t>(npass) * N * g.rows * g.Qp * 16 * 2, 256);
    g.K2_pad = round_up(static_cast<int64_t>(g.kh2) * 64, 128);
    g.ok = N * g.rows * g.Qp * 32 < (1LL << 40);
    return g;
}

// Patch of output pixels that one 128-row tile covers: pbw columns x pbh rows (x pbi whole images when an image fits).
// Among the widths that divide the output width (and the full width), the one that needs the fewest tiles per image;
// ties go to the wider patch (longer contiguous runs in the NCHW result).  112 x 112 outputs: 16 x 8 (98 full tiles)
// instead of 112 x 1 (112 tiles at 7/8 occupancy).
inline void choose_patch(int64_t OW, int64_t OH, int64_t N, int64_t& pbw, int64_t& pbh, int64_t& pbi) {
    pbw = std::min<int64_t>(OW, tc::BM);
    pbh = std::min<int64_t>(OH, tc::BM / pbw);
    int64_t best = ((OW + pbw - 1) / pbw) * ((OH + pbh - 1) / pbh);
    for (int64_t w = pbw - 1; w >= 8; --w) {
        if (OW % w != 0) continue;
        const int64_t h = std::min<int64_t>(OH, tc::BM / w);
        const int64_t tiles = (OW / w) * ((OH + h - 1) / h);
        if (tiles < best) {
            best = tiles;
            pbw = w;
            pbh = h;
        }
    }
    pbi = (pbw == OW && pbh == OH) ? std::max<int64_t>(1, std::min<int64_t>(tc::BM / (pbw * pbh), N)) : 1;
}

int32_t conv_common(const ConvArgs& a, int npass, bool tern_act, float lo, float hi, bool allow_fold = true) {
    TBN_REQUIRE(a.N > 0 && a.C > 0 && a.H > 0 && a.W > 0 && a.M_out > 0 && a.kh > 0 && a.kw > 0, TBN_INVALID_SHAPE,
                "conv2d: dimensions must be positive");
    TBN_REQUIRE(a.sh > 0 && a.sw > 0 && a.dh > 0 && a.dw > 0 && a.ph >= 0 && a.pw >= 0, TBN_INVALID_ARGUMENT,
                "conv2d: strides and dilations must be positive, pads non-negative");
    TBN_REQUIRE(device_error_word() != nullptr, TBN_RUNTIME_ERROR, "tbn_cuda_init was not called on this device");
    // out = (in + 2p - d(k-1) - 1)/s + 1   (conv2d.cpp:114-117)
    const int64_t OH = (a.H + 2 * a.ph - a.dh * (a.kh - 1) - 1) / a.sh + 1;
    const int64_t OW = (a.W + 2 * a.pw - a.dw * (a.kw - 1) - 1) / a.sw + 1;
    TBN_REQUIRE(a.H + 2 * a.ph - a.dh * (a.kh - 1) - 1 >= 0 && a.W + 2 * a.pw - a.dw * (a.kw - 1) - 1 >= 0 && OH > 0 &&
                    OW > 0,
                TBN_INVALID_SHAPE, "conv2d: invalid output dimensions");
    TBN_REQUIRE((a.x || a.x_cl) && (a.neg || a.dense_w) && (a.y || a.y_cl), TBN_INVALID_ARGUMENT, "conv2d: null pointer");
    TBN_REQUIRE(!a.x_cl || (a.weight_order == TBN_CONV_WEIGHTS_TAP_MAJOR && !tern_act), TBN_INVALID_ARGUMENT,
                "conv2d: a channels-last input needs tap-major filters and the float x binary / float modes");
    TBN_REQUIRE(reinterpret_cast<uintptr_t>(a.x_cl) % 16 == 0 && reinterpret_cast<uintptr_t>(a.y_cl) % 16 == 0,
                TBN_INVALID_ARGUMENT, "conv2d: channels-last tensors must be 16-byte aligned");
    TBN_REQUIRE(a.H < 32000 && a.W < 32000 && a.dh * (a.kh - 1) < 32000 && a.dw * (a.kw - 1) < 32000, TBN_INVALID_SHAPE,
                "conv2d: image or dilated kernel too large");
    const int64_t K = a.C * a.kh * a.kw, M = a.N * OH * OW, N = a.M_out;
    TBN_REQUIRE(K < (1LL << 24) && a.C * a.H * a.W < (1LL << 31) && M < (1LL << 31) && OH * OW < (1LL << 31),
                TBN_INVALID_SHAPE, "conv2d: problem too large");
    const int64_t K_pad = round_up(K, 128), N_pad = round_up(N, 8), M_pad = round_up(M, tc::BM);
    const bool fast = a.weight_order == TBN_CONV_WEIGHTS_TAP_MAJOR;
    TBN_REQUIRE(a.weight_order == TBN_CONV_WEIGHTS_REFERENCE || fast, TBN_INVALID_ARGUMENT, "conv2d: unknown weight order");
    const bool f16 = a.f16 && fast && !a.x_cl && !a.y_cl && !a.dense_w && !tern_act && npass == 1;
    TBN_REQUIRE(!fast || a.C % 64 == 0, TBN_INVALID_ARGUMENT,
                "conv2d: tap-major weights need a channel count that is a multiple of 64");
    FoldGeom fold;
    if (!fast && allow_fold) fold = fold_geometry(a.N, a.C, a.H, a.W, a.kh, a.kw, a.sh, a.sw, a.ph, a.pw, a.dh, a.dw, OW, npass);
    const int terms_w = a.dense_w ? 2 : 1;
    // The workspace query sizes the folded form from upper bounds that unusual pads can exceed: when the caller's
    // buffer only covers the gather path, that path runs.
    if (fold.ok && a.ws_bytes < static_cast<size_t>(fold.t_bytes) + scratch_bytes() + (a.dense_w ? 0 : expanded_bytes(K_pad, N_pad)) +
                                    static_cast<size_t>(round_up(terms_w * N_pad * fold.K2_pad * 2, 256)))
        fold = FoldGeom{};
    const size_t folded_w_bytes = fold.ok ? static_cast<size_t>(round_up(terms_w * N_pad * fold.K2_pad * 2, 256)) : 0;
    const size_t front_bytes = fast ? xs_bytes(a.N, a.C, a.H, a.W, npass)
                                    : (fold.ok ? static_cast<size_t>(fold.t_bytes) : table_bytes(K_pad));
    // fp16 mode: a 256-byte slot at the very end holds max |x| of the call.
    const size_t need = front_bytes + scratch_bytes() + (a.dense_w ? 0 : expanded_bytes(K_pad, N_pad)) + folded_w_bytes + (f16 ? 256 : 0);
    uint32_t* amax_slot = f16 ? reinterpret_cast<uint32_t*>(static_cast<uint8_t*>(a.ws) + need - 256) : nullptr;
    TBN_REQUIRE(a.ws && a.ws_bytes >= need, TBN_INVALID_ARGUMENT,
                "conv2d: workspace too small (see tbn_conv2d_workspace_bytes)");
    TBN_REQUIRE(reinterpret_cast<uintptr_t>(a.ws) % 128 == 0, TBN_INVALID_ARGUMENT,
                "conv2d: workspace must be 128-byte aligned");
    TBN_REQUIRE(reinterpret_cast<uintptr_t>(a.neg) % 16 == 0 && (!a.pos || reinterpret_cast<uintptr_t>(a.pos) % 16 == 0) &&
                    reinterpret_cast<uintptr_t>(a.dense_w) % 16 == 0,
                TBN_INVALID_ARGUMENT, "conv2d: weights must be 16-byte aligned");
    TBN_REQUIRE(!(a.ep.flags & TBN_EPI_ADD_RESIDUAL) || a.ep.residual, TBN_INVALID_ARGUMENT,
                "conv2d: TBN_EPI_ADD_RESIDUAL needs a residual tensor");
    EncodeTiledFn encode = encode_tiled_fn();
    TBN_REQUIRE(encode != nullptr, TBN_CUDA_ERROR, "cuTensorMapEncodeTiled is not available from the driver");

    // Folded form: its activation tensor map (overlapping windows) is encoded before anything is launched; if the
    // driver refuses it, or the workspace only covers the gather path, the element-gather path runs instead.
    CUtensorMap fold_map;
    int64_t fold_pbw, fold_pbh, fold_pbi;
    choose_patch(OW, OH, a.N, fold_pbw, fold_pbh, fold_pbi);
    if (fold.ok) {
        const int64_t t_stride = a.N * fold.rows * fold.Qp * 16;
        // Positions (overlapping 64-element windows, 16 elements apart) x folded rows x images x terms.
        const cuuint64_t gdim[5] = {64, static_cast<cuuint64_t>(fold.Qp - 3), static_cast<cuuint64_t>(fold.rows),
                                    static_cast<cuuint64_t>(a.N), static_cast<cuuint64_t>(npass)};
        const cuuint64_t gstride[4] = {32, static_cast<cuuint64_t>(fold.Qp) * 32, static_cast<cuuint64_t>(fold.rows) * fold.Qp * 32,
                                       static_cast<cuuint64_t>(t_stride) * 2};
        const cuuint32_t box[5] = {tc::BK, static_cast<cuuint32_t>(fold_pbw), static_cast<cuuint32_t>(fold_pbh),
                                   static_cast<cuuint32_t>(fold_pbi), 1};
        const cuuint32_t estr[5] = {1, 1, 1, 1, 1};
        const CUresult cr = encode(&fold_map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 5, a.ws, gdim, gstride, box, estr,
                                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (cr != CUDA_SUCCESS) return conv_common(a, npass, tern_act, lo, hi, /*allow_fold=*/false);
    }

    int2* table = static_cast<int2*>(a.ws);
    __nv_bfloat16* xs = a.x_cl ? static_cast<__nv_bfloat16*>(const_cast<void*>(a.x_cl)) : static_cast<__nv_bfloat16*>(a.ws);
    const int64_t term_stride = a.N * a.H * a.W * a.C;
    int32_t rc = TBN_SUCCESS;
    if (a.x_cl) {
        // the producing layer's epilogue wrote this form already
    } else if (fast) {
        const int64_t HW = a.H * a.W, tiles_per_image = (HW + 31) / 32;
        TBN_REQUIRE(HW < (1LL << 31) && a.N * tiles_per_image < (1LL << 31) && a.C / 64 <= 65535, TBN_INVALID_SHAPE,
                    "conv2d: input too large for the pre-pass grid");
        dim3 grid(static_cast<unsigned>(a.N * tiles_per_image), static_cast<unsigned>(a.C / 64));
        profile_begin(kProfSplit, a.st);
        if (f16) {
            TBN_CUDA_TRY(cudaMemsetAsync(amax_slot, 0, sizeof(uint32_t), a.st));
            const int64_t total = a.N * a.C * HW;
            const int vec_ok = total % 4 == 0 && reinterpret_cast<uintptr_t>(a.x) % 16 == 0;
            const int gmax = static_cast<int>(std::max<int64_t>(1, std::min((total / (vec_ok ? 4 : 1) + 255) / 256, static_cast<int64_t>(std::max(sm_count(), 1)) * 16)));
            absmax_kernel<<<gmax, 256, 0, a.st>>>(a.x, 1, total, total, vec_ok, amax_slot);
            rc = launched("absmax_kernel");
            if (rc) return rc;
            nhwc_split_kernel<1, false, true><<<grid, 256, 0, a.st>>>(a.x, static_cast<int>(a.C), static_cast<int>(HW),
                                                                      static_cast<int>(tiles_per_image), xs, term_stride, 0.f, 0.f, amax_slot);
        } else if (tern_act)
            nhwc_split_kernel<1, true><<<grid, 256, 0, a.st>>>(a.x, static_cast<int>(a.C), static_cast<int>(HW),
                                                               static_cast<int>(tiles_per_image), xs, term_stride, lo, hi);
        else if (npass == 1)
            nhwc_split_kernel<1, false><<<grid, 256, 0, a.st>>>(a.x, static_cast<int>(a.C), static_cast<int>(HW),
                                                                static_cast<int>(tiles_per_image), xs, term_stride, 0.f, 0.f);
        else
            nhwc_split_kernel<2, false><<<grid, 256, 0, a.st>>>(a.x, static_cast<int>(a.C), static_cast<int>(HW),
                                                                static_cast<int>(tiles_per_image), xs, term_stride, 0.f, 0.f);
        profile_end(kProfSplit, a.st);
        rc = launched("nhwc_split_kernel");
    } else if (fold.ok) {
        const int64_t total = a.N * fold.rows * fold.Qp;
        const int grid = static_cast<int>(std::max<int64_t>(1, std::min((total + 255) / 256, static_cast<int64_t>(std::max(sm_count(), 1)) * 32)));
        const int64_t t_stride = total * 16;
        profile_begin(kProfSplit, a.st);
        if (tern_act)
            s2d_split_kernel<1, true><<<grid, 256, 0, a.st>>>(a.x, a.N, static_cast<int>(a.C), static_cast<int>(a.H), static_cast<int>(a.W),
                                                              fold.rows, fold.Qp, fold.left, xs, t_stride, lo, hi);
        else if (npass == 1)
            s2d_split_kernel<1, false><<<grid, 256, 0, a.st>>>(a.x, a.N, static_cast<int>(a.C), static_cast<int>(a.H), static_cast<int>(a.W),
                                                               fold.rows, fold.Qp, fold.left, xs, t_stride, 0.f, 0.f);
        else
            s2d_split_kernel<2, false><<<grid, 256, 0, a.st>>>(a.x, a.N, static_cast<int>(a.C), static_cast<int>(a.H), static_cast<int>(a.W),
                                                               fold.rows, fold.Qp, fold.left, xs, t_stride, 0.f, 0.f);
        profile_end(kProfSplit, a.st);
        rc = launched("s2d_split_kernel");
    } else {
        conv_tap_table_kernel<<<static_cast<unsigned>((K_pad + 127) / 128), 128, 0, a.st>>>(
            table, static_cast<int>(K), static_cast<int>(K_pad), static_cast<int>(a.H), static_cast<int>(a.W),
            static_cast<int>(a.kh), static_cast<int>(a.kw), a.dh, a.dw);
        rc = launched("conv_tap_table_kernel");
    }
    if (rc) return rc;

    const int bn = gemm_plan(M, N, K).bn;  // the class's measured column tile, adjusted to this shape's tile count
    TensorMaps maps;
    if (a.dense_w) {
        rc = make_split_map(encode, a.dense_w, K_pad, N_pad, 2, bn, &maps.neg);
        if (rc) return rc;
        maps.pos = maps.neg;
    } else {
        // Packed filters are expanded to bf16 once per call (a few MB at most, L2 resident) and then arrive by TMA
        // like float filters do, so that the build warps spend their instructions on the activation gather only.
        uint4* expanded = reinterpret_cast<uint4*>(static_cast<uint8_t*>(a.ws) + front_bytes + scratch_bytes());
        const int64_t words = N_pad * (K_pad / 32);
        const int grid = static_cast<int>(std::max<int64_t>(1, std::min((words + 255) / 256, static_cast<int64_t>(std::max(sm_count(), 1)) * 8)));
        expand_words_kernel<<<grid, 256, 0, a.st>>>(a.neg, a.pos, words, expanded, f16 ? kOneF16 : kOneBf16);
        rc = launched("expand_words_kernel");
        if (rc) return rc;
        rc = make_split_map(encode, expanded, K_pad, N_pad, 1, bn, &maps.neg);
        if (rc) return rc;
        maps.pos = maps.neg;
    }
    maps.a = maps.neg;  // unused in CONV mode
    if (fold.ok) {
        // Fold the filters (float terms or the bf16 expansion just made) into the space-to-depth order.
        const __nv_bfloat16* w_src = a.dense_w ? static_cast<const __nv_bfloat16*>(a.dense_w)
                                               : reinterpret_cast<const __nv_bfloat16*>(static_cast<uint8_t*>(a.ws) + front_bytes + scratch_bytes());
        __nv_bfloat16* w_fold = reinterpret_cast<__nv_bfloat16*>(static_cast<uint8_t*>(a.ws) + front_bytes + scratch_bytes() +
                                                                 (a.dense_w ? 0 : expanded_bytes(K_pad, N_pad)));
        const int64_t total = static_cast<int64_t>(terms_w) * N_pad * fold.K2_pad;
        const int grid = static_cast<int>(std::max<int64_t>(1, std::min((total + 255) / 256, static_cast<int64_t>(std::max(sm_count(), 1)) * 8)));
        fold_filters_kernel<<<grid, 256, 0, a.st>>>(w_src, terms_w, N_pad, K_pad, static_cast<int>(a.C), static_cast<int>(a.kh),
                                                    static_cast<int>(a.kw), fold.eh, fold.ew, fold.kh2, fold.K2_pad, w_fold);
        rc = launched("fold_filters_kernel");
        if (rc) return rc;
        rc = make_split_map(encode, w_fold, fold.K2_pad, N_pad, terms_w, bn, &maps.neg);
        if (rc) return rc;
        maps.pos = maps.neg;
    }

    tc::Params p = {};
    p.M = static_cast<int>(M);
    p.N = static_cast<int>(N);
    p.num_kb = static_cast<int>((K + tc::BK - 1) / tc::BK);  // k-blocks that hold real k; the operands are zero beyond K
    p.tiles_m = static_cast<int>(M_pad / tc::BM);
    p.tiles_n = static_cast<int>((N + bn - 1) / bn);
    p.K = static_cast<int>(K);
    p.c = a.y;
    p.out_cl = static_cast<__nv_bfloat16*>(a.y_cl);
    p.out_cl_term_stride = M * N;
    p.ldc = N;
    p.out_nchw = 1;
    p.out_hw = static_cast<int>(OH * OW);
    p.ep = a.ep;
    p.err_word = device_error_word();
    p.c_vec_ok = 0;
    set_segments(p, npass);
    p.scratch = reinterpret_cast<float4*>(static_cast<uint8_t*>(a.ws) + front_bytes);
    p.conv.xs = xs;
    p.conv.xs_term_stride = term_stride;
    p.conv.kw = static_cast<int>(a.kw);
    p.conv.taps = static_cast<int>(a.kh * a.kw);
    p.conv.dh = a.dh;
    p.conv.dw = a.dw;
    p.conv.cblocks = static_cast<int>(a.C / 64);
    p.conv.x = a.x;
    p.conv.table = table;
    p.conv.C = static_cast<int>(a.C);
    p.conv.H = static_cast<int>(a.H);
    p.conv.W = static_cast<int>(a.W);
    p.conv.OH = static_cast<int>(OH);
    p.conv.OW = static_cast<int>(OW);
    p.conv.sh = a.sh;
    p.conv.sw = a.sw;
    p.conv.ph = a.ph;
    p.conv.pw = a.pw;
    p.conv.act_lo = lo;
    p.conv.act_hi = hi;
    p.f16 = f16 ? 1 : 0;
    p.amax_bits = amax_slot;
    // Patch mode: when the channels-last copy exists and the geometry fits a TMA box, an m-tile is a rectangle of
    // output pixels (whole output rows first, then several rows, then several images) of at most 128 pixels, and
    // the activation operand of one tap and 64 channels is one tiled TMA load.
    if (fold.ok) {
        const int64_t pbw = fold_pbw, pbh = fold_pbh, pbi = fold_pbi;
        maps.a = fold_map;
        // The kernel sees a stride-1 convolution with kh2 taps of 64 "channels": one k-block per folded filter row.
        p.num_kb = fold.kh2;
        set_segments(p, a.dense_w ? 3 : npass);
        p.conv.kw = 1;
        p.conv.taps = fold.kh2;
        p.conv.dh = 1;
        p.conv.dw = 1;
        p.conv.cblocks = 1;
        p.conv.sh = 1;
        p.conv.sw = 1;
        p.conv.ph = fold.top;
        p.conv.pw = 0;
        p.conv.pbw = static_cast<int>(pbw);
        p.conv.pbh = static_cast<int>(pbh);
        p.conv.pbi = static_cast<int>(pbi);
        p.conv.patches_w = static_cast<int>((OW + pbw - 1) / pbw);
        p.conv.patches_h = static_cast<int>((OH + pbh - 1) / pbh);
        p.conv.a_box_bytes = static_cast<int>(npass * pbw * pbh * pbi * 128);
        const int64_t tiles_m = static_cast<int64_t>(p.conv.patches_w) * p.conv.patches_h * ((a.N + pbi - 1) / pbi);
        TBN_REQUIRE(tiles_m * p.tiles_n < (1LL << 31), TBN_INVALID_SHAPE, "conv2d: too many tiles");
        p.tiles_m = static_cast<int>(tiles_m);
        if (a.dense_w) return dispatch_bn<2, false, 4, false, 1>(bn, maps, p, a.st);
        if (tern_act || npass == 1) return dispatch_bn<1, false, 4, false, 2>(bn, maps, p, a.st);
        return dispatch_bn<2, false, 4, false, 2>(bn, maps, p, a.st);
    }
    if (fast) {
        int64_t pbw, pbh, pbi;
        choose_patch(OW, OH, a.N, pbw, pbh, pbi);
        // Row mode (conv_rows.cuh): stride-1 convolutions with at most three filter columns whose tiles are no
        // emptier than the patch tiles below.  TBN_CONV_ROWS=0 in the environment keeps the patch-mode kernel
        // (for A/B measurements).
        {
            static const bool rows_enabled = [] {
                const char* v = std::getenv("TBN_CONV_ROWS");
                return !(v && v[0] == '0');
            }();
            static const bool stack_rows_enabled = [] {
                const char* v = std::getenv("TBN_CONV_STACK");
                return !(v && v[0] == '0');
            }();
            const int64_t pitch = round_up(OW + a.kw - 1, 8);
            int64_t rpbh = pitch <= tc::BM ? std::min<int64_t>(OH, tc::BM / pitch) : 0;
            // Stacked rows (conv_rows.cuh, Params::stack): tiles of BM / pitch consecutive rows of the sequence
            // img * OH + oh where that needs at least 5 % fewer tiles than whole tiles per image.
            const int64_t spbh = pitch <= tc::BM ? tc::BM / pitch : 0;
            const int64_t plain_tiles = rpbh > 0 ? a.N * ((OH + rpbh - 1) / rpbh) : 0;
            const int64_t stack_tiles = spbh > 0 ? (a.N * OH + spbh - 1) / spbh : 0;
            const bool row_stack = stack_rows_enabled && spbh >= 1 && std::min<int64_t>(spbh, OH) <= 9 &&
                                   stack_tiles * 20 <= plain_tiles * 19 && a.N * OH + tc::BM < (1LL << 31);
            const int64_t row_tiles = row_stack ? stack_tiles : plain_tiles;
            const int64_t row_max_h = row_stack ? std::min<int64_t>(spbh, OH) : rpbh;  // height of the largest box
            if (row_stack) rpbh = spbh;
            const int64_t patch_tiles = ((OW + pbw - 1) / pbw) * ((OH + pbh - 1) / pbh) * ((a.N + pbi - 1) / pbi);
            const bool applicable = rows_enabled && !a.dense_w && a.sh == 1 && a.sw == 1 && a.dw == 1 && a.kw <= rows::kMaxTaps &&
                                    (bn == 64 || bn == 128) && npass * K <= tc::kMaxAccumSteps && rpbh >= 1 &&
                                    row_tiles * 20 <= patch_tiles * 21 &&
                                    a.N * a.H * a.W * a.C * 2 < (1LL << 40) && a.W + a.pw < 32000;
            if (applicable) {
                rows::Params rp = {};
                rp.N = static_cast<int>(N);
                rp.C = static_cast<int>(a.C);
                rp.cblocks = static_cast<int>(a.C / 64);
                rp.kh = static_cast<int>(a.kh);
                rp.kw = static_cast<int>(a.kw);
                rp.dh = a.dh;
                rp.ph = a.ph;
                rp.pw = a.pw;
                rp.H = static_cast<int>(a.H);
                rp.W = static_cast<int>(a.W);
                rp.OH = static_cast<int>(OH);
                rp.OW = static_cast<int>(OW);
                rp.pitch = static_cast<int>(pitch);
                rp.pbh = static_cast<int>(rpbh);
                rp.tiles_per_image = static_cast<int>((OH + rpbh - 1) / rpbh);
                rp.stack = row_stack ? 1 : 0;
                rp.images = static_cast<int>(a.N);
                rp.max_h = static_cast<int>(row_max_h);
                const int64_t tiles_m = row_tiles;
                rp.tiles_n = static_cast<int>((N + bn - 1) / bn);
                rp.a_box_bytes = static_cast<int>(npass * pitch * rpbh * 128);
                rp.n_btiles = static_cast<int>(K / 64);
                rp.f16 = f16 ? 1 : 0;
                rp.amax_bits = amax_slot;
                rp.y = a.y;
                rp.y_cl = static_cast<__nv_bfloat16*>(a.y_cl);
                rp.y_cl_term_stride = M * N;
                rp.ep = a.ep;
                rp.ep.scale = a.ep.scale;
                rp.err_word = device_error_word();
                if (tiles_m * rp.tiles_n < (1LL << 31)) {
                    rp.tiles_m = static_cast<int>(tiles_m);
                    CUtensorMap map_x;
                    const cuuint64_t gdim[5] = {static_cast<cuuint64_t>(a.C), static_cast<cuuint64_t>(a.W), static_cast<cuuint64_t>(a.H),
                                                static_cast<cuuint64_t>(a.N), static_cast<cuuint64_t>(npass)};
                    const cuuint64_t gstride[4] = {static_cast<cuuint64_t>(a.C) * 2, static_cast<cuuint64_t>(a.W * a.C) * 2,
                                                   static_cast<cuuint64_t>(a.H * a.W * a.C) * 2, static_cast<cuuint64_t>(term_stride) * 2};
                    const cuuint32_t box[5] = {tc::BK, static_cast<cuuint32_t>(pitch), static_cast<cuuint32_t>(row_max_h), 1, 1};
                    const cuuint32_t estr[5] = {1, 1, 1, 1, 1};
                    rows::RowMaps row_maps = {};
                    bool maps_ok = true;
                    for (int64_t h = 1; row_stack && h < row_max_h; ++h) {  // the smaller box heights of stacked tiles
                        const cuuint32_t hbox[5] = {tc::BK, static_cast<cuuint32_t>(pitch), static_cast<cuuint32_t>(h), 1, 1};
                        maps_ok = maps_ok && encode(&row_maps.m[h - 1], f16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16,
                                                    5, xs, gdim, gstride, hbox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
                    }
                    const CUresult cr = encode(&map_x, f16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 5, xs, gdim,
                                               gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
                    if (cr == CUDA_SUCCESS && maps_ok) {
                        const bool one_term = tern_act || npass == 1;
                        // Resident filters when one column tile covers all output channels and they fit beside two stages.
                        int st_res = 0, st_str = 0;
                        if (bn == 64) {
                            st_res = rp.tiles_n == 1 ? (one_term ? rows::stages_that_fit<64, 1, true>(rp.n_btiles) : rows::stages_that_fit<64, 2, true>(rp.n_btiles)) : 0;
                            st_str = one_term ? rows::stages_that_fit<64, 1, false>(0) : rows::stages_that_fit<64, 2, false>(0);
                        } else {
                            st_res = rp.tiles_n == 1 ? (one_term ? rows::stages_that_fit<128, 1, true>(rp.n_btiles) : rows::stages_that_fit<128, 2, true>(rp.n_btiles)) : 0;
                            st_str = one_term ? rows::stages_that_fit<128, 1, false>(0) : rows::stages_that_fit<128, 2, false>(0);
                        }
                        const bool resident = st_res >= 2;
                        rp.nstages = resident ? st_res : st_str;
                        // Three filter columns as one 192-column instruction (conv_rows.cuh, WIDE): 64 output channels,
                        // resident filters.  TBN_CONV_WIDE=0 in the environment keeps one instruction per filter tap.
                        static const bool wide_enabled = [] {
                            const char* v = std::getenv("TBN_CONV_WIDE");
                            return !(v && v[0] == '0');
                        }();
                        const int64_t qpr = (OW + rows::kQuarterOutputs - 1) / rows::kQuarterOutputs;
                        const int64_t wide_rows = (qpr == 1 || qpr == 2 || qpr == 4) ? 4 / qpr : 0;  // output rows per tile
                        const int64_t wide_plain = wide_rows > 0 ? a.N * ((OH + wide_rows - 1) / wide_rows) : 0;
                        const int64_t wide_stacked = wide_rows > 0 ? (a.N * OH + wide_rows - 1) / wide_rows : 0;
                        const bool wide_stack = stack_rows_enabled && wide_rows > 0 && wide_stacked * 20 <= wide_plain * 19 &&
                                                a.N * OH + tc::BM < (1LL << 31);
                        const int64_t wide_tiles = wide_stack ? wide_stacked : wide_plain;
                        if (wide_enabled && bn == 64 && N == 64 && a.kw == rows::kMaxTaps && resident && wide_rows > 0 &&
                            wide_tiles * 4 <= row_tiles * 5) {  // at most a quarter more tiles
                            const int st_wide = one_term ? rows::stages_that_fit<64, 1, true, true>(rp.n_btiles)
                                                         : rows::stages_that_fit<64, 2, true, true>(rp.n_btiles);
                            CUtensorMap map_q;  // one lane quarter: 32 pixels of one input row, 64 channels
                            const cuuint32_t qbox[5] = {tc::BK, 32, 1, 1, 1};
                            const CUresult qr = encode(&map_q, f16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 5, xs,
                                                       gdim, gstride, qbox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                                       CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
                            if (st_wide >= 2 && qr == CUDA_SUCCESS && wide_tiles < (1LL << 31)) {
                                rp.nstages = st_wide;
                                rp.qpr = static_cast<int>(qpr);
                                rp.pbh = static_cast<int>(wide_rows);
                                rp.tiles_per_image = static_cast<int>((OH + wide_rows - 1) / wide_rows);
                                rp.stack = wide_stack ? 1 : 0;
                                rp.tiles_m = static_cast<int>(wide_tiles);
                                rp.a_box_bytes = static_cast<int>(npass * tc::BM * 128);
                                return one_term ? rows::launch<64, 1, true, true>(map_q, maps.neg, rp, a.st)
                                                : rows::launch<64, 2, true, true>(map_q, maps.neg, rp, a.st);
                            }
                        }
                        if (rp.nstages >= 2) {
                            if (bn == 64) {
                                if (one_term) return resident ? rows::launch<64, 1, true>(map_x, maps.neg, rp, a.st, &row_maps) : rows::launch<64, 1, false>(map_x, maps.neg, rp, a.st, &row_maps);
                                return resident ? rows::launch<64, 2, true>(map_x, maps.neg, rp, a.st, &row_maps) : rows::launch<64, 2, false>(map_x, maps.neg, rp, a.st, &row_maps);
                            }
                            if (one_term) return resident ? rows::launch<128, 1, true>(map_x, maps.neg, rp, a.st, &row_maps) : rows::launch<128, 1, false>(map_x, maps.neg, rp, a.st, &row_maps);
                            return resident ? rows::launch<128, 2, true>(map_x, maps.neg, rp, a.st, &row_maps) : rows::launch<128, 2, false>(map_x, maps.neg, rp, a.st, &row_maps);
                        }
                    }
                }
            }
        }
        const bool patch_ok = pbw * a.sw <= 256 && pbh * a.sh <= 256 && a.sw <= 8 && a.sh <= 8 && pbi <= 256 &&
                              a.N * a.H * a.W * a.C * 2 < (1LL << 40);
        if (patch_ok) {
            // Stacked rows (gemm_tc.cuh, ConvGeom::stack_rows): tiles of whole output rows of the sequence img * OH + oh,
            // one box per image a tile touches -- where that needs at least 5 % fewer tiles than the rectangles.
            // TBN_CONV_STACK=0 in the environment keeps the rectangles (for A/B measurements).
            static const bool stack_enabled = [] {
                const char* v = std::getenv("TBN_CONV_STACK");
                return !(v && v[0] == '0');
            }();
            const int64_t srows = OW <= tc::BM ? tc::BM / OW : 0;
            const int64_t smax_h = std::min<int64_t>(srows, OH);
            const int64_t patch_tiles_m = ((OW + pbw - 1) / pbw) * ((OH + pbh - 1) / pbh) * ((a.N + pbi - 1) / pbi);
            const int64_t stack_tiles_m = srows > 0 ? (a.N * OH + srows - 1) / srows : 0;
            const bool stacked = stack_enabled && srows >= 2 && smax_h <= 9 && OW * a.sw <= 256 && smax_h * a.sh <= 256 &&
                                 stack_tiles_m * 20 <= patch_tiles_m * 19 && a.N * OH + tc::BM < (1LL << 31);
            if (stacked) {
                pbw = OW;
                pbh = smax_h;  // the activation map carries the largest height
                pbi = 1;
            }
            p.conv.stack_rows = stacked ? static_cast<int>(srows) : 0;
            p.conv.stack_max_h = static_cast<int>(smax_h);
            const cuuint64_t gdim[5] = {static_cast<cuuint64_t>(a.C), static_cast<cuuint64_t>(a.W), static_cast<cuuint64_t>(a.H),
                                        static_cast<cuuint64_t>(a.N), static_cast<cuuint64_t>(npass)};
            const cuuint64_t gstride[4] = {static_cast<cuuint64_t>(a.C) * 2, static_cast<cuuint64_t>(a.W * a.C) * 2,
                                           static_cast<cuuint64_t>(a.H * a.W * a.C) * 2, static_cast<cuuint64_t>(term_stride) * 2};
            const cuuint32_t box[5] = {tc::BK, static_cast<cuuint32_t>(pbw * a.sw), static_cast<cuuint32_t>(pbh * a.sh),
                                       static_cast<cuuint32_t>(pbi), 1};
            const cuuint32_t estr[5] = {1, static_cast<cuuint32_t>(a.sw), static_cast<cuuint32_t>(a.sh), 1, 1};
            for (int64_t h = 1; stacked && h < smax_h; ++h) {  // the smaller heights
                const cuuint32_t hbox[5] = {tc::BK, static_cast<cuuint32_t>(OW * a.sw), static_cast<cuuint32_t>(h * a.sh), 1, 1};
                const CUresult hr = encode(&maps.out.m[h - 1], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 5, xs, gdim, gstride, hbox, estr,
                                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                           CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
                TBN_REQUIRE(hr == CUDA_SUCCESS, TBN_CUDA_ERROR,
                            "cuTensorMapEncodeTiled (activation rows) failed with CUresult " + std::to_string(static_cast<int>(hr)));
            }
            const CUresult cr = encode(&maps.a, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 5, xs, gdim, gstride, box, estr,
                                       CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                       CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            TBN_REQUIRE(cr == CUDA_SUCCESS, TBN_CUDA_ERROR,
                        "cuTensorMapEncodeTiled (activation patches) failed with CUresult " + std::to_string(static_cast<int>(cr)));
            p.conv.pbw = static_cast<int>(pbw);
            p.conv.pbh = static_cast<int>(pbh);
            p.conv.pbi = static_cast<int>(pbi);
            p.conv.patches_w = static_cast<int>((OW + pbw - 1) / pbw);
            p.conv.patches_h = static_cast<int>((OH + pbh - 1) / pbh);
            p.conv.a_box_bytes = static_cast<int>(npass * (stacked ? srows * OW : pbw * pbh * pbi) * 128);
            const int64_t tiles_m = stacked ? stack_tiles_m : static_cast<int64_t>(p.conv.patches_w) * p.conv.patches_h * ((a.N + pbi - 1) / pbi);
            TBN_REQUIRE(tiles_m * p.tiles_n < (1LL << 31), TBN_INVALID_SHAPE, "conv2d: too many tiles");
            p.tiles_m = static_cast<int>(tiles_m);
            if (a.dense_w) {
                set_segments(p, 3);
                return dispatch_bn<2, false, 4, false, 1>(bn, maps, p, a.st);
            }
            if (tern_act || npass == 1) return dispatch_bn<1, false, 4, false, 2>(bn, maps, p, a.st);
            return dispatch_bn<2, false, 4, false, 2>(bn, maps, p, a.st);
        }
    }
    // Weight source: 1 = two-term float filters, 2 = expanded sign filters (binary and ternary alike).
    if (fast) {
        if (a.dense_w) {
            set_segments(p, 3);
            return dispatch_bn<2, false, 2, false, 1>(bn, maps, p, a.st);
        }
        if (tern_act || npass == 1) return dispatch_bn<1, false, 2, false, 2>(bn, maps, p, a.st);
        return dispatch_bn<2, false, 2, false, 2>(bn, maps, p, a.st);
    }
    if (a.dense_w) {
        set_segments(p, 3);
        return dispatch_bn<2, false, 1, false, 1>(bn, maps, p, a.st);
    }
    if (tern_act) return dispatch_bn<1, false, 1, true, 2>(bn, maps, p, a.st);
    if (npass == 1) return dispatch_bn<1, false, 1, false, 2>(bn, maps, p, a.st);
    return dispatch_bn<2, false, 1, false, 2>(bn, maps, p, a.st);
}

}  // namespace
}  // namespace tbn_cuda

using namespace tbn_cuda;

extern "C" {

size_t tbn_conv2d_workspace_bytes(int64_t N, int64_t C, int64_t H, int64_t W, int64_t M_out, int64_t kh, int64_t kw,
                                  int32_t weight_order) {
    if (N <= 0 || C <= 0 || H <= 0 || W <= 0 || M_out <= 0 || kh <= 0 || kw <= 0) return 0;
    const int64_t K_pad = round_up(C * kh * kw, 128);
    size_t front = weight_order == TBN_CONV_WEIGHTS_TAP_MAJOR ? xs_bytes(N, C, H, W, 2) : table_bytes(K_pad);
    size_t folded = 0;
    if (weight_order != TBN_CONV_WEIGHTS_TAP_MAJOR && C <= 4) {
        // Upper bounds of the space-to-depth form (the strides and pads are not known here).
        front = std::max(front, static_cast<size_t>(round_up(2 * N * ((H + 1) / 2) * ((W + 1) / 2 + 16) * 32, 256)));
        folded = static_cast<size_t>(round_up(2 * round_up(M_out, 8) * round_up((kh / 2 + 2) * 64, 128) * 2, 256));
    }
    return front + static_cast<size_t>(std::max(sm_count(), 160)) * tc::BM * 256 * sizeof(float) +
           expanded_bytes(K_pad, round_up(M_out, 8)) + folded + 256;
}

int32_t tbn_permute_filters(const float* d_w, int64_t M, int64_t C, int64_t taps, float* d_out, void* stream) {
    TBN_REQUIRE(M > 0 && C > 0 && taps > 0 && C < (1LL << 31) && taps < (1LL << 31), TBN_INVALID_SHAPE,
                "tbn_permute_filters: bad dimensions");
    TBN_REQUIRE(d_w && d_out && d_w != d_out, TBN_INVALID_ARGUMENT, "tbn_permute_filters: null or aliased pointers");
    const int64_t total = M * C * taps;
    const int grid = static_cast<int>(std::max<int64_t>(1, std::min((total + 255) / 256, static_cast<int64_t>(std::max(sm_count(), 1)) * 16)));
    permute_filters_kernel<<<grid, 256, 0, as_stream(stream)>>>(d_w, M, static_cast<int>(C), static_cast<int>(taps), d_out);
    return launched("permute_filters_kernel");
}

int32_t tbn_conv2d_fxb(const float* d_x, int64_t N, int64_t C, int64_t H, int64_t W, const uint32_t* d_neg,
                       const uint32_t* d_pos, int64_t M_out, int64_t kh, int64_t kw, int32_t sh, int32_t sw, int32_t ph,
                       int32_t pw, int32_t dh, int32_t dw, const float* d_alpha, float scale, const float* d_bias,
                       const float* d_residual, float* d_y, int32_t mode, uint32_t epilogue, int32_t weight_order,
                       void* d_workspace, size_t workspace_bytes, void* stream) {
    TBN_REQUIRE(mode == TBN_MODE_AUTO || mode == TBN_MODE_TC_BF16X1 || mode == TBN_MODE_TC_BF16X2 || mode == TBN_MODE_TC_FP16X1,
                TBN_NOT_IMPLEMENTED, "tbn_conv2d_fxb: modes are AUTO (= two bf16 terms), TC_BF16X1, TC_BF16X2 and TC_FP16X1");
    ConvArgs a{nullptr, d_x, N, C, H, W, d_neg, d_pos, M_out, kh, kw, sh, sw, ph, pw, dh, dw,
               Epilogue{d_alpha, d_bias, d_residual, scale, epilogue}, d_y, d_workspace, workspace_bytes,
               as_stream(stream), weight_order};
    // The one-pass fp16 form exists for the channels-last path; other geometries run the two-term form, which is
    // more accurate than what was asked for.
    a.f16 = mode == TBN_MODE_TC_FP16X1 && weight_order == TBN_CONV_WEIGHTS_TAP_MAJOR;
    return conv_common(a, (mode == TBN_MODE_TC_BF16X1 || a.f16) ? 1 : 2, false, 0.f, 0.f);
}

int32_t tbn_conv2d_fxb_chain(const float* d_x, const void* d_x_cl, int64_t N, int64_t C, int64_t H, int64_t W,
                             const uint32_t* d_neg, const uint32_t* d_pos, int64_t M_out, int64_t kh, int64_t kw, int32_t sh,
                             int32_t sw, int32_t ph, int32_t pw, int32_t dh, int32_t dw, const float* d_alpha, float scale,
                             const float* d_bias, const float* d_residual, float* d_y, void* d_y_cl, int32_t mode,
                             uint32_t epilogue, int32_t weight_order, void* d_workspace, size_t workspace_bytes, void* stream) {
    TBN_REQUIRE(mode == TBN_MODE_AUTO || mode == TBN_MODE_TC_BF16X1 || mode == TBN_MODE_TC_BF16X2, TBN_NOT_IMPLEMENTED,
                "tbn_conv2d_fxb_chain: modes are AUTO (= two bf16 terms), TC_BF16X1 and TC_BF16X2");
    ConvArgs a{nullptr, d_x, N, C, H, W, d_neg, d_pos, M_out, kh, kw, sh, sw, ph, pw, dh, dw,
               Epilogue{d_alpha, d_bias, d_residual, scale, epilogue}, d_y, d_workspace, workspace_bytes,
               as_stream(stream), weight_order};
    a.x_cl = d_x_cl;
    a.y_cl = d_y_cl;
    return conv_common(a, mode == TBN_MODE_TC_BF16X1 ? 1 : 2, false, 0.f, 0.f);
}

int32_t tbn_conv2d_f32_chain(const float* d_x, const void* d_x_cl, int64_t N, int64_t C, int64_t H, int64_t W,
                             const void* d_packed_w, int64_t M_out, int64_t kh, int64_t kw, int32_t sh, int32_t sw, int32_t ph,
                             int32_t pw, int32_t dh, int32_t dw, const float* d_bias, const float* d_residual, float* d_y,
                             void* d_y_cl, uint32_t epilogue, int32_t weight_order, void* d_workspace, size_t workspace_bytes,
                             void* stream) {
    TBN_REQUIRE(d_packed_w != nullptr, TBN_INVALID_ARGUMENT, "tbn_conv2d_f32_chain: null weights");
    ConvArgs a{d_packed_w, d_x, N, C, H, W, nullptr, nullptr, M_out, kh, kw, sh, sw, ph, pw, dh, dw,
               Epilogue{nullptr, d_bias, d_residual, 1.0f, epilogue}, d_y, d_workspace, workspace_bytes,
               as_stream(stream), weight_order};
    a.x_cl = d_x_cl;
    a.y_cl = d_y_cl;
    return conv_common(a, 2, false, 0.f, 0.f);
}

int32_t tbn_conv2d_tbn(const float* d_x, int64_t N, int64_t C, int64_t H, int64_t W, float lo, float hi,
                       const uint32_t* d_neg, int64_t M_out, int64_t kh, int64_t kw, int32_t sh, int32_t sw, int32_t ph,
                       int32_t pw, int32_t dh, int32_t dw, const float* d_alpha, float scale, const float* d_bias,
                       float* d_y, uint32_t epilogue, int32_t weight_order, void* d_workspace, size_t workspace_bytes,
                       void* stream) {
    const ConvArgs a{nullptr, d_x, N, C, H, W, d_neg, nullptr, M_out, kh, kw, sh, sw, ph, pw, dh, dw,
                     Epilogue{d_alpha, d_bias, nullptr, scale, epilogue & ~TBN_EPI_ADD_RESIDUAL}, d_y, d_workspace,
                     workspace_bytes, as_stream(stream), weight_order};
    return conv_common(a, 1, true, lo, hi);
}

int32_t tbn_conv2d_f32(const float* d_x, int64_t N, int64_t C, int64_t H, int64_t W, const void* d_packed_w, int64_t M_out,
                       int64_t kh, int64_t kw, int32_t sh, int32_t sw, int32_t ph, int32_t pw, int32_t dh, int32_t dw,
                       const float* d_bias, const float* d_residual, float* d_y, uint32_t epilogue, int32_t weight_order,
                       void* d_workspace, size_t workspace_bytes, void* stream) {
    TBN_REQUIRE(d_packed_w != nullptr, TBN_INVALID_ARGUMENT, "tbn_conv2d_f32: null weights");
    const ConvArgs a{d_packed_w, d_x, N, C, H, W, nullptr, nullptr, M_out, kh, kw, sh, sw, ph, pw, dh, dw,
                     Epilogue{nullptr, d_bias, d_residual, 1.0f, epilogue}, d_y, d_workspace, workspace_bytes,
                     as_stream(stream), weight_order};
    return conv_common(a, 2, false, 0.f, 0.f);
}

}  // extern "C"
