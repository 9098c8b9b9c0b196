// Glue operators of the CNN graphs, device resident (all HBM-bound, one pass over the data):
// ReLU, Add (the broadcast forms the reference Session accepts), MaxPool / AveragePool,
// GlobalAveragePool / GlobalMaxPool, the Greater / Less / Sub trio of the exported ternary-activation subgraph,
// and a 2-D transpose (Gemm with transA / transB).  Stand in for Session::execute_relu / execute_add /
// execute_greater / execute_less / execute_sub (tbn/runtime/model.hpp:905-1316) and
// tbn-runtime/src/operators/pooling.cpp:10-216.
#include <algorithm>

#include "common.cuh"

namespace tbn_cuda {
namespace {

__global__ void relu_kernel(const float* __restrict__ x, int64_t n, float* __restrict__ y) {
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride)
        y[i] = fmaxf(x[i], 0.0f);  // std::max(0.0f, x): NaN -> 0 as in the reference
}

// out[i] = a[i] + b[(i / inner) % b_n]; b_n == a_n (inner 1) is the same-shape add.
__global__ void add_kernel(const float* __restrict__ a, int64_t a_n, const float* __restrict__ b, int64_t b_n,
                           int64_t inner, float* __restrict__ y, int relu) {
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < a_n; i += stride) {
        const float v = __fadd_rn(a[i], b[(i / inner) % b_n]);
        y[i] = relu ? fmaxf(v, 0.0f) : v;
    }
}

// kind 0: max over the in-range taps (-inf if none); kind 1: average (pooling.cpp:50-76, 116-143).
__global__ void pool2d_kernel(int kind, const float* __restrict__ x, int64_t NC, int H, int W, int OH, int OW, int kh,
                              int kw, int sh, int sw, int ph, int pw, int count_include_pad, float* __restrict__ y) {
    const int64_t total = NC * OH * OW;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total; idx += stride) {
        const int ow = static_cast<int>(idx % OW);
        const int oh = static_cast<int>((idx / OW) % OH);
        const int64_t nc = idx / (static_cast<int64_t>(OW) * OH);
        const float* plane = x + nc * H * W;
        float best = -INFINITY, sum = 0.0f;
        int count = 0;
        for (int i = 0; i < kh; ++i) {
            const int ih = oh * sh - ph + i;
            for (int j = 0; j < kw; ++j) {
                const int iw = ow * sw - pw + j;
                if (ih >= 0 && ih < H && iw >= 0 && iw < W) {
                    const float v = plane[ih * W + iw];
                    best = best > v ? best : v;
                    sum = __fadd_rn(sum, v);
                    ++count;
                } else if (count_include_pad) {
                    ++count;
                }
            }
        }
        y[idx] = kind == 0 ? best : (count > 0 ? __fdiv_rn(sum, static_cast<float>(count)) : 0.0f);
    }
}

// 3 x 3 / stride 2 / pad 1 max pool (the stem pool of the ResNet graphs), W % 4 == 0: one warp per output row of one
// plane.  Each lane loads four input columns of the three input rows as float4 (fully coalesced; neighbouring
// warps of the block share the rows through L1/L2), takes the column to its left from the lane before it, and
// forms two outputs with the comparisons in the same tap order (i, then j) and with the same `best > v ? best : v`
// rule as the general kernel -- bit-identical to it, NaNs included.  HBM bound: every input row is read from DRAM
// once, the output written once.
__global__ void __launch_bounds__(256) maxpool_3x3s2p1_kernel(const float* __restrict__ x, int64_t rows_total, int H, int W,
                                                              int OH, int OW, float* __restrict__ y) {
    const int64_t row = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);  // (plane, oh)
    if (row >= rows_total) return;
    const int lane = threadIdx.x & 31;
    const int64_t plane = row / OH;
    const int oh = static_cast<int>(row - plane * OH);
    const float* in = x + plane * H * W;
    float* out = y + plane * OH * OW + static_cast<int64_t>(oh) * OW;
    for (int c0 = 0; c0 < W; c0 += 128) {
        const int col = c0 + 4 * lane;  // this lane's four input columns; outputs ow0 = col / 2 and ow0 + 1
        float best0 = -INFINITY, best1 = -INFINITY;
#pragma unroll
        for (int i = 0; i < 3; ++i) {
            const int ih = 2 * oh - 1 + i;
            const bool row_in = ih >= 0 && ih < H;  // warp-uniform
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (row_in && col < W) v = __ldg(reinterpret_cast<const float4*>(in + static_cast<int64_t>(ih) * W + col));
            float left = __shfl_up_sync(0xffffffffu, v.w, 1);
            if (lane == 0 && row_in && c0 > 0) left = __ldg(in + static_cast<int64_t>(ih) * W + c0 - 1);
            if (!row_in) continue;
            // output ow0: columns col-1, col, col+1; output ow0+1: columns col+1, col+2, col+3 (all < W when col < W)
            if (col > 0) best0 = best0 > left ? best0 : left;
            best0 = best0 > v.x ? best0 : v.x;
            best0 = best0 > v.y ? best0 : v.y;
            best1 = best1 > v.y ? best1 : v.y;
            best1 = best1 > v.z ? best1 : v.z;
            best1 = best1 > v.w ? best1 : v.w;
        }
        const int ow0 = col >> 1;
        if (col < W) {
            if (ow0 + 1 < OW) *reinterpret_cast<float2*>(out + ow0) = make_float2(best0, best1);
            else if (ow0 < OW) out[ow0] = best0;
        }
    }
}

// One warp per (n, c) plane.
__global__ void global_avgpool_kernel(const float* __restrict__ x, int64_t NC, int64_t HW, float* __restrict__ y) {
    const int64_t plane = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (plane >= NC) return;
    const int lane = threadIdx.x & 31;
    float sum = 0.0f;
    for (int64_t i = lane; i < HW; i += 32) sum += x[plane * HW + i];
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) sum += __shfl_down_sync(0xffffffffu, sum, off);
    if (lane == 0) y[plane] = __fdiv_rn(sum, static_cast<float>(HW));
}

// One warp per (n, c) plane; std::max semantics (a NaN element never replaces the running maximum).
__global__ void global_maxpool_kernel(const float* __restrict__ x, int64_t NC, int64_t HW, float* __restrict__ y) {
    const int64_t plane = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (plane >= NC) return;
    const int lane = threadIdx.x & 31;
    float best = -INFINITY;
    for (int64_t i = lane; i < HW; i += 32) {
        const float v = x[plane * HW + i];
        best = best < v ? v : best;
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        const float other = __shfl_down_sync(0xffffffffu, best, off);
        best = best < other ? other : best;
    }
    if (lane == 0) y[plane] = best;
}

// op 0: y = x > rhs ? 1 : 0; op 1: y = x < rhs ? 1 : 0; op 2: y = x - rhs.  rhs is indexed modulo its length,
// the flat broadcast of the reference Session (model.hpp:1213-1216, 1260-1263, 1309-1311).
__global__ void binary_elementwise_kernel(int op, const float* __restrict__ x, int64_t n, const float* __restrict__ rhs,
                                          int64_t rhs_n, float* __restrict__ y) {
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
        const float a = x[i], b = rhs[rhs_n == n ? i : i % rhs_n];
        y[i] = op == 0 ? (a > b ? 1.0f : 0.0f) : op == 1 ? (a < b ? 1.0f : 0.0f) : __fsub_rn(a, b);
    }
}

// y[c][r] = x[r][c] through a 32 x 33 shared-memory tile (both sides coalesced).
__global__ void transpose2d_kernel(const float* __restrict__ x, int64_t rows, int64_t cols, float* __restrict__ y) {
    __shared__ float tile[32][33];
    const int64_t c0 = static_cast<int64_t>(blockIdx.x) * 32, r0 = static_cast<int64_t>(blockIdx.y) * 32;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8 threads
    for (int i = ty; i < 32; i += 8)
        if (r0 + i < rows && c0 + tx < cols) tile[i][tx] = x[(r0 + i) * cols + c0 + tx];
    __syncthreads();
    for (int i = ty; i < 32; i += 8)
        if (c0 + i < cols && r0 + tx < rows) y[(c0 + i) * rows + r0 + tx] = tile[tx][i];
}

int grid_for(int64_t n) {
    const int64_t cap = static_cast<int64_t>(sm_count() > 0 ? sm_count() : 148) * 16;
    return static_cast<int>(std::max<int64_t>(1, std::min((n + 255) / 256, cap)));
}

}  // namespace
}  // namespace tbn_cuda

using namespace tbn_cuda;

extern "C" {

int32_t tbn_relu(const float* d_x, int64_t n, float* d_y, void* stream) {
    TBN_REQUIRE(n >= 0, TBN_INVALID_ARGUMENT, "tbn_relu: negative size");
    if (n == 0) return TBN_SUCCESS;
    TBN_REQUIRE(d_x && d_y, TBN_INVALID_ARGUMENT, "tbn_relu: null pointer");
    relu_kernel<<<grid_for(n), 256, 0, as_stream(stream)>>>(d_x, n, d_y);
    return launched("relu_kernel");
}

int32_t tbn_add(const float* d_a, int64_t a_n, const float* d_b, int64_t b_n, int64_t inner, int32_t relu, float* d_y,
                void* stream) {
    TBN_REQUIRE(a_n >= 0 && b_n > 0 && inner > 0, TBN_INVALID_ARGUMENT, "tbn_add: bad sizes");
    if (a_n == 0) return TBN_SUCCESS;
    TBN_REQUIRE(d_a && d_b && d_y, TBN_INVALID_ARGUMENT, "tbn_add: null pointer");
    TBN_REQUIRE(a_n == b_n || a_n % (b_n * inner) == 0, TBN_INVALID_SHAPE, "tbn_add: shapes do not broadcast");
    add_kernel<<<grid_for(a_n), 256, 0, as_stream(stream)>>>(d_a, a_n, d_b, b_n, a_n == b_n ? 1 : inner, d_y, relu);
    return launched("add_kernel");
}

int32_t tbn_pool2d(int32_t kind, const float* d_x, int64_t N, int64_t C, int64_t H, int64_t W, int32_t kh, int32_t kw,
                   int32_t sh, int32_t sw, int32_t ph, int32_t pw, int32_t ceil_mode, int32_t count_include_pad,
                   float* d_y, void* stream) {
    TBN_REQUIRE(kind == 0 || kind == 1, TBN_INVALID_ARGUMENT, "tbn_pool2d: kind must be 0 (max) or 1 (average)");
    TBN_REQUIRE(N > 0 && C > 0 && H > 0 && W > 0 && kh > 0 && kw > 0 && sh > 0 && sw > 0 && ph >= 0 && pw >= 0,
                TBN_INVALID_SHAPE, "tbn_pool2d: bad dimensions");
    TBN_REQUIRE(d_x && d_y, TBN_INVALID_ARGUMENT, "tbn_pool2d: null pointer");
    // pooling.cpp:28-34
    const int64_t OH = ceil_mode ? (H + 2 * ph - kh + sh - 1) / sh + 1 : (H + 2 * ph - kh) / sh + 1;
    const int64_t OW = ceil_mode ? (W + 2 * pw - kw + sw - 1) / sw + 1 : (W + 2 * pw - kw) / sw + 1;
    TBN_REQUIRE(OH > 0 && OW > 0 && H < (1 << 30) && W < (1 << 30), TBN_INVALID_SHAPE, "tbn_pool2d: empty output");
    if (kind == 0 && kh == 3 && kw == 3 && sh == 2 && sw == 2 && ph == 1 && pw == 1 && !ceil_mode && W % 4 == 0 &&
        reinterpret_cast<uintptr_t>(d_x) % 16 == 0 && reinterpret_cast<uintptr_t>(d_y) % 8 == 0 && OW % 2 == 0 &&
        N * C * OH < (1LL << 33)) {
        const int64_t rows = N * C * OH;
        maxpool_3x3s2p1_kernel<<<static_cast<unsigned>((rows + 7) / 8), 256, 0, as_stream(stream)>>>(
            d_x, rows, static_cast<int>(H), static_cast<int>(W), static_cast<int>(OH), static_cast<int>(OW), d_y);
        return launched("maxpool_3x3s2p1_kernel");
    }
    pool2d_kernel<<<grid_for(N * C * OH * OW), 256, 0, as_stream(stream)>>>(
        kind, d_x, N * C, static_cast<int>(H), static_cast<int>(W), static_cast<int>(OH), static_cast<int>(OW), kh, kw,
        sh, sw, ph, pw, count_include_pad, d_y);
    return launched("pool2d_kernel");
}

int32_t tbn_global_avgpool2d(const float* d_x, int64_t N, int64_t C, int64_t H, int64_t W, float* d_y, void* stream) {
    TBN_REQUIRE(N > 0 && C > 0 && H > 0 && W > 0, TBN_INVALID_SHAPE, "tbn_global_avgpool2d: bad dimensions");
    TBN_REQUIRE(d_x && d_y, TBN_INVALID_ARGUMENT, "tbn_global_avgpool2d: null pointer");
    const int64_t planes = N * C;
    global_avgpool_kernel<<<static_cast<unsigned>((planes + 7) / 8), 256, 0, as_stream(stream)>>>(d_x, planes, H * W, d_y);
    return launched("global_avgpool_kernel");
}

int32_t tbn_global_maxpool2d(const float* d_x, int64_t N, int64_t C, int64_t H, int64_t W, float* d_y, void* stream) {
    TBN_REQUIRE(N > 0 && C > 0 && H > 0 && W > 0, TBN_INVALID_SHAPE, "tbn_global_maxpool2d: bad dimensions");
    TBN_REQUIRE(d_x && d_y, TBN_INVALID_ARGUMENT, "tbn_global_maxpool2d: null pointer");
    const int64_t planes = N * C;
    global_maxpool_kernel<<<static_cast<unsigned>((planes + 7) / 8), 256, 0, as_stream(stream)>>>(d_x, planes, H * W, d_y);
    return launched("global_maxpool_kernel");
}

int32_t tbn_binary_elementwise(int32_t op, const float* d_x, int64_t n, const float* d_rhs, int64_t rhs_n, float* d_y,
                               void* stream) {
    TBN_REQUIRE(op >= TBN_ELT_GREATER && op <= TBN_ELT_SUB, TBN_INVALID_ARGUMENT, "tbn_binary_elementwise: unknown operation");
    TBN_REQUIRE(n >= 0 && rhs_n > 0, TBN_INVALID_ARGUMENT, "tbn_binary_elementwise: bad sizes");
    if (n == 0) return TBN_SUCCESS;
    TBN_REQUIRE(d_x && d_rhs && d_y, TBN_INVALID_ARGUMENT, "tbn_binary_elementwise: null pointer");
    binary_elementwise_kernel<<<grid_for(n), 256, 0, as_stream(stream)>>>(op, d_x, n, d_rhs, rhs_n, d_y);
    return launched("binary_elementwise_kernel");
}

int32_t tbn_transpose2d(const float* d_x, int64_t rows, int64_t cols, float* d_y, void* stream) {
    TBN_REQUIRE(rows > 0 && cols > 0, TBN_INVALID_SHAPE, "tbn_transpose2d: bad dimensions");
    TBN_REQUIRE(d_x && d_y && d_x != d_y, TBN_INVALID_ARGUMENT, "tbn_transpose2d: null or aliased pointers");
    const int64_t gx = (cols + 31) / 32, gy = (rows + 31) / 32;
    TBN_REQUIRE(gx < (1LL << 31) && gy <= 65535, TBN_INVALID_SHAPE, "tbn_transpose2d: matrix too large");
    transpose2d_kernel<<<dim3(static_cast<unsigned>(gx), static_cast<unsigned>(gy)), 256, 0, as_stream(stream)>>>(d_x, rows, cols, d_y);
    return launched("transpose2d_kernel");
}

}  // extern "C"
