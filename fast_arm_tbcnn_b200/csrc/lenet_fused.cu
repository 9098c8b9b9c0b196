// The LeNet-shaped binary CNN as ONE kernel: Conv 1->C1 5x5 + bias, ReLU, MaxPool 2x2, Conv C1->C2 5x5 + bias, ReLU,
// MaxPool 2x2, Flatten, Gemm C2*16 -> classes + bias on 1 x 28 x 28 inputs, float x binary mode
// (y = (sum +-x) * alpha + bias per layer).  Replaces, for this graph, the eight-node sequence the reference Session
// executes node by node (tbn/runtime/model.hpp:190-228: execute_conv, execute_relu, execute_maxpool, execute_gemm;
// conv2d.cpp:220-369, pooling.cpp:10-80) and the nine launches of the layer-by-layer path here.
//
// The network is launch- and HBM-bound layer by layer (a few KB per image between layers).  Here a block keeps one
// image and all its intermediates in shared memory, the sign bits of all three weight tensors live in registers /
// shared memory, and only the image (3136 B) is read and the logits (4 * classes B) written: the compulsory bytes.
// Arithmetic is add / subtract by sign on the CUDA cores, fp32, taps in the reference's (c, i, j) order.
//   conv1 + ReLU + pool: one thread per pooled output (C1 x 12 x 12), 6 x 6 input window in registers
//   conv2 + ReLU + pool: one thread per pooled output (C2 x 4 x 4 = 256 threads), its filter's sign words in registers
//   Gemm: one warp per class, shuffle reduction
#include <algorithm>

#include "common.cuh"

namespace tbn_cuda {
namespace {

constexpr int kImg = 28, kK = 5, kC1Out = 24, kP1 = 12, kC2Out = 8, kP2 = 4;
constexpr int kThreadsLenet = 256;

__device__ __forceinline__ float signed_add(float acc, float x, uint32_t neg_bit) {
    return __fadd_rn(acc, __uint_as_float(__float_as_uint(x) ^ (neg_bit << 31)));
}

// Packed layouts (see tbn_quant_pack_binary): conv filters [M_out][K_pad/32] with k = (c*5 + i)*5 + j (bit set <=> -1);
// Gemm weights [N_pad][K_pad/32] with k = flattened (c2, py, px).
template <int C1, int C2>
__global__ void __launch_bounds__(kThreadsLenet, 2) lenet_fused_kernel(const float* __restrict__ x, int64_t batch,
                                                                    const uint32_t* __restrict__ w1, const float* __restrict__ a1,
                                                                    const float* __restrict__ b1, const uint32_t* __restrict__ w2,
                                                                    const float* __restrict__ a2, const float* __restrict__ b2,
                                                                    const uint32_t* __restrict__ wf, const float* __restrict__ af,
                                                                    const float* __restrict__ bf, int classes, float* __restrict__ y) {
    static_assert(C2 * kP2 * kP2 == kThreadsLenet, "one thread per pooled output of the second convolution");
    constexpr int K2 = C1 * kK * kK, K2_WORDS = (K2 + 127) / 128 * 4, KF_WORDS = kThreadsLenet / 32;
    __shared__ __align__(16) float img[kImg * kImg];
    __shared__ float p1[C1][kP1][kP1 + 1];
    __shared__ float p2[kThreadsLenet];
    __shared__ uint32_t w1_s[C1];
    __shared__ float a1_s[C1], b1_s[C1];
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    if (t < C1) {
        w1_s[t] = __ldg(w1 + t * 4);  // K = 25 -> K_pad = 128: four words per filter, the first holds all 25 taps
        a1_s[t] = a1 ? __ldg(a1 + t) : 1.0f;
        b1_s[t] = b1 ? __ldg(b1 + t) : 0.0f;
    }
    // This thread's second-layer filter and output position: fixed for the whole kernel.
    const int c2 = t / (kP2 * kP2), py2 = (t / kP2) % kP2, px2 = t % kP2;
    uint32_t w2_r[(K2 + 31) / 32];
#pragma unroll
    for (int i = 0; i < (K2 + 31) / 32; ++i) w2_r[i] = __ldg(w2 + c2 * K2_WORDS + i);
    const float alpha2 = a2 ? __ldg(a2 + c2) : 1.0f, bias2 = b2 ? __ldg(b2 + c2) : 0.0f;
    __syncthreads();

    for (int64_t n = blockIdx.x; n < batch; n += gridDim.x) {
        // ---- image -> shared memory (196 float4)
        const float4* src = reinterpret_cast<const float4*>(x + n * (kImg * kImg));
        if (t < kImg * kImg / 4) reinterpret_cast<float4*>(img)[t] = __ldg(src + t);
        __syncthreads();
        // ---- conv1 + bias + ReLU + 2x2 max pool
        for (int o = t; o < C1 * kP1 * kP1; o += kThreadsLenet) {
            const int c = o / (kP1 * kP1), py = (o / kP1) % kP1, px = o % kP1;
            float win[kK + 1][kK + 1];
#pragma unroll
            for (int i = 0; i <= kK; ++i)
#pragma unroll
                for (int j = 0; j <= kK; ++j) win[i][j] = img[(2 * py + i) * kImg + 2 * px + j];
            const uint32_t bits = w1_s[c];
            float best = 0.0f;  // ReLU then max == max with 0
#pragma unroll
            for (int dy = 0; dy < 2; ++dy)
#pragma unroll
                for (int dx = 0; dx < 2; ++dx) {
                    float acc = 0.0f;
#pragma unroll
                    for (int i = 0; i < kK; ++i)
#pragma unroll
                        for (int j = 0; j < kK; ++j) acc = signed_add(acc, win[dy + i][dx + j], (bits >> (i * kK + j)) & 1u);
                    best = fmaxf(best, __fadd_rn(__fmul_rn(acc, a1_s[c]), b1_s[c]));
                }
            p1[c][py][px] = best;
        }
        __syncthreads();
        // ---- conv2 + bias + ReLU + 2x2 max pool: pooled output (c2, py2, px2)
        {
            float acc[2][2] = {{0.f, 0.f}, {0.f, 0.f}};
#pragma unroll
            for (int c = 0; c < C1; ++c) {
                float win[kK + 1][kK + 1];
#pragma unroll
                for (int i = 0; i <= kK; ++i)
#pragma unroll
                    for (int j = 0; j <= kK; ++j) win[i][j] = p1[c][2 * py2 + i][2 * px2 + j];
#pragma unroll
                for (int i = 0; i < kK; ++i)
#pragma unroll
                    for (int j = 0; j < kK; ++j) {
                        const int k = (c * kK + i) * kK + j;  // compile-time constant after unrolling
                        const uint32_t bit = (w2_r[k >> 5] >> (k & 31)) & 1u;
                        acc[0][0] = signed_add(acc[0][0], win[i][j], bit);
                        acc[0][1] = signed_add(acc[0][1], win[i][j + 1], bit);
                        acc[1][0] = signed_add(acc[1][0], win[i + 1][j], bit);
                        acc[1][1] = signed_add(acc[1][1], win[i + 1][j + 1], bit);
                    }
            }
            float best = 0.0f;
#pragma unroll
            for (int dy = 0; dy < 2; ++dy)
#pragma unroll
                for (int dx = 0; dx < 2; ++dx) best = fmaxf(best, __fadd_rn(__fmul_rn(acc[dy][dx], alpha2), bias2));
            p2[t] = best;  // flattened index (c2, py2, px2) = t: the Flatten order of NCHW
        }
        __syncthreads();
        // ---- Gemm: one warp per class
        for (int cls = warp; cls < classes; cls += kThreadsLenet / 32) {
            float acc = 0.0f;
#pragma unroll
            for (int j = 0; j < KF_WORDS; ++j) {
                const uint32_t word = __ldg(wf + cls * KF_WORDS + j);  // k = 32 j + lane
                acc = signed_add(acc, p2[32 * j + lane], (word >> lane) & 1u);
            }
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, off));
            if (lane == 0) y[n * classes + cls] = __fadd_rn(__fmul_rn(acc, af ? __ldg(af + cls) : 1.0f), bf ? __ldg(bf + cls) : 0.0f);
        }
        // The next iteration's first barrier (after the image load) orders these reads of p2 / p1 before their rewrite:
        // img is rewritten before it, but nothing reads img after the conv1 barrier above.
    }
}

}  // namespace
}  // namespace tbn_cuda

using namespace tbn_cuda;

extern "C" int32_t tbn_lenet_fused_fxb(const float* d_x, int64_t batch, int32_t c1, int32_t c2, int32_t classes,
                                       const uint32_t* d_w1, const float* d_alpha1, const float* d_bias1, const uint32_t* d_w2,
                                       const float* d_alpha2, const float* d_bias2, const uint32_t* d_wf, const float* d_alphaf,
                                       const float* d_biasf, float* d_y, void* stream) {
    TBN_REQUIRE(batch > 0, TBN_INVALID_SHAPE, "tbn_lenet_fused_fxb: batch must be positive");
    TBN_REQUIRE(c1 == 6 && c2 == 16, TBN_NOT_IMPLEMENTED,
                "tbn_lenet_fused_fxb: built for 6 and 16 feature maps (the simple_cnn shape); use the layer entry points otherwise");
    TBN_REQUIRE(classes >= 1 && classes <= 64, TBN_INVALID_SHAPE, "tbn_lenet_fused_fxb: between 1 and 64 classes");
    TBN_REQUIRE(d_x && d_w1 && d_w2 && d_wf && d_y, TBN_INVALID_ARGUMENT, "tbn_lenet_fused_fxb: null pointer");
    TBN_REQUIRE(reinterpret_cast<uintptr_t>(d_x) % 16 == 0, TBN_INVALID_ARGUMENT, "tbn_lenet_fused_fxb: input must be 16-byte aligned");
    const int sms = sm_count() > 0 ? sm_count() : 148;
    const int grid = static_cast<int>(std::min<int64_t>(batch, static_cast<int64_t>(sms) * 8));
    lenet_fused_kernel<6, 16><<<grid, kThreadsLenet, 0, as_stream(stream)>>>(d_x, batch, d_w1, d_alpha1, d_bias1, d_w2, d_alpha2,
                                                                            d_bias2, d_wf, d_alphaf, d_biasf, classes, d_y);
    return launched("lenet_fused_kernel");
}
