// Operator functions of the tbn:: API on the GPU.
//
// Names, argument order and error behaviour follow the reference's operator headers
// (tbn-runtime/include/tbn/operators/{conv2d,gemm,quantized_gemm,pooling}.hpp); every function
// accepts host or device tensors and returns a DEVICE-resident tensor (read it back with
// typed_data<T>()).  All arithmetic runs in libtbn_cuda through the C ABI (include/tbn_cuda.h);
// there is no CPU fallback.  TilingParams arguments are accepted and ignored.
#pragma once

#include <vector>

#include "../runtime/tensor.hpp"

namespace tbn {

// ---- weight quantisation -------------------------------------------------------------------
// quantized_gemm.hpp:86-97 of the reference.
Tensor quantize_to_binary(const Tensor& weights, float threshold = 0.0f);
Tensor quantize_to_ternary(const Tensor& weights, float threshold_low = -0.1f, float threshold_high = 0.1f);
bool is_binary_float_weights(const float* data, size_t count);

// Sign-packed weights ready for the GEMM / convolution kernels: `neg` (and `pos` for ternary) hold
// uint32 [ceil8(N)][ceil128(K)/32] planes in the reference's BinaryMatrix layout, `alpha` the
// per-output-channel scale mean|w|.
struct PackedWeights {
    Tensor neg, pos, alpha;
    int64_t K = 0, N = 0;
    Shape weight_shape;  // original shape ([K,N] matrix or [M,C,kh,kw] filter bank)
    bool ternary = false;
    bool tap_major = false;  // filter banks with C % 64 == 0 are packed in (i, j, c) order for the channels-last path
};
// fp32 weights: a [K,N] matrix (Gemm B) or a [M,C,kh,kw] filter bank.  `ge_zero` selects the Session's
// sign rule (w >= thr is +1) instead of quantize_to_binary's (w > thr).
PackedWeights pack_binary_weights(const Tensor& weights, float threshold = 0.0f, bool ge_zero = false);
PackedWeights pack_ternary_weights(const Tensor& weights, float threshold_low, float threshold_high);
// A BINARY-dtype tensor (1 = +1, 0 = -1), as produced by quantize_to_binary.
PackedWeights pack_binary_tensor(const Tensor& binary_weights);

// Float (non-quantised) weights split once into two bf16 terms for the tensor-core float path.
struct DenseWeights {
    Tensor split;        // [2][ceil8(N)][ceil128(K)] bf16
    int64_t K = 0, N = 0;
    Shape weight_shape;
    bool tap_major = false;
};
DenseWeights pack_dense_weights(const Tensor& weights);  // [K,N] matrix or [M,C,kh,kw] filter bank
// C = alpha * A W + bias and the float-filter convolution, fp32 accuracy.
Tensor matmul_float_dense(const Tensor& a, const DenseWeights& w, const Tensor* bias = nullptr, float alpha = 1.0f);

// ---- GEMM ------------------------------------------------------------------------------------
// Reference "TBN mode" (activations ternarised at +-0.1, exact integer accumulation), bit-equal to
// the reference functions of the same name (quantized_gemm.hpp:42-84).
Tensor qlinear_matmul_binary(const Tensor& a, const Tensor& b_binary, float b_scale, const TilingParams& params);
Tensor qlinear_matmul_binary_float(const Tensor& a, const Tensor& b_binary_float, float b_scale, const TilingParams& params);
// The reference maps ternary 0 to +1 and runs the binary path (quantized_gemm_neon.cpp:506-538); kept as is.
Tensor qlinear_matmul_ternary(const Tensor& a, const Tensor& b_ternary, float b_scale, const TilingParams& params);
Tensor qlinear_matmul_binary_packed(const Tensor& a, const PackedWeights& w, float scale,
                                    float threshold_low = -0.1f, float threshold_high = 0.1f);

// The float x binary / float x ternary product in fp32 accuracy:
//   C = (A * sign(W)) * alpha * scale + bias      (what the reference's float tbn::gemm gives on alpha*sign(W)).
Tensor matmul_float_packed(const Tensor& a, const PackedWeights& w, const Tensor* bias = nullptr, float scale = 1.0f,
                           bool relu = false);
// tbn::gemm (gemm.hpp:11-12): alpha * op(A) op(B) + beta * C with a 1-D C.  A scaled-binary op(B)
// (+-alpha per column) runs on the packed-weight kernel, any other B on the float path; transposed operands
// are materialised on the device first.
Tensor gemm(const Tensor& A, const Tensor& B, const Tensor* C = nullptr, float alpha = 1.0f, float beta = 0.0f,
            bool transA = false, bool transB = false);

// ---- convolution ---------------------------------------------------------------------------
struct Conv2DParams {
    int64_t kernel_h = 3, kernel_w = 3, stride_h = 1, stride_w = 1, pad_h = 0, pad_w = 0, dilation_h = 1,
            dilation_w = 1, groups = 1;
    Conv2DParams() = default;
    Conv2DParams(int64_t kh, int64_t kw, int64_t sh = 1, int64_t sw = 1, int64_t ph = 0, int64_t pw = 0,
                 int64_t dh = 1, int64_t dw = 1, int64_t g = 1)
        : kernel_h(kh), kernel_w(kw), stride_h(sh), stride_w(sw), pad_h(ph), pad_w(pw), dilation_h(dh),
          dilation_w(dw), groups(g) {}
};
// Reference TBN-mode convolutions (conv2d.hpp:44-54): ternarised activations, binary weights, + bias.
Tensor conv2d_binary(const Tensor& input, const Tensor& binary_weights, const Tensor* bias = nullptr,
                     const Conv2DParams& params = Conv2DParams());
Tensor conv2d_binary_with_scales(const Tensor& input, const Tensor& binary_weights, const Tensor* bias,
                                 const Conv2DParams& params, const std::vector<float>& channel_scales);
Tensor conv2d_ternary(const Tensor& input, const Tensor& ternary_weights, const Tensor* bias = nullptr,
                      const Conv2DParams& params = Conv2DParams());
// Float x binary convolution in fp32 accuracy on packed weights, with optional fused residual add and ReLU.
Tensor conv2d_float_packed(const Tensor& input, const PackedWeights& w, const Tensor* bias, const Conv2DParams& params,
                           const Tensor* residual = nullptr, bool relu = false);
// TBN-mode convolution on packed weights with the Session's epilogue (acc + bias) * alpha.
Tensor conv2d_tbn_packed(const Tensor& input, const PackedWeights& w, const Tensor* alpha, const Tensor* bias,
                         const Conv2DParams& params, bool bias_before_alpha);
Tensor conv2d_float_dense(const Tensor& input, const DenseWeights& w, const Tensor* bias, const Conv2DParams& params,
                          const Tensor* residual = nullptr, bool relu = false);
// Convolution inside a layer sequence (tap-major filters only: C % 64 == 0).  The input is the NCHW fp32 tensor `x`
// and / or its channels-last bf16 form `x_cl` written by the previous call; the result comes back as the NCHW
// fp32 tensor (want_y), as the channels-last bf16 form (want_y_cl), or both.  Bit-identical to the plain calls.
struct ConvChainResult {
    Tensor y, y_cl;
};
ConvChainResult conv2d_chain(const Shape& x_shape, const Tensor* x, const Tensor* x_cl, const PackedWeights* packed,
                             const DenseWeights* dense, const Tensor* bias, const Conv2DParams& params,
                             const Tensor* residual, bool relu, bool want_y, bool want_y_cl);
// tbn::conv2d (conv2d.hpp:40-41): scaled-binary filters run on the packed-weight kernel, others on the float path.
Tensor conv2d(const Tensor& input, const Tensor& weights, const Tensor* bias = nullptr,
              const Conv2DParams& params = Conv2DParams());

// ---- pooling / elementwise ---------------------------------------------------------------
struct Pool2DParams {
    int64_t kernel_h = 2, kernel_w = 2, stride_h = 2, stride_w = 2, pad_h = 0, pad_w = 0, dilation_h = 1,
            dilation_w = 1;
    bool ceil_mode = false, count_include_pad = false;
    Pool2DParams() = default;
    Pool2DParams(int64_t kh, int64_t kw, int64_t sh = 2, int64_t sw = 2, int64_t ph = 0, int64_t pw = 0)
        : kernel_h(kh), kernel_w(kw), stride_h(sh), stride_w(sw), pad_h(ph), pad_w(pw) {}
};
Tensor maxpool2d(const Tensor& input, const Pool2DParams& params = Pool2DParams());
Tensor avgpool2d(const Tensor& input, const Pool2DParams& params = Pool2DParams());
Tensor global_avgpool2d(const Tensor& input);
Tensor global_maxpool2d(const Tensor& input);
Tensor relu(const Tensor& input);
Tensor add(const Tensor& a, const Tensor& b);
// The element-wise trio of the exported ternary-activation subgraph (Session::execute_greater / execute_less /
// execute_sub, model.hpp:1176-1316): float 0/1 comparison results, rhs indexed modulo its length.
Tensor greater(const Tensor& lhs, const Tensor& rhs);
Tensor less(const Tensor& lhs, const Tensor& rhs);
Tensor sub(const Tensor& lhs, const Tensor& rhs);
Tensor transpose2d(const Tensor& x);  // [R,C] -> [C,R] on the device

// Per-channel scale of scaled-binary weights (every row of [channels, per] is +-alpha up to rounding),
// summed sequentially like Session::execute_conv (model.hpp:388-394).  Returns false when the weights are
// not of that form (same 1 % / 90 % rule as model.hpp:396-410).
bool scaled_binary_channel_scales(const Tensor& weights, std::vector<float>* scales);

// Waits for all queued GPU work of this library and reports device-side errors.
void synchronize();

}  // namespace tbn
