// Operator functions of the tbn:: API: argument checks as in the reference, work through the C ABI.
#include <cmath>
#include <cstring>

#include "tbn/operators/ops.hpp"
#include "tbn_cuda.h"

namespace tbn {

namespace detail {
void ensure_runtime();
}

namespace {

using detail::check;

// Results that a kernel overwrites completely: no zero fill.
Tensor device_f32(const Shape& shape) { return Tensor::device_uninitialized(shape, DataType::FLOAT32); }

const float* dptr(const Tensor& t) { return static_cast<const float*>(t.device_data()); }
const float* dptr_or_null(const Tensor* t) { return t ? dptr(*t) : nullptr; }

// Scratch buffer reused across calls (grown on demand); the library itself never allocates.
struct Workspace {
    Tensor buf;
    void* get(size_t bytes) {
        if (buf.empty() || buf.data_size() < bytes) buf = Tensor(Shape{static_cast<int64_t>(bytes)}, DataType::UINT8, DeviceType::CUDA);
        return buf.device_data();
    }
};
Workspace& workspace() {
    static thread_local Workspace ws;
    return ws;
}

void require_f32_2d(const Tensor& t, const char* what) {
    TBN_CHECK(t.dtype() == DataType::FLOAT32, InvalidArgumentError, std::string(what) + " must be FLOAT32");
    if (t.shape().dims.size() != 2) throw InvalidShapeError("Both inputs must be 2D matrices");
}

}  // namespace

void synchronize() { check(tbn_cuda_sync(nullptr)); }

// ---------------------------------------------------------------- quantisation

Tensor quantize_to_binary(const Tensor& weights, float threshold) {
    detail::ensure_runtime();
    Tensor out(weights.shape(), DataType::BINARY, DeviceType::CUDA);
    if (weights.dtype() == DataType::FLOAT32) {
        check(tbn_quantize_to_binary(dptr(weights), weights.num_elements(), threshold,
                                     static_cast<uint8_t*>(out.device_data()), nullptr));
        out.mark_device_written();
    } else if (weights.dtype() == DataType::INT8) {
        // Rare path (INT8 sources); a host loop keeps the same rule src > 0.
        const int8_t* src = weights.typed_data<int8_t>();
        Tensor host(weights.shape(), DataType::BINARY);
        uint8_t* dst = host.typed_data<uint8_t>();
        for (int64_t i = 0; i < weights.num_elements(); ++i) dst[i] = src[i] > 0 ? BINARY_ONE : BINARY_ZERO;
        return host.to_device(DeviceType::CUDA);
    } else {
        throw InvalidArgumentError("Unsupported dtype for binary quantization");
    }
    return out;
}

Tensor quantize_to_ternary(const Tensor& weights, float lo, float hi) {
    detail::ensure_runtime();
    if (weights.dtype() != DataType::FLOAT32) throw InvalidArgumentError("Unsupported dtype for ternary quantization");
    Tensor out(weights.shape(), DataType::TERNARY, DeviceType::CUDA);
    check(tbn_quantize_to_ternary(dptr(weights), weights.num_elements(), lo, hi, static_cast<int8_t*>(out.device_data()),
                                  nullptr));
    out.mark_device_written();
    return out;
}

bool is_binary_float_weights(const float* data, size_t count) {
    for (size_t i = 0; i < count; ++i)
        if (data[i] != -1.0f && data[i] != 1.0f && data[i] != 0.0f) return false;
    return true;
}

namespace {

PackedWeights pack_impl(const Tensor& weights, bool ternary, float lo, float hi, bool ge) {
    detail::ensure_runtime();
    TBN_CHECK(weights.dtype() == DataType::FLOAT32, InvalidArgumentError, "weights must be FLOAT32");
    const auto& d = weights.shape().dims;
    TBN_CHECK(d.size() == 2 || d.size() == 4, InvalidShapeError, "weights must be [K,N] or [M,C,kh,kw]");
    PackedWeights p;
    p.weight_shape = weights.shape();
    p.ternary = ternary;
    int layout;
    int64_t ldw;
    Tensor reordered;
    const float* src = dptr(weights);
    if (d.size() == 2) {
        p.K = d[0]; p.N = d[1]; layout = TBN_LAYOUT_KN; ldw = p.N;
    } else {
        p.N = d[0]; p.K = d[1] * d[2] * d[3]; layout = TBN_LAYOUT_NK; ldw = p.K;
        if (d[1] % 64 == 0) {  // channels-last fast path: K ordered (i, j, c)
            reordered = device_f32(Shape{p.N, p.K});
            check(tbn_permute_filters(src, d[0], d[1], d[2] * d[3], static_cast<float*>(reordered.device_data()), nullptr));
            reordered.mark_device_written();
            src = dptr(reordered);
            p.tap_major = true;
        }
    }
    int64_t Kp = 0, Np = 0;
    check(tbn_packed_dims(p.K, p.N, &Kp, &Np));
    p.neg = Tensor(Shape{Np, Kp / 32}, DataType::UINT32, DeviceType::CUDA);
    p.alpha = device_f32(Shape{p.N});
    const size_t ws_bytes = tbn_quant_pack_workspace_bytes(p.K, p.N, ternary ? 1 : 0);
    void* ws = workspace().get(ws_bytes);
    if (ternary) {
        p.pos = Tensor(Shape{Np, Kp / 32}, DataType::UINT32, DeviceType::CUDA);
        check(tbn_quant_pack_ternary(src, p.K, p.N, ldw, layout, lo, hi, nullptr,
                                     static_cast<uint32_t*>(p.pos.device_data()), static_cast<uint32_t*>(p.neg.device_data()),
                                     static_cast<float*>(p.alpha.device_data()), ws, ws_bytes, nullptr));
        p.pos.mark_device_written();
    } else {
        check(tbn_quant_pack_binary(src, p.K, p.N, ldw, layout, lo, ge ? 1 : 0,
                                    static_cast<uint32_t*>(p.neg.device_data()), static_cast<float*>(p.alpha.device_data()), ws,
                                    ws_bytes, nullptr));
    }
    p.neg.mark_device_written();
    p.alpha.mark_device_written();
    return p;
}

}  // namespace

PackedWeights pack_binary_weights(const Tensor& weights, float threshold, bool ge_zero) {
    return pack_impl(weights, false, threshold, 0.0f, ge_zero);
}

PackedWeights pack_ternary_weights(const Tensor& weights, float lo, float hi) { return pack_impl(weights, true, lo, hi, false); }

PackedWeights pack_binary_tensor(const Tensor& b) {
    TBN_CHECK(b.dtype() == DataType::BINARY, InvalidArgumentError, "Input B must be BINARY");
    // 1 -> +1, 0 -> -1 as floats, then the regular packer (bit set <=> -1).
    const uint8_t* src = b.typed_data<uint8_t>();
    Tensor f(b.shape(), DataType::FLOAT32);
    float* dst = f.typed_data<float>();
    for (int64_t i = 0; i < b.num_elements(); ++i) dst[i] = src[i] == BINARY_ONE ? 1.0f : -1.0f;
    return pack_impl(f, false, 0.0f, 0.0f, false);
}

DenseWeights pack_dense_weights(const Tensor& weights) {
    detail::ensure_runtime();
    TBN_CHECK(weights.dtype() == DataType::FLOAT32, InvalidArgumentError, "weights must be FLOAT32");
    const auto& d = weights.shape().dims;
    TBN_CHECK(d.size() == 2 || d.size() == 4, InvalidShapeError, "weights must be [K,N] or [M,C,kh,kw]");
    DenseWeights w;
    w.weight_shape = weights.shape();
    int layout;
    int64_t ldw;
    Tensor reordered;
    const float* src = dptr(weights);
    if (d.size() == 2) {
        w.K = d[0]; w.N = d[1]; layout = TBN_LAYOUT_KN; ldw = w.N;
    } else {
        w.N = d[0]; w.K = d[1] * d[2] * d[3]; layout = TBN_LAYOUT_NK; ldw = w.K;
        if (d[1] % 64 == 0) {
            reordered = device_f32(Shape{w.N, w.K});
            check(tbn_permute_filters(src, d[0], d[1], d[2] * d[3], static_cast<float*>(reordered.device_data()), nullptr));
            reordered.mark_device_written();
            src = dptr(reordered);
            w.tap_major = true;
        }
    }
    w.split = Tensor(Shape{static_cast<int64_t>(tbn_dense_pack_bytes(w.K, w.N))}, DataType::UINT8, DeviceType::CUDA);
    check(tbn_dense_pack(src, w.K, w.N, ldw, layout, w.split.device_data(), nullptr));
    w.split.mark_device_written();
    return w;
}

Tensor matmul_float_dense(const Tensor& a, const DenseWeights& w, const Tensor* bias, float alpha) {
    require_f32_2d(a, "Input A");
    const int64_t M = a.shape().dims[0], K = a.shape().dims[1];
    if (K != w.K) throw InvalidShapeError("Matrix dimensions incompatible: A cols (" + std::to_string(K) + ") != B rows (" +
                                          std::to_string(w.K) + ")");
    if (bias) TBN_CHECK(bias->num_elements() == w.N, InvalidShapeError, "bias must have one entry per output column");
    Tensor out = device_f32(Shape{M, w.N});
    const size_t ws_bytes = tbn_gemm_workspace_bytes(M, K, TBN_MODE_TC_BF16X2);
    check(tbn_gemm_f32(dptr(a), M, K, K, w.split.device_data(), w.N, alpha, dptr_or_null(bias),
                       static_cast<float*>(out.device_data()), w.N, 0u, workspace().get(ws_bytes), ws_bytes, nullptr));
    out.mark_device_written();
    return out;
}

// ---------------------------------------------------------------- GEMM

Tensor qlinear_matmul_binary_packed(const Tensor& a, const PackedWeights& w, float scale, float lo, float hi) {
    require_f32_2d(a, "Input A");
    const int64_t M = a.shape().dims[0], K = a.shape().dims[1];
    if (K != w.K) throw InvalidShapeError("Matrix dimensions incompatible: A cols (" + std::to_string(K) + ") != B rows (" +
                                          std::to_string(w.K) + ")");
    Tensor out = device_f32(Shape{M, w.N});
    const size_t ws_bytes = tbn_gemm_workspace_bytes(M, K, TBN_MODE_TC_BF16X1);
    check(tbn_gemm_tbn(dptr(a), M, K, K, lo, hi, static_cast<const uint32_t*>(w.neg.device_data()), w.N, nullptr, scale, nullptr,
                       static_cast<float*>(out.device_data()), w.N, 0, workspace().get(ws_bytes), ws_bytes, nullptr));
    out.mark_device_written();
    return out;
}

Tensor qlinear_matmul_binary(const Tensor& a, const Tensor& b, float scale, const TilingParams&) {
    TBN_CHECK(a.dtype() == DataType::FLOAT32, InvalidArgumentError, "Input A must be FLOAT32");
    if (a.shape().dims.size() != 2 || b.shape().dims.size() != 2) throw InvalidShapeError("Both inputs must be 2D matrices");
    if (b.dtype() == DataType::FLOAT32) {
        // +-1/0 floats: sign by >= 0 (convert_binary_float_to_int8); other floats: quantize_to_binary's rule.
        const bool pre = is_binary_float_weights(b.typed_data<float>(), static_cast<size_t>(b.num_elements()));
        return qlinear_matmul_binary_packed(a, pack_binary_weights(b, 0.0f, pre), scale);
    }
    TBN_CHECK(b.dtype() == DataType::BINARY, InvalidArgumentError, "Input B must be BINARY or FLOAT32 with binary values");
    return qlinear_matmul_binary_packed(a, pack_binary_tensor(b), scale);
}

Tensor qlinear_matmul_binary_float(const Tensor& a, const Tensor& b, float scale, const TilingParams&) {
    return qlinear_matmul_binary_packed(a, pack_binary_weights(b, 0.0f, true), scale);
}

Tensor qlinear_matmul_ternary(const Tensor& a, const Tensor& b, float scale, const TilingParams& tp) {
    TBN_CHECK(a.dtype() == DataType::FLOAT32, InvalidArgumentError, "Input A must be FLOAT32");
    TBN_CHECK(b.dtype() == DataType::TERNARY, InvalidArgumentError, "Input B must be TERNARY");
    const int8_t* src = b.typed_data<int8_t>();
    Tensor bin(b.shape(), DataType::BINARY);
    uint8_t* dst = bin.typed_data<uint8_t>();
    for (int64_t i = 0; i < b.num_elements(); ++i) dst[i] = src[i] == TERNARY_MINUS_ONE ? BINARY_ZERO : BINARY_ONE;
    return qlinear_matmul_binary(a, bin, scale, tp);
}

Tensor matmul_float_packed(const Tensor& a, const PackedWeights& w, const Tensor* bias, float scale, bool relu_flag) {
    require_f32_2d(a, "Input A");
    const int64_t M = a.shape().dims[0], K = a.shape().dims[1];
    if (K != w.K) throw InvalidShapeError("Matrix dimensions incompatible: A cols (" + std::to_string(K) + ") != B rows (" +
                                          std::to_string(w.K) + ")");
    if (bias) TBN_CHECK(bias->num_elements() == w.N, InvalidShapeError, "bias must have one entry per output column");
    Tensor out = device_f32(Shape{M, w.N});
    const size_t ws_bytes = tbn_gemm_workspace_bytes(M, K, TBN_MODE_AUTO);
    check(tbn_gemm_fxb(dptr(a), M, K, K, static_cast<const uint32_t*>(w.neg.device_data()),
                       w.ternary ? static_cast<const uint32_t*>(w.pos.device_data()) : nullptr, w.N, dptr(w.alpha), scale,
                       dptr_or_null(bias), static_cast<float*>(out.device_data()), w.N, TBN_MODE_AUTO, relu_flag ? TBN_EPI_RELU : 0u,
                       workspace().get(ws_bytes), ws_bytes, nullptr));
    out.mark_device_written();
    return out;
}

bool scaled_binary_channel_scales(const Tensor& weights, std::vector<float>* scales) {
    const float* w = weights.typed_data<float>();
    const int64_t ch = weights.shape().dims[0], per = weights.num_elements() / ch;
    if (scales) scales->assign(static_cast<size_t>(ch), 0.0f);
    bool ok = true;
    for (int64_t c = 0; c < ch; ++c) {
        float sum = 0.0f;
        for (int64_t i = 0; i < per; ++i) sum += std::fabs(w[c * per + i]);
        const float s = sum / static_cast<float>(per);
        if (scales) (*scales)[static_cast<size_t>(c)] = s;
        int64_t near = 0;
        for (int64_t i = 0; i < per; ++i) {
            const float v = w[c * per + i], e = v >= 0 ? s : -s;
            if (std::fabs(v - e) < 0.01f * s || std::fabs(v) < 0.01f) ++near;
        }
        if (near < per * 0.9f) ok = false;
    }
    return ok;
}

Tensor gemm(const Tensor& A, const Tensor& B, const Tensor* C, float alpha, float beta, bool transA, bool transB) {
    TBN_CHECK(A.dtype() == DataType::FLOAT32, InvalidArgumentError, "gemm requires float32 input A");
    TBN_CHECK(B.dtype() == DataType::FLOAT32, InvalidArgumentError, "gemm requires float32 input B");
    require_f32_2d(A, "A");
    require_f32_2d(B, "B");
    if (transA || transB) return gemm(transA ? transpose2d(A) : A, transB ? transpose2d(B) : B, C, alpha, beta, false, false);
    // Columns of a scaled-binary B are +-alpha: check on the transposed view (channels = columns).
    const int64_t K = B.shape().dims[0], N = B.shape().dims[1];
    const float* b = B.typed_data<float>();
    Tensor bt(Shape{N, K}, DataType::FLOAT32);
    float* t = bt.typed_data<float>();
    for (int64_t k = 0; k < K; ++k)
        for (int64_t n = 0; n < N; ++n) t[n * K + k] = b[k * N + n];
    const bool binary = scaled_binary_channel_scales(bt, nullptr);
    Tensor bias;
    if (C && beta != 0.0f) {
        TBN_CHECK(C->shape().dims.size() == 1, NotImplementedError, "gemm: only a 1-D C (bias) is accelerated");
        bias = C->to_device(DeviceType::CPU);
        float* p = bias.typed_data<float>();
        for (int64_t i = 0; i < bias.num_elements(); ++i) p[i] *= beta;
    }
    if (!binary) return matmul_float_dense(A, pack_dense_weights(B), bias.empty() ? nullptr : &bias, alpha);
    return matmul_float_packed(A, pack_binary_weights(B, 0.0f, true), bias.empty() ? nullptr : &bias, alpha);
}

// ---------------------------------------------------------------- convolution

namespace {

struct ConvDims {
    int64_t N, C, H, W, M, kh, kw, OH, OW;
};

ConvDims conv_dims(const Tensor& x, const Shape& wshape, const Conv2DParams& p) {
    TBN_CHECK(x.shape().dims.size() == 4, InvalidShapeError, "Conv2D input must be 4D (NCHW), got " + shape_to_string(x.shape()));
    TBN_CHECK(wshape.dims.size() == 4, InvalidShapeError, "Conv2D weights must be 4D (MCHW), got " + shape_to_string(wshape));
    TBN_CHECK(x.dtype() == DataType::FLOAT32, InvalidArgumentError, "Conv2D requires float32 input");
    ConvDims d{x.shape().dims[0], x.shape().dims[1], x.shape().dims[2], x.shape().dims[3],
               wshape.dims[0], wshape.dims[2], wshape.dims[3], 0, 0};
    TBN_CHECK(d.C == wshape.dims[1], InvalidShapeError,
              "Input channels (" + std::to_string(d.C) + ") must match weight channels (" + std::to_string(wshape.dims[1]) + ")");
    if (p.groups != 1) throw NotImplementedError("Grouped convolution not yet implemented");
    d.OH = (d.H + 2 * p.pad_h - p.dilation_h * (d.kh - 1) - 1) / p.stride_h + 1;
    d.OW = (d.W + 2 * p.pad_w - p.dilation_w * (d.kw - 1) - 1) / p.stride_w + 1;
    TBN_CHECK(d.OH > 0 && d.OW > 0, InvalidShapeError,
              "Invalid output dimensions: " + std::to_string(d.OH) + "x" + std::to_string(d.OW));
    return d;
}

void check_bias(const Tensor* bias, int64_t M) {
    if (!bias) return;
    TBN_CHECK(bias->shape().dims.size() == 1, InvalidShapeError, "Bias must be 1D");
    TBN_CHECK(bias->shape().dims[0] == M, InvalidShapeError, "Bias size must match output channels");
}

}  // namespace

Tensor conv2d_float_packed(const Tensor& x, const PackedWeights& w, const Tensor* bias, const Conv2DParams& p,
                           const Tensor* residual, bool relu_flag) {
    const ConvDims d = conv_dims(x, w.weight_shape, p);
    check_bias(bias, d.M);
    Tensor y = device_f32(Shape{d.N, d.M, d.OH, d.OW});
    if (residual) TBN_CHECK(residual->shape() == y.shape(), InvalidShapeError, "residual must have the output's shape");
    const int32_t order = w.tap_major ? TBN_CONV_WEIGHTS_TAP_MAJOR : TBN_CONV_WEIGHTS_REFERENCE;
    const size_t ws_bytes = tbn_conv2d_workspace_bytes(d.N, d.C, d.H, d.W, d.M, d.kh, d.kw, order);
    uint32_t epi = (relu_flag ? TBN_EPI_RELU : 0u) | (residual ? TBN_EPI_ADD_RESIDUAL : 0u);
    check(tbn_conv2d_fxb(dptr(x), d.N, d.C, d.H, d.W, static_cast<const uint32_t*>(w.neg.device_data()),
                         w.ternary ? static_cast<const uint32_t*>(w.pos.device_data()) : nullptr, d.M, d.kh, d.kw,
                         static_cast<int32_t>(p.stride_h), static_cast<int32_t>(p.stride_w), static_cast<int32_t>(p.pad_h),
                         static_cast<int32_t>(p.pad_w), static_cast<int32_t>(p.dilation_h), static_cast<int32_t>(p.dilation_w),
                         dptr(w.alpha), 1.0f, dptr_or_null(bias), dptr_or_null(residual), static_cast<float*>(y.device_data()),
                         TBN_MODE_AUTO, epi, order, workspace().get(ws_bytes), ws_bytes, nullptr));
    y.mark_device_written();
    return y;
}

Tensor conv2d_tbn_packed(const Tensor& x, const PackedWeights& w, const Tensor* alpha, const Tensor* bias,
                         const Conv2DParams& p, bool bias_before_alpha) {
    const ConvDims d = conv_dims(x, w.weight_shape, p);
    check_bias(bias, d.M);
    Tensor y = device_f32(Shape{d.N, d.M, d.OH, d.OW});
    const int32_t order = w.tap_major ? TBN_CONV_WEIGHTS_TAP_MAJOR : TBN_CONV_WEIGHTS_REFERENCE;
    const size_t ws_bytes = tbn_conv2d_workspace_bytes(d.N, d.C, d.H, d.W, d.M, d.kh, d.kw, order);
    check(tbn_conv2d_tbn(dptr(x), d.N, d.C, d.H, d.W, -0.1f, 0.1f, static_cast<const uint32_t*>(w.neg.device_data()), d.M, d.kh,
                         d.kw, static_cast<int32_t>(p.stride_h), static_cast<int32_t>(p.stride_w), static_cast<int32_t>(p.pad_h),
                         static_cast<int32_t>(p.pad_w), static_cast<int32_t>(p.dilation_h), static_cast<int32_t>(p.dilation_w),
                         dptr_or_null(alpha), 1.0f, dptr_or_null(bias), static_cast<float*>(y.device_data()),
                         bias_before_alpha ? TBN_EPI_BIAS_BEFORE_ALPHA : 0u, order, workspace().get(ws_bytes), ws_bytes, nullptr));
    y.mark_device_written();
    return y;
}

namespace {
PackedWeights pack_binary_filters(const Tensor& bw) {
    TBN_CHECK(bw.dtype() == DataType::BINARY, InvalidArgumentError, "Binary Conv2D requires binary weights");
    TBN_CHECK(bw.shape().dims.size() == 4, InvalidShapeError, "Conv2D weights must be 4D (MCHW)");
    return pack_binary_tensor(bw);
}
}  // namespace

Tensor conv2d_binary(const Tensor& x, const Tensor& bw, const Tensor* bias, const Conv2DParams& p) {
    return conv2d_tbn_packed(x, pack_binary_filters(bw), nullptr, bias, p, false);
}

Tensor conv2d_binary_with_scales(const Tensor& x, const Tensor& bw, const Tensor* bias, const Conv2DParams& p,
                                 const std::vector<float>& scales) {
    TBN_CHECK(bw.shape().dims.size() == 4 && static_cast<int64_t>(scales.size()) == bw.shape().dims[0], InvalidArgumentError,
              "channel_scales size must match output channels");
    Tensor alpha = make_tensor(Shape{static_cast<int64_t>(scales.size())}, scales);
    return conv2d_tbn_packed(x, pack_binary_filters(bw), &alpha, bias, p, false);  // acc*alpha + bias
}

Tensor conv2d_ternary(const Tensor& x, const Tensor& tw, const Tensor* bias, const Conv2DParams& p) {
    TBN_CHECK(tw.dtype() == DataType::TERNARY, InvalidArgumentError, "Ternary Conv2D requires ternary weights");
    const int8_t* src = tw.typed_data<int8_t>();
    Tensor bin(tw.shape(), DataType::BINARY);
    uint8_t* dst = bin.typed_data<uint8_t>();
    for (int64_t i = 0; i < tw.num_elements(); ++i) dst[i] = src[i] < 0 ? BINARY_ZERO : BINARY_ONE;
    return conv2d_binary(x, bin, bias, p);
}

Tensor conv2d(const Tensor& x, const Tensor& w, const Tensor* bias, const Conv2DParams& p) {
    TBN_CHECK(w.dtype() == DataType::FLOAT32, InvalidArgumentError, "Conv2D requires float32 weights");
    TBN_CHECK(w.shape().dims.size() == 4, InvalidShapeError, "Conv2D weights must be 4D (MCHW), got " + shape_to_string(w.shape()));
    if (!scaled_binary_channel_scales(w, nullptr)) return conv2d_float_dense(x, pack_dense_weights(w), bias, p);
    return conv2d_float_packed(x, pack_binary_weights(w, 0.0f, true), bias, p);
}

Tensor conv2d_float_dense(const Tensor& x, const DenseWeights& w, const Tensor* bias, const Conv2DParams& p,
                          const Tensor* residual, bool relu_flag) {
    const ConvDims d = conv_dims(x, w.weight_shape, p);
    check_bias(bias, d.M);
    Tensor y = device_f32(Shape{d.N, d.M, d.OH, d.OW});
    if (residual) TBN_CHECK(residual->shape() == y.shape(), InvalidShapeError, "residual must have the output's shape");
    const int32_t order = w.tap_major ? TBN_CONV_WEIGHTS_TAP_MAJOR : TBN_CONV_WEIGHTS_REFERENCE;
    const size_t ws_bytes = tbn_conv2d_workspace_bytes(d.N, d.C, d.H, d.W, d.M, d.kh, d.kw, order);
    const uint32_t epi = (relu_flag ? TBN_EPI_RELU : 0u) | (residual ? TBN_EPI_ADD_RESIDUAL : 0u);
    check(tbn_conv2d_f32(dptr(x), d.N, d.C, d.H, d.W, w.split.device_data(), d.M, d.kh, d.kw, static_cast<int32_t>(p.stride_h),
                         static_cast<int32_t>(p.stride_w), static_cast<int32_t>(p.pad_h), static_cast<int32_t>(p.pad_w),
                         static_cast<int32_t>(p.dilation_h), static_cast<int32_t>(p.dilation_w), dptr_or_null(bias),
                         dptr_or_null(residual), static_cast<float*>(y.device_data()), epi, order, workspace().get(ws_bytes),
                         ws_bytes, nullptr));
    y.mark_device_written();
    return y;
}

ConvChainResult conv2d_chain(const Shape& x_shape, const Tensor* x, const Tensor* x_cl, const PackedWeights* packed,
                             const DenseWeights* dense, const Tensor* bias, const Conv2DParams& p, const Tensor* residual,
                             bool relu_flag, bool want_y, bool want_y_cl) {
    TBN_CHECK((x || x_cl) && (packed || dense) && (want_y || want_y_cl), InvalidArgumentError, "conv2d_chain: missing operand");
    const Shape& wshape = packed ? packed->weight_shape : dense->weight_shape;
    TBN_CHECK(x_shape.dims.size() == 4 && wshape.dims.size() == 4, InvalidShapeError, "Conv2D input and weights must be 4D");
    TBN_CHECK((packed ? packed->tap_major : dense->tap_major), InvalidArgumentError, "conv2d_chain needs tap-major filters");
    ConvDims d{x_shape.dims[0], x_shape.dims[1], x_shape.dims[2], x_shape.dims[3], wshape.dims[0], wshape.dims[2], wshape.dims[3], 0, 0};
    TBN_CHECK(d.C == wshape.dims[1], InvalidShapeError, "Input channels must match weight channels");
    if (p.groups != 1) throw NotImplementedError("Grouped convolution not yet implemented");
    d.OH = (d.H + 2 * p.pad_h - p.dilation_h * (d.kh - 1) - 1) / p.stride_h + 1;
    d.OW = (d.W + 2 * p.pad_w - p.dilation_w * (d.kw - 1) - 1) / p.stride_w + 1;
    TBN_CHECK(d.OH > 0 && d.OW > 0, InvalidShapeError, "Invalid output dimensions");
    check_bias(bias, d.M);
    ConvChainResult out;
    if (want_y) out.y = device_f32(Shape{d.N, d.M, d.OH, d.OW});
    if (want_y_cl) out.y_cl = Tensor::device_uninitialized(Shape{2, d.N, d.OH, d.OW, d.M}, DataType::BFLOAT16);
    if (residual) TBN_CHECK(residual->shape() == (Shape{d.N, d.M, d.OH, d.OW}), InvalidShapeError, "residual must have the output's shape");
    const size_t ws_bytes = tbn_conv2d_workspace_bytes(d.N, d.C, d.H, d.W, d.M, d.kh, d.kw, TBN_CONV_WEIGHTS_TAP_MAJOR);
    const uint32_t epi = (relu_flag ? TBN_EPI_RELU : 0u) | (residual ? TBN_EPI_ADD_RESIDUAL : 0u);
    const float* xp = x_cl ? nullptr : dptr(*x);
    const void* xclp = x_cl ? x_cl->device_data() : nullptr;
    float* yp = want_y ? static_cast<float*>(out.y.device_data()) : nullptr;
    void* yclp = want_y_cl ? out.y_cl.device_data() : nullptr;
    const int32_t sh = static_cast<int32_t>(p.stride_h), sw = static_cast<int32_t>(p.stride_w), ph = static_cast<int32_t>(p.pad_h),
                  pw = static_cast<int32_t>(p.pad_w), dh = static_cast<int32_t>(p.dilation_h), dw = static_cast<int32_t>(p.dilation_w);
    if (packed) {
        check(tbn_conv2d_fxb_chain(xp, xclp, d.N, d.C, d.H, d.W, static_cast<const uint32_t*>(packed->neg.device_data()),
                                   packed->ternary ? static_cast<const uint32_t*>(packed->pos.device_data()) : nullptr, d.M, d.kh,
                                   d.kw, sh, sw, ph, pw, dh, dw, dptr(packed->alpha), 1.0f, dptr_or_null(bias),
                                   dptr_or_null(residual), yp, yclp, TBN_MODE_AUTO, epi, TBN_CONV_WEIGHTS_TAP_MAJOR,
                                   workspace().get(ws_bytes), ws_bytes, nullptr));
    } else {
        check(tbn_conv2d_f32_chain(xp, xclp, d.N, d.C, d.H, d.W, dense->split.device_data(), d.M, d.kh, d.kw, sh, sw, ph, pw, dh,
                                   dw, dptr_or_null(bias), dptr_or_null(residual), yp, yclp, epi, TBN_CONV_WEIGHTS_TAP_MAJOR,
                                   workspace().get(ws_bytes), ws_bytes, nullptr));
    }
    if (want_y) out.y.mark_device_written();
    if (want_y_cl) out.y_cl.mark_device_written();
    return out;
}

// ---------------------------------------------------------------- pooling / elementwise

namespace {
Tensor pool(int kind, const Tensor& x, const Pool2DParams& p, const char* name) {
    TBN_CHECK(x.shape().dims.size() == 4, InvalidShapeError,
              std::string(name) + " input must be 4D (NCHW), got " + shape_to_string(x.shape()));
    TBN_CHECK(x.dtype() == DataType::FLOAT32, InvalidArgumentError, std::string(name) + " requires float32 input");
    const int64_t N = x.shape().dims[0], C = x.shape().dims[1], H = x.shape().dims[2], W = x.shape().dims[3];
    const int64_t OH = p.ceil_mode ? (H + 2 * p.pad_h - p.kernel_h + p.stride_h - 1) / p.stride_h + 1
                                   : (H + 2 * p.pad_h - p.kernel_h) / p.stride_h + 1;
    const int64_t OW = p.ceil_mode ? (W + 2 * p.pad_w - p.kernel_w + p.stride_w - 1) / p.stride_w + 1
                                   : (W + 2 * p.pad_w - p.kernel_w) / p.stride_w + 1;
    TBN_CHECK(OH > 0 && OW > 0, InvalidShapeError, std::string(name) + ": empty output");
    Tensor y = device_f32(Shape{N, C, OH, OW});
    check(tbn_pool2d(kind, dptr(x), N, C, H, W, static_cast<int32_t>(p.kernel_h), static_cast<int32_t>(p.kernel_w),
                     static_cast<int32_t>(p.stride_h), static_cast<int32_t>(p.stride_w), static_cast<int32_t>(p.pad_h),
                     static_cast<int32_t>(p.pad_w), p.ceil_mode, p.count_include_pad, static_cast<float*>(y.device_data()), nullptr));
    y.mark_device_written();
    return y;
}
}  // namespace

Tensor maxpool2d(const Tensor& x, const Pool2DParams& p) { return pool(0, x, p, "MaxPool2D"); }
Tensor avgpool2d(const Tensor& x, const Pool2DParams& p) { return pool(1, x, p, "AvgPool2D"); }

Tensor global_avgpool2d(const Tensor& x) {
    TBN_CHECK(x.shape().dims.size() == 4, InvalidShapeError, "GlobalAvgPool2D input must be 4D (NCHW)");
    const int64_t N = x.shape().dims[0], C = x.shape().dims[1], H = x.shape().dims[2], W = x.shape().dims[3];
    Tensor y = device_f32(Shape{N, C, 1, 1});
    check(tbn_global_avgpool2d(dptr(x), N, C, H, W, static_cast<float*>(y.device_data()), nullptr));
    y.mark_device_written();
    return y;
}

Tensor global_maxpool2d(const Tensor& x) {
    TBN_CHECK(x.shape().dims.size() == 4, InvalidShapeError, "GlobalMaxPool2D input must be 4D (NCHW)");
    const int64_t N = x.shape().dims[0], C = x.shape().dims[1], H = x.shape().dims[2], W = x.shape().dims[3];
    Tensor y = device_f32(Shape{N, C, 1, 1});
    check(tbn_global_maxpool2d(dptr(x), N, C, H, W, static_cast<float*>(y.device_data()), nullptr));
    y.mark_device_written();
    return y;
}

namespace {
Tensor elementwise(int op, const Tensor& lhs, const Tensor& rhs, const char* what) {
    TBN_CHECK(lhs.dtype() == DataType::FLOAT32 && rhs.dtype() == DataType::FLOAT32, InvalidArgumentError,
              std::string(what) + " requires float32 inputs");
    TBN_CHECK(rhs.num_elements() > 0, InvalidShapeError, std::string(what) + ": empty right-hand side");
    Tensor y = device_f32(lhs.shape());
    check(tbn_binary_elementwise(op, dptr(lhs), lhs.num_elements(), dptr(rhs), rhs.num_elements(),
                                 static_cast<float*>(y.device_data()), nullptr));
    y.mark_device_written();
    return y;
}
}  // namespace

Tensor greater(const Tensor& lhs, const Tensor& rhs) { return elementwise(TBN_ELT_GREATER, lhs, rhs, "Greater"); }
Tensor less(const Tensor& lhs, const Tensor& rhs) { return elementwise(TBN_ELT_LESS, lhs, rhs, "Less"); }
Tensor sub(const Tensor& lhs, const Tensor& rhs) { return elementwise(TBN_ELT_SUB, lhs, rhs, "Sub"); }

Tensor transpose2d(const Tensor& x) {
    require_f32_2d(x, "transpose input");
    const int64_t R = x.shape().dims[0], C = x.shape().dims[1];
    Tensor y = device_f32(Shape{C, R});
    check(tbn_transpose2d(dptr(x), R, C, static_cast<float*>(y.device_data()), nullptr));
    y.mark_device_written();
    return y;
}

Tensor relu(const Tensor& x) {
    Tensor y = device_f32(x.shape());
    check(tbn_relu(dptr(x), x.num_elements(), static_cast<float*>(y.device_data()), nullptr));
    y.mark_device_written();
    return y;
}

Tensor add(const Tensor& a, const Tensor& b) {
    const auto& ad = a.shape().dims;
    const auto& bd = b.shape().dims;
    const Tensor* big = &a;
    const Tensor* small = &b;
    if (b.num_elements() > a.num_elements()) std::swap(big, small);
    const auto& gd = big->shape().dims;
    const auto& sd = small->shape().dims;
    int64_t inner = 1;
    if (ad == bd) {
        inner = 1;
    } else if (gd.size() == 2 && sd.size() == 1 && sd[0] == gd[1]) {
        inner = 1;  // [M,N] + [N]
    } else if (gd.size() == 4 && (sd.size() == 1 || sd.size() == 3) && sd[0] == gd[1] && small->num_elements() == gd[1]) {
        inner = gd[2] * gd[3];  // [N,C,H,W] + [C] or [C,1,1]
    } else {
        throw InvalidShapeError("Add: shapes " + shape_to_string(a.shape()) + " and " + shape_to_string(b.shape()) +
                                " do not broadcast");
    }
    Tensor y = device_f32(big->shape());
    check(tbn_add(dptr(*big), big->num_elements(), dptr(*small), small->num_elements(), inner, 0,
                  static_cast<float*>(y.device_data()), nullptr));
    y.mark_device_written();
    return y;
}

}  // namespace tbn
