// BinaryMatrix / TernaryMatrix / PackedBinaryWeights and the operators on pre-packed operands.
#include "tbn/gemm/packed_matrix.hpp"

#include <cstring>
#include <string>

#include "tbn/operators/ops.hpp"
#include "tbn_cuda.h"

namespace tbn {

namespace detail {
void ensure_runtime();
}

// ---- packing: the checks and messages of GeMM.cpp:29-151 ------------------------------------------------

TernaryMatrix TernaryMatrix::pack(std::span<const std::int8_t> data, std::uint32_t rows, std::uint32_t cols) {
    if (rows % 8 != 0 || cols % 64 != 0) throw std::invalid_argument("TernaryMatrix: rows must be a multiple of 8 and cols of 64");
    if (data.size() != static_cast<std::size_t>(rows) * cols) throw std::invalid_argument("TernaryMatrix: data size mismatch");
    const std::size_t row_bytes = cols / 8;
    std::vector<std::uint8_t> pos(static_cast<std::size_t>(rows) * row_bytes, 0), neg(pos.size(), 0);
    for (std::uint32_t m = 0; m < rows; ++m)
        for (std::uint32_t k = 0; k < cols; ++k) {
            const std::int8_t v = data[static_cast<std::size_t>(m) * cols + k];
            if (v != -1 && v != 0 && v != 1) throw std::invalid_argument("TernaryMatrix: values must be in {-1, 0, +1}");
            if (v > 0) pos[m * row_bytes + k / 8] |= static_cast<std::uint8_t>(1u << (k & 7));
            if (v < 0) neg[m * row_bytes + k / 8] |= static_cast<std::uint8_t>(1u << (k & 7));
        }
    return TernaryMatrix(std::move(pos), std::move(neg), rows, cols);
}

TernaryMatrix TernaryMatrix::pack_from_float(const float* data, std::uint32_t rows, std::uint32_t cols, float lo, float hi) {
    if (rows % 8 != 0 || cols % 64 != 0) throw std::invalid_argument("TernaryMatrix: rows must be a multiple of 8 and cols of 64");
    const std::size_t row_bytes = cols / 8;
    std::vector<std::uint8_t> pos(static_cast<std::size_t>(rows) * row_bytes, 0), neg(pos.size(), 0);
    for (std::uint32_t m = 0; m < rows; ++m)
        for (std::uint32_t k = 0; k < cols; ++k) {
            const float v = data[static_cast<std::size_t>(m) * cols + k];
            if (v > hi) pos[m * row_bytes + k / 8] |= static_cast<std::uint8_t>(1u << (k & 7));
            else if (v < lo) neg[m * row_bytes + k / 8] |= static_cast<std::uint8_t>(1u << (k & 7));
        }
    return TernaryMatrix(std::move(pos), std::move(neg), rows, cols);
}

BinaryMatrix BinaryMatrix::pack(std::span<const std::int8_t> data, std::uint32_t rows, std::uint32_t cols) {
    if (rows % 64 != 0 || cols % 8 != 0) throw std::invalid_argument("BinaryMatrix: rows must be a multiple of 64 and cols of 8");
    if (data.size() != static_cast<std::size_t>(rows) * cols) throw std::invalid_argument("BinaryMatrix: data size mismatch");
    const std::size_t col_bytes = rows / 8;
    std::vector<std::uint8_t> bits(static_cast<std::size_t>(cols) * col_bytes, 0);
    for (std::uint32_t k = 0; k < rows; ++k)
        for (std::uint32_t n = 0; n < cols; ++n) {
            const std::int8_t v = data[static_cast<std::size_t>(k) * cols + n];
            if (v != -1 && v != 1) throw std::invalid_argument("BinaryMatrix: values must be in {-1, +1}");
            if (v < 0) bits[n * col_bytes + k / 8] |= static_cast<std::uint8_t>(1u << (k & 7));
        }
    return BinaryMatrix(std::move(bits), rows, cols);
}

PackedBinaryWeights PackedBinaryWeights::from_int8(std::span<const std::int8_t> weights, std::uint32_t rows_raw,
                                                   std::uint32_t cols_raw, const TilingParams& tiling) {
    const std::uint32_t rows_padded = (rows_raw + 63) / 64 * 64, cols_padded = (cols_raw + 7) / 8 * 8;
    std::vector<std::int8_t> padded(static_cast<std::size_t>(rows_padded) * cols_padded, static_cast<std::int8_t>(1));
    for (std::uint32_t i = 0; i < rows_raw; ++i)
        std::memcpy(&padded[static_cast<std::size_t>(i) * cols_padded], &weights[static_cast<std::size_t>(i) * cols_raw], cols_raw);
    PackedBinaryWeights out;
    out.b_packed = BinaryMatrix::pack(std::span<const std::int8_t>(padded.data(), padded.size()), rows_padded, cols_padded);
    out.tiling = tiling;
    out.original_m = rows_raw;
    out.original_n = cols_raw;
    out.original_k = rows_raw;
    return out;
}

// ---- device copies ---------------------------------------------------------------------------------------

const Tensor& BinaryMatrix::device_words() const {
    if (!device_) {
        // Column n of the host plane is rows_/8 contiguous bytes; the device layout wants ceil128(rows_)/8 per column.
        const std::int64_t k_pad = (static_cast<std::int64_t>(rows_) + 127) / 128 * 128;
        const std::size_t src_bytes = rows_ / 8, dst_bytes = static_cast<std::size_t>(k_pad / 8);
        Tensor host(Shape{static_cast<std::int64_t>(cols_), k_pad / 32}, DataType::INT32);  // zero-filled: padding = +1
        auto* dst = static_cast<std::uint8_t*>(host.data());
        for (std::uint32_t n = 0; n < cols_; ++n) std::memcpy(dst + n * dst_bytes, bits_.data() + n * src_bytes, src_bytes);
        device_ = std::make_shared<Tensor>(host.to_device(DeviceType::CUDA));
    }
    return *device_;
}

const Tensor& TernaryMatrix::device_values() const {
    if (!device_) {
        Tensor host(Shape{static_cast<std::int64_t>(rows_), static_cast<std::int64_t>(cols_)}, DataType::FLOAT32);
        float* dst = host.typed_data<float>();
        const std::size_t row_bytes = cols_ / 8;
        for (std::uint32_t m = 0; m < rows_; ++m)
            for (std::uint32_t k = 0; k < cols_; ++k) {
                const std::uint8_t bit = static_cast<std::uint8_t>(1u << (k & 7));
                const bool p = positive_[m * row_bytes + k / 8] & bit, n = negative_[m * row_bytes + k / 8] & bit;
                dst[static_cast<std::size_t>(m) * cols_ + k] = p ? 1.0f : (n ? -1.0f : 0.0f);
            }
        device_ = std::make_shared<Tensor>(host.to_device(DeviceType::CUDA));
    }
    return *device_;
}

// ---- operators ---------------------------------------------------------------------------------------------

namespace {

// float(acc) * scale over A [M, K] (fp32 on the device, row stride lda) against the packed plane.
Tensor tbn_product(const float* d_a, std::int64_t M, std::int64_t K, std::int64_t lda, const BinaryMatrix& b, std::uint32_t n_orig,
                   float scale, float lo, float hi) {
    TBN_CHECK(n_orig > 0 && n_orig <= b.cols(), InvalidShapeError, "n_orig exceeds the packed matrix's columns");
    TBN_CHECK(K <= static_cast<std::int64_t>(b.rows()), InvalidShapeError,
              "Matrix dimensions incompatible: A cols (" + std::to_string(K) + ") > packed B rows (" + std::to_string(b.rows()) + ")");
    Tensor out = Tensor::device_uninitialized(Shape{M, static_cast<std::int64_t>(n_orig)}, DataType::FLOAT32);
    const size_t ws_bytes = tbn_gemm_workspace_bytes(M, K, TBN_MODE_TC_BF16X1);
    Tensor ws = Tensor::device_uninitialized(Shape{static_cast<std::int64_t>(ws_bytes)}, DataType::UINT8);
    // Columns K .. b.rows() of the padded product meet zero activations in the reference (pad_float_matrix), so
    // running the product over the first K rows of the plane gives the same integers.  The plane's row stride is
    // ceil128(b.rows()) / 32 words, which is the stride tbn_gemm_tbn derives from K only when both round to the same
    // multiple of 128 -- otherwise the product runs over the plane's full K with A's missing columns read as zero.
    const std::int64_t k_plane = static_cast<std::int64_t>(b.rows());
    const bool same_stride = (K + 127) / 128 == (k_plane + 127) / 128;
    const float* a_ptr = d_a;
    std::int64_t k_run = K, lda_run = lda;
    Tensor widened;
    if (!same_stride) {
        widened = Tensor(Shape{M, k_plane}, DataType::FLOAT32, DeviceType::CUDA);  // zero-filled
        for (std::int64_t m = 0; m < M; ++m)
            detail::check(tbn_cuda_d2d(static_cast<float*>(widened.device_data()) + m * k_plane, d_a + m * lda,
                                       static_cast<size_t>(K) * 4, nullptr));
        widened.mark_device_written();
        a_ptr = static_cast<const float*>(widened.device_data());
        k_run = k_plane;
        lda_run = k_plane;
    }
    detail::check(tbn_gemm_tbn(a_ptr, M, k_run, lda_run, lo, hi, static_cast<const std::uint32_t*>(b.device_words().device_data()),
                               n_orig, nullptr, scale, nullptr, static_cast<float*>(out.device_data()), n_orig, 0,
                               ws.device_data(), ws_bytes, nullptr));
    out.mark_device_written();
    return out;
}

}  // namespace

Tensor qlinear_matmul_binary_blocked_packed(const Tensor& a, const BinaryMatrix& b_packed, std::uint32_t n_orig, float scale,
                                            const TilingParams&, float lo, float hi) {
    detail::ensure_runtime();
    TBN_CHECK(a.dtype() == DataType::FLOAT32, InvalidArgumentError, "Input A must be FLOAT32");
    if (a.shape().dims.size() != 2) throw InvalidShapeError("Input A must be a 2D matrix");
    TBN_CHECK(!b_packed.empty(), InvalidArgumentError, "packed B is empty");
    const std::int64_t M = a.shape().dims[0], K = a.shape().dims[1];
    return tbn_product(static_cast<const float*>(a.device_data()), M, K, K, b_packed, n_orig, scale, lo, hi);
}

Tensor qlinear_matmul_binary_blocked_prepacked(const TernaryMatrix& a_packed, const BinaryMatrix& b_packed, std::uint32_t m_orig,
                                               std::uint32_t n_orig, float scale, const TilingParams&) {
    detail::ensure_runtime();
    TBN_CHECK(!a_packed.empty() && !b_packed.empty(), InvalidArgumentError, "packed operand is empty");
    TBN_CHECK(m_orig > 0 && m_orig <= a_packed.rows(), InvalidShapeError, "m_orig exceeds the packed matrix's rows");
    // The planes hold exact -1 / 0 / +1; as fp32 they pass the +-0.5 ternarisation unchanged.
    const Tensor& av = a_packed.device_values();
    return tbn_product(static_cast<const float*>(av.device_data()), m_orig, a_packed.cols(), a_packed.cols(), b_packed, n_orig,
                       scale, -0.5f, 0.5f);
}

}  // namespace tbn
