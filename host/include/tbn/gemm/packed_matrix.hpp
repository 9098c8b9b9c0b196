// Host-side packed matrix types of the reference's GEMM layer, for source compatibility with code that
// pre-packs its operands (reference: GeMM/05-final/GeMM.hpp:48-204):
//   BinaryMatrix        one bit-plane, column-major over [rows = K][cols = N]: byte n*(K/8) + k/8, bit k&7,
//                       bit set <=> -1 (GeMM.cpp:114-151); rows % 64 == 0, cols % 8 == 0, values in {-1, +1}
//   TernaryMatrix       two row-major bit-planes over [rows = M][cols = K]: byte m*(K/8) + k/8, bit k&7
//                       (positive: +1, negative: -1; GeMM.cpp:29-112); rows % 8 == 0, cols % 64 == 0
//   PackedBinaryWeights weights packed once (pads K to 64 and N to 8 with +1), GeMM.cpp:375-402
// The types own HOST byte vectors exactly as in the reference (view() hands out spans of them).  New: each keeps
// a device copy of its planes in the layout the CUDA kernels read (made on first use, then reused), which is
// what qlinear_matmul_binary_blocked_packed / _blocked_prepacked consume -- no arithmetic happens on the host.
#pragma once

#include <cstdint>
#include <memory>
#include <span>
#include <stdexcept>
#include <vector>

#include "../runtime/tensor.hpp"
#include "../runtime/types.hpp"

namespace tbn {

struct TernaryMatrixView {
    std::span<const std::uint8_t> positive;
    std::span<const std::uint8_t> negative;
    std::uint32_t rows{};
    std::uint32_t cols{};
};

struct BinaryMatrixView {
    std::span<const std::uint8_t> bits;
    std::uint32_t rows{};
    std::uint32_t cols{};
};

class TernaryMatrix {
public:
    TernaryMatrix() = default;
    [[nodiscard]] static TernaryMatrix pack(std::span<const std::int8_t> data, std::uint32_t rows, std::uint32_t cols);
    [[nodiscard]] static TernaryMatrix pack_from_float(const float* data, std::uint32_t rows, std::uint32_t cols,
                                                       float threshold_low = -0.1f, float threshold_high = 0.1f);
    [[nodiscard]] static TernaryMatrix from_bitplanes(std::vector<std::uint8_t> positive, std::vector<std::uint8_t> negative,
                                                      std::uint32_t rows, std::uint32_t cols) {
        return TernaryMatrix(std::move(positive), std::move(negative), rows, cols);
    }
    [[nodiscard]] std::uint32_t rows() const noexcept { return rows_; }
    [[nodiscard]] std::uint32_t cols() const noexcept { return cols_; }
    [[nodiscard]] TernaryMatrixView view() const noexcept { return {positive_, negative_, rows_, cols_}; }
    [[nodiscard]] bool empty() const noexcept { return positive_.empty(); }

    // The matrix as fp32 {-1, 0, +1} [rows, cols] on the device (expanded from the planes on first use).
    const Tensor& device_values() const;

private:
    TernaryMatrix(std::vector<std::uint8_t> positive, std::vector<std::uint8_t> negative, std::uint32_t rows, std::uint32_t cols)
        : positive_(std::move(positive)), negative_(std::move(negative)), rows_(rows), cols_(cols) {}
    std::vector<std::uint8_t> positive_, negative_;
    std::uint32_t rows_{}, cols_{};
    mutable std::shared_ptr<Tensor> device_;
};

class BinaryMatrix {
public:
    BinaryMatrix() = default;
    [[nodiscard]] static BinaryMatrix pack(std::span<const std::int8_t> data, std::uint32_t rows, std::uint32_t cols);
    [[nodiscard]] std::uint32_t rows() const noexcept { return rows_; }
    [[nodiscard]] std::uint32_t cols() const noexcept { return cols_; }
    [[nodiscard]] BinaryMatrixView view() const noexcept { return {bits_, rows_, cols_}; }
    [[nodiscard]] bool empty() const noexcept { return bits_.empty(); }

    // The plane as uint32 words [cols][ceil128(rows)/32] on the device: the layout of tbn_gemm_tbn / tbn_gemm_fxb
    // (rows padded with +1 = bit 0).  Uploaded on first use.
    const Tensor& device_words() const;

private:
    BinaryMatrix(std::vector<std::uint8_t> bits, std::uint32_t rows, std::uint32_t cols)
        : bits_(std::move(bits)), rows_(rows), cols_(cols) {}
    std::vector<std::uint8_t> bits_;
    std::uint32_t rows_{}, cols_{};
    mutable std::shared_ptr<Tensor> device_;
};

struct PackedBinaryWeights {
    TernaryMatrix a_packed;
    BinaryMatrix b_packed;
    TilingParams tiling{};
    std::uint32_t original_m{};
    std::uint32_t original_n{};
    std::uint32_t original_k{};
    [[nodiscard]] bool valid() const noexcept { return !b_packed.empty(); }
    [[nodiscard]] static PackedBinaryWeights from_int8(std::span<const std::int8_t> weights, std::uint32_t rows_raw,
                                                       std::uint32_t cols_raw, const TilingParams& tiling);
};

// tbn-runtime/include/tbn/operators/quantized_gemm.hpp:66-84.  Activations ternarised at (threshold_low,
// threshold_high) x pre-packed binary weights, exact integer accumulation, float(acc) * scale: bit-equal to the
// reference functions of the same name.  b_packed.rows() is the (padded) K, which must cover a's columns.
Tensor qlinear_matmul_binary_blocked_packed(const Tensor& a, const BinaryMatrix& b_packed, std::uint32_t n_orig, float scale,
                                            const TilingParams& params, float threshold_low = -0.1f,
                                            float threshold_high = 0.1f);
Tensor qlinear_matmul_binary_blocked_prepacked(const TernaryMatrix& a_packed, const BinaryMatrix& b_packed,
                                               std::uint32_t m_orig, std::uint32_t n_orig, float scale,
                                               const TilingParams& params);

}  // namespace tbn
