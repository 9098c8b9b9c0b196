// Basic types of the tbn:: API (reference: tbn-runtime/include/tbn/runtime/types.hpp).
// DeviceType gains CUDA; everything else keeps the reference's names and values.
#pragma once

#include <cstddef>
#include <cstdint>
#include <initializer_list>
#include <string>
#include <vector>

namespace tbn {

enum class DataType {
    FLOAT32, FLOAT16, BFLOAT16, INT8, INT16, INT32, INT64, UINT8, UINT16, UINT32, UINT64, BOOL,
    TERNARY,  // -1, 0, +1 stored one int8 per element
    BINARY    // 0 (= -1), 1 (= +1) stored one uint8 per element
};

enum class DeviceType { CPU, ARM_NEON, ARM_SVE, CUDA };

struct Shape {
    std::vector<int64_t> dims;
    Shape() = default;
    Shape(std::initializer_list<int64_t> d) : dims(d) {}
    Shape(const std::vector<int64_t>& d) : dims(d) {}
    int64_t size() const {
        int64_t s = 1;
        for (int64_t d : dims) s *= d;
        return s;
    }
    bool operator==(const Shape& o) const { return dims == o.dims; }
    bool operator!=(const Shape& o) const { return dims != o.dims; }
};

struct QuantizationParams {
    float scale = 1.0f;
    int32_t zero_point = 0;
    int32_t bit_width = 8;
};

using TernaryWeight = int8_t;
using BinaryWeight = uint8_t;
constexpr TernaryWeight TERNARY_MINUS_ONE = -1, TERNARY_ZERO = 0, TERNARY_PLUS_ONE = 1;
constexpr BinaryWeight BINARY_ZERO = 0, BINARY_ONE = 1;

inline size_t element_size(DataType t) {
    switch (t) {
        case DataType::FLOAT32: case DataType::INT32: case DataType::UINT32: return 4;
        case DataType::FLOAT16: case DataType::BFLOAT16: case DataType::INT16: case DataType::UINT16: return 2;
        case DataType::INT64: case DataType::UINT64: return 8;
        default: return 1;
    }
}

std::string shape_to_string(const Shape& shape);

// Tiling of the reference's CPU GEMM (GeMM/05-final/GeMM.hpp:16-43).  Accepted everywhere the
// reference accepts it so that callers compile unchanged; the GPU kernels choose their own tiles.
struct TilingParams {
    std::uint32_t mblk, nblk, kblk, mmk, nmk;
    static constexpr TilingParams default_128x128() noexcept { return {64, 64, 128, 32, 32}; }
};

}  // namespace tbn
