// Error types of the tbn:: API (same names, codes and hierarchy as the reference's
// tbn-runtime/include/tbn/utils/errors.hpp:10-93) plus the mapping from C-ABI status codes.
#pragma once

#include <stdexcept>
#include <string>

namespace tbn {

enum class ErrorCode {
    SUCCESS = 0,
    INVALID_ARGUMENT = -1,
    OUT_OF_MEMORY = -2,
    NOT_IMPLEMENTED = -3,
    INVALID_MODEL = -4,
    RUNTIME_ERROR = -5,
    QUANTIZATION_ERROR = -6,
    INVALID_SHAPE = -7,
    DEVICE_NOT_SUPPORTED = -8,
    ONNX_PARSE_ERROR = -9,
    OPERATOR_NOT_SUPPORTED = -10
};

class TBNError : public std::exception {
public:
    TBNError(ErrorCode code, std::string message) : code_(code), message_(std::move(message)) {}
    const char* what() const noexcept override { return message_.c_str(); }
    ErrorCode code() const noexcept { return code_; }

private:
    ErrorCode code_;
    std::string message_;
};

#define TBN_DEFINE_ERROR(NAME, CODE)                                        \
    class NAME : public TBNError {                                          \
    public:                                                                 \
        explicit NAME(const std::string& msg) : TBNError(ErrorCode::CODE, msg) {} \
    };

TBN_DEFINE_ERROR(InvalidArgumentError, INVALID_ARGUMENT)
TBN_DEFINE_ERROR(OutOfMemoryError, OUT_OF_MEMORY)
TBN_DEFINE_ERROR(NotImplementedError, NOT_IMPLEMENTED)
TBN_DEFINE_ERROR(InvalidModelError, INVALID_MODEL)
TBN_DEFINE_ERROR(QuantizationError, QUANTIZATION_ERROR)
TBN_DEFINE_ERROR(InvalidShapeError, INVALID_SHAPE)
TBN_DEFINE_ERROR(RuntimeError, RUNTIME_ERROR)
#undef TBN_DEFINE_ERROR

#define TBN_CHECK(condition, error_type, message) \
    do {                                          \
        if (!(condition)) throw error_type(message); \
    } while (0)

#define TBN_CHECK_NOT_NULL(ptr, error_type) TBN_CHECK((ptr) != nullptr, error_type, #ptr " must not be null")

namespace detail {
// Throws the TBNError subclass that corresponds to a non-zero C-ABI status, with the library's message.
void throw_status(int status);
inline void check(int status) {
    if (status != 0) throw_status(status);
}
}  // namespace detail

}  // namespace tbn
