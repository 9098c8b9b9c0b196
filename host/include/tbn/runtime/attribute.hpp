// Node attributes (reference: tbn-runtime/include/tbn/runtime/attribute.hpp).
#pragma once

#include <string>
#include <unordered_map>
#include <variant>
#include <vector>

#include "tensor.hpp"

namespace tbn {

struct AttributeValue {
    using Value = std::variant<int64_t, float, std::string, Tensor, std::vector<int64_t>, std::vector<float>,
                               std::vector<std::string>>;
    Value value;

    AttributeValue() : value(int64_t(0)) {}
    AttributeValue(int64_t v) : value(v) {}
    AttributeValue(int v) : value(static_cast<int64_t>(v)) {}
    AttributeValue(float v) : value(v) {}
    AttributeValue(double v) : value(static_cast<float>(v)) {}
    AttributeValue(const std::string& v) : value(v) {}
    AttributeValue(const char* v) : value(std::string(v)) {}
    AttributeValue(const Tensor& v) : value(v) {}
    AttributeValue(const std::vector<int64_t>& v) : value(v) {}
    AttributeValue(const std::vector<float>& v) : value(v) {}
    AttributeValue(const std::vector<std::string>& v) : value(v) {}

    bool is_int() const { return std::holds_alternative<int64_t>(value); }
    bool is_float() const { return std::holds_alternative<float>(value); }
    bool is_string() const { return std::holds_alternative<std::string>(value); }
    bool is_tensor() const { return std::holds_alternative<Tensor>(value); }
    bool is_ints() const { return std::holds_alternative<std::vector<int64_t>>(value); }
    bool is_floats() const { return std::holds_alternative<std::vector<float>>(value); }
    int64_t as_int() const { return std::get<int64_t>(value); }
    float as_float() const { return std::get<float>(value); }
    const std::string& as_string() const { return std::get<std::string>(value); }
    const Tensor& as_tensor() const { return std::get<Tensor>(value); }
    const std::vector<int64_t>& as_ints() const { return std::get<std::vector<int64_t>>(value); }
    const std::vector<float>& as_floats() const { return std::get<std::vector<float>>(value); }
    int64_t as_int_or(int64_t d) const { return is_int() ? as_int() : d; }
    float as_float_or(float d) const { return is_float() ? as_float() : d; }
};

using NodeAttributes = std::unordered_map<std::string, AttributeValue>;

}  // namespace tbn
