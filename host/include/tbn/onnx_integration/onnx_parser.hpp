// ONNX model loading for the tbn:: API without libonnx / protobuf.
//
// Same public surface as the reference (tbn-runtime/include/tbn/onnx_integration/onnx_parser.hpp:21-47):
// OnnxParser::parse_from_file / parse_from_buffer / get_graph / get_producer_name / get_producer_version and
// the free functions load_onnx_model / load_onnx_model_from_buffer.  The reference hands the bytes to the
// generated onnx::ModelProto classes; here a reader of the protobuf wire format walks the same messages
// (ModelProto, GraphProto, NodeProto, AttributeProto, TensorProto, ValueInfoProto, TypeProto,
// TensorShapeProto) and fills the same ModelGraph.
//
// Conversion rules kept from the reference (tbn-runtime/src/onnx_integration/onnx_parser.cpp):
//   * open / parse failure -> InvalidModelError (:41-47, :60-62);
//   * graph inputs, outputs and value_info become value_info shapes; a dimension without dim_value
//     (symbolic / dynamic) becomes 1 (:159-175);
//   * initializers: FLOAT, INT32, INT64, UINT8, INT8 keep their type, every other element type is loaded as
//     FLOAT32 (:188-212); data is taken from raw_data, else float_data, else int32_data, else int64_data
//     (:219-237); a tensor whose data lives in an external file stays zero-filled (:236);
//   * nodes: a missing name becomes op_type + "_" + first output (:244-248); attributes of type INT, FLOAT,
//     STRING, TENSOR, INTS, FLOATS, STRINGS are converted, others are dropped (:262-312).
// Differences, all on malformed or unusual input: data longer than the tensor is truncated instead of
// overrunning the buffer; int32_data holding 8-bit elements is narrowed element-wise instead of copied as
// 32-bit words; an attribute without a type field takes the type of the field it carries.
#pragma once

#include <memory>
#include <string>

#include "../runtime/model.hpp"

namespace tbn {

class OnnxParserImpl;

class OnnxParser {
public:
    OnnxParser();
    ~OnnxParser();

    void parse_from_file(const std::string& path);
    void parse_from_buffer(const void* data, size_t size);
    std::shared_ptr<ModelGraph> get_graph();
    std::string get_producer_name() const;
    std::string get_producer_version() const;

private:
    std::unique_ptr<OnnxParserImpl> impl_;
};

TBNModel load_onnx_model(const std::string& path);
TBNModel load_onnx_model_from_buffer(const void* data, size_t size);

}  // namespace tbn
