// Protobuf wire-format reader for the subset of ONNX the tbn:: runtime consumes.
//
// Wire format (public protobuf encoding): a message is a sequence of (tag, payload) with
// tag = field_number << 3 | wire_type; wire types 0 = varint, 1 = 64-bit, 2 = length-delimited, 5 = 32-bit.
// Repeated scalars may be packed (one length-delimited payload) or not; both forms are accepted.
// Field numbers are those of the public onnx.proto (ModelProto.graph = 7, GraphProto.node = 1, ...).
#include "tbn/onnx_integration/onnx_parser.hpp"

#include <cstring>
#include <fstream>
#include <iterator>

namespace tbn {

namespace {

struct Span {
    const uint8_t* p = nullptr;
    const uint8_t* end = nullptr;
    bool done() const { return p >= end; }
    size_t size() const { return static_cast<size_t>(end - p); }
};

[[noreturn]] void malformed(const char* what) { throw InvalidModelError(std::string("Failed to parse ONNX model: ") + what); }

uint64_t read_varint(Span& s) {
    uint64_t v = 0;
    for (int shift = 0; shift < 64; shift += 7) {
        if (s.done()) malformed("truncated varint");
        const uint8_t b = *s.p++;
        v |= static_cast<uint64_t>(b & 0x7f) << shift;
        if (!(b & 0x80)) return v;
    }
    malformed("varint longer than 10 bytes");
}

uint32_t read_fixed32(Span& s) {
    if (s.size() < 4) malformed("truncated 32-bit field");
    uint32_t v;
    std::memcpy(&v, s.p, 4);
    s.p += 4;
    return v;
}

uint64_t read_fixed64(Span& s) {
    if (s.size() < 8) malformed("truncated 64-bit field");
    uint64_t v;
    std::memcpy(&v, s.p, 8);
    s.p += 8;
    return v;
}

Span read_bytes(Span& s) {
    const uint64_t n = read_varint(s);
    if (n > s.size()) malformed("length-delimited field runs past the end of its message");
    Span out{s.p, s.p + n};
    s.p += n;
    return out;
}

std::string to_string(const Span& s) { return std::string(reinterpret_cast<const char*>(s.p), s.size()); }

float bits_to_float(uint32_t u) {
    float f;
    std::memcpy(&f, &u, 4);
    return f;
}

// One decoded field.  `value` holds the varint / fixed payload, `bytes` the length-delimited one.
struct Field {
    uint32_t number = 0;
    uint32_t wire = 0;
    uint64_t value = 0;
    Span bytes;
};

bool next_field(Span& s, Field& f) {
    if (s.done()) return false;
    const uint64_t tag = read_varint(s);
    f.number = static_cast<uint32_t>(tag >> 3);
    f.wire = static_cast<uint32_t>(tag & 7);
    if (f.number == 0) malformed("field number 0");
    switch (f.wire) {
        case 0: f.value = read_varint(s); break;
        case 1: f.value = read_fixed64(s); break;
        case 2: f.bytes = read_bytes(s); break;
        case 5: f.value = read_fixed32(s); break;
        default: malformed("unsupported wire type (groups are not used by ONNX)");
    }
    return true;
}

// Repeated int64 / int32 (varint) field, packed or not.
void append_varints(const Field& f, std::vector<int64_t>& out) {
    if (f.wire == 0) {
        out.push_back(static_cast<int64_t>(f.value));
    } else if (f.wire == 2) {
        Span s = f.bytes;
        while (!s.done()) out.push_back(static_cast<int64_t>(read_varint(s)));
    } else {
        malformed("integer field with a non-integer wire type");
    }
}

// Repeated float field, packed or not.
void append_floats(const Field& f, std::vector<float>& out) {
    if (f.wire == 5) {
        out.push_back(bits_to_float(static_cast<uint32_t>(f.value)));
    } else if (f.wire == 2) {
        if (f.bytes.size() % 4) malformed("packed float field whose length is not a multiple of 4");
        const size_t n = f.bytes.size() / 4, at = out.size();
        out.resize(at + n);
        if (n) std::memcpy(out.data() + at, f.bytes.p, n * 4);
    } else {
        malformed("float field with a non-float wire type");
    }
}

// ---- ONNX messages ------------------------------------------------------------------------------

// TensorProto.DataType values of onnx.proto.
enum OnnxType { kFloat = 1, kUint8 = 2, kInt8 = 3, kInt32 = 6, kInt64 = 7 };

struct RawTensor {
    std::string name;
    std::vector<int64_t> dims;
    int32_t data_type = 0;
    Span raw;
    std::vector<float> float_data;
    std::vector<int64_t> int32_data, int64_data;
};

RawTensor parse_tensor(Span s) {
    RawTensor t;
    Field f;
    while (next_field(s, f)) {
        switch (f.number) {
            case 1: append_varints(f, t.dims); break;
            case 2: t.data_type = static_cast<int32_t>(f.value); break;
            case 4: append_floats(f, t.float_data); break;
            case 5: append_varints(f, t.int32_data); break;
            case 7: append_varints(f, t.int64_data); break;
            case 8: if (f.wire == 2) t.name = to_string(f.bytes); break;
            case 9: if (f.wire == 2) t.raw = f.bytes; break;
            default: break;  // segment, string_data, doc_string, external_data, double_data, ...
        }
    }
    return t;
}

template <typename T>
void store_narrowed(Tensor& dst, const std::vector<int64_t>& src) {
    T* out = dst.typed_data<T>();
    const size_t n = std::min<size_t>(src.size(), static_cast<size_t>(dst.num_elements()));
    for (size_t i = 0; i < n; ++i) out[i] = static_cast<T>(src[i]);
}

Tensor convert_tensor(const RawTensor& t) {
    DataType dtype;
    switch (t.data_type) {
        case kFloat: dtype = DataType::FLOAT32; break;
        case kInt32: dtype = DataType::INT32; break;
        case kInt64: dtype = DataType::INT64; break;
        case kUint8: dtype = DataType::UINT8; break;
        case kInt8: dtype = DataType::INT8; break;
        default: dtype = DataType::FLOAT32; break;
    }
    for (int64_t d : t.dims)
        if (d < 0) malformed("initializer with a negative dimension");
    Tensor tensor(Shape(t.dims), dtype);  // zero-filled
    const size_t capacity = tensor.data_size();
    if (t.raw.size() > 0) {
        std::memcpy(tensor.data(), t.raw.p, std::min(capacity, t.raw.size()));
    } else if (!t.float_data.empty()) {
        std::memcpy(tensor.data(), t.float_data.data(), std::min(capacity, t.float_data.size() * sizeof(float)));
    } else if (!t.int32_data.empty()) {
        switch (dtype) {
            case DataType::INT8: store_narrowed<int8_t>(tensor, t.int32_data); break;
            case DataType::UINT8: store_narrowed<uint8_t>(tensor, t.int32_data); break;
            case DataType::INT64: store_narrowed<int64_t>(tensor, t.int32_data); break;
            default: store_narrowed<int32_t>(tensor, t.int32_data); break;
        }
    } else if (!t.int64_data.empty()) {
        if (dtype == DataType::INT64) store_narrowed<int64_t>(tensor, t.int64_data);
        else store_narrowed<int32_t>(tensor, t.int64_data);
    }
    // else: no inline data (e.g. stored in an external file): stays zero, as in the reference.
    return tensor;
}

// AttributeProto.AttributeType values of onnx.proto.
enum AttrType { kAttrUndefined = 0, kAttrFloat = 1, kAttrInt = 2, kAttrString = 3, kAttrTensor = 4, kAttrFloats = 6,
                kAttrInts = 7, kAttrStrings = 8 };

void parse_attribute(Span s, NodeAttributes& attrs) {
    std::string name, str;
    int type = kAttrUndefined;
    float fval = 0.0f;
    int64_t ival = 0;
    bool has_f = false, has_i = false, has_s = false, has_t = false;
    Span tensor_bytes;
    std::vector<float> floats;
    std::vector<int64_t> ints;
    std::vector<std::string> strings;
    Field f;
    while (next_field(s, f)) {
        switch (f.number) {
            case 1: if (f.wire == 2) name = to_string(f.bytes); break;
            case 2: fval = bits_to_float(static_cast<uint32_t>(f.value)); has_f = true; break;
            case 3: ival = static_cast<int64_t>(f.value); has_i = true; break;
            case 4: if (f.wire == 2) { str = to_string(f.bytes); has_s = true; } break;
            case 5: if (f.wire == 2) { tensor_bytes = f.bytes; has_t = true; } break;
            case 7: append_floats(f, floats); break;
            case 8: append_varints(f, ints); break;
            case 9: if (f.wire == 2) strings.push_back(to_string(f.bytes)); break;
            case 20: type = static_cast<int>(f.value); break;
            default: break;  // g, tensors, graphs, doc_string, ref_attr_name, sparse tensors, type protos
        }
    }
    if (type == kAttrUndefined) {
        if (has_f) type = kAttrFloat;
        else if (has_i) type = kAttrInt;
        else if (has_s) type = kAttrString;
        else if (has_t) type = kAttrTensor;
        else if (!floats.empty()) type = kAttrFloats;
        else if (!ints.empty()) type = kAttrInts;
        else if (!strings.empty()) type = kAttrStrings;
    }
    switch (type) {
        case kAttrInt: attrs[name] = AttributeValue(ival); break;
        case kAttrFloat: attrs[name] = AttributeValue(fval); break;
        case kAttrString: attrs[name] = AttributeValue(str); break;
        case kAttrTensor: attrs[name] = AttributeValue(convert_tensor(parse_tensor(tensor_bytes))); break;
        case kAttrInts: attrs[name] = AttributeValue(ints); break;
        case kAttrFloats: attrs[name] = AttributeValue(floats); break;
        case kAttrStrings: attrs[name] = AttributeValue(strings); break;
        default: break;  // GRAPH, SPARSE_TENSOR, TYPE_PROTO and their lists: not used by this runtime
    }
}

ModelNode parse_node(Span s) {
    ModelNode node;
    Field f;
    while (next_field(s, f)) {
        if (f.wire != 2) continue;
        switch (f.number) {
            case 1: node.inputs.push_back(to_string(f.bytes)); break;
            case 2: node.outputs.push_back(to_string(f.bytes)); break;
            case 3: node.name = to_string(f.bytes); break;
            case 4: node.op_type = to_string(f.bytes); break;
            case 5: parse_attribute(f.bytes, node.attributes); break;
            default: break;
        }
    }
    if (node.name.empty()) node.name = node.op_type + "_" + (node.outputs.empty() ? std::string() : node.outputs[0]);
    return node;
}

// ValueInfoProto -> (name, shape); TypeProto.tensor_type.shape.dim[*].dim_value, dynamic dimensions -> 1.
void parse_value_info(Span s, std::string& name, Shape& shape) {
    Field f;
    while (next_field(s, f)) {
        if (f.wire != 2) continue;
        if (f.number == 1) {
            name = to_string(f.bytes);
        } else if (f.number == 2) {  // TypeProto
            Span type = f.bytes;
            Field tf;
            while (next_field(type, tf)) {
                if (tf.number != 1 || tf.wire != 2) continue;  // tensor_type
                Span tt = tf.bytes;
                Field ttf;
                while (next_field(tt, ttf)) {
                    if (ttf.number != 2 || ttf.wire != 2) continue;  // shape
                    Span sh = ttf.bytes;
                    Field df;
                    while (next_field(sh, df)) {
                        if (df.number != 1 || df.wire != 2) continue;  // dim
                        Span dim = df.bytes;
                        Field vf;
                        int64_t value = 1;
                        while (next_field(dim, vf))
                            if (vf.number == 1 && vf.wire == 0) value = static_cast<int64_t>(vf.value);
                        shape.dims.push_back(value);
                    }
                }
            }
        }
    }
}

}  // namespace

class OnnxParserImpl {
public:
    void parse(const void* data, size_t size) {
        bytes_.assign(static_cast<const uint8_t*>(data), static_cast<const uint8_t*>(data) + size);
        producer_name_.clear();
        producer_version_.clear();
        graph_bytes_ = Span{};
        have_graph_ = false;
        Span s{bytes_.data(), bytes_.data() + bytes_.size()};
        Field f;
        bool any = false;
        while (next_field(s, f)) {
            any = true;
            if (f.wire != 2) continue;
            if (f.number == 2) producer_name_ = to_string(f.bytes);
            else if (f.number == 3) producer_version_ = to_string(f.bytes);
            else if (f.number == 7) { graph_bytes_ = f.bytes; have_graph_ = true; }
        }
        if (!any && size > 0) malformed("no fields");
        // Walk the graph once now so that a malformed file fails at load time, as ParseFromIstream does.
        if (have_graph_) convert();
    }

    std::shared_ptr<ModelGraph> convert() const {
        auto graph = std::make_shared<ModelGraph>();
        if (!have_graph_) return graph;
        Span s = graph_bytes_;
        Field f;
        while (next_field(s, f)) {
            if (f.wire != 2) continue;
            switch (f.number) {
                case 1: graph->nodes.push_back(parse_node(f.bytes)); break;
                case 5: {
                    const RawTensor t = parse_tensor(f.bytes);
                    graph->initializers[t.name] = convert_tensor(t);
                    break;
                }
                case 11: case 12: case 13: {
                    std::string name;
                    Shape shape;
                    parse_value_info(f.bytes, name, shape);
                    graph->value_info[name] = shape;
                    if (f.number == 11) graph->inputs.push_back(name);
                    if (f.number == 12) graph->outputs.push_back(name);
                    break;
                }
                default: break;
            }
        }
        return graph;
    }

    std::string producer_name_, producer_version_;

private:
    std::vector<uint8_t> bytes_;
    Span graph_bytes_;
    bool have_graph_ = false;
};

OnnxParser::OnnxParser() : impl_(std::make_unique<OnnxParserImpl>()) {}
OnnxParser::~OnnxParser() = default;

void OnnxParser::parse_from_file(const std::string& path) {
    std::ifstream input(path, std::ios::binary);
    if (!input) throw InvalidModelError("Failed to open ONNX file: " + path);
    const std::vector<char> bytes((std::istreambuf_iterator<char>(input)), std::istreambuf_iterator<char>());
    try {
        impl_->parse(bytes.data(), bytes.size());
    } catch (const InvalidModelError& e) {
        throw InvalidModelError("Failed to parse ONNX model from: " + path + " (" + e.what() + ")");
    }
}

void OnnxParser::parse_from_buffer(const void* data, size_t size) {
    if (!data && size) throw InvalidModelError("Failed to parse ONNX model from buffer");
    impl_->parse(data, size);
}

std::shared_ptr<ModelGraph> OnnxParser::get_graph() { return impl_->convert(); }
std::string OnnxParser::get_producer_name() const { return impl_->producer_name_; }
std::string OnnxParser::get_producer_version() const { return impl_->producer_version_; }

TBNModel load_onnx_model(const std::string& path) {
    OnnxParser parser;
    parser.parse_from_file(path);
    TBNModel model(parser.get_graph());
    model.set_producer(parser.get_producer_name(), parser.get_producer_version());
    return model;
}

TBNModel load_onnx_model_from_buffer(const void* data, size_t size) {
    OnnxParser parser;
    parser.parse_from_buffer(data, size);
    TBNModel model(parser.get_graph());
    model.set_producer(parser.get_producer_name(), parser.get_producer_version());
    return model;
}

}  // namespace tbn
