// TBNModel / Session on the GPU and the graph-spec reader.  Attribute handling follows the reference
// Session node by node (tbn-runtime/include/tbn/runtime/model.hpp:238-1316); the arithmetic is delegated
// to the operator functions in ops.cpp, i.e. to CUDA kernels behind the C ABI.
#include <algorithm>
#include <sstream>

#include "tbn/onnx_integration/onnx_parser.hpp"
#include "tbn/runtime/model.hpp"
#include "tbn_cuda.h"

namespace tbn {

// ------------------------------------------------------------------------- TBNModel

bool TBNModel::has_input(const std::string& name) const {
    return std::find(graph_->inputs.begin(), graph_->inputs.end(), name) != graph_->inputs.end();
}
bool TBNModel::has_output(const std::string& name) const {
    return std::find(graph_->outputs.begin(), graph_->outputs.end(), name) != graph_->outputs.end();
}
const Shape& TBNModel::get_input_shape(const std::string& name) const {
    auto it = graph_->value_info.find(name);
    TBN_CHECK(it != graph_->value_info.end(), InvalidArgumentError, "Input '" + name + "' not found in model");
    return it->second;
}
const Shape& TBNModel::get_output_shape(const std::string& name) const {
    auto it = graph_->value_info.find(name);
    TBN_CHECK(it != graph_->value_info.end(), InvalidArgumentError, "Output '" + name + "' not found in model");
    return it->second;
}
void TBNModel::validate() const {
    TBN_CHECK(!graph_->inputs.empty(), InvalidModelError, "Model has no inputs");
    TBN_CHECK(!graph_->outputs.empty(), InvalidModelError, "Model has no outputs");
    TBN_CHECK(!graph_->nodes.empty(), InvalidModelError, "Model has no computation nodes");
    for (const auto& n : graph_->inputs)
        TBN_CHECK(graph_->value_info.count(n) > 0, InvalidModelError, "Input '" + n + "' shape not defined");
    for (const auto& n : graph_->outputs)
        TBN_CHECK(graph_->value_info.count(n) > 0, InvalidModelError, "Output '" + n + "' shape not defined");
}

// ------------------------------------------------------------------------- Session

TBNModel::Session::Session(std::shared_ptr<ModelGraph> graph, TilingParams tiling) : graph_(std::move(graph)), tiling_(tiling) {}

void TBNModel::Session::set_input(const std::string& name, const Tensor& tensor) {
    TBN_CHECK(graph_->value_info.count(name) > 0, InvalidArgumentError, "Input '" + name + "' not found in model");
    TBN_CHECK(tensor.shape() == graph_->value_info.at(name), InvalidShapeError, "Input shape mismatch for '" + name + "'");
    tensor.device_data();  // upload now (no-op for a tensor that already lives on the device)
    input_tensors_[name] = tensor;
}

Tensor TBNModel::Session::get_input(const std::string& name) const {
    auto it = input_tensors_.find(name);
    TBN_CHECK(it != input_tensors_.end(), InvalidArgumentError, "Input '" + name + "' not set");
    return it->second;
}

Tensor TBNModel::Session::get_output(const std::string& name) const {
    auto it = output_tensors_.find(name);
    TBN_CHECK(it != output_tensors_.end(), InvalidArgumentError, "Output '" + name + "' not available");
    return it->second;
}

const Tensor& TBNModel::Session::value(const std::string& name) const {
    auto it = intermediate_tensors_.find(name);
    TBN_CHECK(it != intermediate_tensors_.end(), RuntimeError, "Input tensor '" + name + "' not found");
    return it->second;
}

void TBNModel::Session::run() {
    size_t user_inputs = 0;
    for (const auto& n : graph_->inputs)
        if (graph_->initializers.find(n) == graph_->initializers.end()) ++user_inputs;
    TBN_CHECK(input_tensors_.size() == user_inputs, InvalidArgumentError,
              "Not all inputs provided (expected " + std::to_string(user_inputs) + ", got " +
                  std::to_string(input_tensors_.size()) + ")");
    output_tensors_.clear();
    intermediate_tensors_.clear();
    cl_tensors_.clear();
    value_shapes_.clear();
    readers_.clear();
    skip_.clear();
    for (const auto& kv : input_tensors_) intermediate_tensors_[kv.first] = kv.second;
    for (const auto& kv : graph_->initializers) intermediate_tensors_[kv.first] = kv.second;
    if (optimize_ && !use_quantization_ && run_lenet_fused()) {
        synchronize();
        return;
    }
    const auto& nodes = graph_->nodes;
    std::unordered_map<std::string, size_t> last_use;
    for (size_t i = 0; i < nodes.size(); ++i)
        for (const auto& in : nodes[i].inputs) {
            readers_[in].push_back(i);
            last_use[in] = i;
        }
    const std::unordered_set<std::string> outputs(graph_->outputs.begin(), graph_->outputs.end());
    for (size_t i = 0; i < nodes.size(); ++i) {
        if (!skip_.count(i)) {
            if (nodes[i].op_type == "Conv") execute_conv(nodes[i], i);
            else execute_node(nodes[i]);
        }
        if (optimize_) {
            // Values whose last reader has run are freed (graph inputs, outputs and weights stay).
            for (const auto& in : nodes[i].inputs) {
                auto lu = last_use.find(in);
                if (lu == last_use.end() || lu->second != i) continue;
                if (outputs.count(in) || input_tensors_.count(in) || graph_->initializers.count(in)) continue;
                intermediate_tensors_.erase(in);
                cl_tensors_.erase(in);
            }
        }
    }
    for (const auto& out : graph_->outputs) {
        auto it = intermediate_tensors_.find(out);
        TBN_CHECK(it != intermediate_tensors_.end(), RuntimeError, "Output '" + out + "' was not produced");
        output_tensors_[out] = it->second;
    }
    cl_tensors_.clear();
    synchronize();
}

// The LeNet-shaped graph (Conv 5x5, Relu, MaxPool 2x2, Conv 5x5, Relu, MaxPool 2x2, Flatten, Gemm on 1 x 28 x 28
// inputs with 6 and 16 feature maps, all three weight tensors binary) runs as one kernel in float x binary mode:
// the whole-network fusion of Session::execute_* (tbn/runtime/model.hpp:190-228).  Returns false when the graph is
// anything else; the node-by-node path then runs.
bool TBNModel::Session::run_lenet_fused() {
    const auto& nodes = graph_->nodes;
    static const char* kOps[8] = {"Conv", "Relu", "MaxPool", "Conv", "Relu", "MaxPool", "Flatten", "Gemm"};
    if (nodes.size() != 8 || graph_->outputs.size() != 1 || input_tensors_.size() != 1) return false;
    for (size_t i = 0; i < 8; ++i) {
        if (nodes[i].op_type != kOps[i] || nodes[i].outputs.size() != 1 || nodes[i].inputs.empty()) return false;
        if (i > 0 && nodes[i].inputs[0] != nodes[i - 1].outputs[0]) return false;
    }
    if (nodes[7].outputs[0] != graph_->outputs[0] || input_tensors_.count(nodes[0].inputs[0]) == 0) return false;
    auto ints_are = [](const ModelNode& n, const char* key, std::initializer_list<int64_t> want, bool absent_ok) {
        auto a = n.attributes.find(key);
        if (a == n.attributes.end()) return absent_ok;
        if (!a->second.is_ints()) return false;
        const auto& v = a->second.as_ints();
        if (v.size() < want.size()) return false;
        size_t i = 0;
        for (int64_t w : want)
            if (v[i++] != w) return false;
        for (; i < v.size(); ++i)
            if (v[i] != (std::string(key) == "pads" ? 0 : 1)) return false;
        return true;
    };
    auto int_is = [](const ModelNode& n, const char* key, int64_t want) {
        auto a = n.attributes.find(key);
        return a == n.attributes.end() || (a->second.is_int() && a->second.as_int() == want);
    };
    auto float_is = [](const ModelNode& n, const char* key, float want) {
        auto a = n.attributes.find(key);
        return a == n.attributes.end() || (a->second.is_float() && a->second.as_float() == want);
    };
    for (size_t c : {size_t(0), size_t(3)}) {
        const ModelNode& n = nodes[c];
        if (n.inputs.size() < 2 || !ints_are(n, "strides", {1, 1}, true) || !ints_are(n, "pads", {0, 0}, true) ||
            !ints_are(n, "dilations", {1, 1}, true) || !int_is(n, "group", 1))
            return false;
        auto ap = n.attributes.find("auto_pad");
        if (ap != n.attributes.end() && ap->second.is_string() && ap->second.as_string() != "NOTSET" && ap->second.as_string() != "VALID")
            return false;
    }
    for (size_t c : {size_t(2), size_t(5)}) {
        const ModelNode& n = nodes[c];
        if (!ints_are(n, "kernel_shape", {2, 2}, true) || !ints_are(n, "strides", {2, 2}, true) || !ints_are(n, "pads", {0, 0}, true) ||
            !int_is(n, "ceil_mode", 0))
            return false;
    }
    if (!int_is(nodes[6], "axis", 1)) return false;
    const ModelNode& fc = nodes[7];
    if (fc.inputs.size() < 2 || !int_is(fc, "transA", 0) || !int_is(fc, "transB", 0) || !float_is(fc, "alpha", 1.0f) ||
        !float_is(fc, "beta", 1.0f))
        return false;
    const Tensor& X = input_tensors_.at(nodes[0].inputs[0]);
    auto init = [&](const std::string& name) -> const Tensor* {
        auto it = graph_->initializers.find(name);
        return it == graph_->initializers.end() ? nullptr : &it->second;
    };
    const Tensor *W1 = init(nodes[0].inputs[1]), *W2 = init(nodes[3].inputs[1]), *WF = init(fc.inputs[1]);
    if (!W1 || !W2 || !WF || X.dtype() != DataType::FLOAT32) return false;
    const auto& xs = X.shape().dims;
    if (xs.size() != 4 || xs[1] != 1 || xs[2] != 28 || xs[3] != 28) return false;
    if (W1->shape().dims != std::vector<int64_t>{6, 1, 5, 5} || W2->shape().dims != std::vector<int64_t>{16, 6, 5, 5}) return false;
    const auto& fs = WF->shape().dims;
    if (fs.size() != 2 || fs[0] != 256 || fs[1] < 1 || fs[1] > 64) return false;
    const Tensor* bias[3] = {nullptr, nullptr, nullptr};
    const ModelNode* owners[3] = {&nodes[0], &nodes[3], &fc};
    for (int i = 0; i < 3; ++i)
        if (owners[i]->inputs.size() >= 3) {
            bias[i] = init(owners[i]->inputs[2]);
            const int64_t want = i == 0 ? 6 : (i == 1 ? 16 : fs[1]);
            if (!bias[i] || bias[i]->dtype() != DataType::FLOAT32 || bias[i]->num_elements() != want) return false;
        }
    const CachedWeights* c1 = weights_for(nodes[0].inputs[1], *W1, true);
    const CachedWeights* c2 = weights_for(nodes[3].inputs[1], *W2, true);
    const CachedWeights* cf = weights_for(fc.inputs[1], *WF, false);
    if (!c1 || !c2 || !cf || c1->dense || c2->dense || cf->dense || c1->packed.tap_major || c2->packed.tap_major) return false;
    const int64_t batch = xs[0], classes = fs[1];
    Tensor out = Tensor::device_uninitialized(Shape{batch, classes}, DataType::FLOAT32);
    auto words = [](const PackedWeights& w) { return static_cast<const uint32_t*>(w.neg.device_data()); };
    auto f32 = [](const Tensor* t) { return t ? static_cast<const float*>(t->device_data()) : nullptr; };
    detail::check(tbn_lenet_fused_fxb(static_cast<const float*>(X.device_data()), batch, 6, 16, static_cast<int32_t>(classes),
                                      words(c1->packed), f32(&c1->packed.alpha), f32(bias[0]), words(c2->packed),
                                      f32(&c2->packed.alpha), f32(bias[1]), words(cf->packed), f32(&cf->packed.alpha), f32(bias[2]),
                                      static_cast<float*>(out.device_data()), nullptr));
    out.mark_device_written();
    intermediate_tensors_[graph_->outputs[0]] = out;
    output_tensors_[graph_->outputs[0]] = out;
    return true;
}

const TBNModel::Session::CachedWeights* TBNModel::Session::weights_for(const std::string& name, const Tensor& w, bool conv) {
    auto it = weight_cache_.find(name);
    if (it != weight_cache_.end()) return &it->second;
    if (w.dtype() != DataType::FLOAT32) return nullptr;
    CachedWeights cw;
    // "^T" marks the materialised transpose of a Gemm weight: declarations are made under the graph's name.
    const bool is_t = name.size() > 2 && name.compare(name.size() - 2, 2, "^T") == 0;
    const bool declared = declared_binary_.count(is_t ? name.substr(0, name.size() - 2) : name) > 0;
    if (conv) {
        std::vector<float> scales;
        cw.scaled_binary = scaled_binary_channel_scales(w, &scales);
        if (!cw.scaled_binary && !declared) {
            cw.dense = true;
            cw.dense_w = pack_dense_weights(w);
            return &weight_cache_.emplace(name, std::move(cw)).first->second;
        }
        // Scaled-binary: sign by >= 0 (model.hpp:433).  Declared raw weights: quantize_to_binary's w > 0.
        cw.packed = pack_binary_weights(w, 0.0f, cw.scaled_binary);
        if (cw.scaled_binary) cw.alpha_tbn = make_tensor(Shape{static_cast<int64_t>(scales.size())}, scales);
        else cw.alpha_tbn = cw.packed.alpha;
    } else {
        const int64_t K = w.shape().dims[0], N = w.shape().dims[1];
        const float* b = w.typed_data<float>();
        Tensor bt(Shape{N, K}, DataType::FLOAT32);
        float* t = bt.typed_data<float>();
        for (int64_t k = 0; k < K; ++k)
            for (int64_t n = 0; n < N; ++n) t[n * K + k] = b[k * N + n];
        cw.scaled_binary = scaled_binary_channel_scales(bt, nullptr);
        if (!cw.scaled_binary && !declared) {
            cw.dense = true;
            cw.dense_w = pack_dense_weights(w);
            return &weight_cache_.emplace(name, std::move(cw)).first->second;
        }
        cw.packed = pack_binary_weights(w, 0.0f, false);  // w > 0, as quantize_to_binary (model.hpp:840)
    }
    return &weight_cache_.emplace(name, std::move(cw)).first->second;
}

void TBNModel::Session::execute_conv(const ModelNode& node, size_t idx) {
    TBN_CHECK(node.inputs.size() >= 2, InvalidArgumentError, "Conv expects at least 2 inputs");
    TBN_CHECK(node.outputs.size() == 1, InvalidArgumentError, "Conv expects 1 output");
    // The input may exist only in its channels-last form (written by the previous convolution's epilogue).
    auto x_it = intermediate_tensors_.find(node.inputs[0]);
    auto xcl_it = cl_tensors_.find(node.inputs[0]);
    TBN_CHECK(x_it != intermediate_tensors_.end() || xcl_it != cl_tensors_.end(), RuntimeError,
              "Input tensor '" + node.inputs[0] + "' not found");
    const Tensor* Xp = x_it != intermediate_tensors_.end() ? &x_it->second : nullptr;
    const Tensor* Xcl = xcl_it != cl_tensors_.end() ? &xcl_it->second : nullptr;
    const Shape x_shape = Xp ? Xp->shape() : value_shapes_.at(node.inputs[0]);
    const Tensor& W = value(node.inputs[1]);
    TBN_CHECK(W.shape().dims.size() == 4, InvalidShapeError, "Conv2D weights must be 4D (MCHW)");
    Conv2DParams p;
    p.kernel_h = W.shape().dims[2];
    p.kernel_w = W.shape().dims[3];
    auto a = node.attributes.find("strides");
    if (a != node.attributes.end() && a->second.is_ints() && a->second.as_ints().size() >= 2) {
        p.stride_h = a->second.as_ints()[0];
        p.stride_w = a->second.as_ints()[1];
    }
    a = node.attributes.find("pads");  // begin_h, begin_w are the ones honoured (model.hpp:313-321)
    if (a != node.attributes.end() && a->second.is_ints() && a->second.as_ints().size() >= 4) {
        p.pad_h = a->second.as_ints()[0];
        p.pad_w = a->second.as_ints()[1];
    }
    a = node.attributes.find("auto_pad");
    if (a != node.attributes.end() && a->second.is_string() &&
        (a->second.as_string() == "SAME_UPPER" || a->second.as_string() == "SAME_LOWER")) {
        p.pad_h = (p.kernel_h - 1) * p.dilation_h / 2;
        p.pad_w = (p.kernel_w - 1) * p.dilation_w / 2;
    }
    a = node.attributes.find("dilations");
    if (a != node.attributes.end() && a->second.is_ints() && a->second.as_ints().size() >= 2) {
        p.dilation_h = a->second.as_ints()[0];
        p.dilation_w = a->second.as_ints()[1];
    }
    a = node.attributes.find("group");
    if (a != node.attributes.end() && a->second.is_int()) p.groups = a->second.as_int();
    const Tensor* B = nullptr;
    if (node.inputs.size() >= 3) {
        auto it = intermediate_tensors_.find(node.inputs[2]);
        if (it != intermediate_tensors_.end()) B = &it->second;
    }
    const auto& nodes = graph_->nodes;
    std::string out_name = node.outputs[0];
    Tensor result;
    if (W.dtype() == DataType::BINARY || W.dtype() == DataType::TERNARY) {
        TBN_CHECK(Xp != nullptr, RuntimeError, "Input tensor '" + node.inputs[0] + "' not found");
        result = W.dtype() == DataType::BINARY ? conv2d_binary(*Xp, W, B, p) : conv2d_ternary(*Xp, W, B, p);
        intermediate_tensors_[out_name] = result;
        return;
    }
    const CachedWeights* cw = weights_for(node.inputs[1], W, true);
    if (use_quantization_) {
        TBN_CHECK(Xp != nullptr, RuntimeError, "Input tensor '" + node.inputs[0] + "' not found");
        if (cw && cw->scaled_binary) {
            result = conv2d_tbn_packed(*Xp, cw->packed, &cw->alpha_tbn, B, p, true);  // (acc + bias) * alpha
        } else {
            // model.hpp:560-563: quantize_to_binary + conv2d_binary (no per-channel scale).
            result = conv2d_binary(*Xp, quantize_to_binary(W), B, p);
        }
        intermediate_tensors_[out_name] = result;
        return;
    }
    if (!cw) throw NotImplementedError("Conv '" + node.name + "': weights must be FLOAT32");
    // Float mode.  Fold a following Relu, or Add (with an existing fp32 tensor) + Relu, into the epilogue.
    bool relu_fused = false;
    const Tensor* residual = nullptr;
    // A value that is also a graph output must exist under its own name: nothing is folded over it.
    auto is_graph_output = [&](const std::string& name) {
        return std::find(graph_->outputs.begin(), graph_->outputs.end(), name) != graph_->outputs.end();
    };
    if (optimize_ && readers_[out_name].size() == 1 && !is_graph_output(out_name) && idx + 1 < nodes.size()) {
        const ModelNode& nxt = nodes[idx + 1];
        if (nxt.op_type == "Relu" && nxt.inputs.size() == 1 && nxt.inputs[0] == out_name) {
            relu_fused = true;
            skip_.insert(idx + 1);
            out_name = nxt.outputs.at(0);
        } else if (nxt.op_type == "Add" && nxt.inputs.size() == 2 && (nxt.inputs[0] == out_name || nxt.inputs[1] == out_name) &&
                   idx + 2 < nodes.size() && nodes[idx + 2].op_type == "Relu" && nodes[idx + 2].inputs.size() == 1 &&
                   nodes[idx + 2].inputs[0] == nxt.outputs.at(0) && readers_[nxt.outputs[0]].size() == 1 &&
                   !is_graph_output(nxt.outputs[0])) {
            const std::string& other = nxt.inputs[0] == out_name ? nxt.inputs[1] : nxt.inputs[0];
            auto rit = intermediate_tensors_.find(other);
            if (other != out_name && rit != intermediate_tensors_.end() && rit->second.dtype() == DataType::FLOAT32) {
                residual = &rit->second;
                relu_fused = true;
                skip_.insert(idx + 1);
                skip_.insert(idx + 2);
                out_name = nodes[idx + 2].outputs.at(0);
            }
        }
    }
    const bool tap_major = cw->dense ? cw->dense_w.tap_major : cw->packed.tap_major;
    if (optimize_ && tap_major) {
        // Chaining: channels-last convolutions among the readers take the bf16 form from this epilogue; any other
        // reader (a residual add, a pool, a graph output) needs the fp32 NCHW tensor.
        size_t cl_readers = 0;
        const auto& rd = readers_[out_name];
        for (size_t r : rd) {
            const ModelNode& rn = nodes[r];
            if (rn.op_type != "Conv" || rn.inputs.at(0) != out_name || rn.inputs.size() < 2) continue;
            auto wi = graph_->initializers.find(rn.inputs[1]);
            if (wi == graph_->initializers.end() || wi->second.dtype() != DataType::FLOAT32 || wi->second.shape().dims.size() != 4)
                continue;
            if (wi->second.shape().dims[1] % 64 == 0) ++cl_readers;  // what pack_*_weights lay out tap-major
        }
        const bool is_output = std::find(graph_->outputs.begin(), graph_->outputs.end(), out_name) != graph_->outputs.end();
        const bool want_cl = cl_readers > 0;
        const bool want_y = cl_readers != rd.size() || rd.empty() || is_output;
        ConvChainResult r = conv2d_chain(x_shape, Xcl ? nullptr : Xp, Xcl, cw->dense ? nullptr : &cw->packed,
                                         cw->dense ? &cw->dense_w : nullptr, B, p, residual, relu_fused, want_y, want_cl);
        if (want_cl) cl_tensors_[out_name] = r.y_cl;
        if (want_y) intermediate_tensors_[out_name] = r.y;
        const Shape& ws = W.shape();
        const int64_t OH = (x_shape.dims[2] + 2 * p.pad_h - p.dilation_h * (ws.dims[2] - 1) - 1) / p.stride_h + 1;
        const int64_t OW = (x_shape.dims[3] + 2 * p.pad_w - p.dilation_w * (ws.dims[3] - 1) - 1) / p.stride_w + 1;
        value_shapes_[out_name] = Shape{x_shape.dims[0], ws.dims[0], OH, OW};
        return;
    }
    TBN_CHECK(Xp != nullptr, RuntimeError, "Input tensor '" + node.inputs[0] + "' not found");
    result = cw->dense ? conv2d_float_dense(*Xp, cw->dense_w, B, p, residual, relu_fused)
                       : conv2d_float_packed(*Xp, cw->packed, B, p, residual, relu_fused);
    intermediate_tensors_[out_name] = result;
}

void TBNModel::Session::execute_gemm(const ModelNode& node) {
    TBN_CHECK(node.inputs.size() >= 2, InvalidArgumentError, "Gemm expects at least 2 inputs");
    TBN_CHECK(node.outputs.size() == 1, InvalidArgumentError, "Gemm expects 1 output");
    const Tensor& A = value(node.inputs[0]);
    const Tensor& Bw = value(node.inputs[1]);
    float alpha = 1.0f, beta = 1.0f;
    bool transA = false, transB = false;
    auto a = node.attributes.find("alpha");
    if (a != node.attributes.end() && a->second.is_float()) alpha = a->second.as_float();
    a = node.attributes.find("beta");
    if (a != node.attributes.end() && a->second.is_float()) beta = a->second.as_float();
    a = node.attributes.find("transA");
    if (a != node.attributes.end() && a->second.is_int()) transA = a->second.as_int() != 0;
    a = node.attributes.find("transB");
    if (a != node.attributes.end() && a->second.is_int()) transB = a->second.as_int() != 0;
    const Tensor* C = nullptr;
    if (node.inputs.size() >= 3) {
        auto it = intermediate_tensors_.find(node.inputs[2]);
        if (it != intermediate_tensors_.end()) C = &it->second;
    }
    TBN_CHECK(Bw.shape().dims.size() == 2, InvalidShapeError, "Gemm B must be 2D");
    if (transA || transB) {
        // The reference sends every transposed Gemm to its float tbn::gemm, quantisation on or off
        // (model.hpp:763: the binary path requires !transA && !transB).  Here: op(B) is materialised once per
        // weight tensor, op(A) per call, and the product runs on the float x binary kernel when op(B) is
        // scaled-binary, on the float path otherwise.
        const std::string key = transB ? node.inputs[1] + "^T" : node.inputs[1];
        if (transB && !transposed_.count(key)) transposed_[key] = transpose2d(Bw);
        const Tensor& Bop = transB ? transposed_.at(key) : Bw;
        const Tensor Aop = transA ? transpose2d(A) : A;
        const CachedWeights* cwt = weights_for(key, Bop, false);
        if (!cwt) throw NotImplementedError("Gemm '" + node.name + "': weights must be FLOAT32");
        Tensor bias_t;
        if (C && beta != 0.0f) {
            TBN_CHECK(C->shape().dims.size() == 1, NotImplementedError, "Gemm: only a 1-D C (bias) is accelerated");
            if (beta == 1.0f) {
                bias_t = *C;
            } else {
                bias_t = C->to_device(DeviceType::CPU);
                float* pb = bias_t.typed_data<float>();
                for (int64_t i = 0; i < bias_t.num_elements(); ++i) pb[i] *= beta;
            }
        }
        intermediate_tensors_[node.outputs[0]] =
            cwt->dense ? matmul_float_dense(Aop, cwt->dense_w, bias_t.empty() ? nullptr : &bias_t, alpha)
                       : matmul_float_packed(Aop, cwt->packed, bias_t.empty() ? nullptr : &bias_t, alpha);
        return;
    }
    const CachedWeights* cw = weights_for(node.inputs[1], Bw, false);
    if (!cw) throw NotImplementedError("Gemm '" + node.name + "': float weights that are neither scaled-binary nor declared with "
                                       "mark_binary() are not on the accelerated path");
    Tensor bias;
    if (C && beta != 0.0f) {
        TBN_CHECK(C->shape().dims.size() == 1, NotImplementedError, "Gemm: only a 1-D C (bias) is accelerated");
        if (beta == 1.0f) {
            bias = *C;
        } else {
            bias = C->to_device(DeviceType::CPU);
            float* pb = bias.typed_data<float>();
            for (int64_t i = 0; i < bias.num_elements(); ++i) pb[i] *= beta;
        }
    }
    Tensor result;
    if (cw->dense && !use_quantization_) {
        result = matmul_float_dense(A, cw->dense_w, bias.empty() ? nullptr : &bias, alpha);
    } else if (use_quantization_) {
        // model.hpp:835-869: binary GEMM with scale 1, then * alpha, + beta * C.  Plain float weights are
        // binarised on the fly by sign, as the reference does (model.hpp:839-841).
        result = qlinear_matmul_binary_packed(A, cw->dense ? pack_binary_weights(Bw, 0.0f, false) : cw->packed, alpha);
        if (!bias.empty()) result = add(result, bias);
    } else {
        result = matmul_float_packed(A, cw->packed, bias.empty() ? nullptr : &bias, alpha);
    }
    intermediate_tensors_[node.outputs[0]] = result;
}

void TBNModel::Session::execute_pool(const ModelNode& node, bool is_max) {
    const Tensor& X = value(node.inputs.at(0));
    Pool2DParams p;
    auto a = node.attributes.find("kernel_shape");
    if (a != node.attributes.end() && a->second.is_ints() && a->second.as_ints().size() >= 2) {
        p.kernel_h = a->second.as_ints()[0];
        p.kernel_w = a->second.as_ints()[1];
    }
    p.stride_h = p.kernel_h;
    p.stride_w = p.kernel_w;
    a = node.attributes.find("strides");
    if (a != node.attributes.end() && a->second.is_ints() && a->second.as_ints().size() >= 2) {
        p.stride_h = a->second.as_ints()[0];
        p.stride_w = a->second.as_ints()[1];
    }
    a = node.attributes.find("pads");
    if (a != node.attributes.end() && a->second.is_ints() && a->second.as_ints().size() >= 2) {
        p.pad_h = a->second.as_ints()[0];
        p.pad_w = a->second.as_ints()[1];
    }
    a = node.attributes.find("ceil_mode");
    if (a != node.attributes.end() && a->second.is_int()) p.ceil_mode = a->second.as_int() != 0;
    a = node.attributes.find("count_include_pad");
    if (a != node.attributes.end() && a->second.is_int()) p.count_include_pad = a->second.as_int() != 0;
    intermediate_tensors_[node.outputs.at(0)] = is_max ? maxpool2d(X, p) : avgpool2d(X, p);
}

void TBNModel::Session::execute_node(const ModelNode& node) {
    const std::string& op = node.op_type;
    if (op == "Gemm") {
        execute_gemm(node);
    } else if (op == "Relu") {
        TBN_CHECK(node.inputs.size() == 1, InvalidArgumentError, "ReLU expects 1 input");
        intermediate_tensors_[node.outputs.at(0)] = relu(value(node.inputs[0]));
    } else if (op == "MaxPool") {
        execute_pool(node, true);
    } else if (op == "AveragePool" || op == "AvgPool") {
        execute_pool(node, false);
    } else if (op == "GlobalAveragePool" || op == "GlobalAvgPool") {
        intermediate_tensors_[node.outputs.at(0)] = global_avgpool2d(value(node.inputs.at(0)));
    } else if (op == "GlobalMaxPool") {
        intermediate_tensors_[node.outputs.at(0)] = global_maxpool2d(value(node.inputs.at(0)));
    } else if (op == "MatMul") {
        // model.hpp:879-903: 2-D only, plain float product.
        TBN_CHECK(node.inputs.size() == 2, InvalidArgumentError, "MatMul expects 2 inputs");
        const Tensor& A = value(node.inputs[0]);
        const Tensor& B = value(node.inputs[1]);
        if (A.shape().dims.size() != 2 || B.shape().dims.size() != 2)
            throw NotImplementedError("MatMul for non-2D tensors not implemented");
        const CachedWeights* cw = graph_->initializers.count(node.inputs[1]) ? weights_for(node.inputs[1], B, false) : nullptr;
        if (cw) intermediate_tensors_[node.outputs.at(0)] = cw->dense ? matmul_float_dense(A, cw->dense_w) : matmul_float_packed(A, cw->packed);
        else intermediate_tensors_[node.outputs.at(0)] = gemm(A, B);
    } else if (op == "Greater" || op == "Less") {
        // model.hpp:1176-1270: the right-hand side is a tensor (usually a scalar initializer) or, when absent
        // from the tensor map, the node's "value" attribute.
        TBN_CHECK(node.inputs.size() == 2, InvalidArgumentError, op + " expects 2 inputs");
        const Tensor& lhs = value(node.inputs[0]);
        Tensor rhs;
        auto it = intermediate_tensors_.find(node.inputs[1]);
        if (it != intermediate_tensors_.end()) {
            rhs = it->second;
        } else {
            float scalar = 0.0f;
            auto a = node.attributes.find("value");
            if (a != node.attributes.end()) scalar = a->second.as_float();
            rhs = make_tensor(Shape{1}, std::vector<float>{scalar});
        }
        intermediate_tensors_[node.outputs.at(0)] = op == "Greater" ? greater(lhs, rhs) : less(lhs, rhs);
    } else if (op == "Sub") {
        TBN_CHECK(node.inputs.size() == 2, InvalidArgumentError, "Sub expects 2 inputs");
        intermediate_tensors_[node.outputs.at(0)] = sub(value(node.inputs[0]), value(node.inputs[1]));
    } else if (op == "Add") {
        TBN_CHECK(node.inputs.size() == 2, InvalidArgumentError, "Add expects 2 inputs");
        intermediate_tensors_[node.outputs.at(0)] = add(value(node.inputs[0]), value(node.inputs[1]));
    } else if (op == "Flatten") {
        const Tensor& X = value(node.inputs.at(0));
        int64_t axis = 1;
        auto a = node.attributes.find("axis");
        if (a != node.attributes.end() && a->second.is_int()) axis = a->second.as_int();
        int64_t outer = 1;
        for (int64_t i = 0; i < axis && i < static_cast<int64_t>(X.shape().dims.size()); ++i) outer *= X.shape().dims[i];
        intermediate_tensors_[node.outputs.at(0)] = X.reshaped(Shape{outer, X.num_elements() / std::max<int64_t>(outer, 1)});
    } else if (op == "Reshape") {
        const Tensor& X = value(node.inputs.at(0));
        const Tensor& S = value(node.inputs.at(1));
        const int64_t* sd = S.typed_data<int64_t>();
        std::vector<int64_t> dims(sd, sd + S.num_elements());
        int64_t known = 1, infer = -1;
        for (size_t i = 0; i < dims.size(); ++i) {
            if (dims[i] == -1) infer = static_cast<int64_t>(i);
            else known *= dims[i];
        }
        if (infer >= 0) dims[static_cast<size_t>(infer)] = X.num_elements() / std::max<int64_t>(known, 1);
        intermediate_tensors_[node.outputs.at(0)] = X.reshaped(Shape(dims));
    } else if (op == "Cast") {
        intermediate_tensors_[node.outputs.at(0)] = value(node.inputs.at(0));
    } else {
        throw NotImplementedError("Operator '" + op + "' not implemented");
    }
}

// ------------------------------------------------------------------------- loaders

TBNModel load_model(const std::string& model_path) { return load_onnx_model(model_path); }
TBNModel load_model_from_buffer(const void* data, size_t size) { return load_onnx_model_from_buffer(data, size); }
const char* get_version() { return "0.1.0"; }

namespace {
std::vector<std::string> split(const std::string& s, char sep) {
    std::vector<std::string> out;
    std::string cur;
    std::istringstream is(s);
    while (std::getline(is, cur, sep))
        if (!cur.empty()) out.push_back(cur);
    return out;
}
std::vector<int64_t> ints(const std::string& s) {
    std::vector<int64_t> v;
    for (const auto& p : split(s, ',')) v.push_back(std::stoll(p));
    return v;
}
}  // namespace

TBNModel parse_graph_spec(const std::string& spec, const float* blob, const int64_t* iblob, std::vector<std::string>* binary_names) {
    auto graph = std::make_shared<ModelGraph>();
    std::istringstream lines(spec);
    std::string line;
    while (std::getline(lines, line)) {
        const auto tok = split(line, ' ');
        if (tok.empty() || tok[0][0] == '#') continue;
        if ((tok[0] == "input" || tok[0] == "output" || tok[0] == "value") && tok.size() >= 3) {
            graph->value_info[tok[1]] = Shape(ints(tok[2]));
            if (tok[0] == "input") graph->inputs.push_back(tok[1]);
            if (tok[0] == "output") graph->outputs.push_back(tok[1]);
        } else if (tok[0] == "init" && tok.size() >= 5) {
            const Shape shape(ints(tok[3]));
            const int64_t off = std::stoll(tok[4]);
            if (tok[2] == "f32") graph->initializers[tok[1]] = Tensor(shape, DataType::FLOAT32, blob + off);
            else if (tok[2] == "i64") graph->initializers[tok[1]] = Tensor(shape, DataType::INT64, iblob + off);
            else throw InvalidModelError("graph spec: unknown initializer type in '" + line + "'");
        } else if (tok[0] == "node" && tok.size() >= 5) {
            ModelNode node;
            node.op_type = tok[1];
            node.name = tok[2];
            node.inputs = split(tok[3], ',');
            node.outputs = split(tok[4], ',');
            for (size_t i = 5; i < tok.size(); ++i) {
                const auto eq = tok[i].find('=');
                if (eq == std::string::npos || eq + 3 > tok[i].size()) throw InvalidModelError("graph spec: bad attribute '" + tok[i] + "'");
                const std::string key = tok[i].substr(0, eq), val = tok[i].substr(eq + 3);
                switch (tok[i][eq + 1]) {
                    case 'i': node.attributes[key] = AttributeValue(static_cast<int64_t>(std::stoll(val))); break;
                    case 'f': node.attributes[key] = AttributeValue(std::stof(val)); break;
                    case 's': node.attributes[key] = AttributeValue(val); break;
                    case 'I': node.attributes[key] = AttributeValue(ints(val)); break;
                    default: throw InvalidModelError("graph spec: bad attribute kind in '" + tok[i] + "'");
                }
            }
            graph->nodes.push_back(std::move(node));
        } else if (tok[0] == "binary" && tok.size() >= 2) {
            if (binary_names)
                for (const auto& n : split(tok[1], ',')) binary_names->push_back(n);
        } else {
            throw InvalidModelError("graph spec: cannot parse '" + line + "'");
        }
    }
    return TBNModel(graph);
}

}  // namespace tbn
