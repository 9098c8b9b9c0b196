// Graph IR, model and Session of the tbn:: API, executing on the GPU.
//
// Same public surface as the reference (tbn-runtime/include/tbn/runtime/model.hpp:21-1330):
// ModelNode / ModelGraph are plain structs to be filled by a loader or by hand; TBNModel wraps a graph;
// TBNModel::create_session(TilingParams) returns a Session with set_quantization / set_tiling /
// set_input / get_input / run / get_output and the same exception types.
//
// What changed underneath: the Session's tensor map lives in HBM (set_input uploads, get_output returns a
// device tensor whose typed_data() downloads), the per-weight caches are packed once on the device, and
// every node runs a CUDA kernel through the C ABI.
//
// Numeric modes, selected by the reference's own switch:
//   set_quantization(false)  Conv/Gemm evaluate y = x * W in fp32 accuracy.  A scaled-binary W (+-alpha per
//                            output channel, i.e. a dequantised TBN model) or one declared with mark_binary()
//                            (raw fp32 weights; sign and alpha = mean|w| derived here) runs on the packed-weight
//                            kernels; any other float W runs on the float path (two bf16 terms per operand).
//   set_quantization(true)   the reference's TBN mode, bit-equal: activations ternarised at +-0.1, exact
//                            integer GEMM, Conv epilogue (acc + bias) * alpha, Gemm quantised on the fly.
#pragma once

#include <memory>
#include <string>
#include <unordered_map>
#include <unordered_set>
#include <vector>

#include "../operators/ops.hpp"
#include "attribute.hpp"
#include "tensor.hpp"

namespace tbn {

struct ModelNode {
    std::string name;
    std::string op_type;
    std::vector<std::string> inputs;
    std::vector<std::string> outputs;
    NodeAttributes attributes;
};

struct ModelGraph {
    std::vector<ModelNode> nodes;
    std::unordered_map<std::string, Tensor> initializers;
    std::unordered_map<std::string, Shape> value_info;
    std::vector<std::string> inputs;
    std::vector<std::string> outputs;
};

class TBNModel {
public:
    TBNModel() : graph_(std::make_shared<ModelGraph>()) {}
    explicit TBNModel(std::shared_ptr<ModelGraph> graph) : graph_(std::move(graph)) {}

    const ModelGraph& graph() const { return *graph_; }
    ModelGraph& graph() { return *graph_; }
    const std::vector<std::string>& inputs() const { return graph_->inputs; }
    const std::vector<std::string>& outputs() const { return graph_->outputs; }
    bool has_input(const std::string& name) const;
    bool has_output(const std::string& name) const;
    const Shape& get_input_shape(const std::string& name) const;
    const Shape& get_output_shape(const std::string& name) const;
    void validate() const;
    void set_producer(const std::string& name, const std::string& version) {
        producer_name_ = name;
        producer_version_ = version;
    }
    const std::string& producer_name() const { return producer_name_; }
    const std::string& producer_version() const { return producer_version_; }

    class Session {
    public:
        explicit Session(std::shared_ptr<ModelGraph> graph, TilingParams tiling = TilingParams::default_128x128());

        void set_quantization(bool enable) { use_quantization_ = enable; }
        bool is_quantization_enabled() const { return use_quantization_; }
        void set_tiling(const TilingParams& p) { tiling_ = p; }
        const TilingParams& get_tiling() const { return tiling_; }

        // Declares a weight initializer as raw fp32 weights to be binarised by sign with the per-output-channel
        // scale mean|w| (extension; the reference only recognises weights that are already +-alpha).
        void mark_binary(const std::string& weight_name) { declared_binary_.insert(weight_name); }
        // Graph-level optimisations of the float mode, on by default; results are bit-identical either way.
        //   fusion   a Relu, or an Add with the block input followed by a Relu, that only consumes a Conv's result
        //            runs in that convolution's epilogue;
        //   chaining a Conv whose result feeds channels-last convolutions writes the bf16 channels-last form from its
        //            epilogue (and no fp32 tensor when nothing else reads it); those convolutions skip their pre-pass;
        //   release  intermediates are freed after their last reader (outputs and inputs are kept).
        void set_graph_optimizations(bool enable) { optimize_ = enable; }

        void set_input(const std::string& name, const Tensor& tensor);
        Tensor get_input(const std::string& name) const;
        void run();
        Tensor get_output(const std::string& name) const;

    private:
        struct CachedWeights {
            PackedWeights packed;   // sign planes (+ alpha for the float x binary mode)
            Tensor alpha_tbn;       // sequentially summed scale of the dequantised weights (TBN-mode Conv)
            bool scaled_binary = false;
            bool dense = false;     // plain float weights: `dense_w` is used instead of `packed`
            DenseWeights dense_w;
        };
        const CachedWeights* weights_for(const std::string& name, const Tensor& w, bool conv);
        bool run_lenet_fused();
        void execute_node(const ModelNode& node);
        void execute_conv(const ModelNode& node, size_t idx);
        void execute_gemm(const ModelNode& node);
        void execute_pool(const ModelNode& node, bool is_max);
        const Tensor& value(const std::string& name) const;

        std::shared_ptr<ModelGraph> graph_;
        std::unordered_map<std::string, Tensor> input_tensors_, output_tensors_, intermediate_tensors_;
        std::unordered_map<std::string, CachedWeights> weight_cache_;
        std::unordered_map<std::string, Tensor> transposed_;  // op(B) of Gemm nodes with transB, once per weight
        // State of one run(): channels-last forms and shapes of values, readers of every value, fused-away nodes.
        std::unordered_map<std::string, Tensor> cl_tensors_;
        std::unordered_map<std::string, Shape> value_shapes_;
        std::unordered_map<std::string, std::vector<size_t>> readers_;
        std::unordered_set<size_t> skip_;
        bool optimize_ = true;
        std::unordered_set<std::string> declared_binary_;
        bool use_quantization_ = false;
        TilingParams tiling_;
    };

    Session create_session(TilingParams tiling = TilingParams::default_128x128()) const { return Session(graph_, tiling); }

private:
    std::shared_ptr<ModelGraph> graph_;
    std::string producer_name_, producer_version_;
};

// Loader entry points of the reference (model.hpp:1328-1330; implemented over the ONNX reader in
// onnx_integration/onnx_parser.hpp).  Both throw InvalidModelError when the file cannot be opened or parsed.
TBNModel load_model(const std::string& model_path);
TBNModel load_model_from_buffer(const void* data, size_t size);
const char* get_version();  // "0.1.0", as the reference

// Builds a graph from a line-oriented description (one declaration per line):
//   input|output|value <name> <d0,d1,..>
//   init <name> f32|i64 <d0,d1,..> <offset>      offset into `blob` (4-byte units) / `iblob` (8-byte units)
//   node <op_type> <name> <in0,in1,..> <out0,..> [key=i:<int>|f:<float>|s:<str>|I:<i0,i1,..>]...
//   binary <name0,name1,..>                       weight names to pass to Session::mark_binary
TBNModel parse_graph_spec(const std::string& spec, const float* blob, const int64_t* iblob,
                          std::vector<std::string>* binary_names = nullptr);

}  // namespace tbn
