// Python module `_tbn` over the GPU Session.
//
// Same Python surface as the reference's module (tbn-runtime/python/bindings.cpp:53-168): Shape (dims, repr),
// Model(path, mblk, nblk, kblk, mmk, nmk) with run(input, use_quantization=False), run_quantized(input),
// input_names(), output_names(), input_shape(name), and load_model(path, ...).  The tiling arguments are
// accepted and ignored (the GPU kernels choose their own tiles).  The Session is created once per Model and
// reused, so packed weights are cached across run() calls as in the reference.
//
// Extension: when the array's leading dimension is a multiple of the model's declared batch (and the rest of
// the shape matches), run() feeds it through the Session slice by slice and concatenates the outputs.
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <cstring>
#include <memory>

#include "tbn/tbn.hpp"

namespace py = pybind11;
using namespace tbn;

namespace {

Tensor array_to_tensor(const float* data, const Shape& shape) { return Tensor(shape, DataType::FLOAT32, data); }

class PyModel {
public:
    PyModel(const std::string& path, uint32_t mblk, uint32_t nblk, uint32_t kblk, uint32_t mmk, uint32_t nmk)
        : model_(load_onnx_model(path)),
          session_(std::make_unique<TBNModel::Session>(model_.create_session(TilingParams{mblk, nblk, kblk, mmk, nmk}))) {}

    py::array_t<float> run(py::array_t<float, py::array::c_style | py::array::forcecast> input, bool use_quantization) {
        const auto& in_names = model_.graph().inputs;
        const auto& out_names = model_.graph().outputs;
        if (in_names.empty()) throw std::runtime_error("Model has no inputs");
        if (out_names.empty()) throw std::runtime_error("Model has no outputs");
        // The first graph input that is not an initializer is the data input (old exports list weights too).
        std::string in_name = in_names[0];
        for (const auto& n : in_names)
            if (!model_.graph().initializers.count(n)) { in_name = n; break; }
        const Shape& want = model_.get_input_shape(in_name);
        py::buffer_info buf = input.request();
        Shape got;
        for (py::ssize_t i = 0; i < buf.ndim; ++i) got.dims.push_back(buf.shape[i]);
        session_->set_quantization(use_quantization);

        int64_t slices = 1;
        if (got != want && !got.dims.empty() && got.dims.size() == want.dims.size() && want.dims[0] > 0 &&
            got.dims[0] % want.dims[0] == 0 && std::equal(got.dims.begin() + 1, got.dims.end(), want.dims.begin() + 1))
            slices = got.dims[0] / want.dims[0];
        const Shape slice_shape = slices > 1 ? want : got;  // a mismatch is reported by set_input, as in the reference
        const int64_t slice_elems = slice_shape.size();
        std::vector<Tensor> outs;
        for (int64_t s = 0; s < slices; ++s) {
            session_->set_input(in_name, array_to_tensor(static_cast<const float*>(buf.ptr) + s * slice_elems, slice_shape));
            session_->run();
            outs.push_back(session_->get_output(out_names[0]));
        }
        Shape out_shape = outs[0].shape();
        const int64_t out_elems = outs[0].num_elements();
        if (slices > 1 && !out_shape.dims.empty()) out_shape.dims[0] *= slices;
        std::vector<py::ssize_t> dims(out_shape.dims.begin(), out_shape.dims.end());
        py::array_t<float> result(dims);
        float* dst = static_cast<float*>(result.request().ptr);
        for (int64_t s = 0; s < slices; ++s)
            std::memcpy(dst + s * out_elems, outs[static_cast<size_t>(s)].typed_data<float>(), static_cast<size_t>(out_elems) * sizeof(float));
        return result;
    }

    py::array_t<float> run_quantized(py::array_t<float, py::array::c_style | py::array::forcecast> input) {
        return run(std::move(input), true);
    }
    std::vector<std::string> input_names() const { return model_.graph().inputs; }
    std::vector<std::string> output_names() const { return model_.graph().outputs; }
    Shape input_shape(const std::string& name) const {
        auto it = model_.graph().value_info.find(name);
        if (it == model_.graph().value_info.end()) throw std::runtime_error("Input not found: " + name);
        return it->second;
    }
    void mark_binary(const std::string& weight_name) { session_->mark_binary(weight_name); }
    std::string producer() const { return model_.producer_name() + " " + model_.producer_version(); }

private:
    TBNModel model_;
    std::unique_ptr<TBNModel::Session> session_;
};

}  // namespace

PYBIND11_MODULE(_tbn, m) {
    m.doc() = "TBN runtime on B200: inference for ternary-binary neural networks (GPU Session behind the reference's Python API)";
    py::register_exception<TBNError>(m, "TBNError");

    py::class_<Shape>(m, "Shape")
        .def(py::init<>())
        .def(py::init<std::vector<int64_t>>())
        .def_readwrite("dims", &Shape::dims)
        .def("__repr__", [](const Shape& s) {
            std::string str = "Shape([";
            for (size_t i = 0; i < s.dims.size(); ++i) str += (i ? ", " : "") + std::to_string(s.dims[i]);
            return str + "])";
        });

    py::class_<PyModel>(m, "Model")
        .def(py::init<const std::string&, uint32_t, uint32_t, uint32_t, uint32_t, uint32_t>(), py::arg("path"),
             py::arg("mblk") = 64, py::arg("nblk") = 64, py::arg("kblk") = 128, py::arg("mmk") = 32, py::arg("nmk") = 32,
             "Load an ONNX model.  The tiling arguments of the CPU runtime are accepted and ignored.")
        .def("run", &PyModel::run, py::arg("input"), py::arg("use_quantization") = false)
        .def("run_quantized", &PyModel::run_quantized, py::arg("input"))
        .def("input_names", &PyModel::input_names)
        .def("output_names", &PyModel::output_names)
        .def("input_shape", &PyModel::input_shape, py::arg("name"))
        .def("mark_binary", &PyModel::mark_binary, py::arg("weight_name"),
             "Declare raw fp32 weights as binary (sign + mean|w| scale derived on the device).")
        .def("producer", &PyModel::producer);

    m.def("load_model",
          [](const std::string& path, uint32_t mblk, uint32_t nblk, uint32_t kblk, uint32_t mmk, uint32_t nmk) {
              return std::make_unique<PyModel>(path, mblk, nblk, kblk, mmk, nmk);
          },
          py::arg("path"), py::arg("mblk") = 64, py::arg("nblk") = 64, py::arg("kblk") = 128, py::arg("mmk") = 32,
          py::arg("nmk") = 32, "Load an ONNX model.");
    m.def("get_version", []() { return std::string(get_version()); });
}
