// Test driver for the C++ host API: reads a graph spec + weight blob + input from files, runs it through
// tbn::TBNModel::Session and writes the output.  Usage:
//   run_graph <spec.txt> <blob.f32> <input.f32> <input name> <output name> <quantization 0|1> <out.f32> [repeat]
// Also exercises the error paths a reference user relies on (exception types), printing "errors ok".
#include <cstdio>
#include <cstring>
#include <fstream>
#include <iostream>
#include <sstream>
#include <vector>

#include "tbn/tbn.hpp"

static std::vector<char> read_file(const char* path) {
    std::ifstream f(path, std::ios::binary);
    if (!f) throw std::runtime_error(std::string("cannot open ") + path);
    return std::vector<char>((std::istreambuf_iterator<char>(f)), std::istreambuf_iterator<char>());
}

static int error_paths() {
    using namespace tbn;
    int bad = 0;
    auto graph = std::make_shared<ModelGraph>();
    graph->inputs = {"x"};
    graph->outputs = {"y"};
    graph->value_info["x"] = Shape{1, 4};
    graph->value_info["y"] = Shape{1, 4};
    graph->nodes.push_back(ModelNode{"n0", "Softmax", {"x"}, {"y"}, {}});
    TBNModel model(graph);
    auto s = model.create_session();
    try { s.set_input("nope", Tensor(Shape{1, 4}, DataType::FLOAT32)); ++bad; } catch (const InvalidArgumentError&) {}
    try { s.set_input("x", Tensor(Shape{1, 5}, DataType::FLOAT32)); ++bad; } catch (const InvalidShapeError&) {}
    try { s.run(); ++bad; } catch (const InvalidArgumentError&) {}   // no inputs set
    s.set_input("x", Tensor(Shape{1, 4}, DataType::FLOAT32));
    try { s.run(); ++bad; } catch (const NotImplementedError&) {}   // unknown operator
    try { s.get_output("y"); ++bad; } catch (const InvalidArgumentError&) {}
    try { load_onnx_model("missing.onnx"); ++bad; } catch (const InvalidModelError&) {}
    try { qlinear_matmul_binary(Tensor(Shape{2, 3}, DataType::FLOAT32), Tensor(Shape{4, 2}, DataType::BINARY), 1.0f,
                                TilingParams::default_128x128()); ++bad; } catch (const InvalidShapeError&) {}
    // 2x2 float x binary with scale 0.7, the shape of the reference's operator smoke test
    // (tbn-runtime/tests/test_quantized_operators.cpp:160-195) evaluated in TBN mode: activations > 0.1 -> +1.
    Tensor a = make_tensor(Shape{2, 2}, std::vector<float>{1.0f, 2.0f, 3.0f, 4.0f});
    Tensor b = make_tensor(Shape{2, 2}, std::vector<BinaryWeight>{1, 0, 0, 1});
    Tensor c = qlinear_matmul_binary(a, b, 0.7f, TilingParams::default_128x128());
    const float* cd = c.typed_data<float>();
    if (cd[0] != 0.0f || cd[1] != 0.0f || cd[2] != 0.0f || cd[3] != 0.0f) ++bad;  // (+1)(+1) + (+1)(-1) = 0
    std::printf(bad ? "errors FAILED (%d)\n" : "errors ok\n", bad);
    return bad;
}

int main(int argc, char** argv) {
    try {
        if (argc == 2 && std::strcmp(argv[1], "--errors") == 0) return error_paths();
        if (argc < 8) {
            std::fprintf(stderr, "usage: run_graph spec blob input in_name out_name quant out [repeat]\n");
            return 2;
        }
        const auto spec = read_file(argv[1]);
        const auto blob = read_file(argv[2]);
        const auto input = read_file(argv[3]);
        std::vector<std::string> binary;
        const int64_t none = 0;
        tbn::TBNModel model = tbn::parse_graph_spec(std::string(spec.begin(), spec.end()),
                                                    reinterpret_cast<const float*>(blob.data()), &none, &binary);
        model.validate();
        auto session = model.create_session();
        for (const auto& n : binary) session.mark_binary(n);
        session.set_quantization(std::atoi(argv[6]) != 0);
        tbn::Tensor x(model.get_input_shape(argv[4]), tbn::DataType::FLOAT32, input.data());
        session.set_input(argv[4], x);
        const int repeat = argc > 8 ? std::atoi(argv[8]) : 1;
        for (int i = 0; i < repeat; ++i) session.run();
        tbn::Tensor y = session.get_output(argv[5]);
        std::ofstream out(argv[7], std::ios::binary);
        out.write(static_cast<const char*>(static_cast<const void*>(y.typed_data<float>())), static_cast<std::streamsize>(y.data_size()));
        std::printf("ok %s\n", tbn::shape_to_string(y.shape()).c_str());
        return 0;
    } catch (const tbn::TBNError& e) {
        std::fprintf(stderr, "TBNError %d: %s\n", static_cast<int>(e.code()), e.what());
        return 1;
    } catch (const std::exception& e) {
        std::fprintf(stderr, "error: %s\n", e.what());
        return 1;
    }
}
