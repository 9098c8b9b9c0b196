// Test driver for the C++ host API: reads a graph spec + weight blob + input from files, runs it through
// tbn::TBNModel::Session and writes the output.  Usage:
//   run_graph <spec.txt> <blob.f32> <input.f32> <input name> <output name> <quantization 0|1> <out.f32> [repeat [noopt]]
//     (repeat > 1 prints the wall time per Session::run after the first; noopt switches the graph optimisations off)
//   run_graph --onnx <model.onnx> <input.f32> <input name> <output name> <quantization 0|1> <out.f32> [binary names]
//   run_graph --dump-onnx <model.onnx>     canonical text listing of the loaded graph (no GPU work)
// Also exercises the error paths a reference user relies on (exception types), printing "errors ok".
#include <algorithm>
#include <array>
#include <cstdint>
#include <chrono>
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

static uint64_t fnv1a(const void* data, size_t n) {
    const unsigned char* p = static_cast<const unsigned char*>(data);
    uint64_t h = 1469598103934665603ull;
    for (size_t i = 0; i < n; ++i) h = (h ^ p[i]) * 1099511628211ull;
    return h;
}

static std::string join(const std::vector<std::string>& v) {
    std::string out;
    for (size_t i = 0; i < v.size(); ++i) out += (i ? "," : "") + v[i];
    return out;
}

static std::string dims_of(const tbn::Shape& s) {
    std::string out;
    for (size_t i = 0; i < s.dims.size(); ++i) out += (i ? "," : "") + std::to_string(s.dims[i]);
    return out.empty() ? "-" : out;
}

// One line per graph element, sorted where the container is unordered, so that two loaders can be compared.
static int dump_onnx(const char* path) {
    using namespace tbn;
    TBNModel model = load_onnx_model(path);
    const ModelGraph& g = model.graph();
    std::printf("producer %s|%s\n", model.producer_name().c_str(), model.producer_version().c_str());
    for (const auto& n : g.inputs) std::printf("input %s %s\n", n.c_str(), dims_of(g.value_info.at(n)).c_str());
    for (const auto& n : g.outputs) std::printf("output %s %s\n", n.c_str(), dims_of(g.value_info.at(n)).c_str());
    std::vector<std::string> names;
    for (const auto& kv : g.value_info) names.push_back(kv.first);
    std::sort(names.begin(), names.end());
    for (const auto& n : names) std::printf("value %s %s\n", n.c_str(), dims_of(g.value_info.at(n)).c_str());
    names.clear();
    for (const auto& kv : g.initializers) names.push_back(kv.first);
    std::sort(names.begin(), names.end());
    for (const auto& n : names) {
        const Tensor& t = g.initializers.at(n);
        std::printf("init %s dtype=%d dims=%s bytes=%zu fnv=%016llx\n", n.c_str(), static_cast<int>(t.dtype()),
                    dims_of(t.shape()).c_str(), t.data_size(), static_cast<unsigned long long>(fnv1a(t.data(), t.data_size())));
    }
    for (const auto& node : g.nodes) {
        std::printf("node %s %s [%s] -> [%s]", node.op_type.c_str(), node.name.c_str(), join(node.inputs).c_str(),
                    join(node.outputs).c_str());
        std::vector<std::string> keys;
        for (const auto& kv : node.attributes) keys.push_back(kv.first);
        std::sort(keys.begin(), keys.end());
        for (const auto& k : keys) {
            const AttributeValue& a = node.attributes.at(k);
            std::printf(" %s=", k.c_str());
            if (a.is_int()) std::printf("i:%lld", static_cast<long long>(a.as_int()));
            else if (a.is_float()) std::printf("f:%.9g", a.as_float());
            else if (a.is_string()) std::printf("s:%s", a.as_string().c_str());
            else if (a.is_ints()) { std::printf("I:"); for (size_t i = 0; i < a.as_ints().size(); ++i) std::printf(i ? ",%lld" : "%lld", static_cast<long long>(a.as_ints()[i])); }
            else if (a.is_floats()) { std::printf("F:"); for (size_t i = 0; i < a.as_floats().size(); ++i) std::printf(i ? ",%.9g" : "%.9g", a.as_floats()[i]); }
            else if (a.is_tensor()) std::printf("t:%s:%016llx", dims_of(a.as_tensor().shape()).c_str(),
                                                static_cast<unsigned long long>(fnv1a(a.as_tensor().data(), a.as_tensor().data_size())));
            else { std::printf("S:"); const auto& v = std::get<std::vector<std::string>>(a.value); for (size_t i = 0; i < v.size(); ++i) std::printf(i ? ",%s" : "%s", v[i].c_str()); }
        }
        std::printf("\n");
    }
    return 0;
}

static int run_onnx(int argc, char** argv) {
    // argv: --onnx model input in_name out_name quant out [binary names]
    tbn::TBNModel model = tbn::load_model(argv[2]);
    model.validate();
    const auto input = read_file(argv[3]);
    auto session = model.create_session();
    if (argc > 8) {
        std::stringstream ss(argv[8]);
        std::string name;
        while (std::getline(ss, name, ',')) if (!name.empty()) session.mark_binary(name);
    }
    session.set_quantization(std::atoi(argv[6]) != 0);
    tbn::Tensor x(model.get_input_shape(argv[4]), tbn::DataType::FLOAT32, input.data());
    if (x.data_size() != input.size()) throw std::runtime_error("input file size does not match the model's input shape");
    session.set_input(argv[4], x);
    session.run();
    tbn::Tensor y = session.get_output(argv[5]);
    std::ofstream out(argv[7], std::ios::binary);
    out.write(static_cast<const char*>(static_cast<const void*>(y.typed_data<float>())), static_cast<std::streamsize>(y.data_size()));
    std::printf("ok %s\n", tbn::shape_to_string(y.shape()).c_str());
    return 0;
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

// Known-answer vectors of the packed layouts (host types only, no GPU): the three vectors the oracle is pinned on.
static int packed_layout() {
    using namespace tbn;
    int bad = 0;
    std::vector<std::int8_t> w(128 * 8, 1);
    w[37 * 8 + 3] = -1;
    w[64 * 8 + 0] = -1;
    BinaryMatrix b = BinaryMatrix::pack(w, 128, 8);
    std::vector<std::uint32_t> words(b.view().bits.size() / 4);
    std::memcpy(words.data(), b.view().bits.data(), b.view().bits.size());
    for (size_t i = 0; i < words.size(); ++i)
        if (words[i] != (i == 13 ? 0x20u : (i == 2 ? 0x1u : 0u))) ++bad;
    std::vector<float> a(8 * 64, 0.0f);
    a[1 * 64 + 9] = 0.5f; a[2 * 64 + 33] = -0.5f; a[0] = 0.1f; a[1] = -0.1f;
    TernaryMatrix t = TernaryMatrix::pack_from_float(a.data(), 8, 64);
    std::vector<std::uint32_t> pos(t.view().positive.size() / 4), neg(pos.size());
    std::memcpy(pos.data(), t.view().positive.data(), t.view().positive.size());
    std::memcpy(neg.data(), t.view().negative.data(), t.view().negative.size());
    for (size_t i = 0; i < pos.size(); ++i) {
        if (pos[i] != (i == 2 ? 0x200u : 0u)) ++bad;
        if (neg[i] != (i == 5 ? 0x2u : 0u)) ++bad;
    }
    try { (void)BinaryMatrix::pack(std::vector<std::int8_t>(60 * 8, 1), 60, 8); ++bad; } catch (const std::invalid_argument&) {}
    try { (void)BinaryMatrix::pack(std::vector<std::int8_t>(64 * 8, 0), 64, 8); ++bad; } catch (const std::invalid_argument&) {}
    try { (void)TernaryMatrix::pack(std::vector<std::int8_t>(8 * 64, 2), 8, 64); ++bad; } catch (const std::invalid_argument&) {}
    PackedBinaryWeights pw = PackedBinaryWeights::from_int8(std::vector<std::int8_t>(70 * 5, -1), 70, 5, TilingParams::default_128x128());
    if (!pw.valid() || pw.b_packed.rows() != 128 || pw.b_packed.cols() != 8 || pw.original_n != 5) ++bad;
    std::printf(bad ? "packed layout FAILED (%d)\n" : "packed layout ok\n", bad);
    return bad;
}

// Operators on pre-packed operands (GPU): both must equal qlinear_matmul_binary on the unpacked operands, bit for bit.
static int prepacked() {
    using namespace tbn;
    int bad = 0;
    const TilingParams tp = TilingParams::default_128x128();
    std::uint64_t s = 88172645463325252ull;
    auto rnd = [&]() { s ^= s << 13; s ^= s >> 7; s ^= s << 17; return s; };
    for (const auto& dims : std::vector<std::array<int, 3>>{{40, 200, 24}, {130, 576, 128}, {16, 64, 8}, {33, 300, 20}}) {
        const int M = dims[0], K = dims[1], N = dims[2];
        const int Kp = (K + 127) / 128 * 128, Np = (N + 7) / 8 * 8, Mp = (M + 15) / 16 * 16;
        std::vector<float> a(static_cast<size_t>(M) * K);
        for (auto& v : a) v = static_cast<float>(static_cast<int>(rnd() % 2001) - 1000) / 2000.0f;   // [-0.5, 0.5]
        std::vector<BinaryWeight> bq(static_cast<size_t>(K) * N);
        for (auto& v : bq) v = static_cast<BinaryWeight>(rnd() & 1);
        Tensor A = make_tensor(Shape{M, K}, a), B = make_tensor(Shape{K, N}, bq);
        Tensor expect = qlinear_matmul_binary(A, B, 0.37f, tp);
        // pad K to 128 and N to 8 with +1, as the reference's callers do (quantized_gemm_neon.cpp:199-214)
        std::vector<std::int8_t> bi(static_cast<size_t>(Kp) * Np, 1);
        for (int k = 0; k < K; ++k)
            for (int n = 0; n < N; ++n) bi[static_cast<size_t>(k) * Np + n] = bq[static_cast<size_t>(k) * N + n] ? 1 : -1;
        BinaryMatrix Bp = BinaryMatrix::pack(bi, Kp, Np);
        Tensor got = qlinear_matmul_binary_blocked_packed(A, Bp, N, 0.37f, tp);
        if (std::memcmp(got.typed_data<float>(), expect.typed_data<float>(), static_cast<size_t>(M) * N * 4) != 0) ++bad;
        std::vector<float> ap(static_cast<size_t>(Mp) * Kp, 0.0f);
        for (int m = 0; m < M; ++m) std::memcpy(&ap[static_cast<size_t>(m) * Kp], &a[static_cast<size_t>(m) * K], static_cast<size_t>(K) * 4);
        TernaryMatrix Ap = TernaryMatrix::pack_from_float(ap.data(), Mp, Kp);
        Tensor got2 = qlinear_matmul_binary_blocked_prepacked(Ap, Bp, M, N, 0.37f, tp);
        if (std::memcmp(got2.typed_data<float>(), expect.typed_data<float>(), static_cast<size_t>(M) * N * 4) != 0) ++bad;
        // weights padded only to 64 rows (PackedBinaryWeights::from_int8): K = 200 -> 256 plane rows vs 256: same; K = 64 -> 64 vs 128
        std::vector<std::int8_t> braw(static_cast<size_t>(K) * N);
        for (size_t i = 0; i < braw.size(); ++i) braw[i] = bq[i] ? 1 : -1;
        PackedBinaryWeights pw = PackedBinaryWeights::from_int8(braw, K, N, tp);
        Tensor got3 = qlinear_matmul_binary_blocked_packed(A, pw.b_packed, N, 0.37f, tp);
        if (std::memcmp(got3.typed_data<float>(), expect.typed_data<float>(), static_cast<size_t>(M) * N * 4) != 0) ++bad;
    }
    std::printf(bad ? "prepacked FAILED (%d)\n" : "prepacked ok\n", bad);
    return bad;
}

int main(int argc, char** argv) {
    try {
        if (argc == 2 && std::strcmp(argv[1], "--errors") == 0) return error_paths();
        if (argc == 2 && std::strcmp(argv[1], "--packed-layout") == 0) return packed_layout();
        if (argc == 2 && std::strcmp(argv[1], "--prepacked") == 0) return prepacked();
        if (argc == 3 && std::strcmp(argv[1], "--dump-onnx") == 0) return dump_onnx(argv[2]);
        if (argc >= 8 && std::strcmp(argv[1], "--onnx") == 0) return run_onnx(argc, argv);
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
        if (argc > 9 && std::strcmp(argv[9], "noopt") == 0) session.set_graph_optimizations(false);
        session.run();  // first run: packs and caches the weights
        const auto t0 = std::chrono::steady_clock::now();
        for (int i = 1; i < repeat; ++i) session.run();
        if (repeat > 1)
            std::printf("ms_per_run %.4f\n",
                        std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count() / (repeat - 1));
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
