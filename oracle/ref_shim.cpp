// C-callable wrappers around the UNMODIFIED reference sources (fast-arm-tbcnn).
//
// TEST INFRASTRUCTURE ONLY.  This file is compiled together with the reference's
// own translation units (taken from where they lie, never copied) into
// oracle/_ref/libtbn_ref.so by oracle/Makefile.  It is used to (1) validate the
// plain-C restatement in oracle/tbn_oracle.c, (2) generate golden fixtures and
// (3) time the reference CPU path as the benchmark's reference arm.  Nothing in
// the product (the CUDA library or its host layer) links or loads it.
//
// Every wrapper returns 0 on success or a negative tbn::ErrorCode value; the
// message of the last failure is available through ref_last_error().

#include "tbn/runtime/model.hpp"
#include "tbn/operators/conv2d.hpp"
#include "tbn/operators/gemm.hpp"
#include "tbn/operators/pooling.hpp"
#include "tbn/operators/quantized_gemm.hpp"
#include "tbn/memory/packed_weights.hpp"

#include <cstdint>
#include <cstring>
#include <sstream>
#include <string>
#include <vector>

namespace tbn {
// Defined (non-static) in quantized_gemm_neon.cpp but declared in no header.
Tensor qlinear_matmul_binary_naive(const Tensor& a, const Tensor& b_binary, float scale);
// Declared in model.hpp, defined in onnx_parser.cpp which is not built here
// (needs protobuf).  Graphs are hand-built, so this is never reached.
TBNModel load_onnx_model(const std::string&) {
    throw NotImplementedError("ONNX parser is not part of the oracle build");
}
TBNModel load_onnx_model_from_buffer(const void*, size_t) {
    throw NotImplementedError("ONNX parser is not part of the oracle build");
}
namespace impl {
Tensor im2col(const Tensor& input, int64_t kernel_h, int64_t kernel_w,
              int64_t stride_h, int64_t stride_w, int64_t pad_h, int64_t pad_w,
              int64_t dilation_h, int64_t dilation_w);
TernaryMatrix im2col_ternary_packed(
    const float* input, int64_t N, int64_t C, int64_t H, int64_t W,
    int64_t kernel_h, int64_t kernel_w, int64_t stride_h, int64_t stride_w,
    int64_t pad_h, int64_t pad_w, int64_t dilation_h, int64_t dilation_w,
    uint32_t m_padded, uint32_t k_padded, float threshold_low, float threshold_high);
}  // namespace impl
}  // namespace tbn

namespace {

thread_local std::string g_last_error;

template <typename F>
int guarded(F&& f) {
    try {
        f();
        return 0;
    } catch (const tbn::TBNError& e) {
        g_last_error = e.what();
        return static_cast<int>(e.code());
    } catch (const std::invalid_argument& e) {
        g_last_error = e.what();
        return -1;
    } catch (const std::exception& e) {
        g_last_error = e.what();
        return -5;
    }
}

tbn::Tensor f32_tensor(const std::vector<int64_t>& dims, const float* data) {
    return tbn::Tensor(tbn::Shape(dims), tbn::DataType::FLOAT32, data);
}

tbn::TilingParams tiling_from(const uint32_t* t) {
    return tbn::TilingParams{t[0], t[1], t[2], t[3], t[4]};
}

std::vector<std::string> split(const std::string& s, char sep) {
    std::vector<std::string> out;
    std::string cur;
    std::istringstream is(s);
    while (std::getline(is, cur, sep)) {
        if (!cur.empty()) out.push_back(cur);
    }
    return out;
}

std::vector<int64_t> parse_ints(const std::string& s) {
    std::vector<int64_t> v;
    for (const auto& p : split(s, ',')) v.push_back(std::stoll(p));
    return v;
}

}  // namespace

extern "C" {

const char* ref_last_error() { return g_last_error.c_str(); }

// tbn::quantize_to_binary (quantized_gemm_neon.cpp:544-565)
int ref_quantize_to_binary(const float* w, int64_t n, float thr, uint8_t* out) {
    return guarded([&] {
        tbn::Tensor t = f32_tensor({n}, w);
        tbn::Tensor b = tbn::quantize_to_binary(t, thr);
        std::memcpy(out, b.data(), static_cast<size_t>(n));
    });
}

// tbn::quantize_to_ternary (quantized_gemm_neon.cpp:570-597)
int ref_quantize_to_ternary(const float* w, int64_t n, float lo, float hi, int8_t* out) {
    return guarded([&] {
        tbn::Tensor t = f32_tensor({n}, w);
        tbn::Tensor q = tbn::quantize_to_ternary(t, lo, hi);
        std::memcpy(out, q.data(), static_cast<size_t>(n));
    });
}

// tbn::BinaryMatrix::pack (GeMM.cpp:114-151); bits_out holds rows*cols/8 bytes.
int ref_binary_pack(const int8_t* data, uint32_t rows, uint32_t cols, uint8_t* bits_out) {
    return guarded([&] {
        auto m = tbn::BinaryMatrix::pack({data, static_cast<size_t>(rows) * cols}, rows, cols);
        auto v = m.view();
        std::memcpy(bits_out, v.bits.data(), v.bits.size());
    });
}

// tbn::TernaryMatrix::pack (GeMM.cpp:29-69)
int ref_ternary_pack(const int8_t* data, uint32_t rows, uint32_t cols, uint8_t* pos, uint8_t* neg) {
    return guarded([&] {
        auto m = tbn::TernaryMatrix::pack({data, static_cast<size_t>(rows) * cols}, rows, cols);
        auto v = m.view();
        std::memcpy(pos, v.positive.data(), v.positive.size());
        std::memcpy(neg, v.negative.data(), v.negative.size());
    });
}

// tbn::TernaryMatrix::pack_from_float (GeMM.cpp:71-112)
int ref_ternary_pack_from_float(const float* data, uint32_t rows, uint32_t cols, float lo, float hi,
                                uint8_t* pos, uint8_t* neg) {
    return guarded([&] {
        auto m = tbn::TernaryMatrix::pack_from_float(data, rows, cols, lo, hi);
        auto v = m.view();
        std::memcpy(pos, v.positive.data(), v.positive.size());
        std::memcpy(neg, v.negative.data(), v.negative.size());
    });
}

// tbn::TernaryPackedWeights::set_weight loop (packed_weights.hpp:53-71); out holds (n+3)/4 bytes.
int ref_ternary_codes(const int8_t* t, int64_t n, uint8_t* out) {
    return guarded([&] {
        tbn::TernaryPackedWeights p(tbn::Shape({n}));
        for (int64_t i = 0; i < n; ++i) p.set_weight(i, t[i]);
        std::memcpy(out, p.data(), static_cast<size_t>(p.packed_size()));
    });
}

// tbn::GemmEngine::compute (GeMM.cpp:303-363).  a_rows x a_cols ternary planes, a_cols x b_cols binary bits.
int ref_gemm_engine(const uint8_t* pos, const uint8_t* neg, uint32_t a_rows, uint32_t a_cols,
                    const uint8_t* bits, uint32_t b_cols, const uint32_t* tiling,
                    int32_t* c_out, uint64_t* flops_out) {
    return guarded([&] {
        const size_t a_bytes = static_cast<size_t>(a_rows) * (a_cols / 8);
        const size_t b_bytes = static_cast<size_t>(b_cols) * (a_cols / 8);
        tbn::TernaryMatrixView av{{pos, a_bytes}, {neg, a_bytes}, a_rows, a_cols};
        tbn::BinaryMatrixView bv{{bits, b_bytes}, a_cols, b_cols};
        tbn::GemmEngine engine;
        tbn::Int32Matrix c = engine.compute(av, bv, tiling_from(tiling));
        std::memcpy(c_out, c.data().data(), c.size() * sizeof(int32_t));
        if (flops_out) *flops_out = engine.last_flops();
    });
}

// tbn::qlinear_matmul_binary (quantized_gemm_neon.cpp:380-430) with a BINARY-dtype B[K,N] (1 => +1, 0 => -1).
int ref_qlinear_matmul_binary(const float* a, int64_t M, int64_t K, const uint8_t* b, int64_t N,
                              float scale, const uint32_t* tiling, float* c_out) {
    return guarded([&] {
        tbn::Tensor at = f32_tensor({M, K}, a);
        tbn::Tensor bt(tbn::Shape({K, N}), tbn::DataType::BINARY, b);
        tbn::Tensor c = tbn::qlinear_matmul_binary(at, bt, scale, tiling_from(tiling));
        std::memcpy(c_out, c.data(), static_cast<size_t>(M * N) * sizeof(float));
    });
}

// Weights packed once, the way the Session caches them (model.hpp:810-833): BINARY bytes [K,N]
// -> +-1 int8 padded with +1 to [ceil128(K), ceil8(N)] -> BinaryMatrix::pack.  Returns a handle
// for ref_qlinear_matmul_binary_packed, or NULL on failure.
void* ref_pack_binary_weights(const uint8_t* b, uint32_t K, uint32_t N) {
    tbn::BinaryMatrix* out = nullptr;
    const int rc = guarded([&] {
        const uint32_t Kp = (K + 127) / 128 * 128, Np = (N + 7) / 8 * 8;
        std::vector<int8_t> padded(static_cast<size_t>(Kp) * Np, 1);
        for (uint32_t i = 0; i < K; ++i)
            for (uint32_t j = 0; j < N; ++j)
                padded[static_cast<size_t>(i) * Np + j] = (b[static_cast<size_t>(i) * N + j] == tbn::BINARY_ONE) ? 1 : -1;
        out = new tbn::BinaryMatrix(tbn::BinaryMatrix::pack({padded.data(), padded.size()}, Kp, Np));
    });
    return rc == 0 ? out : nullptr;
}

void ref_free_binary_weights(void* handle) { delete static_cast<tbn::BinaryMatrix*>(handle); }

// tbn::qlinear_matmul_binary_blocked_packed (quantized_gemm_neon.cpp:249-309): the per-inference
// part of the reference's "float x binary" path with cached weights.
int ref_qlinear_matmul_binary_packed(const float* a, int64_t M, int64_t K, const void* handle, uint32_t N,
                                     float scale, const uint32_t* tiling, float* c_out) {
    return guarded([&] {
        tbn::Tensor at = f32_tensor({M, K}, a);
        tbn::Tensor c = tbn::qlinear_matmul_binary_blocked_packed(
            at, *static_cast<const tbn::BinaryMatrix*>(handle), N, scale, tiling_from(tiling));
        std::memcpy(c_out, c.data(), static_cast<size_t>(M) * N * sizeof(float));
    });
}

// tbn::qlinear_matmul_binary_naive (quantized_gemm_neon.cpp:63-90): the true float x binary product.
int ref_fxb_naive(const float* a, int64_t M, int64_t K, const uint8_t* b, int64_t N, float scale,
                  float* c_out) {
    return guarded([&] {
        tbn::Tensor at = f32_tensor({M, K}, a);
        tbn::Tensor bt(tbn::Shape({K, N}), tbn::DataType::BINARY, b);
        tbn::Tensor c = tbn::qlinear_matmul_binary_naive(at, bt, scale);
        std::memcpy(c_out, c.data(), static_cast<size_t>(M * N) * sizeof(float));
    });
}

// tbn::gemm (gemm.cpp:349-360).  c_ndim: 0 = no C, 1 = C[N], 2 = C[M,N].
int ref_gemm_f32(const float* a, int64_t a_rows, int64_t a_cols, const float* b, int64_t b_rows,
                 int64_t b_cols, const float* c, int c_ndim, float alpha, float beta, int transA,
                 int transB, float* out) {
    return guarded([&] {
        tbn::Tensor at = f32_tensor({a_rows, a_cols}, a);
        tbn::Tensor bt = f32_tensor({b_rows, b_cols}, b);
        const int64_t M = transA ? a_cols : a_rows;
        const int64_t N = transB ? b_rows : b_cols;
        tbn::Tensor ct;
        if (c_ndim == 1) ct = f32_tensor({N}, c);
        if (c_ndim == 2) ct = f32_tensor({M, N}, c);
        tbn::Tensor r = tbn::gemm(at, bt, c_ndim ? &ct : nullptr, alpha, beta, transA != 0, transB != 0);
        std::memcpy(out, r.data(), static_cast<size_t>(M * N) * sizeof(float));
    });
}

// tbn::conv2d (conv2d.cpp:78-192); p = {sh, sw, ph, pw, dh, dw}.  out_dims receives {N, M, OH, OW}.
int ref_conv2d_f32(const float* x, int64_t N, int64_t C, int64_t H, int64_t W, const float* w,
                   int64_t M, int64_t kh, int64_t kw, const float* bias, const int64_t* p,
                   float* out, int64_t* out_dims) {
    return guarded([&] {
        tbn::Tensor xt = f32_tensor({N, C, H, W}, x);
        tbn::Tensor wt = f32_tensor({M, C, kh, kw}, w);
        tbn::Tensor bt;
        if (bias) bt = f32_tensor({M}, bias);
        tbn::Conv2DParams cp(kh, kw, p[0], p[1], p[2], p[3], p[4], p[5]);
        tbn::Tensor r = tbn::conv2d(xt, wt, bias ? &bt : nullptr, cp);
        for (int i = 0; i < 4; ++i) out_dims[i] = r.shape().dims[i];
        if (out) std::memcpy(out, r.data(), r.data_size());
    });
}

// tbn::impl::im2col (conv2d.cpp:420-507); out is [N*OH*OW, C*kh*kw].
int ref_im2col(const float* x, int64_t N, int64_t C, int64_t H, int64_t W, int64_t kh, int64_t kw,
               const int64_t* p, float* out) {
    return guarded([&] {
        tbn::Tensor xt = f32_tensor({N, C, H, W}, x);
        tbn::Tensor r = tbn::impl::im2col(xt, kh, kw, p[0], p[1], p[2], p[3], p[4], p[5]);
        std::memcpy(out, r.data(), r.data_size());
    });
}

// tbn::impl::im2col_ternary_packed (conv2d.cpp:511-601)
int ref_im2col_ternary_packed(const float* x, int64_t N, int64_t C, int64_t H, int64_t W, int64_t kh,
                              int64_t kw, const int64_t* p, uint32_t m_padded, uint32_t k_padded,
                              float lo, float hi, uint8_t* pos, uint8_t* neg) {
    return guarded([&] {
        auto m = tbn::impl::im2col_ternary_packed(x, N, C, H, W, kh, kw, p[0], p[1], p[2], p[3], p[4],
                                                  p[5], m_padded, k_padded, lo, hi);
        auto v = m.view();
        std::memcpy(pos, v.positive.data(), v.positive.size());
        std::memcpy(neg, v.negative.data(), v.negative.size());
    });
}

// tbn::maxpool2d / avgpool2d / global_avgpool2d (pooling.cpp:10-216); p = {kh, kw, sh, sw, ph, pw}.
// kind: 0 = max, 1 = avg, 2 = global avg, 3 = global max.
int ref_pool2d(int kind, const float* x, int64_t N, int64_t C, int64_t H, int64_t W, const int64_t* p,
               int ceil_mode, int count_include_pad, float* out, int64_t* out_dims) {
    return guarded([&] {
        tbn::Tensor xt = f32_tensor({N, C, H, W}, x);
        tbn::Tensor r;
        if (kind == 2) {
            r = tbn::global_avgpool2d(xt);
        } else if (kind == 3) {
            r = tbn::global_maxpool2d(xt);
        } else {
            tbn::Pool2DParams pp(p[0], p[1], p[2], p[3], p[4], p[5]);
            pp.ceil_mode = ceil_mode != 0;
            pp.count_include_pad = count_include_pad != 0;
            r = kind == 0 ? tbn::maxpool2d(xt, pp) : tbn::avgpool2d(xt, pp);
        }
        for (size_t i = 0; i < 4; ++i) out_dims[i] = i < r.shape().dims.size() ? r.shape().dims[i] : 1;
        if (out) std::memcpy(out, r.data(), r.data_size());
    });
}

// Runs a hand-built ModelGraph through tbn::TBNModel::Session (model.hpp:119-1316).
//
// `spec` is a line-oriented description (same grammar as the product's graph runner):
//   input  <name> <d0,d1,..>
//   output <name> <d0,d1,..>
//   value  <name> <d0,d1,..>                      (optional value_info for intermediates)
//   init   <name> f32|i64 <d0,d1,..> <offset>     (offset in 4-byte units into `blob` for f32,
//                                                  in 8-byte units into `iblob` for i64)
//   node   <op_type> <name> <in0,in1,..> <out0,..> [key=i:<int>|f:<float>|s:<str>|I:<i0,i1,..>]...
// One input tensor and one output tensor are exchanged as fp32.
int ref_session_run(const char* spec, const float* blob, const int64_t* iblob, const char* input_name,
                    const float* input, const char* output_name, float* output, int64_t output_elems,
                    int quantization, const uint32_t* tiling, int repeats) {
    return guarded([&] {
        auto graph = std::make_shared<tbn::ModelGraph>();
        std::istringstream lines(spec);
        std::string line;
        while (std::getline(lines, line)) {
            auto tok = split(line, ' ');
            if (tok.empty() || tok[0][0] == '#') continue;
            if (tok[0] == "input" || tok[0] == "output" || tok[0] == "value") {
                graph->value_info[tok[1]] = tbn::Shape(parse_ints(tok[2]));
                if (tok[0] == "input") graph->inputs.push_back(tok[1]);
                if (tok[0] == "output") graph->outputs.push_back(tok[1]);
            } else if (tok[0] == "init") {
                auto dims = parse_ints(tok[3]);
                const int64_t off = std::stoll(tok[4]);
                if (tok[2] == "f32") {
                    graph->initializers[tok[1]] = tbn::Tensor(tbn::Shape(dims), tbn::DataType::FLOAT32, blob + off);
                } else {
                    graph->initializers[tok[1]] = tbn::Tensor(tbn::Shape(dims), tbn::DataType::INT64, iblob + off);
                }
            } else if (tok[0] == "node") {
                tbn::ModelNode node;
                node.op_type = tok[1];
                node.name = tok[2];
                node.inputs = split(tok[3], ',');
                node.outputs = split(tok[4], ',');
                for (size_t i = 5; i < tok.size(); ++i) {
                    const auto eq = tok[i].find('=');
                    const std::string key = tok[i].substr(0, eq);
                    const char kind = tok[i][eq + 1];
                    const std::string val = tok[i].substr(eq + 3);
                    if (kind == 'i') node.attributes[key] = tbn::AttributeValue(static_cast<int64_t>(std::stoll(val)));
                    else if (kind == 'f') node.attributes[key] = tbn::AttributeValue(std::stof(val));
                    else if (kind == 's') node.attributes[key] = tbn::AttributeValue(val);
                    else if (kind == 'I') node.attributes[key] = tbn::AttributeValue(parse_ints(val));
                    else throw tbn::InvalidModelError("bad attribute kind in graph spec: " + tok[i]);
                }
                graph->nodes.push_back(std::move(node));
            } else {
                throw tbn::InvalidModelError("bad graph spec line: " + line);
            }
        }
        tbn::TBNModel model(graph);
        auto session = model.create_session(tiling_from(tiling));
        session.set_quantization(quantization != 0);
        tbn::Tensor in(graph->value_info.at(input_name), tbn::DataType::FLOAT32, input);
        session.set_input(input_name, in);
        for (int r = 0; r < (repeats < 1 ? 1 : repeats); ++r) session.run();
        tbn::Tensor out = session.get_output(output_name);
        if (out.num_elements() != output_elems) {
            throw tbn::InvalidShapeError("output element count mismatch");
        }
        std::memcpy(output, out.data(), static_cast<size_t>(output_elems) * sizeof(float));
    });
}

}  // extern "C"
