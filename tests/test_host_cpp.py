"""The C++ host layer (tbn:: API mirror in host/): builds with g++, exports the reference's entry points,
and -- on a GPU -- runs the benchmark graphs through tbn::TBNModel::Session with the same results as the
oracle (float x binary mode) and the stored reference outputs (TBN mode)."""
import os
import subprocess

import numpy as np
import pytest

from util import rel_l2


@pytest.fixture(scope="module")
def host():
    from fast_arm_tbcnn_b200 import host_build
    lib, driver = host_build.build()
    return lib, driver


def test_host_layer_builds_and_exports_reference_names(host):
    lib, driver = host
    out = subprocess.run(["nm", "-DC", lib], capture_output=True, text=True, check=True).stdout
    for name in ["tbn::qlinear_matmul_binary(", "tbn::quantize_to_binary(", "tbn::quantize_to_ternary(",
                 "tbn::conv2d_binary(", "tbn::conv2d_binary_with_scales(", "tbn::conv2d(", "tbn::gemm(",
                 "tbn::maxpool2d(", "tbn::avgpool2d(", "tbn::global_avgpool2d(", "tbn::global_maxpool2d(", "tbn::load_onnx_model(",
                 "tbn::load_onnx_model_from_buffer(", "tbn::load_model(", "tbn::load_model_from_buffer(", "tbn::get_version(",
                 "tbn::OnnxParser::parse_from_file(", "tbn::OnnxParser::parse_from_buffer(", "tbn::OnnxParser::get_graph(",
                 "tbn::TBNModel::Session::set_input(", "tbn::TBNModel::Session::run(",
                 "tbn::TBNModel::Session::get_output(", "tbn::Tensor::to_device(",
                 "tbn::qlinear_matmul_binary_blocked_packed(", "tbn::qlinear_matmul_binary_blocked_prepacked(",
                 "tbn::BinaryMatrix::pack(", "tbn::TernaryMatrix::pack_from_float(", "tbn::TernaryMatrix::pack(",
                 "tbn::PackedBinaryWeights::from_int8(", "tbn::ShardedGemm::ShardedGemm(", "tbn::ShardedGemm::connect(",
                 "tbn::ShardedGemm::multiply(", "tbn::ShardedGemm::export_result("]:
        assert name in out, name
    assert os.access(driver, os.X_OK)


def _run(driver, tmp_path, net, x, quant, out_shape, dequantised, repeat=1, extra=()):
    from oracle import graphs
    spec, blob, _ = graphs.to_spec(net, dequantised=dequantised)
    (tmp_path / "spec.txt").write_text(spec)
    blob.tofile(tmp_path / "blob.f32")
    np.ascontiguousarray(x, dtype=np.float32).tofile(tmp_path / "x.f32")
    out = tmp_path / f"out_{quant}.f32"
    proc = subprocess.run([driver, str(tmp_path / "spec.txt"), str(tmp_path / "blob.f32"), str(tmp_path / "x.f32"), "input",
                           "output", str(int(quant)), str(out), str(repeat)] + list(extra), capture_output=True, text=True)
    assert proc.returncode == 0, proc.stderr
    return np.fromfile(out, dtype=np.float32).reshape(out_shape)


@pytest.mark.gpu
def test_error_paths_throw_the_reference_exception_types(host):
    proc = subprocess.run([host[1], "--errors"], capture_output=True, text=True)
    assert proc.returncode == 0 and "errors ok" in proc.stdout, proc.stdout + proc.stderr


@pytest.mark.gpu
@pytest.mark.parametrize("dequantised", [False, True])
def test_lenet_through_cpp_session(host, oracle, golden, tmp_path, dequantised):
    """Raw fp32 weights declared binary (mark_binary) and a dequantised TBN model (+-alpha weights, detected)
    give the same float x binary result; TBN mode on the dequantised model is bit-equal to the reference."""
    from oracle import graphs
    net = graphs.lenet(batch=1, seed=1)
    x = golden["ref_outputs_small"]["lenet_x"]
    expect = graphs.run_float(net, x, oracle)
    got = _run(host[1], tmp_path, net, x, False, (1, 10), dequantised, repeat=2)
    assert rel_l2(got, expect) <= 1e-5
    assert got.argmax() == expect.argmax()
    if dequantised:
        got_q = _run(host[1], tmp_path, net, x, True, (1, 10), True)
        assert np.array_equal(got_q, golden["ref_outputs_small"]["lenet_tbn_session"])


@pytest.mark.gpu
def test_conv_layer_through_cpp_session(host, oracle, tmp_path):
    from oracle import graphs
    net = graphs.conv_layer(batch=3)
    x = np.random.default_rng(0).standard_normal((3, 64, 14, 14), dtype=np.float32)
    got = _run(host[1], tmp_path, net, x, False, (3, 128, 14, 14), True)
    assert rel_l2(got, graphs.run_float(net, x, oracle)) <= 1e-5
    got_q = _run(host[1], tmp_path, net, x, True, (3, 128, 14, 14), True)
    wq = graphs.dequantise(net["inits"]["w"])
    assert np.array_equal(got_q, oracle.conv2d_tbn_session(x, wq, net["inits"]["b"], (1, 1, 1, 1, 1, 1)))


@pytest.mark.gpu
def test_resnet18_through_cpp_session(host, oracle, tmp_path):
    """Float stem / shortcut convolutions / classifier on the float path, binary 3x3 convolutions on the packed
    path, all through tbn::TBNModel::Session."""
    from oracle import graphs
    net = graphs.resnet18(batch=1, seed=2, image=64, classes=100)
    x = np.random.default_rng(0).standard_normal((1, 3, 64, 64), dtype=np.float32)
    expect = graphs.run_float(net, x, oracle)
    for dequantised in (False, True):
        got = _run(host[1], tmp_path, net, x, False, (1, 100), dequantised)
        assert rel_l2(got, expect) <= 1e-5
        assert got.argmax() == expect.argmax()


def _run_onnx(driver, tmp_path, model_bytes, x, quant, out_shape, binary=""):
    (tmp_path / "model.onnx").write_bytes(model_bytes)
    np.ascontiguousarray(x, dtype=np.float32).tofile(tmp_path / "x.f32")
    out = tmp_path / f"onnx_out_{quant}.f32"
    cmd = [driver, "--onnx", str(tmp_path / "model.onnx"), str(tmp_path / "x.f32"), "input", "output", str(int(quant)), str(out)]
    proc = subprocess.run(cmd + ([binary] if binary else []), capture_output=True, text=True)
    assert proc.returncode == 0, proc.stderr
    return np.fromfile(out, dtype=np.float32).reshape(out_shape)


@pytest.mark.gpu
@pytest.mark.parametrize("storage", ["raw", "typed_fields"])
def test_exported_tbn_cnn_from_onnx_file(host, golden, tmp_path, storage):
    """load_model on an ONNX file of the exported MNIST TBN CNN (ternary-activation subgraph written as
    Greater / Cast / Less / Cast / Sub, Reshape, Gemm with transB = 1), then Session::run: float mode within
    1e-5 of the reference Session's stored output; quantised mode: the integer convolutions are bit-equal, the
    final transposed Gemm is the reference's float gemm, so 1e-5 there too, and the classes agree."""
    import onnx_schema
    from fast_arm_tbcnn_b200 import graphs
    net = graphs.exported_tbn_cnn(batch=2, seed=3)
    extra = {"float_data": ("conv1_w", "conv2_b", "thr_hi", "flat_shape")} if storage == "typed_fields" else {}
    model = onnx_schema.net_to_onnx(net, **extra)
    ref = golden["ref_outputs_exported_cnn"]
    got = _run_onnx(host[1], tmp_path, model, ref["x"], False, (2, 10))
    assert rel_l2(got, ref["float_session"]) <= 1e-5
    assert np.array_equal(got.argmax(axis=1), ref["float_session"].argmax(axis=1))
    got_q = _run_onnx(host[1], tmp_path, model, ref["x"], True, (2, 10))
    assert rel_l2(got_q, ref["tbn_session"]) <= 1e-5
    assert np.array_equal(got_q.argmax(axis=1), ref["tbn_session"].argmax(axis=1))


@pytest.mark.gpu
def test_lenet_from_onnx_file_matches_the_spec_path(host, oracle, golden, tmp_path):
    """The same LeNet through both loaders (ONNX file, text spec) gives identical bits; raw weights are declared
    binary by name on the command line."""
    import onnx_schema
    from oracle import graphs
    net = graphs.lenet(batch=1, seed=1)
    x = golden["ref_outputs_small"]["lenet_x"]
    via_spec = _run(host[1], tmp_path, net, x, False, (1, 10), False)
    via_onnx = _run_onnx(host[1], tmp_path, onnx_schema.net_to_onnx(net), x, False, (1, 10), binary=",".join(sorted(net["binary"])))
    assert np.array_equal(via_spec, via_onnx)
    assert rel_l2(via_onnx, graphs.run_float(net, x, oracle)) <= 1e-5


@pytest.mark.gpu
def test_cpp_session_graph_optimisations_change_no_bit(host, tmp_path):
    """Epilogue fusion, layer chaining and early release in tbn::TBNModel::Session (on by default) against the
    node-by-node execution: identical output bits on a ResNet-18 whose stages have 64..512 channels."""
    from oracle import graphs
    net = graphs.resnet18(batch=2, seed=2, image=64, classes=10)
    x = np.random.default_rng(3).standard_normal((2, 3, 64, 64), dtype=np.float32)
    fast = _run(host[1], tmp_path, net, x, False, (2, 10), False, repeat=2)
    plain = _run(host[1], tmp_path, net, x, False, (2, 10), False, repeat=2, extra=["noopt"])
    assert np.array_equal(fast, plain) and np.abs(fast).sum() > 0


@pytest.mark.gpu
def test_conv_output_that_is_also_a_graph_output(host, oracle, tmp_path):
    """Conv -> Relu where the convolution's own result is a graph output too: the Relu must not be folded into
    the convolution's epilogue (the pre-activation values would be lost); both outputs come back, from the C++
    Session and from the Python one."""
    from oracle import graphs
    from fast_arm_tbcnn_b200.session import Session
    net = graphs.conv_layer(batch=2)
    net["nodes"][0]["outputs"] = ["pre"]
    net["nodes"].append({"op": "Relu", "name": "act", "inputs": ["pre"], "outputs": ["output"], "attrs": {}})
    net["outputs"] = {"pre": (2, 128, 14, 14), "output": (2, 128, 14, 14)}
    x = np.random.default_rng(4).standard_normal((2, 64, 14, 14), dtype=np.float32)
    keep = {}
    expect_out = graphs.run_float(net, x, oracle, keep=keep)
    from oracle import graphs as og
    spec, blob, _ = og.to_spec(net, dequantised=True)
    (tmp_path / "spec.txt").write_text(spec)
    blob.tofile(tmp_path / "blob.f32")
    x.tofile(tmp_path / "x.f32")
    for name, expect in (("pre", keep["pre"]), ("output", keep["output"])):
        out = tmp_path / f"{name}.f32"
        proc = subprocess.run([host[1], str(tmp_path / "spec.txt"), str(tmp_path / "blob.f32"), str(tmp_path / "x.f32"),
                               "input", name, "0", str(out)], capture_output=True, text=True)
        assert proc.returncode == 0, proc.stderr
        assert rel_l2(np.fromfile(out, dtype=np.float32).reshape(expect.shape), expect) <= 1e-5
    sess = Session(net)
    sess.set_input("input", x)
    sess.run()
    assert rel_l2(sess.get_output("pre").cpu().numpy(), keep["pre"]) <= 1e-5
    assert rel_l2(sess.get_output("output").cpu().numpy(), keep["output"]) <= 1e-5
    assert float(sess.get_output("pre").min()) < 0.0   # really the pre-activation values


def test_packed_matrix_types_layout_known_answers(host):
    """BinaryMatrix / TernaryMatrix / PackedBinaryWeights of the C++ layer (host types, no GPU needed): the layout
    known-answer vectors the oracle is pinned on, and the reference's std::invalid_argument checks."""
    proc = subprocess.run([host[1], "--packed-layout"], capture_output=True, text=True)
    assert proc.returncode == 0 and "packed layout ok" in proc.stdout, proc.stdout + proc.stderr


@pytest.mark.gpu
def test_operators_on_prepacked_operands(host):
    """qlinear_matmul_binary_blocked_packed / _blocked_prepacked == qlinear_matmul_binary (itself bit-equal to the
    oracle) on the same operands, including weights padded to 64 instead of 128 rows."""
    proc = subprocess.run([host[1], "--prepacked"], capture_output=True, text=True)
    assert proc.returncode == 0 and "prepacked ok" in proc.stdout, proc.stdout + proc.stderr


@pytest.mark.gpu
def test_cpp_sharded_gemm_two_processes(host, tmp_path):
    """tbn::ShardedGemm with one process per GPU: handles exchanged through files, each rank's fused kernel stores
    its column slab into both result matrices (its own and, over NVLink, the peer's); every rank's C must equal
    the single-GPU product bit for bit.  Needs two GPUs (skipped on a one-GPU box); with world size 1 the same
    driver checks the single-rank path."""
    import torch
    from fast_arm_tbcnn_b200 import host_build
    world = 2 if torch.cuda.device_count() >= 2 else 1
    procs = []
    for rank in range(world):
        env = dict(os.environ, TBN_DEVICE=str(rank))
        procs.append(subprocess.Popen([host_build.SHARDED_GEMM, str(rank), str(world), str(tmp_path), "300", "640", "512"],
                                      stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, env=env))
    for rank, p in enumerate(procs):
        out, err = p.communicate(timeout=180)
        assert p.returncode == 0 and "sharded gemm ok" in out, (rank, out, err)
