"""The ONNX reader of the C++ host layer (load_onnx_model / load_model / OnnxParser) on CPU: its graph equals
what google.protobuf reads from the same bytes under the reference's conversion rules
(tbn-runtime/src/onnx_integration/onnx_parser.cpp), for files written here and — where the reference tree is
present — for every .onnx fixture the reference ships."""
import glob
import os
import subprocess

import numpy as np
import pytest

from fast_arm_tbcnn_b200 import graphs, host_build

import onnx_schema

from oracle import cpu_oracle

REFERENCE_TREE = cpu_oracle.reference_tree()


@pytest.fixture(scope="module")
def run_graph():
    _, exe = host_build.build()
    return exe


def dump(run_graph, path):
    proc = subprocess.run([run_graph, "--dump-onnx", str(path)], capture_output=True, text=True)
    assert proc.returncode == 0, proc.stderr
    return proc.stdout


VARIANTS = {
    "raw": {},
    "typed_fields": {"float_data": ("conv1_w", "fc_b", "flat_shape", "thr_hi")},
    "external_and_dynamic": {"external": ("conv2_w", "fc_w"), "dynamic_batch": True},
    "unnamed_nodes_extra_attributes": {
        "unnamed_nodes": True,
        "extra_attrs": {"conv1": {"scales": [0.5, 1.25, -3.0], "tags": ["a", "bc"], "probe": np.arange(6, dtype=np.float32).reshape(2, 3)},
                        "fc": {"alpha": 0.75}}},
}


@pytest.mark.parametrize("variant", sorted(VARIANTS))
def test_written_models_round_trip(run_graph, tmp_path, variant):
    net = graphs.exported_tbn_cnn(batch=2, seed=4)
    data = onnx_schema.net_to_onnx(net, **VARIANTS[variant])
    path = tmp_path / "model.onnx"
    path.write_bytes(data)
    text = dump(run_graph, path)
    assert text == onnx_schema.canonical_dump(data)
    if variant == "external_and_dynamic":
        assert "input input 1,1,28,28" in text           # symbolic batch -> 1
        zero32 = onnx_schema._fnv1a(bytes(32 * 16 * 5 * 5 * 4))
        assert f"init conv2_w dtype=0 dims=32,16,5,5 bytes=51200 fnv={zero32:016x}" in text  # external data stays zero
    if variant == "unnamed_nodes_extra_attributes":
        assert "node Conv Conv_c1 " in text               # op_type + "_" + first output


def test_lenet_and_resnet_recipes_round_trip(run_graph, tmp_path):
    for name, net in (("lenet", graphs.lenet(batch=1)), ("resnet", graphs.resnet18(batch=1, image=32, classes=10, width=8))):
        data = onnx_schema.net_to_onnx(net)
        path = tmp_path / (name + ".onnx")
        path.write_bytes(data)
        assert dump(run_graph, path) == onnx_schema.canonical_dump(data)


def test_loader_errors(run_graph, tmp_path):
    proc = subprocess.run([run_graph, "--dump-onnx", str(tmp_path / "missing.onnx")], capture_output=True, text=True)
    assert proc.returncode == 1 and "Failed to open ONNX file" in proc.stderr and "TBNError -4" in proc.stderr
    data = onnx_schema.net_to_onnx(graphs.lenet(batch=1))
    for label, blob in (("truncated", data[: len(data) // 2 + 3]), ("garbage", bytes(range(255, 0, -1)) * 8),
                        ("length past end", b"\x3a\xff\xff\x03abc")):
        path = tmp_path / "bad.onnx"
        path.write_bytes(blob)
        proc = subprocess.run([run_graph, "--dump-onnx", str(path)], capture_output=True, text=True)
        assert proc.returncode == 1 and "Failed to parse ONNX model" in proc.stderr, (label, proc.stdout[:200], proc.stderr)


@pytest.mark.skipif(not os.path.isdir(REFERENCE_TREE), reason="reference tree not present on this machine")
def test_reference_fixtures_load_identically(run_graph):
    files = sorted(glob.glob(os.path.join(REFERENCE_TREE, "tests", "**", "*.onnx"), recursive=True))
    assert len(files) >= 10
    for path in files:
        expect = onnx_schema.canonical_dump(open(path, "rb").read())
        assert dump(run_graph, path) == expect, path
    # Facts about those files the reference's own tests rely on: the exported CNN has 12 nodes with
    # transB = 1 on every Gemm, and the trained MNIST model carries the ternary-activation subgraph.
    cnn = dump(run_graph, os.path.join(REFERENCE_TREE, "tests/models/cnn/onnx/simple_cnn.onnx"))
    assert cnn.count("\nnode ") == 12 and cnn.count("transB=i:1") == 3
    mnist = dump(run_graph, os.path.join(REFERENCE_TREE, "tests/train/mnist/mnist_tbn.onnx"))
    assert [l.split()[1] for l in mnist.splitlines() if l.startswith("node ")] == [
        "Conv", "Relu", "MaxPool", "Conv", "Greater", "Cast", "Less", "Cast", "Sub", "MaxPool", "Reshape", "Gemm"]
