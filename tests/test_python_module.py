"""The `_tbn` Python module (pybind11 over the GPU Session): same surface as the reference's module
(tbn-runtime/python/bindings.cpp:53-168) — Shape, Model(path, tiling...).run / run_quantized / input_names /
output_names / input_shape, load_model."""
import os
import sys

import numpy as np
import pytest

from util import rel_l2

import onnx_schema


@pytest.fixture(scope="module")
def tbn_module():
    from fast_arm_tbcnn_b200 import host_build
    host_build.build()
    sys.path.insert(0, os.path.dirname(host_build.PY_MODULE))
    import _tbn
    return _tbn


@pytest.fixture()
def exported_model(tmp_path):
    from fast_arm_tbcnn_b200 import graphs
    path = tmp_path / "exported.onnx"
    path.write_bytes(onnx_schema.net_to_onnx(graphs.exported_tbn_cnn(batch=2, seed=3)))
    return str(path)


def test_module_surface_and_loading(tbn_module, exported_model):
    m = tbn_module
    assert m.get_version() == "0.1.0"
    assert repr(m.Shape([1, 2, 3])) == "Shape([1, 2, 3])" and m.Shape([4]).dims == [4]
    model = m.Model(exported_model, mblk=64, nblk=64, kblk=128, mmk=16, nmk=8)
    assert model.input_names() == ["input"] and model.output_names() == ["output"]
    assert model.input_shape("input").dims == [2, 1, 28, 28]
    assert model.producer() == "recipe-writer 1.0"
    with pytest.raises(RuntimeError):
        model.input_shape("nope")
    with pytest.raises(m.TBNError, match="Failed to open ONNX file"):
        m.load_model("missing.onnx")
    assert m.load_model(exported_model).output_names() == ["output"]


@pytest.mark.gpu
def test_model_run_matches_the_reference_session(tbn_module, exported_model, golden):
    ref = golden["ref_outputs_exported_cnn"]
    model = tbn_module.Model(exported_model)
    out = model.run(ref["x"])
    assert out.dtype == np.float32 and out.shape == (2, 10)
    assert rel_l2(out, ref["float_session"]) <= 1e-5
    out_q = model.run_quantized(ref["x"])
    assert rel_l2(out_q, ref["tbn_session"]) <= 1e-5
    assert np.array_equal(out_q, model.run(ref["x"], use_quantization=True))
    assert np.array_equal(out, model.run(ref["x"].astype(np.float64)))     # cast like py::array_t<float>
    # a batch that is a multiple of the model's: slices are run one after the other
    big = np.concatenate([ref["x"], ref["x"][::-1], ref["x"]], axis=0)
    out_big = model.run(big)
    assert out_big.shape == (6, 10)
    assert np.array_equal(out_big[:2], out) and np.array_equal(out_big[4:], out) and np.array_equal(out_big[2:4], out[::-1])
    with pytest.raises(tbn_module.TBNError, match="shape mismatch"):
        model.run(np.zeros((3, 1, 28, 28), dtype=np.float32))
