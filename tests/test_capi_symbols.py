"""The C-ABI library loads without a GPU and exports every symbol the header declares."""
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "tbn_cuda.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(tbn_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported_and_bound():
    from fast_arm_tbcnn_b200 import capi
    handle = capi.load()
    names = declared_symbols()
    assert len(names) >= 15
    for name in names:
        assert hasattr(handle, name), f"{name} declared in include/tbn_cuda.h but not exported"
        assert name in capi.SIGNATURES, f"{name} has no ctypes signature"
    assert sorted(capi.SIGNATURES) == names


def test_no_cpu_fallback_without_device():
    """Without a CUDA device the library refuses to initialise instead of computing on the host."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    from fast_arm_tbcnn_b200 import capi
    handle = capi.load()
    status = handle.tbn_cuda_init(0)
    assert status == -8  # DEVICE_NOT_SUPPORTED
    assert "no CPU fallback" in capi.last_error()


def test_pure_host_helpers():
    import ctypes as C
    from fast_arm_tbcnn_b200 import capi
    handle = capi.load()
    kp, np_ = C.c_int64(), C.c_int64()
    assert handle.tbn_packed_dims(576, 6, C.byref(kp), C.byref(np_)) == 0
    assert (kp.value, np_.value) == (640, 8)
    assert handle.tbn_packed_dims(-1, 6, C.byref(kp), C.byref(np_)) == -1
    assert handle.tbn_gemm_workspace_bytes(100, 70, capi.MODE_TC_BF16X2) == 2 * 128 * 128 * 2 + 160 * 128 * 256 * 4 + 256
    assert handle.tbn_gemm_workspace_bytes(100, 70, capi.MODE_SIMT) == 0
    assert handle.tbn_quant_pack_workspace_bytes(200, 37, 0) == 2 * 37 * 4
    assert handle.tbn_quant_pack_workspace_bytes(200, 37, 1) == 2 * 2 * 37 * 4


def test_gemm_plan_table_choices():
    """The compiled-in per-shape table (host code, no GPU): the benchmark shapes get the tensor-core kernel with
    the column tile the sweep and the wave model give, tiny products the CUDA-core kernel, and an override is
    reported back and can be cleared."""
    from fast_arm_tbcnn_b200 import capi
    L = capi.lib
    capi.load()
    assert L.gemm_plan(16384, 16384, 16384)["kernel"] == "tcgen05" and L.gemm_plan(16384, 16384, 16384)["bn"] == 256
    assert L.gemm_plan(4096, 11008, 4096)["bn"] == 256
    assert L.gemm_plan(4096, 4096, 4096) == dict(L.gemm_plan(4096, 4096, 4096), kernel="tcgen05", bn=256, fused_split=False)
    assert L.gemm_plan(3136, 512, 2304)["bn"] == 128      # 25 x 2 tiles of 256 would leave two thirds of the SMs idle
    assert L.gemm_plan(8, 4096, 4096)["bn"] == 64
    assert L.gemm_plan(1, 10, 256)["kernel"] == "cuda-core"
    assert L.gemm_plan(200704, 64, 576)["fused_split"] is True
    assert L.gemm_plan(16384, 16384, 16384)["fused_split"] is False
    try:
        L.gemm_plan_override(kernel=1, bn=64, group_m=7, fused_split=0)
        assert L.gemm_plan(16384, 16384, 16384) == {"kernel": "cuda-core", "bn": 64, "group_m": 7, "fused_split": False}
    finally:
        L.gemm_plan_override()
    assert L.gemm_plan(16384, 16384, 16384)["kernel"] == "tcgen05"
    import pytest
    with pytest.raises(capi.TbnError):
        L.gemm_plan_override(bn=100)
    assert L.wave_model_bn(8192, 256, 256) == 128 and L.wave_model_bn(16384, 16384, 256) == 256
