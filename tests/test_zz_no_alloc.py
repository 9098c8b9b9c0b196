"""The entry point that allocates nothing (tbn_quant_pack_binary_noalloc) against the regular one.

For hosts that budget all GPU memory at start-up and cannot call cudaMalloc on the request path:
the scratch for the per-column scales comes from an array built into the library.  Collected last
on purpose (file name), so a run that stops at the first failure has already run everything else;
it must also pass alone in a fresh process.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def tbn():
    import torch
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    from fast_arm_tbcnn_b200 import capi
    capi.lib.init()
    return capi


def _both(tbn, w, layout, ge):
    import torch
    K, N = (w.shape if layout == tbn.LAYOUT_KN else (w.shape[1], w.shape[0]))
    Kp, Np = tbn.lib.packed_dims(K, N)
    ref_words, ref_alpha = tbn.lib.quant_pack_binary(w, layout, 0.0, ge)
    words = torch.full((Np, Kp // 32), 0x5A5A5A5A, dtype=torch.int32, device=w.device)
    alpha = torch.full((N,), -1.0, dtype=torch.float32, device=w.device)
    tbn.lib.quant_pack_binary_noalloc(w, words, alpha, layout, 0.0, ge)
    tbn.lib.sync()
    return ref_words, ref_alpha, words, alpha


def test_two_calls_in_a_row_match_the_regular_entry_point(tbn):
    import torch
    g = torch.Generator(device="cuda").manual_seed(11)
    # First call: large enough to fill a good part of the built-in scratch (64 chunks x 4096 columns).
    w1 = torch.randn((8192, 4096), generator=g, device="cuda")
    r_words, r_alpha, words, alpha = _both(tbn, w1, tbn.LAYOUT_KN, False)
    assert torch.equal(words, r_words)
    torch.testing.assert_close(alpha, r_alpha, rtol=1e-5, atol=0)
    # Second call right after it, other shape, layout and sign rule: whatever the first call left in
    # the shared scratch must not leak into this result.
    w2 = torch.randn((300, 1000), generator=g, device="cuda") * 3.0
    r_words, r_alpha, words, alpha = _both(tbn, w2, tbn.LAYOUT_NK, True)
    assert torch.equal(words, r_words)
    torch.testing.assert_close(alpha, r_alpha, rtol=1e-5, atol=0)
    # ... and against an independent evaluation of the scale.
    torch.testing.assert_close(alpha, w2.abs().mean(dim=1), rtol=1e-5, atol=0)


def test_alpha_is_optional(tbn):
    import torch
    w = torch.randn((129, 9), device="cuda")
    Kp, Np = tbn.lib.packed_dims(129, 9)
    words = torch.zeros((Np, Kp // 32), dtype=torch.int32, device="cuda")
    tbn.lib.quant_pack_binary_noalloc(w, words, None)
    tbn.lib.sync()
    expect, _ = tbn.lib.quant_pack_binary(w, want_alpha=False)
    tbn.lib.sync()
    assert torch.equal(words, expect)


def test_sizes_beyond_the_built_in_scratch_are_refused(tbn):
    import torch
    K, N = 16384, 16384  # 128 chunks x 16384 columns = 2 Mi partial sums > 1 Mi
    w = torch.zeros((8, 8), device="cuda")  # never read: the call is refused on its sizes alone
    words = torch.zeros((8, 8), dtype=torch.int32, device="cuda")
    alpha = torch.zeros(8, device="cuda")
    status = tbn.lib.h.tbn_quant_pack_binary_noalloc(w.data_ptr(), K, N, N, tbn.LAYOUT_KN, 0.0, 0, words.data_ptr(),
                                                     alpha.data_ptr(), None)
    assert status == -1
    assert "exceeds the built-in scratch" in tbn.last_error() and str(128 * 16384) in tbn.last_error()


def test_words_match_the_oracle_and_device_memory_is_untouched(tbn, oracle):
    """The packed words against the CPU oracle (not only against the regular entry point), and -- after one
    warm-up call has loaded the kernels -- the free device memory reported by the driver is the same before
    and after a call: nothing was allocated or freed."""
    import torch
    from util import u32
    rng = np.random.default_rng(21)
    W = rng.standard_normal((1000, 520), dtype=np.float32)
    w = torch.from_numpy(W).cuda()
    Kp, Np = tbn.lib.packed_dims(1000, 520)
    words = torch.zeros((Np, Kp // 32), dtype=torch.int32, device="cuda")
    alpha = torch.zeros(520, dtype=torch.float32, device="cuda")
    tbn.lib.quant_pack_binary_noalloc(w, words, alpha)      # warm-up: loads this shape class's kernels
    tbn.lib.sync()
    words.zero_()
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    tbn.lib.quant_pack_binary_noalloc(w, words, alpha)
    tbn.lib.sync()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before
    assert np.array_equal(u32(words), oracle.binary_pack_padded(oracle.quantize_to_binary(W)))
    np.testing.assert_allclose(alpha.cpu().numpy(), oracle.column_abs_mean(W), rtol=1e-5)
