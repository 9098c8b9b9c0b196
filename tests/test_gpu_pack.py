"""Parity of the CUDA quantise-and-pack kernels with the oracle (bit-exact), through the C ABI."""
import numpy as np
import pytest

from util import pack_plane, special_weights, u32

pytestmark = pytest.mark.gpu

# The reference sums |w| sequentially in fp32 (model.hpp:388-394), which itself carries a rounding
# error of about sqrt(K) * 2^-24; the kernel sums 128-row chunks, so the two agree to that level.
ALPHA_RTOL = 1e-5

# The last three are large enough (K*N >= 2^22) for the TMA-streamed kernel: ragged K, N off the 512-column
# job width, and an exact multiple.
SHAPES = [(64, 8), (128, 8), (200, 37), (576, 128), (1, 1), (129, 9), (1000, 300), (4608, 512),
          (2500, 1700), (2049, 2052), (4096, 1024)]


@pytest.fixture(scope="module")
def tbn():
    import torch
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    from fast_arm_tbcnn_b200 import capi
    capi.lib.init()
    return capi


@pytest.mark.parametrize("K,N", SHAPES)
@pytest.mark.parametrize("ge", [False, True])
def test_binary_pack_kn(tbn, oracle, K, N, ge):
    import torch
    rng = np.random.default_rng(K * 7 + N)
    w = special_weights(rng, K, N)
    words, alpha = tbn.lib.quant_pack_binary(torch.from_numpy(w).cuda(), tbn.LAYOUT_KN, 0.0, ge)
    tbn.lib.sync()
    if ge:
        expect = pack_plane(oracle.sign_ge0(w) == -1)
    else:
        expect = oracle.binary_pack_padded(oracle.quantize_to_binary(w, 0.0))
        assert np.array_equal(expect, pack_plane(~(w > 0)))
    assert np.array_equal(u32(words), expect)
    finite = np.where(np.isfinite(w), w, 0).astype(np.float32)
    ref_alpha = oracle.column_abs_mean(finite)
    cols = np.all(np.isfinite(w), axis=0)
    np.testing.assert_allclose(alpha.cpu().numpy()[cols], ref_alpha[cols], rtol=ALPHA_RTOL, atol=0)


@pytest.mark.parametrize("K,N", SHAPES)
def test_binary_pack_nk_conv_layout(tbn, oracle, K, N):
    """Conv weights [M_out, C*kh*kw]: the Session transposes to [K, M_out] before packing
    (model.hpp:464-472); the NK layout packs the same words without the transpose."""
    import torch
    rng = np.random.default_rng(K * 3 + N)
    w_nk = np.ascontiguousarray(special_weights(rng, K, N).T)
    words, alpha = tbn.lib.quant_pack_binary(torch.from_numpy(w_nk).cuda(), tbn.LAYOUT_NK, 0.0, True)
    tbn.lib.sync()
    assert np.array_equal(u32(words), pack_plane((oracle.sign_ge0(w_nk) == -1).T))
    rows = np.all(np.isfinite(w_nk), axis=1)
    np.testing.assert_allclose(alpha.cpu().numpy()[rows], oracle.channel_abs_mean(w_nk)[rows], rtol=ALPHA_RTOL)


def test_binary_pack_threshold_and_stride(tbn, oracle):
    import torch
    rng = np.random.default_rng(9)
    big = rng.standard_normal((130, 96), dtype=np.float32)
    view = torch.from_numpy(big).cuda()[:, :50]  # row stride 96, 50 used columns
    words, _ = tbn.lib.quant_pack_binary(view, tbn.LAYOUT_KN, 0.25, False, want_alpha=False)
    tbn.lib.sync()
    assert np.array_equal(u32(words), oracle.binary_pack_padded(oracle.quantize_to_binary(big[:, :50], 0.25)))


def test_layout_known_answers_on_device(tbn, golden):
    import torch
    k = golden["layout_kats"]
    w = k["bin_in"].astype(np.float32)
    words, _ = tbn.lib.quant_pack_binary(torch.from_numpy(w).cuda(), want_alpha=False)
    tbn.lib.sync()
    assert np.array_equal(u32(words).reshape(-1), k["bin_words"])
    t = k["tern_in"].astype(np.float32).reshape(1, 16)
    codes, _, _, _ = tbn.lib.quant_pack_ternary(torch.from_numpy(t).cuda(), -0.5, 0.5, want_alpha=False)
    tbn.lib.sync()
    assert u32(codes)[0] == 0x00AA05A4


@pytest.mark.parametrize("K,N", SHAPES)
@pytest.mark.parametrize("layout", ["kn", "nk"])
def test_ternary_pack(tbn, oracle, K, N, layout):
    import torch
    rng = np.random.default_rng(K + 31 * N)
    w = special_weights(rng, K, N)
    delta = np.float32(0.7) * np.float32(np.nanmean(np.abs(np.where(np.isfinite(w), w, 0))))
    lo, hi = float(-delta), float(delta)
    src = w if layout == "kn" else np.ascontiguousarray(w.T)
    codes, pos, neg, alpha = tbn.lib.quant_pack_ternary(torch.from_numpy(src).cuda(), lo, hi,
                                                       tbn.LAYOUT_KN if layout == "kn" else tbn.LAYOUT_NK)
    tbn.lib.sync()
    t = oracle.quantize_to_ternary(w, lo, hi)
    assert np.array_equal(u32(codes).view(np.uint8)[: (K * N + 3) // 4], oracle.ternary_codes(t))
    assert np.array_equal(u32(pos), pack_plane(t == 1))
    assert np.array_equal(u32(neg), pack_plane(t == -1))
    cols = np.all(np.isfinite(w), axis=0)
    ref_alpha = oracle.column_abs_mean_nonzero(np.where(np.isfinite(w), w, 0).astype(np.float32), lo, hi)
    np.testing.assert_allclose(alpha.cpu().numpy()[cols], ref_alpha[cols], rtol=ALPHA_RTOL)


def test_quantize_byte_tensors(tbn, oracle):
    import torch
    rng = np.random.default_rng(4)
    w = special_weights(rng, 333, 17)
    d = torch.from_numpy(w).cuda()
    for thr in (0.0, -0.3):
        assert np.array_equal(tbn.lib.quantize_to_binary(d, thr).cpu().numpy(), oracle.quantize_to_binary(w, thr))
    for lo, hi in ((-0.1, 0.1), (-0.5, 0.7)):
        assert np.array_equal(tbn.lib.quantize_to_ternary(d, lo, hi).cpu().numpy(), oracle.quantize_to_ternary(w, lo, hi))
    assert tbn.lib.quantize_to_binary(torch.empty(0, device="cuda")).numel() == 0


def _popcount(words):
    import torch
    pop = 0
    for chunk in words.view(torch.uint8).reshape(-1).split(1 << 26):
        x = chunk.to(torch.int32)
        x = x - ((x >> 1) & 0x55)
        x = (x & 0x33) + ((x >> 2) & 0x33)
        pop += int(((x + (x >> 4)) & 0x0F).sum())
    return pop


def test_pack_full_size_properties(tbn):
    """16384 x 16384 (the benchmark size): checked through properties that need no CPU pass over
    the matrix -- the number of set bits equals the number of non-positive weights, and packing -W
    sets exactly the complementary bits (exact zeros are -1 under both signs)."""
    import torch
    g = torch.Generator(device="cuda").manual_seed(1)
    K = N = 16384
    w = torch.randn((K, N), generator=g, device="cuda")
    words, alpha = tbn.lib.quant_pack_binary(w)
    words_neg, _ = tbn.lib.quant_pack_binary(-w, want_alpha=False)
    tbn.lib.sync()
    zeros = int((w == 0).sum())
    assert _popcount(words) == int((w <= 0).sum())
    assert _popcount(words_neg) == int((w >= 0).sum())
    assert _popcount(words & words_neg) == zeros
    assert _popcount(~(words | words_neg)) == 0
    torch.testing.assert_close(alpha, w.abs().mean(dim=0), rtol=1e-5, atol=0)
