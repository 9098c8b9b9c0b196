"""Parity of the implicit-GEMM convolution, the glue operators and the device Session with the oracle."""
import numpy as np
import pytest

from util import rel_l2

pytestmark = pytest.mark.gpu

TOL_FP32 = 1e-5


@pytest.fixture(scope="module")
def tbn():
    import torch
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    from fast_arm_tbcnn_b200 import capi
    capi.lib.init()
    return capi


# (N, C, H, W, M_out, kh, kw, (sh, sw, ph, pw, dh, dw))
CONV_CASES = [
    (1, 64, 14, 14, 128, 3, 3, (1, 1, 1, 1, 1, 1)),   # the benchmark layer
    (2, 3, 13, 12, 5, 3, 3, (1, 1, 1, 1, 1, 1)),
    (2, 3, 13, 12, 5, 3, 3, (2, 2, 3, 3, 1, 1)),
    (2, 3, 13, 12, 5, 3, 3, (1, 2, 0, 1, 2, 1)),
    (1, 1, 28, 28, 6, 5, 5, (1, 1, 0, 0, 1, 1)),       # LeNet conv1
    (3, 6, 12, 12, 16, 5, 5, (1, 1, 0, 0, 1, 1)),      # LeNet conv2
    (5, 16, 9, 9, 40, 1, 1, (1, 1, 0, 0, 1, 1)),
    (2, 3, 32, 32, 64, 7, 7, (2, 2, 3, 3, 1, 1)),
    (33, 8, 7, 5, 24, 3, 3, (1, 1, 1, 1, 1, 1)),
    (2, 512, 4, 4, 300, 3, 3, (1, 1, 1, 1, 1, 1)),     # K = 4608: three accumulation segments
    # stride 2 over <= 4 channels: the space-to-depth (folded) path of the image stems
    (2, 3, 20, 20, 8, 7, 7, (2, 2, 3, 3, 1, 1)),
    (1, 1, 13, 17, 4, 5, 5, (2, 2, 2, 2, 1, 1)),
    (3, 4, 9, 8, 3, 3, 3, (2, 2, 1, 1, 1, 1)),
    (2, 2, 12, 12, 3, 2, 2, (2, 2, 0, 0, 1, 1)),
    (1, 3, 31, 40, 4, 7, 5, (2, 2, 0, 1, 1, 1)),
    (130, 3, 6, 6, 2, 3, 3, (2, 2, 1, 1, 1, 1)),
    (4, 3, 64, 64, 64, 7, 7, (2, 2, 3, 3, 1, 1)),
    (1, 3, 8, 8, 4, 3, 3, (2, 2, 40, 40, 1, 1)),        # pads far beyond the image
]


def _conv_inputs(case, seed=0):
    N, C, H, W, M, kh, kw, p = case
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((N, C, H, W), dtype=np.float32)
    w = (rng.standard_normal((M, C, kh, kw), dtype=np.float32) * np.float32(0.05)).astype(np.float32)
    b = (rng.standard_normal(M, dtype=np.float32) * np.float32(0.05)).astype(np.float32)
    return x, w, b, p


@pytest.mark.parametrize("case", CONV_CASES)
@pytest.mark.parametrize("mode", ["x2", "x1"])
def test_conv_fxb_vs_float_conv(tbn, oracle, case, mode):
    import torch
    from oracle import graphs
    x, w, b, p = _conv_inputs(case)
    dw = torch.from_numpy(w).cuda()
    words, alpha = tbn.lib.quant_pack_binary(dw.reshape(w.shape[0], -1), tbn.LAYOUT_NK)
    m = tbn.MODE_TC_BF16X2 if mode == "x2" else tbn.MODE_TC_BF16X1
    y = tbn.lib.conv2d_fxb(torch.from_numpy(x).cuda(), words, w.shape, p, alpha=alpha, bias=torch.from_numpy(b).cuda(),
                           mode=m)
    tbn.lib.sync()
    expect = oracle.conv2d_f32(x, graphs.dequantise(w), b, p)
    assert tuple(y.shape) == expect.shape
    err = rel_l2(y.cpu().numpy(), expect)
    assert err <= (TOL_FP32 if mode == "x2" else 2.5e-3), err


@pytest.mark.parametrize("case", CONV_CASES)
def test_conv_tbn_bit_exact(tbn, oracle, case):
    """Ternarised activations x binary weights, (acc + bias) * alpha: the Session's cached conv path."""
    import torch
    from oracle import graphs
    x, w, b, p = _conv_inputs(case, seed=3)
    x.reshape(-1)[:4] = [0.1, -0.1, 0.100001, -0.100001]
    wq = graphs.dequantise(w)  # what the reference sees: alpha * sign(w)
    dwq = torch.from_numpy(wq).cuda()
    words, _ = tbn.lib.quant_pack_binary(dwq.reshape(w.shape[0], -1), tbn.LAYOUT_NK, 0.0, True, want_alpha=False)
    alpha = tbn.lib.channel_abs_mean(dwq)
    y = tbn.lib.conv2d_tbn(torch.from_numpy(x).cuda(), words, w.shape, p, alpha=alpha, bias=torch.from_numpy(b).cuda(),
                           epilogue=tbn.EPI_BIAS_BEFORE_ALPHA)
    tbn.lib.sync()
    assert np.array_equal(alpha.cpu().numpy(), oracle.channel_abs_mean(wq))
    assert np.array_equal(y.cpu().numpy(), oracle.conv2d_tbn_session(x, wq, b, p))


# Channel counts that are multiples of 64: the channels-last fast path (tap-major weights).
FAST_CASES = [
    (1, 64, 14, 14, 128, 3, 3, (1, 1, 1, 1, 1, 1)),
    (3, 64, 9, 11, 40, 3, 3, (2, 2, 1, 1, 1, 1)),
    (2, 128, 8, 8, 64, 1, 1, (2, 2, 0, 0, 1, 1)),
    (2, 64, 12, 10, 70, 3, 2, (1, 1, 2, 1, 2, 1)),
    (2, 512, 4, 4, 300, 3, 3, (1, 1, 1, 1, 1, 1)),
    (70, 64, 7, 7, 64, 3, 3, (1, 1, 1, 1, 1, 1)),
    (5, 64, 7, 7, 64, 3, 3, (1, 1, 1, 1, 1, 1)),        # several whole images per tile, last tile partly empty
    (2, 64, 56, 56, 64, 3, 3, (1, 1, 1, 1, 1, 1)),      # two output rows per tile
    (1, 64, 150, 9, 16, 3, 3, (1, 1, 1, 1, 1, 1)),      # rows shorter than a tile, several rows per tile
    (1, 64, 5, 300, 16, 1, 3, (1, 2, 0, 1, 1, 1)),      # output rows longer than one tile
    (2, 128, 28, 28, 64, 1, 1, (2, 2, 0, 0, 1, 1)),     # strided 1x1 (the shortcut convolutions)
    (2, 64, 40, 40, 8, 3, 3, (9, 9, 1, 1, 1, 1)),       # stride beyond the TMA element-stride range: cp.async path
    # tiles of whole output rows that run on into the next image (one TMA box per image a tile touches)
    (5, 64, 14, 14, 256, 3, 3, (1, 1, 1, 1, 1, 1)),     # nine rows per tile, 14 per image
    (3, 64, 28, 28, 256, 3, 3, (2, 2, 1, 1, 1, 1)),     # the same with stride 2
    (9, 128, 7, 7, 256, 3, 3, (1, 1, 1, 1, 1, 1)),      # eighteen rows per tile: up to four images in one tile
    (5, 64, 14, 14, 128, 3, 3, (1, 1, 1, 1, 1, 1)),     # row mode: eight rows per tile running on into the next image
    (3, 64, 10, 28, 64, 3, 3, (1, 1, 1, 1, 1, 1)),      # the same in the three-column kernel (four rows per tile, 10 per image)
    # 64 output channels, three filter columns: one 192-column instruction per filter row, tiles laid out by lane quarters
    (2, 64, 28, 28, 64, 3, 3, (1, 1, 1, 1, 1, 1)),      # one quarter per output row, four rows per tile
    (1, 128, 30, 60, 64, 3, 3, (1, 1, 1, 1, 1, 1)),     # two quarters per row (30 + 30 outputs), two channel blocks
    (1, 64, 9, 40, 64, 3, 3, (1, 1, 1, 1, 1, 1)),       # second quarter partly empty, last tile half empty
    (1, 64, 6, 112, 64, 3, 3, (1, 1, 1, 1, 1, 1)),      # four quarters per row
    (1, 64, 10, 30, 64, 3, 3, (1, 1, 0, 0, 1, 1)),      # no padding
    (1, 64, 5, 58, 64, 1, 3, (1, 1, 0, 1, 1, 1)),       # one filter row
]


@pytest.mark.parametrize("case", FAST_CASES)
def test_conv_declared_fp16_variant(tbn, oracle, case):
    """tbn_conv2d_fxb in the declared one-pass fp16 mode (channels-last path) stays within 1e-3 of the reference's
    float convolution, also when the input is scaled far outside fp16's own range."""
    import torch
    from oracle import graphs
    x, w, b, p = _conv_inputs(case, seed=12)
    dw_, db = torch.from_numpy(w).cuda(), torch.from_numpy(b).cuda()
    words, alpha = tbn.lib.quant_pack_binary(tbn.lib.permute_filters(dw_), tbn.LAYOUT_NK)
    for scale in (1.0, 2.0 ** 40):
        xs = (x * np.float32(scale)).astype(np.float32)
        y = tbn.lib.conv2d_fxb(torch.from_numpy(xs).cuda(), words, w.shape, p, alpha=alpha, bias=db, mode=tbn.MODE_TC_FP16X1,
                               order=tbn.CONV_WEIGHTS_TAP_MAJOR)
        tbn.lib.sync()
        assert rel_l2(y.cpu().numpy(), oracle.conv2d_f32(xs, graphs.dequantise(w), b, p)) <= 1e-3, scale
    # reference filter order: the library runs its two-term form, inside the fp32 bar
    words_r, alpha_r = tbn.lib.quant_pack_binary(dw_.reshape(w.shape[0], -1), tbn.LAYOUT_NK)
    y = tbn.lib.conv2d_fxb(torch.from_numpy(x).cuda(), words_r, w.shape, p, alpha=alpha_r, bias=db, mode=tbn.MODE_TC_FP16X1)
    tbn.lib.sync()
    assert rel_l2(y.cpu().numpy(), oracle.conv2d_f32(x, graphs.dequantise(w), b, p)) <= TOL_FP32


@pytest.mark.parametrize("case", FAST_CASES)
def test_conv_channels_last_path(tbn, oracle, case):
    """Tap-major weights + channels-last activation copy: same results as the reference's float convolution
    (float x binary and float filters) and, in TBN mode, bit-equal to the Session's integer path."""
    import torch
    from oracle import graphs
    x, w, b, p = _conv_inputs(case, seed=12)
    dx, dw_, db = torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda(), torch.from_numpy(b).cuda()
    flat = tbn.lib.permute_filters(dw_)
    assert torch.equal(flat.reshape(w.shape[0], w.shape[2] * w.shape[3], w.shape[1]),
                       dw_.reshape(w.shape[0], w.shape[1], -1).transpose(1, 2))
    order = tbn.CONV_WEIGHTS_TAP_MAJOR
    words, alpha = tbn.lib.quant_pack_binary(flat, tbn.LAYOUT_NK)
    y = tbn.lib.conv2d_fxb(dx, words, w.shape, p, alpha=alpha, bias=db, order=order)
    tbn.lib.sync()
    assert rel_l2(y.cpu().numpy(), oracle.conv2d_f32(x, graphs.dequantise(w), b, p)) <= TOL_FP32
    # float filters
    yd = tbn.lib.conv2d_f32(dx, tbn.lib.dense_pack(flat, tbn.LAYOUT_NK), w.shape, p, bias=db, order=order)
    tbn.lib.sync()
    assert rel_l2(yd.cpu().numpy(), oracle.conv2d_f32(x, w, b, p)) <= TOL_FP32
    # TBN mode on the dequantised filters
    wq = graphs.dequantise(w)
    dwq = torch.from_numpy(wq).cuda()
    words_q, _ = tbn.lib.quant_pack_binary(tbn.lib.permute_filters(dwq), tbn.LAYOUT_NK, 0.0, True, want_alpha=False)
    yq = tbn.lib.conv2d_tbn(dx, words_q, w.shape, p, alpha=tbn.lib.channel_abs_mean(dwq), bias=db,
                            epilogue=tbn.EPI_BIAS_BEFORE_ALPHA, order=order)
    tbn.lib.sync()
    assert np.array_equal(yq.cpu().numpy(), oracle.conv2d_tbn_session(x, wq, b, p))
    # and the two weight orders agree with each other bit for bit in the integer mode
    words_r, _ = tbn.lib.quant_pack_binary(dwq.reshape(w.shape[0], -1), tbn.LAYOUT_NK, 0.0, True, want_alpha=False)
    yr = tbn.lib.conv2d_tbn(dx, words_r, w.shape, p, alpha=tbn.lib.channel_abs_mean(dwq), bias=db,
                            epilogue=tbn.EPI_BIAS_BEFORE_ALPHA)
    tbn.lib.sync()
    assert torch.equal(yq, yr)


def test_channels_last_prepass_beyond_65535_rows(tbn):
    """batch x height above 65535 (the limit of two of the three launch-grid dimensions): the channels-last
    path agrees with the element-wise path bit for bit in the integer mode."""
    import torch
    g = torch.Generator(device="cuda").manual_seed(5)
    x = torch.randn((1200, 64, 56, 8), device="cuda", generator=g)
    w = torch.randn((64, 64, 3, 3), device="cuda", generator=g)
    p = (1, 1, 1, 1, 1, 1)
    alpha = tbn.lib.channel_abs_mean(w)
    words_t, _ = tbn.lib.quant_pack_binary(tbn.lib.permute_filters(w), tbn.LAYOUT_NK, 0.0, True, want_alpha=False)
    words_r, _ = tbn.lib.quant_pack_binary(w.reshape(64, -1), tbn.LAYOUT_NK, 0.0, True, want_alpha=False)
    yt = tbn.lib.conv2d_tbn(x, words_t, tuple(w.shape), p, alpha=alpha, order=tbn.CONV_WEIGHTS_TAP_MAJOR)
    yr = tbn.lib.conv2d_tbn(x, words_r, tuple(w.shape), p, alpha=alpha)
    tbn.lib.sync()
    assert yt.shape == (1200, 64, 56, 8) and torch.equal(yt, yr)
    assert float(yt.abs().sum()) > 0


def test_tap_major_needs_64_channels(tbn):
    import torch
    x = torch.zeros((1, 48, 8, 8), device="cuda")
    words = torch.zeros((8, 16), dtype=torch.int32, device="cuda")
    with pytest.raises(tbn.TbnError) as e:
        tbn.lib.conv2d_fxb(x, words, (8, 48, 3, 3), (1, 1, 1, 1, 1, 1), order=tbn.CONV_WEIGHTS_TAP_MAJOR)
    assert e.value.status == -1


def test_conv_residual_relu_epilogue(tbn, oracle):
    import torch
    from oracle import graphs
    case = (3, 16, 10, 10, 16, 3, 3, (1, 1, 1, 1, 1, 1))
    x, w, b, p = _conv_inputs(case, seed=5)
    res = np.random.default_rng(6).standard_normal((3, 16, 10, 10), dtype=np.float32)
    dw = torch.from_numpy(w).cuda()
    words, alpha = tbn.lib.quant_pack_binary(dw.reshape(16, -1), tbn.LAYOUT_NK)
    y = tbn.lib.conv2d_fxb(torch.from_numpy(x).cuda(), words, w.shape, p, alpha=alpha, bias=torch.from_numpy(b).cuda(),
                           residual=torch.from_numpy(res).cuda(), epilogue=tbn.EPI_RELU)
    tbn.lib.sync()
    expect = oracle.relu(oracle.add(oracle.conv2d_f32(x, graphs.dequantise(w), b, p), res))
    assert rel_l2(y.cpu().numpy(), expect) <= TOL_FP32


def test_conv_argument_errors(tbn):
    import torch
    x = torch.zeros((1, 3, 4, 4), device="cuda")
    words = torch.zeros((8, 4), dtype=torch.int32, device="cuda")
    with pytest.raises(tbn.TbnError) as e:
        tbn.lib.conv2d_fxb(x, words, (5, 3, 7, 7), (1, 1, 0, 0, 1, 1))  # kernel larger than the image
    assert e.value.status == -7
    with pytest.raises(tbn.TbnError) as e:
        tbn.lib.conv2d_fxb(x, words, (5, 3, 3, 3), (0, 1, 0, 0, 1, 1))
    assert e.value.status == -1
    with pytest.raises(tbn.TbnError) as e:
        tbn.lib.conv2d_fxb(x, words, (5, 3, 3, 3), (1, 1, 0, 0, 1, 1), mode=tbn.MODE_TC_BF16X3)
    assert e.value.status == -3


def test_glue_operators(tbn, oracle):
    import torch
    rng = np.random.default_rng(11)
    x = rng.standard_normal((2, 3, 9, 10), dtype=np.float32)
    x[0, 0, 0, 0] = np.nan
    d = torch.from_numpy(x).cuda()
    assert np.array_equal(tbn.lib.relu(d).cpu().numpy(), oracle.relu(x))
    x = np.nan_to_num(x)
    d = torch.from_numpy(x).cuda()
    for p in [(2, 2, 2, 2, 0, 0), (3, 3, 2, 2, 1, 1), (3, 2, 1, 2, 1, 0)]:
        for ceil_mode in (False, True):
            assert np.array_equal(tbn.lib.pool2d(0, d, p, ceil_mode).cpu().numpy(), oracle.pool2d(0, x, p, ceil_mode))
            for cip in (False, True):
                assert np.array_equal(tbn.lib.pool2d(1, d, p, ceil_mode, cip).cpu().numpy(),
                                      oracle.pool2d(1, x, p, ceil_mode, cip))
    np.testing.assert_allclose(tbn.lib.global_avgpool2d(d).cpu().numpy(), oracle.pool2d(2, x, None), rtol=1e-6, atol=1e-7)
    y = rng.standard_normal((2, 3, 9, 10), dtype=np.float32)
    ch = rng.standard_normal(3, dtype=np.float32)
    assert np.array_equal(tbn.lib.add(d, torch.from_numpy(y).cuda()).cpu().numpy(), oracle.add(x, y))
    assert np.array_equal(tbn.lib.add(d, torch.from_numpy(ch).cuda()).cpu().numpy(), oracle.add(x, ch))
    m = rng.standard_normal((5, 7), dtype=np.float32)
    row = rng.standard_normal(7, dtype=np.float32)
    assert np.array_equal(tbn.lib.add(torch.from_numpy(m).cuda(), torch.from_numpy(row).cuda()).cpu().numpy(), m + row)
    assert np.array_equal(tbn.lib.add(d, torch.from_numpy(y).cuda(), relu=True).cpu().numpy(), np.maximum(x + y, 0))


@pytest.mark.parametrize("shape", [(2, 5, 20, 24), (1, 3, 112, 112), (3, 2, 7, 132), (1, 1, 1, 4), (2, 2, 9, 260)])
def test_stem_maxpool_fast_kernel_is_bit_exact(tbn, oracle, shape):
    """3 x 3 / stride 2 / pad 1 max pooling with W % 4 == 0 runs a row-per-warp kernel: bit-identical to the
    reference's maxpool2d (pooling.cpp:10-80), NaN and infinite inputs included (same tap order, same compare)."""
    import torch
    rng = np.random.default_rng(31)
    x = rng.standard_normal(shape, dtype=np.float32)
    flat = x.reshape(-1)
    idx = rng.choice(flat.size, size=max(1, flat.size // 50), replace=False)
    flat[idx] = np.resize(np.array([np.nan, np.inf, -np.inf, 0.0, -0.0], dtype=np.float32), idx.size)
    got = tbn.lib.pool2d(0, torch.from_numpy(x).cuda(), (3, 3, 2, 2, 1, 1)).cpu().numpy()
    tbn.lib.sync()
    expect = oracle.pool2d(0, x, (3, 3, 2, 2, 1, 1))
    assert got.shape == expect.shape
    assert np.array_equal(got, expect, equal_nan=True)
    assert np.array_equal(np.signbit(got), np.signbit(expect))


@pytest.mark.parametrize("batch", [1, 7, 256])
def test_lenet_session_float_binary(tbn, oracle, batch):
    """The simple_cnn-shaped binary CNN: every layer within 1e-5 of the reference's float path on the
    dequantised weights, and the predicted classes identical."""
    from fast_arm_tbcnn_b200.session import Session
    from oracle import graphs
    net = graphs.lenet(batch=batch, seed=1)
    x = np.random.default_rng(0).random((batch, 1, 28, 28), dtype=np.float32)
    keep = {}
    expect = graphs.run_float(net, x, oracle, keep)
    for fuse in (True, False):
        s = Session(net, fuse=fuse)
        s.set_input("input", x)
        s.run()
        tbn.lib.sync()
        got = s.get_output("output").cpu().numpy()
        assert rel_l2(got, expect) <= TOL_FP32
        assert np.array_equal(got.argmax(axis=1), expect.argmax(axis=1))
        if not fuse:
            for name, ref in keep.items():
                assert rel_l2(s.intermediates[name].cpu().numpy().reshape(ref.shape), ref) <= TOL_FP32, name
    with pytest.raises(ValueError):
        s.set_input("input", x[:, :, :27])
    with pytest.raises(KeyError):
        s.set_input("nope", x)


@pytest.mark.parametrize("batch", [1, 7, 2500])
def test_lenet_whole_network_kernel(tbn, oracle, batch):
    """The LeNet-shaped graph as ONE kernel (Session with no intermediates wanted): logits within 1e-5 of the
    reference's float path on the dequantised weights, predicted classes identical, and equal (to rounding) to the
    layer-by-layer execution.  2500 images: several images per block and a ragged last wave."""
    from fast_arm_tbcnn_b200.session import Session
    from oracle import graphs
    net = graphs.lenet(batch=batch, seed=1)
    x = np.random.default_rng(0).random((batch, 1, 28, 28), dtype=np.float32)
    sub = min(batch, 64)   # the CPU oracle on a sample of the images
    pick = np.sort(np.random.default_rng(1).choice(batch, size=sub, replace=False))
    net_sub = graphs.lenet(batch=sub, seed=1)
    expect = graphs.run_float(net_sub, x[pick], oracle)
    s = Session(net)
    s.keep_intermediates = False
    assert s._lenet is not None
    launches0 = tbn.lib.launch_count()
    s.set_input("input", x)
    s.run()
    tbn.lib.sync()
    assert tbn.lib.launch_count() - launches0 == 1   # the whole network is one launch
    got = s.get_output("output").cpu().numpy()
    assert rel_l2(got[pick], expect) <= 1e-5
    assert np.array_equal(got[pick].argmax(axis=1), expect.argmax(axis=1))
    layered = Session(net)
    layered.whole_net = False
    layered.keep_intermediates = False
    layered.set_input("input", x)
    layered.run()
    tbn.lib.sync()
    assert rel_l2(got, layered.get_output("output").cpu().numpy()) <= 1e-5


def test_lenet_session_tbn_mode_bit_exact(tbn, golden):
    """Quantisation on: bit-equal to the reference Session's output stored in the golden fixture."""
    from fast_arm_tbcnn_b200.session import Session
    from oracle import graphs
    r = golden["ref_outputs_small"]
    net = graphs.lenet(batch=1, seed=1)
    net = dict(net, inits={k: (graphs.dequantise(v) if k in net["binary"] else v) for k, v in net["inits"].items()})
    s = Session(net)
    s.set_quantization(True)
    s.set_input("input", r["lenet_x"])
    s.run()
    tbn.lib.sync()
    assert np.array_equal(s.get_output("output").cpu().numpy(), r["lenet_tbn_session"])


@pytest.mark.parametrize("batch", [1, 64])
def test_conv_layer_session_both_modes(tbn, oracle, batch):
    """64x14x14 -> 128x14x14, 3x3, stride 1, pad 1, with bias."""
    from fast_arm_tbcnn_b200.session import Session
    from oracle import graphs
    net = graphs.conv_layer(batch=batch)
    x = np.random.default_rng(0).standard_normal((batch, 64, 14, 14), dtype=np.float32)
    s = Session(net)
    s.set_input("input", x)
    s.run()
    tbn.lib.sync()
    assert rel_l2(s.get_output("output").cpu().numpy(), graphs.run_float(net, x, oracle)) <= TOL_FP32
    # TBN mode on the dequantised model (+-alpha weights), which is what the reference Session is given.
    wq = graphs.dequantise(net["inits"]["w"])
    net_q = dict(net, inits=dict(net["inits"], w=wq))
    s = Session(net_q)
    s.set_quantization(True)
    s.set_input("input", x)
    s.run()
    tbn.lib.sync()
    expect = oracle.conv2d_tbn_session(x, wq, net["inits"]["b"], (1, 1, 1, 1, 1, 1))
    assert np.array_equal(s.get_output("output").cpu().numpy(), expect)


def test_conv_full_batch_properties(tbn):
    """Batch 4096 of the benchmark layer (M = 802816 GEMM rows): batch independence -- every image's
    output equals the output of the same image run alone -- and linearity in the input."""
    import torch
    from fast_arm_tbcnn_b200 import capi
    g = torch.Generator(device="cuda").manual_seed(0)
    B = 4096
    x = torch.randn((B, 64, 14, 14), generator=g, device="cuda")
    w = torch.randn((128, 64, 3, 3), generator=g, device="cuda") * 0.05
    bias = torch.randn(128, generator=g, device="cuda") * 0.05
    p = (1, 1, 1, 1, 1, 1)
    for order, flat in ((capi.CONV_WEIGHTS_REFERENCE, w.reshape(128, -1)), (capi.CONV_WEIGHTS_TAP_MAJOR, tbn.lib.permute_filters(w))):
        words, alpha = tbn.lib.quant_pack_binary(flat.contiguous(), capi.LAYOUT_NK)
        y = tbn.lib.conv2d_fxb(x, words, w.shape, p, alpha=alpha, bias=bias, order=order)
        tbn.lib.sync()
        for i in (0, 1, 2047, 4095):
            yi = tbn.lib.conv2d_fxb(x[i:i + 1].contiguous(), words, w.shape, p, alpha=alpha, bias=bias, order=order)
            tbn.lib.sync()
            assert torch.equal(yi[0], y[i])
        y_neg = tbn.lib.conv2d_fxb(-x, words, w.shape, p, alpha=alpha, order=order)
        y_pos = tbn.lib.conv2d_fxb(x, words, w.shape, p, alpha=alpha, order=order)
        tbn.lib.sync()
        assert torch.equal(y_neg, -y_pos)


# ------------------------------------------------------------------ float weights (dense path)

@pytest.mark.parametrize("M,K,N", [(128, 128, 128), (200, 300, 77), (64, 512, 1000), (1000, 147, 64), (3, 4608, 10)])
def test_gemm_f32_vs_reference_float_gemm(tbn, oracle, M, K, N):
    """tbn_gemm_f32 (bf16 hi/lo on both operands) against tbn::gemm's blocked fp32 loop."""
    import torch
    rng = np.random.default_rng(M + K + N)
    A = rng.standard_normal((M, K), dtype=np.float32)
    W = rng.standard_normal((K, N), dtype=np.float32) * np.float32(0.1)
    bias = rng.standard_normal(N, dtype=np.float32)
    pw = tbn.lib.dense_pack(torch.from_numpy(W).cuda(), tbn.LAYOUT_KN)
    out = tbn.lib.gemm_f32(torch.from_numpy(A).cuda(), pw, N, alpha=0.7, bias=torch.from_numpy(bias).cuda())
    tbn.lib.sync()
    expect = oracle.gemm_f32(A, W, bias, 0.7, 1.0)
    assert rel_l2(out.cpu().numpy(), expect) <= TOL_FP32
    # the NK layout packs the same operand from the transposed matrix
    pw_t = tbn.lib.dense_pack(torch.from_numpy(np.ascontiguousarray(W.T)).cuda(), tbn.LAYOUT_NK)
    assert torch.equal(pw, pw_t)


@pytest.mark.parametrize("case", [CONV_CASES[1], CONV_CASES[2], CONV_CASES[6], CONV_CASES[7], CONV_CASES[9]])
def test_conv_f32_vs_reference_float_conv(tbn, oracle, case):
    import torch
    x, w, b, p = _conv_inputs(case, seed=9)
    pw = tbn.lib.dense_pack(torch.from_numpy(w).cuda().reshape(w.shape[0], -1), tbn.LAYOUT_NK)
    y = tbn.lib.conv2d_f32(torch.from_numpy(x).cuda(), pw, w.shape, p, bias=torch.from_numpy(b).cuda())
    tbn.lib.sync()
    assert rel_l2(y.cpu().numpy(), oracle.conv2d_f32(x, w, b, p)) <= TOL_FP32


@pytest.mark.parametrize("batch,image", [(2, 64), (1, 224)])
def test_resnet18_session(tbn, oracle, batch, image):
    """Binary ResNet-18-style CNN (fp32 stem / shortcut convolutions / classifier, binary 3x3 convolutions,
    residual adds) against the reference's float path on the dequantised weights.  The predicted class is
    identical; the logits agree to 3e-5 end to end (each of the 21 weight layers contributes about 2.5e-6, the
    two-term activation split); fused (Conv+ReLU, Conv+Add+ReLU epilogues) and unfused execution agree."""
    from fast_arm_tbcnn_b200.session import Session
    from oracle import graphs
    net = graphs.resnet18(batch=batch, seed=2, image=image, classes=1000 if image == 224 else 100)
    x = np.random.default_rng(0).standard_normal((batch, 3, image, image), dtype=np.float32)
    expect = graphs.run_float(net, x, oracle)
    outs = []
    for fuse, fast in ((True, True), (False, True), (True, False)):
        s = Session(net, fuse=fuse, fast=fast)
        s.set_input("input", x)
        s.run()
        tbn.lib.sync()
        outs.append(s.get_output("output").cpu().numpy())
        assert rel_l2(outs[-1], expect) <= 3e-5
        assert np.array_equal(outs[-1].argmax(axis=1), expect.argmax(axis=1))
    assert rel_l2(outs[0], outs[1]) <= 1e-6


@pytest.mark.gpu
def test_resnet18_at_the_benchmark_microbatch_against_a_seeded_subset(tbn, oracle):
    """The network as the benchmark runs it -- 512 images of 224 x 224 per Session.run, layer chaining on, no
    intermediates kept -- against the reference's float path on 32 of those images (every 16th; the network treats
    images independently, so the oracle runs them alone): logits within the end-to-end 3e-5, classes identical."""
    import torch
    from fast_arm_tbcnn_b200.session import Session
    from oracle import graphs
    batch, step = 512, 16
    rng = np.random.default_rng(1000)
    x = rng.standard_normal((batch, 3, 224, 224), dtype=np.float32)
    sess = Session(graphs.resnet18(batch=batch, seed=2, image=224, classes=1000))
    sess.keep_intermediates = False
    sess.set_input("input", torch.from_numpy(x).cuda())
    sess.run()
    tbn.lib.sync()
    got = sess.get_output("output").cpu().numpy()[::step]
    sub = np.ascontiguousarray(x[::step])
    expect = graphs.run_float(graphs.resnet18(batch=sub.shape[0], seed=2, image=224, classes=1000), sub, oracle)
    assert got.shape == expect.shape == (batch // step, 1000)
    assert rel_l2(got, expect) <= 3e-5
    for i in range(got.shape[0]):
        assert rel_l2(got[i], expect[i]) <= 1e-4, i   # no single image far off
    assert np.array_equal(got.argmax(axis=1), expect.argmax(axis=1))


def test_resnet18_every_weight_layer_on_reference_inputs(tbn, oracle):
    """Per-layer bar: every Conv and Gemm of the network, fed the reference's own input to that layer, is
    within 1e-5 of the reference's output of that layer (channels-last and element-wise conv paths)."""
    from fast_arm_tbcnn_b200.session import Session
    from oracle import graphs
    net = graphs.resnet18(batch=2, seed=2, image=64, classes=100)
    x = np.random.default_rng(0).standard_normal((2, 3, 64, 64), dtype=np.float32)
    keep = {"input": x}
    graphs.run_float(net, x, oracle, keep)
    checked = 0
    for node in net["nodes"]:
        if node["op"] not in ("Conv", "Gemm"):
            continue
        src, out = node["inputs"][0], node["outputs"][0]
        sub = {"inputs": {src: keep[src].shape}, "outputs": {out: keep[out].shape}, "values": {},
               "inits": {k: net["inits"][k] for k in node["inputs"][1:]},
               "binary": {k for k in node["inputs"][1:] if k in net["binary"]}, "nodes": [node]}
        for fast in (True, False):
            s = Session(sub, fast=fast)
            s.set_input(src, keep[src])
            s.run()
            tbn.lib.sync()
            err = rel_l2(s.get_output(out).cpu().numpy(), keep[out])
            assert err <= TOL_FP32, (node["name"], fast, err)
        checked += 1
    assert checked == 21


@pytest.mark.gpu
def test_elementwise_transpose_and_global_maxpool(tbn):
    """Greater / Less / Sub with the reference Session's flat modulo broadcast (model.hpp:1176-1316), the 2-D
    transpose behind transposed Gemm operands, GlobalMaxPool (pooling.cpp:150-181): exact against numpy."""
    import torch
    g = torch.Generator(device="cuda").manual_seed(9)
    x = torch.randn((3, 5, 7, 6), device="cuda", generator=g)
    x[0, 0, 0, 0] = float("nan")
    for rhs in (torch.tensor([0.25], device="cuda"), torch.randn(6, device="cuda", generator=g), torch.randn_like(x)):
        xn, rn = x.cpu().numpy(), np.resize(rhs.cpu().numpy().reshape(-1), x.numel()).reshape(x.shape)
        with np.errstate(invalid="ignore"):
            assert np.array_equal(tbn.lib.binary_elementwise(tbn.ELT_GREATER, x, rhs).cpu().numpy(), (xn > rn).astype(np.float32))
            assert np.array_equal(tbn.lib.binary_elementwise(tbn.ELT_LESS, x, rhs).cpu().numpy(), (xn < rn).astype(np.float32))
            assert np.array_equal(tbn.lib.binary_elementwise(tbn.ELT_SUB, x, rhs).cpu().numpy(), xn - rn, equal_nan=True)
    for shape in ((1, 1), (33, 65), (256, 10), (1000, 31)):
        m = torch.randn(shape, device="cuda", generator=g)
        assert torch.equal(tbn.lib.transpose2d(m), m.t().contiguous())
    xm = x.clone()
    got = tbn.lib.global_maxpool2d(xm).cpu().numpy()
    ref = np.full((3, 5, 1, 1), -np.inf, dtype=np.float32)
    xn = xm.cpu().numpy()
    for n in range(3):
        for c in range(5):
            best = -np.inf
            for v in xn[n, c].reshape(-1):
                best = v if best < v else best      # std::max(best, v): a NaN never wins
            ref[n, c, 0, 0] = best
    assert np.array_equal(got, ref)
    tbn.lib.sync()


@pytest.mark.gpu
@pytest.mark.parametrize("weights", ["binary", "float"])
def test_chained_convolutions_are_bit_identical(tbn, weights):
    """tbn_conv2d_*_chain: the channels-last bf16 result written by one convolution's epilogue, fed to the next
    convolution instead of the fp32 tensor, gives the same bits as the unchained sequence; it equals the split of
    the fp32 result; and the fp32 tensor can be left out altogether."""
    import torch
    g = torch.Generator(device="cuda").manual_seed(21)
    x = torch.randn((3, 64, 14, 14), device="cuda", generator=g)
    w1 = torch.randn((128, 64, 3, 3), device="cuda", generator=g) * 0.05
    w2 = torch.randn((64, 128, 3, 3), device="cuda", generator=g) * 0.05
    b1 = torch.randn(128, device="cuda", generator=g) * 0.1
    res = torch.randn((3, 64, 7, 7), device="cuda", generator=g)
    p1, p2 = (1, 1, 1, 1, 1, 1), (2, 2, 1, 1, 1, 1)

    def prep(w):
        flat = tbn.lib.permute_filters(w)
        if weights == "binary":
            words, alpha = tbn.lib.quant_pack_binary(flat, tbn.LAYOUT_NK)
            return {"words": words}, alpha
        return {"split": tbn.lib.dense_pack(flat, tbn.LAYOUT_NK)}, None

    k1, a1 = prep(w1)
    k2, a2 = prep(w2)
    y1, y1_cl = tbn.lib.conv2d_chain(tuple(x.shape), k1, tuple(w1.shape), p1, x=x, want_y=True, want_y_cl=True, alpha=a1,
                                     bias=b1, epilogue=tbn.EPI_RELU)
    none_y, y1_cl_only = tbn.lib.conv2d_chain(tuple(x.shape), k1, tuple(w1.shape), p1, x=x, want_y=False, want_y_cl=True,
                                              alpha=a1, bias=b1, epilogue=tbn.EPI_RELU)
    tbn.lib.sync()
    assert none_y is None and torch.equal(y1_cl, y1_cl_only)
    hi = y1.permute(0, 2, 3, 1).bfloat16()
    assert torch.equal(y1_cl[0], hi)
    assert torch.equal(y1_cl[1], (y1.permute(0, 2, 3, 1) - hi.float()).bfloat16())
    plain, _ = tbn.lib.conv2d_chain(tuple(y1.shape), k2, tuple(w2.shape), p2, x=y1, alpha=a2, residual=res)
    chained, _ = tbn.lib.conv2d_chain(tuple(y1.shape), k2, tuple(w2.shape), p2, x_cl=y1_cl, alpha=a2, residual=res)
    tbn.lib.sync()
    assert torch.equal(plain, chained) and float(plain.abs().sum()) > 0


def _random_fast_cases(count, seed):
    """Seeded random channels-last convolution shapes: sizes chosen so that every tile geometry the library picks from
    (rectangular patches, stacked rows, row mode with and without stacking, the three-column kernel, strided and 1x1
    filters) is hit several times."""
    rng = np.random.default_rng(seed)
    cases = []
    while len(cases) < count:
        c = int(rng.choice([64, 128]))
        m = int(rng.choice([64, 64, 128, 256, 40]))
        k = int(rng.choice([1, 3, 3, 3]))
        s = int(rng.choice([1, 1, 1, 2]))
        h, w = int(rng.integers(3, 40)), int(rng.integers(3, 62))
        n = int(rng.integers(1, 7))
        pad = int(rng.integers(0, 2)) if k == 3 else 0
        if (h + 2 * pad - k) // s + 1 < 1 or (w + 2 * pad - k) // s + 1 < 1:
            continue
        cases.append((n, c, h, w, m, k, k, (s, s, pad, pad, 1, 1)))
    return cases


@pytest.mark.gpu
@pytest.mark.parametrize("case", _random_fast_cases(36, seed=77))
def test_conv_channels_last_random_shapes(tbn, oracle, case):
    """Float x binary convolution with tap-major filters on random shapes, with bias, residual and ReLU in the epilogue,
    against the reference's float convolution on the dequantised filters; the channels-last result form equals the
    split of the fp32 result."""
    import torch
    from oracle import graphs
    x, w, b, p = _conv_inputs(case, seed=case[2] * 100 + case[3])
    dx, dw_, db = torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda(), torch.from_numpy(b).cuda()
    words, alpha = tbn.lib.quant_pack_binary(tbn.lib.permute_filters(dw_), tbn.LAYOUT_NK)
    expect = oracle.conv2d_f32(x, graphs.dequantise(w), b, p)
    res = np.random.default_rng(5).standard_normal(expect.shape, dtype=np.float32)
    y, y_cl = tbn.lib.conv2d_chain(tuple(x.shape), {"words": words}, tuple(w.shape), p, x=dx, want_y=True, want_y_cl=True,
                                   alpha=alpha, bias=db, residual=torch.from_numpy(res).cuda(), epilogue=tbn.EPI_RELU)
    tbn.lib.sync()
    assert rel_l2(y.cpu().numpy(), np.maximum(expect + res, 0.0)) <= TOL_FP32
    hi = y.permute(0, 2, 3, 1).bfloat16()
    assert torch.equal(y_cl[0], hi) and torch.equal(y_cl[1], (y.permute(0, 2, 3, 1) - hi.float()).bfloat16())


@pytest.mark.gpu
@pytest.mark.parametrize("case", _random_fast_cases(16, seed=78))
def test_conv_float_filters_and_tbn_mode_random_shapes(tbn, oracle, case):
    """The same random shapes with float filters (two terms on both sides: within 1e-5 of the reference's float
    convolution) and in TBN mode (ternarised activations x sign filters: bit-equal to the Session's integer path)."""
    import torch
    from oracle import graphs
    x, w, b, p = _conv_inputs(case, seed=case[2] * 100 + case[3] + 1)
    dx, dw_, db = torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda(), torch.from_numpy(b).cuda()
    order = tbn.CONV_WEIGHTS_TAP_MAJOR
    yd = tbn.lib.conv2d_f32(dx, tbn.lib.dense_pack(tbn.lib.permute_filters(dw_), tbn.LAYOUT_NK), w.shape, p, bias=db, order=order)
    tbn.lib.sync()
    assert rel_l2(yd.cpu().numpy(), oracle.conv2d_f32(x, w, b, p)) <= TOL_FP32
    wq = graphs.dequantise(w)
    dwq = torch.from_numpy(wq).cuda()
    words_q, _ = tbn.lib.quant_pack_binary(tbn.lib.permute_filters(dwq), tbn.LAYOUT_NK, 0.0, True, want_alpha=False)
    yq = tbn.lib.conv2d_tbn(dx, words_q, w.shape, p, alpha=tbn.lib.channel_abs_mean(dwq), bias=db,
                            epilogue=tbn.EPI_BIAS_BEFORE_ALPHA, order=order)
    tbn.lib.sync()
    assert np.array_equal(yq.cpu().numpy(), oracle.conv2d_tbn_session(x, wq, b, p))


@pytest.mark.gpu
def test_three_column_instruction_with_residual_and_both_result_forms(tbn, oracle):
    """64 -> 64 channels, 3x3, stride 1 (the layers that run one 192-column instruction per filter row): input taken
    as channels-last terms, residual added, ReLU, fp32 NCHW and channels-last results written -- against the
    reference's float convolution on the dequantised filters, and the two result forms against each other."""
    import torch
    from oracle import graphs
    rng = np.random.default_rng(33)
    x = rng.standard_normal((3, 64, 28, 28), dtype=np.float32)
    w = (rng.standard_normal((64, 64, 3, 3), dtype=np.float32) * np.float32(0.05)).astype(np.float32)
    b = (rng.standard_normal(64, dtype=np.float32) * np.float32(0.05)).astype(np.float32)
    res = rng.standard_normal((3, 64, 28, 28), dtype=np.float32)
    p = (1, 1, 1, 1, 1, 1)
    dx, dw_, db, dres = (torch.from_numpy(a).cuda() for a in (x, w, b, res))
    words, alpha = tbn.lib.quant_pack_binary(tbn.lib.permute_filters(dw_), tbn.LAYOUT_NK)
    k = {"words": words}
    # a first layer only to obtain the channels-last form of its ReLU output
    y0, y0_cl = tbn.lib.conv2d_chain(tuple(x.shape), k, tuple(w.shape), p, x=dx, want_y=True, want_y_cl=True, alpha=alpha,
                                     bias=db, epilogue=tbn.EPI_RELU)
    y1, y1_cl = tbn.lib.conv2d_chain(tuple(x.shape), k, tuple(w.shape), p, x_cl=y0_cl, want_y=True, want_y_cl=True,
                                     alpha=alpha, bias=db, residual=dres, epilogue=tbn.EPI_RELU)
    only_cl = tbn.lib.conv2d_chain(tuple(x.shape), k, tuple(w.shape), p, x_cl=y0_cl, want_y=False, want_y_cl=True,
                                   alpha=alpha, bias=db, residual=dres, epilogue=tbn.EPI_RELU)[1]
    tbn.lib.sync()
    wq = graphs.dequantise(w)
    e0 = np.maximum(oracle.conv2d_f32(x, wq, b, p), 0.0)
    assert rel_l2(y0.cpu().numpy(), e0) <= TOL_FP32
    e1 = np.maximum(oracle.conv2d_f32(y0.cpu().numpy(), wq, b, p) + res, 0.0)
    assert rel_l2(y1.cpu().numpy(), e1) <= TOL_FP32
    hi = y1.permute(0, 2, 3, 1).bfloat16()
    assert torch.equal(y1_cl[0], hi) and torch.equal(y1_cl[1], (y1.permute(0, 2, 3, 1) - hi.float()).bfloat16())
    assert torch.equal(only_cl, y1_cl)


@pytest.mark.gpu
def test_session_layer_chaining_changes_no_bit(tbn, oracle):
    """ResNet-18 through the Session with and without layer chaining (epilogues writing the channels-last form,
    pre-passes skipped, fp32 tensors left out where only convolutions read them): identical outputs."""
    import torch
    from fast_arm_tbcnn_b200 import graphs
    from fast_arm_tbcnn_b200.session import Session
    net = graphs.resnet18(batch=3, seed=2, image=64, classes=10)
    x = torch.randn((3, 3, 64, 64), device="cuda", generator=torch.Generator(device="cuda").manual_seed(4))
    outs = []
    for chain, keep in ((False, True), (True, True), (True, False)):
        s = Session(net, chain=chain)
        s.keep_intermediates = keep
        s.set_input("input", x)
        s.run()
        outs.append(s.get_output("output").clone())
    tbn.lib.sync()
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
