"""Pins the CPU oracle (oracle/tbn_oracle.c): against the reference's own golden
vectors, the layout known-answer vectors, stored outputs of the compiled reference,
and -- where oracle/_ref was built -- differentially against the reference itself."""
import numpy as np
import pytest

from oracle import graphs


def rel_l2(a, b):
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


# ------------------------------------------------------------ golden vectors

@pytest.mark.parametrize("name", ["gemm_tbn_128", "gemm_tbn_64"])
def test_golden_sign_vectors(oracle, golden, name):
    """GeMM/05-final/test_final.cpp:23-70: sign(C) of the ternary x binary product."""
    g = golden[name]
    A, B, Cs = g["A"], g["B"], g["C"]
    m, k = A.shape
    n = B.shape[1]
    # 64x64 set: pad K to 64 is already satisfied; rows%8, cols%64 hold for both sets.
    pos, neg = oracle.ternary_pack(A)
    bits = oracle.binary_pack(B)
    C = oracle.gemm_tbn(pos, neg, bits, m, k, n)
    assert np.array_equal(C, A.astype(np.int32) @ B.astype(np.int32))
    assert np.array_equal(np.sign(C).astype(np.int8), Cs)


def test_golden_through_reference_engine(reference, golden):
    g = golden["gemm_tbn_128"]
    pos, neg = reference.ternary_pack(g["A"])
    bits = reference.binary_pack(g["B"])
    for tiling in [(128, 128, 128, 64, 64), (64, 64, 128, 32, 32), (32, 32, 128, 16, 16)]:
        C, flops = reference.gemm_engine(pos, neg, 128, 128, bits, 128, tiling)
        assert flops == 2 * 128 ** 3
        assert np.array_equal(np.sign(C).astype(np.int8), g["C"])


def test_layout_known_answers(oracle, golden):
    k = golden["layout_kats"]
    words = oracle.binary_pack(k["bin_in"]).view("<u4")
    assert np.array_equal(words, k["bin_words"])
    assert words[13] == 0x20 and words[2] == 0x1 and np.count_nonzero(words) == 2
    pos, neg = oracle.ternary_pack_from_float(k["act_in"], -0.1, 0.1)
    assert np.array_equal(pos.view("<u4"), k["act_pos"]) and np.array_equal(neg.view("<u4"), k["act_neg"])
    assert pos.view("<u4")[2] == 0x200 and neg.view("<u4")[5] == 0x2
    codes = oracle.ternary_codes(k["tern_in"]).view("<u4")
    assert codes[0] == 0x00AA05A4 and np.array_equal(codes, k["tern_codes"])


def test_pack_rejects_bad_input(oracle):
    """GeMM/05-final/test_final.cpp:76-118 error paths."""
    with pytest.raises(RuntimeError):
        oracle.binary_pack(np.ones((60, 8), dtype=np.int8))
    with pytest.raises(RuntimeError):
        oracle.binary_pack(np.zeros((64, 8), dtype=np.int8))
    with pytest.raises(RuntimeError):
        oracle.ternary_pack(np.full((8, 64), 2, dtype=np.int8))
    with pytest.raises(RuntimeError):
        oracle.ternary_pack(np.zeros((7, 64), dtype=np.int8))


# ------------------------------------------- stored outputs of the reference

def test_against_stored_reference_outputs(oracle, golden):
    r = golden["ref_outputs_small"]
    W, A = r["W"], r["A"]
    qb = oracle.quantize_to_binary(W, 0.0)
    assert np.array_equal(qb, r["W_bin"])
    assert qb[3, 5] == 0 and qb[4, 5] == 0 and qb[5, 5] == 0  # +0, -0, NaN -> -1
    assert np.array_equal(oracle.binary_pack_padded(qb).reshape(-1), r["W_words"])
    qt = oracle.quantize_to_ternary(W, -0.4, 0.4)
    assert np.array_equal(qt, r["W_tern"])
    assert np.array_equal(oracle.ternary_codes(qt), r["W_tern_codes"])
    assert np.array_equal(oracle.fxb_naive(A, qb, 0.37), r["fxb_naive"])
    assert np.array_equal(oracle.qlinear_matmul_binary(A, qb, 0.37), r["s1_gemm"])
    Wd = np.where(qb == 1, 1.0, -1.0).astype(np.float32) * np.float32(0.37)
    assert np.array_equal(oracle.gemm_f32(A, Wd, r["gemm_bias"], 1.0, 1.0), r["gemm_f32"])
    x, w, b = r["conv_x"], r["conv_w"], r["conv_b"]
    assert np.array_equal(oracle.conv2d_f32(x, w, b, (1, 1, 1, 1, 1, 1)), r["conv_f32_s1p1"])
    assert np.array_equal(oracle.conv2d_f32(x, w, None, (2, 2, 0, 0, 1, 1)), r["conv_f32_s2p0d1"])
    assert np.array_equal(oracle.conv2d_f32(x, w, b, (1, 1, 2, 2, 2, 2)), r["conv_f32_s1p2d2"])
    assert np.array_equal(oracle.pool2d(0, x, (3, 3, 2, 2, 1, 1)), r["maxpool_k3s2p1"])
    assert np.array_equal(oracle.pool2d(1, x, (2, 2, 2, 2, 0, 0)), r["avgpool_k2s2"])
    assert np.array_equal(oracle.pool2d(2, x, None), r["gap"])


def test_lenet_float_session_matches_stored(oracle, golden):
    r = golden["ref_outputs_small"]
    net = graphs.lenet(batch=1, seed=1)
    out = graphs.run_float(net, r["lenet_x"], oracle)
    assert np.array_equal(out, r["lenet_float_session"])


def test_lenet_tbn_session_matches_stored(oracle, golden):
    """Session with quantisation on (model.hpp:375-559 conv path, :763-870 Gemm path)."""
    r = golden["ref_outputs_small"]
    net = graphs.lenet(batch=1, seed=1)
    w = {k: (graphs.dequantise(v) if k in net["binary"] else v) for k, v in net["inits"].items()}
    x = r["lenet_x"]
    y = oracle.conv2d_tbn_session(x, w["w1"], w["b1"], (1, 1, 0, 0, 1, 1))
    y = oracle.pool2d(0, oracle.relu(y), (2, 2, 2, 2, 0, 0))
    y = oracle.conv2d_tbn_session(y, w["w2"], w["b2"], (1, 1, 0, 0, 1, 1))
    y = oracle.pool2d(0, oracle.relu(y), (2, 2, 2, 2, 0, 0)).reshape(1, -1)
    # Gemm weights alpha*sign are not exactly +-1, so the Session quantises them on the
    # fly (model.hpp:839-841): quantize_to_binary then qlinear_matmul_binary, scale 1.
    qb = oracle.quantize_to_binary(w["wf"], 0.0)
    y = oracle.qlinear_matmul_binary(y, qb, 1.0) + w["bf"][None, :]
    assert np.array_equal(y.astype(np.float32), r["lenet_tbn_session"])


# ---------------------------------------- differential against the reference

@pytest.mark.parametrize("K,N", [(64, 8), (128, 8), (200, 37), (576, 128), (1, 1), (129, 9)])
def test_diff_binary_pack(oracle, reference, K, N):
    rng = np.random.default_rng(K * 1000 + N)
    W = rng.standard_normal((K, N), dtype=np.float32)
    W.flat[:: max(1, W.size // 7)] = 0.0
    for thr in (0.0, 0.25):
        qb = oracle.quantize_to_binary(W, thr)
        assert np.array_equal(qb, reference.quantize_to_binary(W, thr))
    Kp, Np = (K + 127) // 128 * 128, (N + 7) // 8 * 8
    padded = np.ones((Kp, Np), dtype=np.int8)
    padded[:K, :N] = np.where(qb == 1, 1, -1)
    assert np.array_equal(oracle.binary_pack_padded(qb).reshape(-1), reference.binary_pack(padded).view("<u4"))


@pytest.mark.parametrize("M,K,N", [(1, 1, 1), (5, 70, 3), (16, 128, 8), (33, 300, 20), (64, 256, 64)])
def test_diff_gemms(oracle, reference, M, K, N):
    rng = np.random.default_rng(M + 10 * K + 100 * N)
    A = rng.standard_normal((M, K), dtype=np.float32)
    W = rng.standard_normal((K, N), dtype=np.float32)
    qb = oracle.quantize_to_binary(W)
    assert np.array_equal(oracle.fxb_naive(A, qb, 0.5), reference.fxb_naive(A, qb, 0.5))
    assert np.array_equal(oracle.qlinear_matmul_binary(A, qb, 0.5), reference.qlinear_matmul_binary(A, qb, 0.5))
    bias = rng.standard_normal(N, dtype=np.float32)
    for tA, tB in [(False, False), (False, True), (True, False)]:
        a = A.T.copy() if tA else A
        b = W.T.copy() if tB else W
        assert np.array_equal(oracle.gemm_f32(a, b, bias, 0.7, 1.3, tA, tB),
                              reference.gemm_f32(a, b, bias, 0.7, 1.3, tA, tB))
    full = rng.standard_normal((M, N), dtype=np.float32)
    assert np.array_equal(oracle.gemm_f32(A, W, full, 1.0, 1.0), reference.gemm_f32(A, W, full, 1.0, 1.0))
    assert np.array_equal(oracle.gemm_f32(A, W), reference.gemm_f32(A, W))


def test_diff_ternary(oracle, reference):
    rng = np.random.default_rng(5)
    W = rng.standard_normal((96, 40), dtype=np.float32)
    for lo, hi in [(-0.1, 0.1), (-0.56, 0.56)]:
        qt = oracle.quantize_to_ternary(W, lo, hi)
        assert np.array_equal(qt, reference.quantize_to_ternary(W, lo, hi))
        assert np.array_equal(oracle.ternary_codes(qt), reference.ternary_codes(qt))
    A = rng.standard_normal((24, 192), dtype=np.float32)
    po, no = oracle.ternary_pack_from_float(A)
    pr, nr = reference.ternary_pack_from_float(A)
    assert np.array_equal(po, pr) and np.array_equal(no, nr)


@pytest.mark.parametrize("p", [(1, 1, 1, 1, 1, 1), (2, 2, 3, 3, 1, 1), (1, 2, 0, 1, 2, 1), (1, 1, 0, 0, 1, 1)])
def test_diff_conv(oracle, reference, p):
    rng = np.random.default_rng(sum(p))
    x = rng.standard_normal((2, 3, 13, 12), dtype=np.float32)
    w = rng.standard_normal((5, 3, 3, 3), dtype=np.float32)
    b = rng.standard_normal(5, dtype=np.float32)
    ref = reference.conv2d_f32(x, w, b, p)
    assert np.array_equal(oracle.conv2d_f32(x, w, b, p), ref)
    rows = ref.shape[0] * ref.shape[2] * ref.shape[3]
    assert np.array_equal(oracle.im2col(x, 3, 3, p), reference.im2col(x, 3, 3, p, rows))
    mp, kp = (rows + 15) // 16 * 16, 128
    po, no = oracle.im2col_ternary_packed(x, 3, 3, p, mp, kp)
    pr, nr = reference.im2col_ternary_packed(x, 3, 3, p, mp, kp)
    assert np.array_equal(po, pr) and np.array_equal(no, nr)


def test_diff_pools(oracle, reference):
    rng = np.random.default_rng(11)
    x = rng.standard_normal((2, 3, 9, 10), dtype=np.float32)
    for p in [(2, 2, 2, 2, 0, 0), (3, 3, 2, 2, 1, 1), (3, 2, 1, 2, 1, 0)]:
        for ceil_mode in (False, True):
            assert np.array_equal(oracle.pool2d(0, x, p, ceil_mode), reference.pool2d(0, x, p, ceil_mode))
            for cip in (False, True):
                assert np.array_equal(oracle.pool2d(1, x, p, ceil_mode, cip), reference.pool2d(1, x, p, ceil_mode, cip))
    assert np.array_equal(oracle.pool2d(2, x, None), reference.pool2d(2, x, None))


def test_diff_sessions(oracle, reference):
    """LeNet and the single conv layer through the reference Session, both modes."""
    net = graphs.lenet(batch=2, seed=1)
    x = np.random.default_rng(0).random((2, 1, 28, 28), dtype=np.float32)
    spec, blob, iblob = graphs.to_spec(net, dequantised=True)
    ref = reference.session_run(spec, blob, iblob, "input", x, "output", (2, 10), False)
    assert np.array_equal(graphs.run_float(net, x, oracle), ref)

    net = graphs.conv_layer(batch=1)
    x = np.random.default_rng(0).standard_normal((1, 64, 14, 14), dtype=np.float32)
    spec, blob, iblob = graphs.to_spec(net, dequantised=True)
    ref = reference.session_run(spec, blob, iblob, "input", x, "output", (1, 128, 14, 14), False)
    assert np.array_equal(graphs.run_float(net, x, oracle), ref)
    ref_q = reference.session_run(spec, blob, iblob, "input", x, "output", (1, 128, 14, 14), True)
    wq = graphs.dequantise(net["inits"]["w"])
    assert np.array_equal(oracle.conv2d_tbn_session(x, wq, net["inits"]["b"], (1, 1, 1, 1, 1, 1)), ref_q)
    # The two semantics really are different functions (ternarised activations).
    assert rel_l2(ref_q, ref) > 0.1


def test_float_binary_equals_float_gemm_on_dequantised(oracle):
    """The float x binary product with a per-column scale is the float Gemm on alpha*sign(W)
    up to fp32 summation order."""
    rng = np.random.default_rng(3)
    A = rng.standard_normal((8, 300), dtype=np.float32)
    W = rng.standard_normal((300, 16), dtype=np.float32)
    alpha = oracle.column_abs_mean(W)
    assert np.array_equal(alpha, graphs.binary_alpha(W))
    qb = oracle.quantize_to_binary(W)
    c1 = oracle.fxb_naive(A, qb, 1.0) * alpha[None, :]
    c2 = oracle.gemm_f32(A, graphs.dequantise(W))
    assert rel_l2(c1, c2) < 1e-6
