"""Generates the committed golden fixtures under tests/golden/.

Run once in a container that has the reference tree (its location: environment variable TBN_REFERENCE) and
the compiled reference (oracle/_ref/libtbn_ref.so, `make -C oracle ref`):

    python tests/golden/make_golden.py

Fixtures written:
  gemm_tbn_128.npz / gemm_tbn_64.npz
      The reference's own golden matrices, parsed as text from
      GeMM/05-final/matrices_to_test.hpp and GeMM/03-blocked/matrices_64x64.hpp:
      ternary A, binary B (+-1) and C = sign(A @ B).
  layout_kats.npz
      Known-answer vectors for the three packed layouts, produced by running the
      compiled reference packers on small hand-placed inputs.
  ref_outputs_small.npz
      Outputs of the compiled reference on small seeded inputs (packing, scales,
      float GEMM, float conv, TBN-mode GEMM, a LeNet graph in both session modes),
      so that machines without the reference can still check the oracle and the
      CUDA path against what the reference itself produced.
"""
import os
import re
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from oracle import cpu_oracle as co  # noqa: E402
from oracle import graphs  # noqa: E402


def parse_cpp_arrays(path):
    text = open(path, encoding="utf-8").read()
    out = {}
    for name, body in re.findall(r"int8_t\s+(\w+)\[\]\s*=\s*\{([^}]*)\}", text):
        out[name] = np.array([int(v) for v in body.split(",")], dtype=np.int8)
    return out


def main():
    ref_root = co.reference_tree()
    ref = co.Reference()

    arrs = parse_cpp_arrays(os.path.join(ref_root, "GeMM/05-final/matrices_to_test.hpp"))
    np.savez_compressed(os.path.join(HERE, "gemm_tbn_128.npz"),
                        A=arrs["A"].reshape(128, 128), B=arrs["B"].reshape(128, 128),
                        C=arrs["C"].reshape(128, 128))
    arrs = parse_cpp_arrays(os.path.join(ref_root, "GeMM/03-blocked/matrices_64x64.hpp"))
    keys = sorted(arrs)
    a64, b64, c64 = (arrs[k] for k in keys)
    np.savez_compressed(os.path.join(HERE, "gemm_tbn_64.npz"),
                        A=a64.reshape(64, 64), B=b64.reshape(64, 64), C=c64.reshape(64, 64),
                        names=np.array(keys))

    # ---- layout known-answer vectors (reference packers on hand-placed inputs)
    wb = np.ones((128, 8), dtype=np.int8)
    wb[37, 3] = -1
    wb[64, 0] = -1
    bin_words = ref.binary_pack(wb).view("<u4")
    act = np.zeros((8, 64), dtype=np.float32)
    act[1, 9], act[2, 33], act[0, 0], act[0, 1] = 0.5, -0.5, 0.1, -0.1
    pos, neg = ref.ternary_pack_from_float(act, -0.1, 0.1)
    tern = np.array([-1, 0, 1, 1, 0, 0, -1, -1, 1, 1, 1, 1, -1, -1, -1, -1], dtype=np.int8)
    codes = ref.ternary_codes(tern)
    np.savez_compressed(os.path.join(HERE, "layout_kats.npz"),
                        bin_in=wb, bin_words=bin_words, act_in=act, act_pos=pos.view("<u4"),
                        act_neg=neg.view("<u4"), tern_in=tern, tern_codes=codes.view("<u4"))

    # ---- reference outputs on small seeded inputs
    out = {}
    rng = np.random.default_rng(1234)
    K, N, M = 200, 37, 19
    W = rng.standard_normal((K, N), dtype=np.float32)
    W[3, 5], W[4, 5], W[5, 5] = 0.0, -0.0, np.nan
    A = rng.standard_normal((M, K), dtype=np.float32)
    out["W"], out["A"] = W, A
    qb = ref.quantize_to_binary(W, 0.0)
    out["W_bin"] = qb
    Kp, Np = (K + 127) // 128 * 128, (N + 7) // 8 * 8
    padded = np.ones((Kp, Np), dtype=np.int8)
    padded[:K, :N] = np.where(qb == 1, 1, -1)
    out["W_words"] = ref.binary_pack(padded).view("<u4")
    qt = ref.quantize_to_ternary(W, -0.4, 0.4)
    out["W_tern"] = qt
    out["W_tern_codes"] = ref.ternary_codes(qt.reshape(-1))
    out["fxb_naive"] = ref.fxb_naive(A, qb, 0.37)
    out["s1_gemm"] = ref.qlinear_matmul_binary(A, qb, 0.37)
    Wd = np.where(qb == 1, 1.0, -1.0).astype(np.float32) * np.float32(0.37)
    bias = rng.standard_normal(N, dtype=np.float32)
    out["gemm_bias"] = bias
    out["gemm_f32"] = ref.gemm_f32(A, Wd, bias, 1.0, 1.0, False, False)
    x = rng.standard_normal((2, 5, 9, 11), dtype=np.float32)
    w = (rng.standard_normal((7, 5, 3, 3), dtype=np.float32) * np.float32(0.05))
    cb = rng.standard_normal(7, dtype=np.float32)
    out["conv_x"], out["conv_w"], out["conv_b"] = x, w, cb
    out["conv_f32_s1p1"] = ref.conv2d_f32(x, w, cb, (1, 1, 1, 1, 1, 1))
    out["conv_f32_s2p0d1"] = ref.conv2d_f32(x, w, None, (2, 2, 0, 0, 1, 1))
    out["conv_f32_s1p2d2"] = ref.conv2d_f32(x, w, cb, (1, 1, 2, 2, 2, 2))
    out["maxpool_k3s2p1"] = ref.pool2d(0, x, (3, 3, 2, 2, 1, 1))
    out["avgpool_k2s2"] = ref.pool2d(1, x, (2, 2, 2, 2, 0, 0))
    out["gap"] = ref.pool2d(2, x, None)

    # LeNet (the simple_cnn shape) with weights already of the form alpha*sign(w)
    net = graphs.lenet(batch=1, seed=1)
    xin = np.random.default_rng(0).random((1, 1, 28, 28), dtype=np.float32)
    out["lenet_x"] = xin
    spec, blob, iblob = graphs.to_spec(net, dequantised=True)
    out["lenet_float_session"] = ref.session_run(spec, blob, iblob, "input", xin, "output", (1, 10), False)
    out["lenet_tbn_session"] = ref.session_run(spec, blob, iblob, "input", xin, "output", (1, 10), True)
    np.savez_compressed(os.path.join(HERE, "ref_outputs_small.npz"), **out)

    # The exported MNIST TBN CNN (ternary-activation subgraph, Reshape, Gemm with transB = 1) through the
    # reference Session, float and quantised, batch 2.
    net = graphs.exported_tbn_cnn(batch=2, seed=3)
    xin = np.random.default_rng(5).random((2, 1, 28, 28), dtype=np.float32)
    spec, blob, iblob = graphs.to_spec(net)
    np.savez_compressed(os.path.join(HERE, "ref_outputs_exported_cnn.npz"), x=xin,
                        float_session=ref.session_run(spec, blob, iblob, "input", xin, "output", (2, 10), False),
                        tbn_session=ref.session_run(spec, blob, iblob, "input", xin, "output", (2, 10), True))
    print("golden fixtures written to", HERE)


if __name__ == "__main__":
    main()
