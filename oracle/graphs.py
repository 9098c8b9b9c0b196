"""CPU evaluation of the benchmark networks with the oracle primitives.

TEST INFRASTRUCTURE ONLY.  The network recipes themselves (plain dicts, no computation) live in the
package's graphs module and are re-exported here.  A network is a plain dict

    {"inputs": {name: shape}, "outputs": {name: shape}, "values": {name: shape},
     "inits": {name: ndarray}, "binary": {weight name, ...},
     "nodes": [{"op", "name", "inputs", "outputs", "attrs"}]}

mirroring the reference's ModelGraph (tbn/runtime/model.hpp:21-35).  ``to_spec``
serialises it into the line format understood by ref_session_run (ref_shim.cpp)
and by the product's own graph runner; ``run_float`` evaluates it with the
oracle primitives the way the reference Session does with quantisation off
(model.hpp:566, :873): exact fp32 operators on the dequantised weights
alpha * sign(w).

Weight conventions (declared choices where the configuration leaves them open):
  * binary weights: sign by ``w > 0`` (tbn::quantize_to_binary), alpha = mean |w| per
    output channel (conv: over C*kh*kw; Gemm stored [K,N]: per column);
  * draws come from numpy ``default_rng(seed)`` in topological order, weight then bias.
"""
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from fast_arm_tbcnn_b200 import graphs as _recipes  # noqa: E402
from fast_arm_tbcnn_b200.graphs import conv_layer, exported_tbn_cnn, lenet, resnet18  # noqa: E402,F401


def binary_alpha(w):
    """alpha per output channel: conv [M,C,kh,kw] -> over C*kh*kw; Gemm [K,N] -> per column.
    fp32 sequential sums, as model.hpp:388-394."""
    w = np.asarray(w, dtype=np.float32)
    if w.ndim == 4:
        flat = np.abs(w.reshape(w.shape[0], -1))
        acc = np.zeros(w.shape[0], dtype=np.float32)
        for i in range(flat.shape[1]):
            acc = (acc + flat[:, i]).astype(np.float32)
        return (acc / np.float32(flat.shape[1])).astype(np.float32)
    acc = np.zeros(w.shape[1], dtype=np.float32)
    aw = np.abs(w)
    for k in range(w.shape[0]):
        acc = (acc + aw[k]).astype(np.float32)
    return (acc / np.float32(w.shape[0])).astype(np.float32)


def dequantise(w):
    """alpha * sign(w) with sign by w > 0 (everything else, incl. +-0 and NaN, -> -1)."""
    w = np.asarray(w, dtype=np.float32)
    a = binary_alpha(w)
    s = np.where(w > 0, np.float32(1), np.float32(-1)).astype(np.float32)
    if w.ndim == 4:
        return (s * a[:, None, None, None]).astype(np.float32)
    return (s * a[None, :]).astype(np.float32)


def to_spec(net, dequantised=False):
    """-> (spec text, fp32 blob, int64 blob).  With ``dequantised`` the binary weights are
    replaced by alpha*sign(w), which is how the reference sees a trained TBN model."""
    replace = {name: dequantise(net["inits"][name]) for name in net["binary"]} if dequantised else None
    return _recipes.to_spec(net, replace=replace, mark_binary=not dequantised)


def strip_product_lines(spec):
    """Removes the lines only the product's runner understands (``binary ...``)."""
    return "\n".join(l for l in spec.splitlines() if not l.startswith("binary ")) + "\n"


def run_float(net, x, oracle, keep=None):
    """Evaluates the graph as the reference Session does with quantisation off, on
    dequantised weights.  ``keep``: optional dict receiving every intermediate."""
    vals = {next(iter(net["inputs"])): np.asarray(x, dtype=np.float32)}
    for name, arr in net["inits"].items():
        if np.asarray(arr).dtype == np.int64:
            vals[name] = np.asarray(arr)
        else:
            vals[name] = dequantise(arr) if name in net["binary"] else np.asarray(arr, dtype=np.float32)
    for n in net["nodes"]:
        ins = [vals[i] for i in n["inputs"]]
        a = n["attrs"]
        op = n["op"]
        if op == "Conv":
            st = a.get("strides", [1, 1])
            pd = a.get("pads", [0, 0, 0, 0])
            dl = a.get("dilations", [1, 1])
            p = (st[0], st[1], pd[0], pd[1], dl[0], dl[1])
            out = oracle.conv2d_f32(ins[0], ins[1], ins[2] if len(ins) > 2 else None, p)
        elif op == "Relu":
            out = oracle.relu(ins[0])
        elif op in ("MaxPool", "AveragePool"):
            ks = a.get("kernel_shape", [2, 2])
            st = a.get("strides", ks)
            pd = a.get("pads", [0, 0, 0, 0])
            out = oracle.pool2d(0 if op == "MaxPool" else 1, ins[0], (ks[0], ks[1], st[0], st[1], pd[0], pd[1]),
                                bool(a.get("ceil_mode", 0)), bool(a.get("count_include_pad", 0)))
        elif op == "GlobalAveragePool":
            out = oracle.pool2d(2, ins[0], None)
        elif op == "Flatten":
            ax = a.get("axis", 1)
            out = ins[0].reshape(int(np.prod(ins[0].shape[:ax])), -1).copy()
        elif op == "Add":
            out = oracle.add(ins[0], ins[1])
        elif op == "Gemm":
            out = oracle.gemm_f32(ins[0], ins[1], ins[2] if len(ins) > 2 else None, a.get("alpha", 1.0),
                                  a.get("beta", 1.0), bool(a.get("transA", 0)), bool(a.get("transB", 0)))
        elif op in ("Greater", "Less"):  # model.hpp:1176-1270: float 0/1, rhs indexed modulo its length
            rhs = np.resize(ins[1].reshape(-1), ins[0].size).reshape(ins[0].shape)
            out = ((ins[0] > rhs) if op == "Greater" else (ins[0] < rhs)).astype(np.float32)
        elif op == "Cast":               # model.hpp:1272-1287: pass-through
            out = ins[0]
        elif op == "Sub":                # model.hpp:1289-1316
            out = (ins[0] - np.resize(ins[1].reshape(-1), ins[0].size).reshape(ins[0].shape)).astype(np.float32)
        elif op == "Reshape":            # model.hpp:1039-1091
            out = ins[0].reshape([int(d) for d in ins[1]]).copy()
        elif op == "MatMul":             # model.hpp:879-903
            out = oracle.gemm_f32(ins[0], ins[1])
        elif op == "GlobalMaxPool":      # pooling.cpp:150-181
            out = ins[0].max(axis=(2, 3), keepdims=True).astype(np.float32)
        else:
            raise NotImplementedError(op)
        vals[n["outputs"][0]] = out
        if keep is not None:
            keep[n["outputs"][0]] = out
    return vals[next(iter(net["outputs"]))]
