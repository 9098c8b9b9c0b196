"""Graph recipes of the benchmark networks and their serialisation for the graph runners.

A network is a plain dict

    {"inputs": {name: shape}, "outputs": {name: shape}, "values": {name: shape},
     "inits": {name: ndarray}, "binary": {weight name, ...},
     "nodes": [{"op", "name", "inputs", "outputs", "attrs"}]}

mirroring the reference's ModelGraph (tbn/runtime/model.hpp:21-35); ``Session`` (session.py) and the C++
host layer's ``parse_graph_spec`` consume it.  Nothing here computes: weights are drawn, nodes are listed,
``to_spec`` writes the line format.

Weight conventions (declared choices where the configuration leaves them open):
  * binary weights: sign by ``w > 0`` (tbn::quantize_to_binary), alpha = mean |w| per
    output channel (conv: over C*kh*kw; Gemm stored [K,N]: per column);
  * draws come from numpy ``default_rng(seed)`` in topological order, weight then bias.
"""
import numpy as np


def _node(op, name, inputs, outputs, **attrs):
    return {"op": op, "name": name, "inputs": list(inputs), "outputs": list(outputs), "attrs": attrs}


def lenet(batch=1, seed=1, sigma=0.1):
    """The simple_cnn shape (tests/models/cnn/create_cnn_model.py:11-42), binary weights."""
    rng = np.random.default_rng(seed)

    def draw(*shape):
        return (rng.standard_normal(shape, dtype=np.float32) * np.float32(sigma)).astype(np.float32)

    w1, b1 = draw(6, 1, 5, 5), draw(6)
    w2, b2 = draw(16, 6, 5, 5), draw(16)
    wf_t, bf = draw(10, 256), draw(10)
    net = {
        "inputs": {"input": (batch, 1, 28, 28)},
        "outputs": {"output": (batch, 10)},
        "values": {},
        "inits": {"w1": w1, "b1": b1, "w2": w2, "b2": b2, "wf": np.ascontiguousarray(wf_t.T), "bf": bf},
        "binary": {"w1", "w2", "wf"},
        "nodes": [
            _node("Conv", "c1", ["input", "w1", "b1"], ["c1_out"], strides=[1, 1], pads=[0, 0, 0, 0]),
            _node("Relu", "r1", ["c1_out"], ["r1_out"]),
            _node("MaxPool", "p1", ["r1_out"], ["p1_out"], kernel_shape=[2, 2], strides=[2, 2]),
            _node("Conv", "c2", ["p1_out", "w2", "b2"], ["c2_out"], strides=[1, 1], pads=[0, 0, 0, 0]),
            _node("Relu", "r2", ["c2_out"], ["r2_out"]),
            _node("MaxPool", "p2", ["r2_out"], ["p2_out"], kernel_shape=[2, 2], strides=[2, 2]),
            _node("Flatten", "fl", ["p2_out"], ["fl_out"], axis=1),
            _node("Gemm", "fc", ["fl_out", "wf", "bf"], ["output"], transB=0),
        ],
    }
    return net


def conv_layer(batch=1, cin=64, hw=14, cout=128, k=3, stride=1, pad=1, seed=1, sigma=0.05):
    """Single binary Conv2D layer, e.g. 64x14x14 -> 128x14x14, 3x3, stride 1, pad 1, with bias."""
    rng = np.random.default_rng(seed)
    w = (rng.standard_normal((cout, cin, k, k), dtype=np.float32) * np.float32(sigma)).astype(np.float32)
    b = (rng.standard_normal(cout, dtype=np.float32) * np.float32(sigma)).astype(np.float32)
    oh = (hw + 2 * pad - (k - 1) - 1) // stride + 1
    return {
        "inputs": {"input": (batch, cin, hw, hw)},
        "outputs": {"output": (batch, cout, oh, oh)},
        "values": {},
        "inits": {"w": w, "b": b},
        "binary": {"w"},
        "nodes": [_node("Conv", "conv", ["input", "w", "b"], ["output"], strides=[stride, stride],
                        pads=[pad, pad, pad, pad])],
    }


def resnet18(batch=1, seed=2, image=224, classes=1000, width=64):
    """Binary ResNet-18-style CNN: fp32 stem, 4 stages x 2 basic blocks with binary 3x3
    convolutions, fp32 1x1 stride-2 downsample shortcuts at the entry of stages 2-4
    (stage 1: stride 1, identity shortcut), BatchNorm folded into the conv biases,
    GlobalAveragePool, fp32 Gemm.  Weights N(0, sqrt(2/fan_in)), biases N(0, 0.01)."""
    rng = np.random.default_rng(seed)
    inits, nodes, binary = {}, [], set()

    def conv(name, src, cin, cout, k, stride, pad, is_binary):
        fan_in = cin * k * k
        w = (rng.standard_normal((cout, cin, k, k), dtype=np.float32) * np.float32(np.sqrt(2.0 / fan_in)))
        b = (rng.standard_normal(cout, dtype=np.float32) * np.float32(0.01))
        inits[name + "_w"], inits[name + "_b"] = w.astype(np.float32), b.astype(np.float32)
        if is_binary:
            binary.add(name + "_w")
        nodes.append(_node("Conv", name, [src, name + "_w", name + "_b"], [name + "_out"],
                           strides=[stride, stride], pads=[pad, pad, pad, pad]))
        return name + "_out"

    def relu(name, src):
        nodes.append(_node("Relu", name, [src], [name + "_out"]))
        return name + "_out"

    cur = conv("stem", "input", 3, width, 7, 2, 3, False)
    cur = relu("stem_relu", cur)
    nodes.append(_node("MaxPool", "stem_pool", [cur], ["stem_pool_out"], kernel_shape=[3, 3], strides=[2, 2],
                       pads=[1, 1, 1, 1]))
    cur = "stem_pool_out"
    cin = width
    for stage in range(4):
        cout = width << stage
        for block in range(2):
            stride = 2 if (stage > 0 and block == 0) else 1
            tag = f"s{stage + 1}b{block + 1}"
            y = conv(tag + "_conv1", cur, cin, cout, 3, stride, 1, True)
            y = relu(tag + "_relu1", y)
            y = conv(tag + "_conv2", y, cout, cout, 3, 1, 1, True)
            shortcut = cur
            if stride != 1 or cin != cout:
                shortcut = conv(tag + "_down", cur, cin, cout, 1, stride, 0, False)
            nodes.append(_node("Add", tag + "_add", [y, shortcut], [tag + "_add_out"]))
            cur = relu(tag + "_relu2", tag + "_add_out")
            cin = cout
    nodes.append(_node("GlobalAveragePool", "gap", [cur], ["gap_out"]))
    nodes.append(_node("Flatten", "flat", ["gap_out"], ["flat_out"], axis=1))
    wf = (rng.standard_normal((cin, classes), dtype=np.float32) * np.float32(np.sqrt(2.0 / cin)))
    bf = (rng.standard_normal(classes, dtype=np.float32) * np.float32(0.01))
    inits["fc_w"], inits["fc_b"] = wf.astype(np.float32), bf.astype(np.float32)
    nodes.append(_node("Gemm", "fc", ["flat_out", "fc_w", "fc_b"], ["output"], transB=0))
    return {
        "inputs": {"input": (batch, 3, image, image)},
        "outputs": {"output": (batch, classes)},
        "values": {},
        "inits": inits,
        "binary": binary,
        "nodes": nodes,
    }


def exported_tbn_cnn(batch=1, seed=3, sigma=0.1):
    """The MNIST TBN CNN as the reference's training script exports it to ONNX (tests/train/mnist:
    Conv 1->16 5x5 pad 2, ReLU, MaxPool, Conv 16->32 5x5 pad 2, the ternary activation written as
    Greater / Cast / Less / Cast / Sub against scalar thresholds, MaxPool 14 -> 4 by ceil-less 3x3 stride 3,
    Reshape, Gemm with transB = 1).  Weights are scaled-binary (+-alpha per output channel), i.e. a trained
    TBN model after dequantisation, so the Session recognises them in both modes."""
    rng = np.random.default_rng(seed)

    def scaled_binary(*shape):
        w = (rng.standard_normal(shape, dtype=np.float32) * np.float32(sigma)).astype(np.float32)
        flat = np.abs(w.reshape(shape[0], -1))
        alpha = (flat.sum(axis=1, dtype=np.float32) / np.float32(flat.shape[1])).astype(np.float32)
        sign = np.where(w > 0, np.float32(1), np.float32(-1))
        return (sign * alpha.reshape((-1,) + (1,) * (len(shape) - 1))).astype(np.float32)

    def draw(*shape):
        return (rng.standard_normal(shape, dtype=np.float32) * np.float32(sigma)).astype(np.float32)

    w1, b1 = scaled_binary(16, 1, 5, 5), draw(16)
    w2, b2 = scaled_binary(32, 16, 5, 5), draw(32)
    wf, bf = scaled_binary(10, 512), draw(10)  # [N, K]: used with transB = 1
    return {
        "inputs": {"input": (batch, 1, 28, 28)},
        "outputs": {"output": (batch, 10)},
        "values": {},
        "inits": {"conv1_w": w1, "conv1_b": b1, "conv2_w": w2, "conv2_b": b2, "fc_w": wf, "fc_b": bf,
                  "thr_hi": np.array(0.05, dtype=np.float32), "thr_lo": np.array(-0.05, dtype=np.float32),
                  "flat_shape": np.array([batch, 512], dtype=np.int64)},
        "binary": set(),
        "nodes": [
            _node("Conv", "conv1", ["input", "conv1_w", "conv1_b"], ["c1"], group=1, pads=[2, 2, 2, 2], strides=[1, 1],
                  auto_pad="NOTSET", dilations=[1, 1]),
            _node("Relu", "relu1", ["c1"], ["r1"]),
            _node("MaxPool", "pool1", ["r1"], ["p1"], ceil_mode=0, pads=[0, 0, 0, 0], kernel_shape=[2, 2], strides=[2, 2]),
            _node("Conv", "conv2", ["p1", "conv2_w", "conv2_b"], ["c2"], group=1, pads=[2, 2, 2, 2], strides=[1, 1],
                  auto_pad="NOTSET", dilations=[1, 1]),
            _node("Greater", "gt", ["c2", "thr_hi"], ["gt_out"]),
            _node("Cast", "cast_gt", ["gt_out"], ["gt_f"], to=1),
            _node("Less", "lt", ["c2", "thr_lo"], ["lt_out"]),
            _node("Cast", "cast_lt", ["lt_out"], ["lt_f"], to=1),
            _node("Sub", "tern", ["gt_f", "lt_f"], ["t2"]),
            _node("MaxPool", "pool2", ["t2"], ["p2"], ceil_mode=0, pads=[0, 0, 0, 0], kernel_shape=[3, 3], strides=[3, 3]),
            _node("Reshape", "view", ["p2", "flat_shape"], ["flat"], allowzero=0),
            _node("Gemm", "fc", ["flat", "fc_w", "fc_b"], ["output"], alpha=1.0, beta=1.0, transA=0, transB=1),
        ],
    }


def to_spec(net, replace=None, mark_binary=True):
    """-> (spec text, fp32 blob, int64 blob).  ``replace`` maps initialiser names to arrays that are
    written instead of the network's own; ``mark_binary`` adds the line naming the binary weights."""
    replace = replace or {}
    lines, chunks, ichunks, off, ioff = [], [], [], 0, 0
    for name, shape in net["inputs"].items():
        lines.append(f"input {name} {','.join(map(str, shape))}")
    for name, shape in net["outputs"].items():
        lines.append(f"output {name} {','.join(map(str, shape))}")
    for name, shape in net.get("values", {}).items():
        lines.append(f"value {name} {','.join(map(str, shape))}")
    for name, arr in net["inits"].items():
        a = np.asarray(replace.get(name, arr))
        dims = ",".join(map(str, a.shape)) if a.ndim else "1"
        if a.dtype == np.int64:  # shape operands of Reshape
            lines.append(f"init {name} i64 {dims} {ioff}")
            ichunks.append(a.reshape(-1))
            ioff += a.size
            continue
        a = a.astype(np.float32)
        lines.append(f"init {name} f32 {dims} {off}")
        chunks.append(a.reshape(-1))
        off += a.size
    for n in net["nodes"]:
        parts = ["node", n["op"], n["name"], ",".join(n["inputs"]), ",".join(n["outputs"])]
        for k, v in n["attrs"].items():
            if isinstance(v, (list, tuple)):
                parts.append(f"{k}=I:{','.join(map(str, v))}")
            elif isinstance(v, float):
                parts.append(f"{k}=f:{v!r}")
            elif isinstance(v, str):
                parts.append(f"{k}=s:{v}")
            else:
                parts.append(f"{k}=i:{int(v)}")
        lines.append(" ".join(parts))
    blob = np.concatenate(chunks) if chunks else np.zeros(1, dtype=np.float32)
    binary_line = "binary " + ",".join(sorted(net["binary"])) if net["binary"] and mark_binary else ""
    text = "\n".join(lines + ([binary_line] if binary_line else [])) + "\n"
    iblob = np.concatenate(ichunks) if ichunks else np.zeros(1, dtype=np.int64)
    return text, blob.astype(np.float32), iblob.astype(np.int64)
