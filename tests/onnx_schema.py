"""ONNX files for the loader tests, written and read with google.protobuf — an implementation of the wire
format that shares nothing with the C++ reader under test.

The message classes are built at run time from field numbers of the public onnx.proto (only the fields the
runtime consumes, plus external_data so that such tensors can be produced).  ``net_to_onnx`` serialises a
network recipe dict (fast_arm_tbcnn_b200.graphs) into ModelProto bytes; ``canonical_dump`` renders any ONNX
file in the same one-line-per-element text the C++ driver prints with ``run_graph --dump-onnx``, following the
reference's conversion rules (tbn-runtime/src/onnx_integration/onnx_parser.cpp:159-312).
"""
import numpy as np
from google.protobuf import descriptor_pb2, descriptor_pool, message_factory

_F = descriptor_pb2.FieldDescriptorProto
_O, _R = _F.LABEL_OPTIONAL, _F.LABEL_REPEATED

# TensorProto.DataType / AttributeProto.AttributeType values
FLOAT, UINT8, INT8, INT32, INT64, DOUBLE = 1, 2, 3, 6, 7, 11
A_FLOAT, A_INT, A_STRING, A_TENSOR, A_FLOATS, A_INTS, A_STRINGS = 1, 2, 3, 4, 6, 7, 8
# tbn::DataType enumerator values printed by the dump
_TBN_DTYPE = {FLOAT: 0, INT8: 3, INT32: 5, INT64: 6, UINT8: 7}
_NP = {0: np.float32, 3: np.int8, 5: np.int32, 6: np.int64, 7: np.uint8}


def _classes():
    fd = descriptor_pb2.FileDescriptorProto(name="onnx_subset.proto", package="onnx_subset", syntax="proto2")

    def msg(name, fields):
        m = fd.message_type.add(name=name)
        for fname, num, ftype, label, tname, packed in fields:
            f = m.field.add(name=fname, number=num, type=ftype, label=label)
            if tname:
                f.type_name = ".onnx_subset." + tname
            if packed:
                f.options.packed = True

    msg("Dimension", [("dim_value", 1, _F.TYPE_INT64, _O, None, False), ("dim_param", 2, _F.TYPE_STRING, _O, None, False)])
    msg("TensorShapeProto", [("dim", 1, _F.TYPE_MESSAGE, _R, "Dimension", False)])
    msg("TypeTensor", [("elem_type", 1, _F.TYPE_INT32, _O, None, False),
                       ("shape", 2, _F.TYPE_MESSAGE, _O, "TensorShapeProto", False)])
    msg("TypeProto", [("tensor_type", 1, _F.TYPE_MESSAGE, _O, "TypeTensor", False)])
    msg("ValueInfoProto", [("name", 1, _F.TYPE_STRING, _O, None, False), ("type", 2, _F.TYPE_MESSAGE, _O, "TypeProto", False)])
    msg("StringStringEntryProto", [("key", 1, _F.TYPE_STRING, _O, None, False), ("value", 2, _F.TYPE_STRING, _O, None, False)])
    msg("TensorProto", [("dims", 1, _F.TYPE_INT64, _R, None, False), ("data_type", 2, _F.TYPE_INT32, _O, None, False),
                        ("float_data", 4, _F.TYPE_FLOAT, _R, None, True), ("int32_data", 5, _F.TYPE_INT32, _R, None, True),
                        ("int64_data", 7, _F.TYPE_INT64, _R, None, True), ("name", 8, _F.TYPE_STRING, _O, None, False),
                        ("raw_data", 9, _F.TYPE_BYTES, _O, None, False),
                        ("external_data", 13, _F.TYPE_MESSAGE, _R, "StringStringEntryProto", False),
                        ("data_location", 14, _F.TYPE_INT32, _O, None, False)])
    msg("AttributeProto", [("name", 1, _F.TYPE_STRING, _O, None, False), ("f", 2, _F.TYPE_FLOAT, _O, None, False),
                           ("i", 3, _F.TYPE_INT64, _O, None, False), ("s", 4, _F.TYPE_BYTES, _O, None, False),
                           ("t", 5, _F.TYPE_MESSAGE, _O, "TensorProto", False), ("floats", 7, _F.TYPE_FLOAT, _R, None, False),
                           ("ints", 8, _F.TYPE_INT64, _R, None, False), ("strings", 9, _F.TYPE_BYTES, _R, None, False),
                           ("type", 20, _F.TYPE_INT32, _O, None, False)])
    msg("NodeProto", [("input", 1, _F.TYPE_STRING, _R, None, False), ("output", 2, _F.TYPE_STRING, _R, None, False),
                      ("name", 3, _F.TYPE_STRING, _O, None, False), ("op_type", 4, _F.TYPE_STRING, _O, None, False),
                      ("attribute", 5, _F.TYPE_MESSAGE, _R, "AttributeProto", False),
                      ("doc_string", 6, _F.TYPE_STRING, _O, None, False), ("domain", 7, _F.TYPE_STRING, _O, None, False)])
    msg("GraphProto", [("node", 1, _F.TYPE_MESSAGE, _R, "NodeProto", False), ("name", 2, _F.TYPE_STRING, _O, None, False),
                       ("initializer", 5, _F.TYPE_MESSAGE, _R, "TensorProto", False),
                       ("doc_string", 10, _F.TYPE_STRING, _O, None, False),
                       ("input", 11, _F.TYPE_MESSAGE, _R, "ValueInfoProto", False),
                       ("output", 12, _F.TYPE_MESSAGE, _R, "ValueInfoProto", False),
                       ("value_info", 13, _F.TYPE_MESSAGE, _R, "ValueInfoProto", False)])
    msg("OperatorSetIdProto", [("domain", 1, _F.TYPE_STRING, _O, None, False), ("version", 2, _F.TYPE_INT64, _O, None, False)])
    msg("ModelProto", [("ir_version", 1, _F.TYPE_INT64, _O, None, False), ("producer_name", 2, _F.TYPE_STRING, _O, None, False),
                       ("producer_version", 3, _F.TYPE_STRING, _O, None, False), ("domain", 4, _F.TYPE_STRING, _O, None, False),
                       ("model_version", 5, _F.TYPE_INT64, _O, None, False), ("doc_string", 6, _F.TYPE_STRING, _O, None, False),
                       ("graph", 7, _F.TYPE_MESSAGE, _O, "GraphProto", False),
                       ("opset_import", 8, _F.TYPE_MESSAGE, _R, "OperatorSetIdProto", False)])
    pool = descriptor_pool.DescriptorPool()
    pool.Add(fd)
    return {n: message_factory.GetMessageClass(pool.FindMessageTypeByName("onnx_subset." + n))
            for n in ("ModelProto", "TensorProto")}


_CLS = None


def classes():
    global _CLS
    if _CLS is None:
        _CLS = _classes()
    return _CLS


def _fill_value_info(vi, name, shape, dynamic_first=False):
    vi.name = name
    vi.type.tensor_type.elem_type = FLOAT
    for i, d in enumerate(shape):
        dim = vi.type.tensor_type.shape.dim.add()
        if dynamic_first and i == 0:
            dim.dim_param = "batch"
        else:
            dim.dim_value = int(d)


def net_to_onnx(net, float_data=(), external=(), dynamic_batch=False, unnamed_nodes=False, extra_attrs=None,
                producer=("recipe-writer", "1.0")):
    """Recipe dict -> ModelProto bytes.  ``float_data``: initialiser names stored in the typed float_data /
    int64_data fields instead of raw_data; ``external``: names stored as external-data references (no bytes in
    the file); ``dynamic_batch``: the first input/output dimension becomes symbolic; ``unnamed_nodes``: node
    names are left empty; ``extra_attrs``: {node name: {attr: value}} added on top (floats / strings lists,
    tensors as numpy arrays)."""
    m = classes()["ModelProto"]()
    m.ir_version = 8
    m.producer_name, m.producer_version = producer
    m.doc_string = "written by tests/onnx_schema.py"
    op = m.opset_import.add()
    op.domain, op.version = "", 18
    g = m.graph
    g.name = "main_graph"
    for name, shape in net["inputs"].items():
        _fill_value_info(g.input.add(), name, shape, dynamic_batch)
    for name, shape in net["outputs"].items():
        _fill_value_info(g.output.add(), name, shape, dynamic_batch)
    for name, shape in net.get("values", {}).items():
        _fill_value_info(g.value_info.add(), name, shape)
    for name, arr in net["inits"].items():
        a = np.asarray(arr)
        t = g.initializer.add()
        t.name = name
        t.dims.extend(int(d) for d in a.shape)
        t.data_type = INT64 if a.dtype == np.int64 else FLOAT
        if name in external:
            t.data_location = 1
            for k, v in (("location", "weights.bin"), ("offset", "0"), ("length", str(a.nbytes))):
                e = t.external_data.add()
                e.key, e.value = k, v
        elif name in float_data:
            if a.dtype == np.int64:
                t.int64_data.extend(int(v) for v in a.reshape(-1))
            else:
                t.float_data.extend(float(v) for v in a.astype(np.float32).reshape(-1))
        else:
            t.raw_data = (a if a.dtype == np.int64 else a.astype(np.float32)).tobytes()
    for n in net["nodes"]:
        node = g.node.add()
        node.op_type = n["op"]
        if not unnamed_nodes:
            node.name = n["name"]
        node.input.extend(n["inputs"])
        node.output.extend(n["outputs"])
        attrs = dict(n["attrs"])
        attrs.update((extra_attrs or {}).get(n["name"], {}))
        for k, v in attrs.items():
            a = node.attribute.add()
            a.name = k
            if isinstance(v, np.ndarray):
                a.type = A_TENSOR
                a.t.dims.extend(int(d) for d in v.shape)
                a.t.data_type = FLOAT
                a.t.raw_data = v.astype(np.float32).tobytes()
            elif isinstance(v, (list, tuple)) and v and isinstance(v[0], float):
                a.type = A_FLOATS
                a.floats.extend(v)
            elif isinstance(v, (list, tuple)) and v and isinstance(v[0], str):
                a.type = A_STRINGS
                a.strings.extend(s.encode() for s in v)
            elif isinstance(v, (list, tuple)):
                a.type = A_INTS
                a.ints.extend(int(x) for x in v)
            elif isinstance(v, float):
                a.type = A_FLOAT
                a.f = v
            elif isinstance(v, str):
                a.type = A_STRING
                a.s = v.encode()
            else:
                a.type = A_INT
                a.i = int(v)
    return m.SerializeToString()


def _fnv1a(data):
    h = 1469598103934665603
    for b in bytes(data):
        h = ((h ^ b) * 1099511628211) & 0xFFFFFFFFFFFFFFFF
    return h


def _tensor_bytes(t):
    """TensorProto -> (tbn dtype enumerator, dims, bytes) under the reference's conversion rules."""
    dtype = _TBN_DTYPE.get(t.data_type, 0)
    npt = _NP[dtype]
    dims = [int(d) for d in t.dims]
    count = int(np.prod(dims)) if dims else 1
    out = np.zeros(count, dtype=npt)
    raw = bytes(t.raw_data)
    if raw:
        buf = bytearray(out.tobytes())
        n = min(len(buf), len(raw))
        buf[:n] = raw[:n]
        return dtype, dims, bytes(buf)
    for src in (t.float_data, t.int32_data, t.int64_data):
        if len(src):
            vals = np.asarray(list(src))
            if src is t.float_data:
                buf = bytearray(out.tobytes())
                rawf = vals.astype(np.float32).tobytes()
                n = min(len(buf), len(rawf))
                buf[:n] = rawf[:n]
                return dtype, dims, bytes(buf)
            tgt = npt if not (src is t.int64_data and dtype != 6) else np.int32
            n = min(count, len(vals))
            conv = np.zeros(count, dtype=tgt)
            conv[:n] = vals[:n].astype(tgt)
            return dtype, dims, conv.tobytes()[:out.nbytes]
    return dtype, dims, out.tobytes()


def _dims_text(dims):
    return ",".join(str(d) for d in dims) if len(dims) else "-"


def _g9(x):
    return "%.9g" % float(np.float32(x))


def canonical_dump(model_bytes):
    m = classes()["ModelProto"]()
    m.ParseFromString(model_bytes)
    g = m.graph
    lines = [f"producer {m.producer_name}|{m.producer_version}"]
    info = {}

    def shape_of(vi):
        return [int(d.dim_value) if d.HasField("dim_value") else 1 for d in vi.type.tensor_type.shape.dim]

    for vi in g.input:
        info[vi.name] = shape_of(vi)
    for vi in g.output:
        info[vi.name] = shape_of(vi)
    for vi in g.value_info:
        info[vi.name] = shape_of(vi)
    lines += [f"input {vi.name} {_dims_text(info[vi.name])}" for vi in g.input]
    lines += [f"output {vi.name} {_dims_text(info[vi.name])}" for vi in g.output]
    lines += [f"value {k} {_dims_text(info[k])}" for k in sorted(info)]
    inits = {}
    for t in g.initializer:
        inits[t.name] = _tensor_bytes(t)
    for name in sorted(inits):
        dtype, dims, data = inits[name]
        lines.append(f"init {name} dtype={dtype} dims={_dims_text(dims)} bytes={len(data)} fnv={_fnv1a(data):016x}")
    for n in g.node:
        name = n.name or (n.op_type + "_" + (n.output[0] if len(n.output) else ""))
        parts = [f"node {n.op_type} {name} [{','.join(n.input)}] -> [{','.join(n.output)}]"]
        rendered = {}
        for a in n.attribute:
            if a.type == A_INT:
                rendered[a.name] = f"i:{a.i}"
            elif a.type == A_FLOAT:
                rendered[a.name] = "f:" + _g9(a.f)
            elif a.type == A_STRING:
                rendered[a.name] = "s:" + a.s.decode()
            elif a.type == A_INTS:
                rendered[a.name] = "I:" + ",".join(str(v) for v in a.ints)
            elif a.type == A_FLOATS:
                rendered[a.name] = "F:" + ",".join(_g9(v) for v in a.floats)
            elif a.type == A_STRINGS:
                rendered[a.name] = "S:" + ",".join(v.decode() for v in a.strings)
            elif a.type == A_TENSOR:
                _, dims, data = _tensor_bytes(a.t)
                rendered[a.name] = f"t:{_dims_text(dims)}:{_fnv1a(data):016x}"
        parts += [f"{k}={rendered[k]}" for k in sorted(rendered)]
        lines.append(" ".join(parts))
    return "\n".join(lines) + "\n"
