"""A few dozen lines of protobuf wire format: enough to WRITE small frozen TensorFlow GraphDefs
for the parser tests and to READ one back, without TensorFlow.  Written independently of the C++
reader in forward_b200/csrc/tf_cvt/tf_graph.cpp so that the two check each other.

Field numbers (TensorFlow's published graph.proto / node_def.proto / attr_value.proto /
tensor.proto / tensor_shape.proto): GraphDef.node = 1; NodeDef name 1, op 2, input 3, attr 5
(map entry: key 1, value 2); AttrValue s 2, i 3, f 4, b 5, type 6, shape 7, tensor 8;
TensorProto dtype 1, tensor_shape 2, tensor_content 4, float_val 5, int_val 7;
TensorShapeProto dim 2 (size 1).
"""
from __future__ import annotations

import struct

import numpy as np

DT_FLOAT, DT_INT32, DT_HALF = 1, 3, 19
_NP = {DT_FLOAT: np.float32, DT_INT32: np.int32, DT_HALF: np.float16}
_DT = {np.dtype(np.float32): DT_FLOAT, np.dtype(np.int32): DT_INT32, np.dtype(np.float16): DT_HALF}


# ---- writing ---------------------------------------------------------------------------------

def _varint(v: int) -> bytes:
    v &= (1 << 64) - 1
    out = bytearray()
    while True:
        b = v & 0x7F
        v >>= 7
        if v:
            out.append(b | 0x80)
        else:
            out.append(b)
            return bytes(out)


def _key(field: int, wire: int) -> bytes:
    return _varint(field << 3 | wire)


def _ld(field: int, payload: bytes) -> bytes:
    return _key(field, 2) + _varint(len(payload)) + payload


def _vi(field: int, v: int) -> bytes:
    return _key(field, 0) + _varint(v)


def shape_proto(dims) -> bytes:
    return b"".join(_ld(2, _vi(1, int(d))) for d in dims)


def tensor_proto(arr: np.ndarray, *, as_values: bool = False, repeat_last: int = 0) -> bytes:
    """tensor_content by default; `as_values` writes float_val / int_val instead (packed), and
    `repeat_last` = N drops all but the first N values (readers must repeat the last one)."""
    arr = np.asarray(arr)
    dt = _DT[arr.dtype]
    out = _vi(1, dt) + _ld(2, shape_proto(arr.shape))
    if not as_values:
        return out + _ld(4, arr.tobytes())
    flat = arr.reshape(-1)
    if repeat_last:
        flat = flat[:repeat_last]
    if dt == DT_FLOAT:
        return out + _ld(5, b"".join(struct.pack("<f", float(x)) for x in flat))
    return out + _ld(7, b"".join(_varint(int(x)) for x in flat))


def attr_tensor(arr, **kw) -> bytes:
    return _ld(8, tensor_proto(arr, **kw))


def attr_type(dt: int) -> bytes:
    return _vi(6, dt)


def attr_shape(dims) -> bytes:
    return _ld(7, shape_proto(dims))


def attr_bool(v: bool) -> bytes:
    return _vi(5, 1 if v else 0)


def attr_int(v: int) -> bytes:
    return _vi(3, v)


def node(name: str, op: str, inputs=(), **attrs) -> bytes:
    body = _ld(1, name.encode()) + _ld(2, op.encode())
    for i in inputs:
        body += _ld(3, i.encode())
    for k, v in attrs.items():
        body += _ld(5, _ld(1, k.encode()) + _ld(2, v))
    return _ld(1, body)


def const(name: str, arr, **kw) -> bytes:
    arr = np.asarray(arr)
    return node(name, "Const", value=attr_tensor(arr, **kw), dtype=attr_type(_DT[arr.dtype]))


def fm_graph(table: np.ndarray, length: int, *, identity: bool = True, gather_axis: int = 0,
             sum_axis: int = 1, keep_dims: bool = False, table_placeholder: bool = False,
             weights_node: np.ndarray | None = None, table_as_values: bool = False) -> bytes:
    """The second-order factorisation-machine term  (sum_l e)^2 - sum_l e^2  over a gathered
    [batch, length, dim] tensor e = table[indices] * mask, laid out like the graph the reference
    tests with (GatherV2 -> Identity -> Mul -> Sum / Square -> Sum; output "sub")."""
    g = b""
    if table_placeholder:
        g += node("emb/table", "Placeholder", dtype=attr_type(DT_FLOAT), shape=attr_shape(table.shape))
    else:
        g += const("emb/table", table, as_values=table_as_values)
    if weights_node is not None:
        g += const("emb_weights", weights_node)
    g += node("emb/read", "Identity", ["emb/table"], T=attr_type(_DT[np.asarray(table).dtype]))
    g += node("ids", "Placeholder", dtype=attr_type(DT_INT32), shape=attr_shape([-1, length]))
    g += const("emb/axis", np.array(gather_axis, dtype=np.int32), as_values=True)
    g += node("emb/gather", "GatherV2", ["emb/read", "ids", "emb/axis"], batch_dims=attr_int(0))
    src = "emb/gather"
    if identity:
        g += node("emb/gather/Identity", "Identity", [src])
        src = "emb/gather/Identity"
    g += const("mask", np.ones((length, 1), dtype=np.float32), as_values=True, repeat_last=1)
    g += node("mul", "Mul", [src, "mask"])
    g += const("Sum/axes", np.array(sum_axis, dtype=np.int32), as_values=True)
    g += node("Sum", "Sum", ["mul", "Sum/axes"], keep_dims=attr_bool(keep_dims))
    g += node("Square", "Square", ["mul"])
    g += const("Sum_1/axes", np.array(1, dtype=np.int32), as_values=True)
    g += node("Sum_1", "Sum", ["Square", "Sum_1/axes:0"], keep_dims=attr_bool(False))
    g += node("Square_1", "Square", ["Sum"])
    g += node("sub", "Sub", ["Square_1", "Sum_1", "^ids"])
    return g


def gather_graph(table: np.ndarray, length: int) -> bytes:
    g = const("w", table)
    g += node("ids", "Placeholder", dtype=attr_type(DT_INT32), shape=attr_shape([-1, length]))
    g += const("axis", np.array(0, dtype=np.int32), as_values=True)
    g += node("lookup", "GatherV2", ["w", "ids", "axis"])
    g += node("out", "Identity", ["lookup"])
    return g


# ---- reading -----------------------------------------------------------------------------------

def _read_varint(b: bytes, i: int):
    r = s = 0
    while True:
        c = b[i]
        i += 1
        r |= (c & 0x7F) << s
        s += 7
        if not c & 0x80:
            return r, i


def fields(b: bytes):
    i, out = 0, []
    while i < len(b):
        key, i = _read_varint(b, i)
        f, w = key >> 3, key & 7
        if w == 0:
            v, i = _read_varint(b, i)
        elif w == 2:
            n, i = _read_varint(b, i)
            v = b[i:i + n]
            i += n
        elif w == 5:
            v = b[i:i + 4]
            i += 4
        elif w == 1:
            v = b[i:i + 8]
            i += 8
        else:
            raise ValueError(f"wire type {w}")
        out.append((f, w, v))
    return out


def read_nodes(graph: bytes) -> dict:
    """{name: {"op": str, "inputs": [str], "attrs": {key: raw AttrValue bytes}}}"""
    nodes = {}
    for f, w, v in fields(graph):
        if f != 1:
            continue
        n = {"op": "", "inputs": [], "attrs": {}}
        name = ""
        for ff, ww, x in fields(v):
            if ff == 1:
                name = x.decode()
            elif ff == 2:
                n["op"] = x.decode()
            elif ff == 3:
                n["inputs"].append(x.decode())
            elif ff == 5:
                kv = fields(x)
                n["attrs"][kv[0][2].decode()] = kv[1][2]
        nodes[name] = n
    return nodes


def const_value(attr_value: bytes) -> np.ndarray:
    """The dense array of a Const node's `value` attribute (tensor_content only)."""
    tensor = [x for f, w, x in fields(attr_value) if f == 8][0]
    dtype, dims, content = None, [], None
    for f, w, x in fields(tensor):
        if f == 1:
            dtype = x
        elif f == 2:
            dims = [[y for g, _, y in fields(d) if g == 1][0] for ff, _, d in fields(x) if ff == 2]
        elif f == 4:
            content = x
    return np.frombuffer(content, dtype=_NP[dtype]).reshape(dims).copy()
