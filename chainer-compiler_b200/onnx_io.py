"""Minimal ONNX reader / writer: the protobuf wire format of ModelProto, GraphProto, NodeProto, AttributeProto,
ValueInfoProto and TensorProto, enough to load the models and test directories `run_onnx` takes (reference:
tools/run_onnx_util.cc:41-175, compiler/model.cc, compiler/tensor.cc) and to write test directories of the same format.
No `onnx` / `protobuf` package is involved.

Tensor payload rules mirrored from compiler/tensor.cc:95-137,179-207: `raw_data` excludes the typed fields; otherwise
bool / int8 / int16 / int32 / uint8 / float16 bits come from `int32_data`, int64 from `int64_data`, float from `float_data`,
double from `double_data`; the writer emits typed fields, as the reference does, not `raw_data`."""
import os
import struct

import numpy as np

# TensorProto.DataType
FLOAT, UINT8, INT8, UINT16, INT16, INT32, INT64, STRING, BOOL, FLOAT16, DOUBLE = 1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11
_NP = {FLOAT: np.float32, UINT8: np.uint8, INT8: np.int8, UINT16: np.uint16, INT16: np.int16, INT32: np.int32, INT64: np.int64, BOOL: np.bool_,
       FLOAT16: np.float16, DOUBLE: np.float64}
_CODE = {np.dtype(v): k for k, v in _NP.items()}


class OnnxError(ValueError):
    pass


# ---- wire format -----------------------------------------------------------------------------------------------------
def _varint(buf, i):
    r = s = 0
    while True:
        if i >= len(buf):
            raise OnnxError("truncated varint")
        c = buf[i]
        i += 1
        r |= (c & 0x7F) << s
        s += 7
        if c < 0x80:
            return r, i
        if s > 70:
            raise OnnxError("varint too long")


def _fields(buf):
    """Yields (field number, wire type, value): int for varints, bytes for the rest."""
    i, n = 0, len(buf)
    while i < n:
        key, i = _varint(buf, i)
        f, w = key >> 3, key & 7
        if w == 0:
            v, i = _varint(buf, i)
        elif w == 1:
            v, i = bytes(buf[i:i + 8]), i + 8
        elif w == 2:
            ln, i = _varint(buf, i)
            if i + ln > n:
                raise OnnxError("truncated length-delimited field %d" % f)
            v, i = bytes(buf[i:i + ln]), i + ln
        elif w == 5:
            v, i = bytes(buf[i:i + 4]), i + 4
        else:
            raise OnnxError("unsupported wire type %d" % w)
        yield f, w, v


def _signed(v):
    return v - (1 << 64) if v >= (1 << 63) else v


def _packed_varints(w, v):
    if w == 0:
        return [_signed(v)]
    out, i = [], 0
    while i < len(v):
        x, i = _varint(v, i)
        out.append(_signed(x))
    return out


def _enc_varint(v):
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


def _enc_field(f, w, payload):
    if w == 0:
        return _enc_varint((f << 3) | 0) + _enc_varint(payload)
    if w == 2:
        return _enc_varint((f << 3) | 2) + _enc_varint(len(payload)) + payload
    if w == 5:
        return _enc_varint((f << 3) | 5) + payload
    raise OnnxError("unsupported wire type %d" % w)


# ---- TensorProto -----------------------------------------------------------------------------------------------------
def parse_tensor(buf):
    """TensorProto bytes -> (name, numpy array)."""
    dims, dtype, name, raw = [], None, "", None
    f32, i32, i64, f64 = [], [], [], []
    for f, w, v in _fields(buf):
        if f == 1:
            dims += _packed_varints(w, v)
        elif f == 2:
            dtype = v
        elif f == 4:
            f32.append(v if w == 2 else v)  # packed floats or one fixed32
        elif f == 5:
            i32 += _packed_varints(w, v)
        elif f == 7:
            i64 += _packed_varints(w, v)
        elif f == 8:
            name = v.decode()
        elif f == 9:
            raw = v
        elif f == 10:
            f64.append(v)
    if dtype not in _NP:
        raise OnnxError("tensor %r: unsupported data type %r" % (name, dtype))
    np_dt = np.dtype(_NP[dtype])
    typed = bool(f32 or i32 or i64 or f64)
    if raw is not None and typed:
        raise OnnxError("tensor %r: raw_data together with typed data" % name)
    if raw is not None:
        arr = np.frombuffer(raw, dtype=np_dt.newbyteorder("<")).astype(np_dt)
    elif dtype == FLOAT:
        arr = np.frombuffer(b"".join(f32), dtype="<f4").astype(np.float32)
    elif dtype == DOUBLE:
        arr = np.frombuffer(b"".join(f64), dtype="<f8").astype(np.float64)
    elif dtype == INT64:
        arr = np.array(i64, dtype=np.int64)
    elif dtype == FLOAT16:
        arr = np.array(i32, dtype=np.int64).astype(np.uint16).view(np.float16)
    else:
        arr = np.array(i32, dtype=np.int64).astype(np_dt)
    n = int(np.prod(dims)) if dims else 1
    if arr.size != n:
        raise OnnxError("tensor %r: %d values for shape %r" % (name, arr.size, dims))
    return name, arr.reshape(dims)


def serialize_tensor(arr, name=""):
    """numpy array -> TensorProto bytes with typed data fields."""
    arr = np.asarray(arr)
    if arr.dtype not in _CODE:
        raise OnnxError("unsupported dtype %s" % arr.dtype)
    code = _CODE[arr.dtype]
    out = bytearray()
    for d in arr.shape:
        out += _enc_field(1, 0, int(d))
    out += _enc_field(2, 0, code)
    flat = np.ascontiguousarray(arr).reshape(-1)
    if code == FLOAT:
        out += _enc_field(4, 2, flat.astype("<f4").tobytes())
    elif code == DOUBLE:
        out += _enc_field(10, 2, flat.astype("<f8").tobytes())
    elif code == INT64:
        out += _enc_field(7, 2, b"".join(_enc_varint(int(v)) for v in flat))
    elif code == FLOAT16:
        out += _enc_field(5, 2, b"".join(_enc_varint(int(v)) for v in flat.view(np.uint16)))
    else:
        out += _enc_field(5, 2, b"".join(_enc_varint(int(v)) for v in flat.astype(np.int64)))
    if name:
        out += _enc_field(8, 2, name.encode())
    return bytes(out)


# ---- graph -----------------------------------------------------------------------------------------------------------
class Node:
    def __init__(self, op_type, inputs, outputs, attrs, name=""):
        self.op_type, self.inputs, self.outputs, self.attrs, self.name = op_type, list(inputs), list(outputs), dict(attrs), name

    def __repr__(self):
        return "%s(%s) -> %s %s" % (self.op_type, ", ".join(self.inputs), ", ".join(self.outputs), self.attrs or "")


class Model:
    def __init__(self, nodes, initializers, inputs, outputs, ir_version=3, opset=8, name="graph"):
        self.nodes, self.initializers, self.inputs, self.outputs = nodes, initializers, inputs, outputs
        self.ir_version, self.opset, self.name = ir_version, opset, name


def _parse_attr(buf):
    name, f, i, s, t, floats, ints, typ = "", None, None, None, None, [], [], None
    for fld, w, v in _fields(buf):
        if fld == 1:
            name = v.decode()
        elif fld == 2:
            f = struct.unpack("<f", v)[0]
        elif fld == 3:
            i = _signed(v)
        elif fld == 4:
            s = v
        elif fld == 5:
            t = parse_tensor(v)[1]
        elif fld == 7:
            floats += list(np.frombuffer(v, "<f4")) if w == 2 else [struct.unpack("<f", v)[0]]
        elif fld == 8:
            ints += _packed_varints(w, v)
        elif fld == 20:
            typ = v
    if typ == 1 or (typ is None and f is not None):
        return name, float(f)
    if typ == 2 or (typ is None and i is not None):
        return name, int(i)
    if typ == 3 or (typ is None and s is not None):
        return name, s.decode(errors="replace")
    if typ == 4 or (typ is None and t is not None):
        return name, t
    if typ == 6 or (typ is None and floats):
        return name, [float(x) for x in floats]
    if typ == 7 or (typ is None and ints):
        return name, [int(x) for x in ints]
    return name, None


def _parse_value_info_name(buf):
    for f, w, v in _fields(buf):
        if f == 1:
            return v.decode()
    return ""


def parse_model(buf):
    ir_version, opset, graph = 0, 0, None
    for f, w, v in _fields(buf):
        if f == 1:
            ir_version = v
        elif f == 7:
            graph = v
        elif f == 8:
            for ff, ww, vv in _fields(v):
                if ff == 2:
                    opset = vv
    if graph is None:
        raise OnnxError("no graph in the model")
    nodes, inits, inputs, outputs, gname = [], {}, [], [], "graph"
    for f, w, v in _fields(graph):
        if f == 1:
            op, ins, outs, attrs, nname = "", [], [], {}, ""
            for ff, ww, vv in _fields(v):
                if ff == 1:
                    ins.append(vv.decode())
                elif ff == 2:
                    outs.append(vv.decode())
                elif ff == 3:
                    nname = vv.decode()
                elif ff == 4:
                    op = vv.decode()
                elif ff == 5:
                    k, val = _parse_attr(vv)
                    attrs[k] = val
            nodes.append(Node(op, ins, outs, attrs, nname))
        elif f == 2:
            gname = v.decode()
        elif f == 5:
            n, a = parse_tensor(v)
            inits[n] = a
        elif f == 11:
            inputs.append(_parse_value_info_name(v))
        elif f == 12:
            outputs.append(_parse_value_info_name(v))
    return Model(nodes, inits, [i for i in inputs if i not in inits], outputs, ir_version, opset, gname)


def _ser_attr(name, val):
    out = bytearray(_enc_field(1, 2, name.encode()))
    if isinstance(val, float):
        out += _enc_field(2, 5, struct.pack("<f", val)) + _enc_field(20, 0, 1)
    elif isinstance(val, (int, np.integer)):
        out += _enc_field(3, 0, int(val)) + _enc_field(20, 0, 2)
    elif isinstance(val, str):
        out += _enc_field(4, 2, val.encode()) + _enc_field(20, 0, 3)
    elif isinstance(val, np.ndarray):
        out += _enc_field(5, 2, serialize_tensor(val)) + _enc_field(20, 0, 4)
    elif isinstance(val, (list, tuple)) and val and isinstance(val[0], float):
        for x in val:
            out += _enc_field(7, 5, struct.pack("<f", x))
        out += _enc_field(20, 0, 6)
    elif isinstance(val, (list, tuple)):
        for x in val:
            out += _enc_field(8, 0, int(x))
        out += _enc_field(20, 0, 7)
    else:
        raise OnnxError("attribute %s: unsupported value %r" % (name, val))
    return bytes(out)


def serialize_model(model):
    g = bytearray()
    for n in model.nodes:
        nb = bytearray()
        for i in n.inputs:
            nb += _enc_field(1, 2, i.encode())
        for o in n.outputs:
            nb += _enc_field(2, 2, o.encode())
        if n.name:
            nb += _enc_field(3, 2, n.name.encode())
        nb += _enc_field(4, 2, n.op_type.encode())
        for k, v in n.attrs.items():
            if v is not None:
                nb += _enc_field(5, 2, _ser_attr(k, v))
        g += _enc_field(1, 2, bytes(nb))
    g += _enc_field(2, 2, model.name.encode())
    for name, arr in model.initializers.items():
        g += _enc_field(5, 2, serialize_tensor(arr, name))
    for name in list(model.inputs) + list(model.initializers):
        g += _enc_field(11, 2, _enc_field(1, 2, name.encode()))
    for name in model.outputs:
        g += _enc_field(12, 2, _enc_field(1, 2, name.encode()))
    out = bytearray(_enc_field(1, 0, model.ir_version))
    out += _enc_field(7, 2, bytes(g))
    out += _enc_field(8, 2, _enc_field(1, 2, b"") + _enc_field(2, 0, model.opset))
    return bytes(out)


# ---- test directories (tools/run_onnx_util.cc:41-175) ------------------------------------------------------------------
def load_model(path):
    with open(path, "rb") as f:
        return parse_model(f.read())


def load_test_dir(test_dir):
    """Returns (model, [(inputs: {name: array} in file order, outputs: [(name, array)])...]) of DIR/model.onnx and
    DIR/test_data_set_*/{input,output}_*.pb.  Unnamed input tensors take the graph's input names in order, as the reference
    does."""
    model = load_model(os.path.join(test_dir, "model.onnx"))
    cases = []
    for d in sorted(os.listdir(test_dir)):
        full = os.path.join(test_dir, d)
        if not (os.path.isdir(full) and d.startswith("test_data_set_")):
            continue
        ins, outs = [], []
        for kind, dst in (("input", ins), ("output", outs)):
            idx = 0
            while os.path.exists(os.path.join(full, "%s_%d.pb" % (kind, idx))):
                with open(os.path.join(full, "%s_%d.pb" % (kind, idx)), "rb") as f:
                    dst.append(parse_tensor(f.read()))
                idx += 1
        named_in = {}
        for k, (name, arr) in enumerate(ins):
            named_in[name if name in model.inputs else model.inputs[k]] = arr
        named_out = [(name if name else model.outputs[k], arr) for k, (name, arr) in enumerate(outs)]
        cases.append((named_in, named_out))
    return model, cases


def write_test_dir(test_dir, model, cases):
    os.makedirs(test_dir, exist_ok=True)
    with open(os.path.join(test_dir, "model.onnx"), "wb") as f:
        f.write(serialize_model(model))
    for k, (ins, outs) in enumerate(cases):
        d = os.path.join(test_dir, "test_data_set_%d" % k)
        os.makedirs(d, exist_ok=True)
        for i, (name, arr) in enumerate(ins.items()):
            with open(os.path.join(d, "input_%d.pb" % i), "wb") as f:
                f.write(serialize_tensor(arr, name))
        for i, (name, arr) in enumerate(outs):
            with open(os.path.join(d, "output_%d.pb" % i), "wb") as f:
                f.write(serialize_tensor(arr, name))
