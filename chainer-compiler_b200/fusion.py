"""Elementwise fusion: grouping and kernel-source generation.

Thin Python front of the C++ implementations in ``csrc/fusion.cc`` (grouping, the counterpart of
``compiler/fusion_elementwise.cc:10-40`` + ``compiler/fusion.cc:165-214``) and ``csrc/eltwise.cc``
(source generation, the counterpart of ``compiler/nvrtc_builder.cc:91-206``).  A graph is a list of
``Node`` in any order; values are identified by their names, as in ONNX.
"""
import ctypes
from collections import namedtuple

from . import _lib
from ._lib import EW_OPS, EwNode, GraphNode, GraphValue, check, lib

Node = namedtuple("Node", ["op_type", "inputs", "outputs", "value", "is_grad"])
Node.__new__.__defaults__ = (None, False)

FusionGroup = namedtuple("FusionGroup", ["fusion_id", "node_indices", "inputs", "outputs", "temps"])

_DTYPE_CODES = {None: 0, "float16": _lib.FLOAT16, "float32": _lib.FLOAT32, "float64": _lib.FLOAT64, "int8": _lib.INT8, "uint8": _lib.UINT8,
                "int32": _lib.INT32, "int64": _lib.INT64, "bool": _lib.BOOL, "int16": _lib.INT16}


def _value_table(nodes):
    names = []
    index = {}
    for nd in nodes:
        for v in list(nd.inputs) + list(nd.outputs):
            if v is not None and v not in index:
                index[v] = len(names)
                names.append(v)
    return names, index


def classify_values(nodes, member_indices, graph_outputs=()):
    """Inputs, outputs and temporaries of a node set, each sorted by value name (compiler/topology.cc:15-58)."""
    members = set(member_indices)
    users = {}
    for i, nd in enumerate(nodes):
        for v in nd.inputs:
            users.setdefault(v, []).append(i)
    produced, read = set(), set()
    for i in members:
        produced.update(nodes[i].outputs)
        read.update(v for v in nodes[i].inputs if v is not None)
    inputs = sorted(read - produced)
    outputs = []
    for v in sorted(produced):
        outside = [u for u in users.get(v, []) if u not in members]
        if outside or v in graph_outputs:
            outputs.append(v)
    temps = sorted(produced - set(outputs))
    return inputs, outputs, temps


def fuse_elementwise(nodes, value_dtypes=None, graph_outputs=()):
    """Returns the list of FusionGroup the reference's --fuse_operations pass would form over `nodes`."""
    value_dtypes = value_dtypes or {}
    names, index = _value_table(nodes)
    gvals = (GraphValue * max(1, len(names)))()
    for i, nm in enumerate(names):
        gvals[i].dtype = _DTYPE_CODES[value_dtypes.get(nm)]
        gvals[i].is_graph_output = int(nm in graph_outputs)
    gnodes = (GraphNode * max(1, len(nodes)))()
    keep = []
    for i, nd in enumerate(nodes):
        ins = (ctypes.c_int32 * max(1, len(nd.inputs)))(*[index[v] if v is not None else -1 for v in nd.inputs])
        outs = (ctypes.c_int32 * max(1, len(nd.outputs)))(*[index[v] for v in nd.outputs])
        keep.extend([ins, outs])
        gnodes[i].op_type = nd.op_type.encode()
        gnodes[i].inputs, gnodes[i].n_inputs = ins, len(nd.inputs)
        gnodes[i].outputs, gnodes[i].n_outputs = outs, len(nd.outputs)
        gnodes[i].is_grad = int(bool(nd.is_grad))
        if nd.op_type == "Constant":
            import numpy as np
            arr = np.asarray(nd.value)
            gnodes[i].const_is_float = int(arr.dtype.kind == "f")
            gnodes[i].const_num_elements = int(arr.size)
    group_of = (ctypes.c_int32 * max(1, len(nodes)))()
    n_groups = ctypes.c_int32(0)
    check(lib().chxq_fuse_elementwise(gnodes, len(nodes), gvals, len(names), group_of, ctypes.byref(n_groups)))
    groups = []
    for gid in range(1, n_groups.value + 1):
        idx = [i for i in range(len(nodes)) if group_of[i] == gid]
        ins, outs, temps = classify_values(nodes, idx, graph_outputs)
        groups.append(FusionGroup(gid, idx, ins, outs, temps))
    return groups


def build_program(nodes, fusion_id, inputs, outputs, dtype="float32"):
    """CUDA source of one fused group: `nodes` (any order), its input and output value names.

    Same contract as BuildNvrtcProgram (compiler/nvrtc_builder.cc:91): kernel `fusion<id>(n, inputs..., outputs...)`
    with the arguments in the given order.
    """
    import numpy as np
    names, index = _value_table(nodes)
    for v in list(inputs) + list(outputs):
        if v not in index:
            raise _lib.ChxqError(_lib.ERR_INVALID_ARGUMENT, "value %r does not occur in the group" % v)
    arr = (EwNode * len(nodes))()
    for i, nd in enumerate(nodes):
        if nd.op_type not in EW_OPS:
            raise _lib.ChxqError(_lib.ERR_UNSUPPORTED, "Cannot build a fused kernel for %s" % nd.op_type)  # nvrtc_builder.cc:84-86
        arr[i].op = EW_OPS[nd.op_type]
        ins = [index[v] for v in nd.inputs]
        arr[i].inputs[0] = ins[0] if len(ins) > 0 else -1
        arr[i].inputs[1] = ins[1] if len(ins) > 1 else -1
        arr[i].output = index[nd.outputs[0]]
        if nd.op_type == "Constant":
            v = np.asarray(nd.value)
            if v.size != 1:
                raise _lib.ChxqError(_lib.ERR_INVALID_ARGUMENT, "fused constants must have one element")  # nvrtc_builder.cc:168
            arr[i].constant = float(v.reshape(-1)[0])
    in_ids = (ctypes.c_int32 * len(inputs))(*[index[v] for v in inputs])
    out_ids = (ctypes.c_int32 * len(outputs))(*[index[v] for v in outputs])
    cnames = (ctypes.c_char_p * len(names))(*[n.encode() for n in names])
    needed = ctypes.c_size_t(0)
    code = _lib.DTYPE_BY_NAME[dtype]
    check(lib().chxq_eltwise_codegen(arr, len(nodes), in_ids, len(inputs), out_ids, len(outputs), cnames, len(names), code, fusion_id, None, 0,
                                     ctypes.byref(needed)))
    buf = ctypes.create_string_buffer(needed.value)
    check(lib().chxq_eltwise_codegen(arr, len(nodes), in_ids, len(inputs), out_ids, len(outputs), cnames, len(names), code, fusion_id, buf,
                                     needed.value, ctypes.byref(needed)))
    return buf.value.decode()


def lstm_cell_group():
    """The pointwise part of an LSTM cell as a node list (testcases/ch2o_tests/model/StatelessLSTM.py:26-37 in the
    reference): c' = tanh(a) * sigmoid(i) + sigmoid(f) * c ; h = sigmoid(o) * tanh(c')."""
    N = Node
    return [
        N("Tanh", ["a"], ["ta"]),
        N("Sigmoid", ["i"], ["si"]),
        N("Sigmoid", ["f"], ["sf"]),
        N("Sigmoid", ["o"], ["so"]),
        N("Mul", ["ta", "si"], ["m1"]),
        N("Mul", ["sf", "c_prev"], ["m2"]),
        N("Add", ["m1", "m2"], ["c_next"]),
        N("Tanh", ["c_next"], ["tc"]),
        N("Mul", ["so", "tc"], ["h"]),
    ]
