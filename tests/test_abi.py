"""The C-ABI library on a host without a GPU: it loads, exports every symbol include/chxq.h declares, and its host-only
entry points (geometry, weight quantizer, fusion grouping, source generator, argument validation) behave as the reference's."""
import ctypes
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_header_symbols_exported(pkg):
    from chainer_compiler_b200 import _lib
    import glob
    headers = sorted(glob.glob(os.path.join(ROOT, "include", "*.h")))
    assert len(headers) >= 2
    text = "".join(open(h).read() for h in headers)
    declared = set(re.findall(r"\b(chxq_[a-z0-9_]+)\s*\(", text))
    declared -= {"chxq_conv_geom", "chxq_qconv_params", "chxq_ew_node", "chxq_graph_node", "chxq_graph_value"}
    assert len(declared) >= 25
    raw = ctypes.CDLL(_lib.LIB_PATH)
    for name in sorted(declared):
        assert hasattr(raw, name), "libchxq.so does not export %s" % name
    assert declared == set(_lib.SIGNATURES), "binding table and header disagree: %s" % (declared ^ set(_lib.SIGNATURES))
    assert pkg.lib().chxq_version() >= 100


def test_missing_library_fails_loudly(pkg, monkeypatch):
    from chainer_compiler_b200 import _lib
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", "/nonexistent/libchxq.so")
    with pytest.raises(_lib.ChxqLibraryError):
        _lib.lib()


def test_ops_refuse_cpu_tensors(ops):
    import torch
    with pytest.raises(ops.ChxqError):
        ops.QuantizeLinear(torch.zeros(4), 1.0)
    with pytest.raises(ops.ChxqError):
        ops.MatMulInteger(torch.zeros(2, 2, dtype=torch.uint8), torch.zeros(2, 2, dtype=torch.int8))


def _geom(pkg, N, C, H, W, M, Cg, KH, KW, strides, pads, group, auto_pad):
    from chainer_compiler_b200 import _lib
    g = _lib.ConvGeom()
    s = (ctypes.c_int64 * 2)(*(list(strides) + [1, 1])[:2])
    p = (ctypes.c_int64 * 2)(*(list(pads) + [0, 0])[:2])
    rc = pkg.lib().chxq_conv_resolve_geometry(N, C, H, W, M, Cg, KH, KW, s, len(strides), p, len(pads), group, auto_pad.encode(), ctypes.byref(g))
    return rc, g


@pytest.mark.parametrize("H,W,k,strides,pads,auto_pad", [(28, 28, 5, (), (), "SAME_UPPER"), (7, 9, 2, (1, 1), (), "SAME_UPPER"),
                                                        (10, 10, 3, (2, 2), (), "SAME_UPPER"), (224, 224, 7, (2, 2), (3, 3), ""),
                                                        (56, 56, 3, (), (1, 1), "NOTSET"), (9, 9, 1, (2, 2), (), "SAME_UPPER")])
def test_conv_geometry_matches_oracle(pkg, orc, H, W, k, strides, pads, auto_pad):
    rc, g = _geom(pkg, 2, 8, H, W, 16, 8, k, k, strides, pads, 1, auto_pad)
    assert rc == 0
    o = orc.conv_geometry(H, W, k, k, strides, pads, "" if auto_pad == "NOTSET" else auto_pad)
    assert (g.stride_h, g.stride_w, g.pad_top, g.pad_left, g.pad_bottom, g.pad_right, g.Ho, g.Wo) == tuple(
        o[n] for n in ("sh", "sw", "pt", "pl", "pb", "pr", "Ho", "Wo"))


def test_conv_geometry_rejects(pkg):
    rc, _ = _geom(pkg, 1, 8, 8, 8, 8, 8, 3, 3, (), (), 1, "SAME_LOWER")  # CalculateAutoPad CHECKs SAME_UPPER
    assert rc == 1 and b"SAME_UPPER" in pkg.lib().chxq_last_error()
    rc, _ = _geom(pkg, 1, 8, 8, 8, 8, 3, 3, 3, (), (), 2, "")  # C != Cg * group
    assert rc == 1
    rc, _ = _geom(pkg, 1, 8, 2, 2, 8, 8, 3, 3, (), (), 1, "")  # kernel larger than input
    assert rc == 1


@pytest.mark.parametrize("to_int8", [True, False])
@pytest.mark.parametrize("per_channel", [True, False])
def test_weight_quantizer_matches_oracle(pkg, orc, to_int8, per_channel):
    from chainer_compiler_b200 import models
    rng = np.random.default_rng(7)
    w = (rng.standard_normal((12, 5, 3, 3)) * 0.02).astype(np.float32)
    w[3] = np.abs(w[3])  # an all-positive channel: the range must still include 0
    q, s, z = models.quantize_weights(w, per_channel=per_channel, to_int8=to_int8)
    if per_channel:
        qo, so, zo = orc.quantize_weight_per_channel(w, to_int8)
    else:
        qo, so, zo = orc.quantize_data(w, to_int8)
        so, zo = np.array([so], np.float32), np.array([zo], np.int32)
    assert np.array_equal(q, qo) and np.array_equal(s, so) and np.array_equal(z, zo)
    if to_int8:
        assert q.min() >= -127  # 254 steps, never -128 (compiler/quantize.cc:79)


def test_validation_without_gpu(pkg):
    """Checks that are made on the host before any CUDA call."""
    L = pkg.lib()
    assert L.chxq_quantize_linear(None, 4, 1.0, 300, 6, 0, None, None) == 1  # zero point outside uint8 (quantize.cc:26-27)
    assert L.chxq_quantize_linear(None, 4, 1.0, -129, 2, 0, None, None) == 1
    assert L.chxq_quantize_linear(None, 4, 1.0, 0, 8, 0, None, None) == 1  # zero point dtype must be uint8 / int8 (:19-25)
    assert L.chxq_quantize_linear(None, 0, 1.0, 0, 6, 0, None, None) == 0  # empty tensor
    assert L.chxq_dequantize_linear(None, 8, 4, 1.0, 0, None, None) == 1
    assert L.chxq_matmul_integer(None, 6, None, 2, 1, 4, 4, 4, None, 3, None, 0, None, None, 0, 0, None) == 1  # zp length 3 with null ptr
    assert L.chxq_matmul_integer(None, 6, None, 2, 1, 0, 4, 4, None, 0, None, 0, None, None, 0, 0, None) == 0  # empty M
    assert L.chxq_matmul_integer(None, 8, None, 2, 1, 4, 4, 4, None, 0, None, 0, None, None, 0, 0, None) == 1  # float operand
    assert L.chxq_eltwise_run(b"", 0, None, 0, None, 0, 4, 8, None) == 1
    assert L.chxq_matmul_integer_workspace(1, 1024, 1024, 1024) >= 1024 * 1024


def test_fusion_grouping(pkg):
    from chainer_compiler_b200.fusion import Node, fuse_elementwise
    f32 = "float32"
    # compiler/fusion_test.cc:11-30: Tanh -> Sigmoid forms one group holding both nodes
    nodes = [Node("Tanh", ["x"], ["t"]), Node("Sigmoid", ["t"], ["y"])]
    groups = fuse_elementwise(nodes, {"x": f32, "t": f32, "y": f32}, graph_outputs=["y"])
    assert len(groups) == 1 and groups[0].node_indices == [0, 1] and groups[0].inputs == ["x"] and groups[0].outputs == ["y"]
    # a single calculating node is not worth a kernel (min_fuse_ops = 2); Identity / Constant do not count
    assert fuse_elementwise([Node("Tanh", ["x"], ["t"]), Node("Identity", ["t"], ["y"])], {}, ["y"]) == []
    # integer inputs are not fused (fusion_elementwise.cc:30-35); Div and Relu are not in the fusable set (:12-21)
    assert fuse_elementwise([Node("Add", ["a", "b"], ["c"]), Node("Mul", ["c", "b"], ["d"])], {"a": "int32", "b": "int32", "c": "int32"}, ["d"]) == []
    assert fuse_elementwise([Node("Div", ["a", "b"], ["c"]), Node("Relu", ["c"], ["d"])], {}, ["d"]) == []
    # scalar float constants join their user's group; unused or integer constants do not (fusion.cc:60-79, fusion_elementwise.cc:24-27)
    nodes = [Node("Constant", [], ["k"], np.float32(2.0)), Node("Mul", ["x", "k"], ["m"]), Node("Exp", ["m"], ["e"]),
             Node("Constant", [], ["unused"], np.float32(1.0)), Node("Constant", [], ["ki"], np.int64(3))]
    g = fuse_elementwise(nodes, {"x": f32}, ["e"])
    assert len(g) == 1 and g[0].node_indices == [0, 1, 2] and g[0].inputs == ["x"] and g[0].outputs == ["e"]
    # a member that depends on the group through a non-member would close a cycle and is rejected (fusion.cc:26-58)
    nodes = [Node("Tanh", ["x"], ["a"]), Node("Exp", ["a"], ["b"]), Node("Relu", ["b"], ["r"]), Node("Add", ["a", "r"], ["y"]),
             Node("Sigmoid", ["y"], ["z"])]
    g = fuse_elementwise(nodes, {}, ["z"])
    assert [grp.node_indices for grp in g] == [[0, 1], [3, 4]]
    # two disconnected chains form two groups, numbered in node order; inputs are sorted by name (topology.cc:55-58)
    nodes = [Node("Add", ["q", "p"], ["s"]), Node("Tanh", ["s"], ["t"]), Node("Sub", ["v", "u"], ["w"]), Node("Exp", ["w"], ["z"])]
    g = fuse_elementwise(nodes, {}, ["t", "z"])
    assert [grp.fusion_id for grp in g] == [1, 2] and g[0].inputs == ["p", "q"] and g[1].inputs == ["u", "v"]
    # forward and gradient nodes do not mix (fusion.cc:181,189)
    nodes = [Node("Tanh", ["x"], ["a"]), Node("Exp", ["a"], ["b"]), Node("Mul", ["b", "g"], ["c"], None, True), Node("Add", ["c", "g"], ["d"], None, True)]
    g = fuse_elementwise(nodes, {}, ["d"])
    assert [grp.node_indices for grp in g] == [[0, 1], [2, 3]]


def test_lstm_group_and_generated_source(pkg):
    from chainer_compiler_b200.fusion import build_program, fuse_elementwise, lstm_cell_group
    nodes = lstm_cell_group()
    g = fuse_elementwise(nodes, {}, ["c_next", "h"])
    assert len(g) == 1 and len(g[0].node_indices) == 9
    assert g[0].inputs == ["a", "c_prev", "f", "i", "o"] and g[0].outputs == ["c_next", "h"]
    code = build_program(nodes, 7, g[0].inputs, g[0].outputs)
    assert 'extern "C" __global__' in code and "fusion7(" in code and "fusion7_s(" in code
    # argument order: inputs then outputs, each in the given (name-sorted) order, as nvrtc_builder.cc:139-147
    sig = code[code.index("fusion7(size_t n"):]
    order = [sig.index(s) for s in ("i_a", "i_c_prev", "i_f", "i_i", "i_o", "o_c_next", "o_h")]
    assert order == sorted(order)
    assert code.count("// Sigmoid") == 3 and code.count("// Tanh") == 2 and code.count("// Mul") == 3 and code.count("// Add") == 1
    assert "uint4" in code  # 128-bit vector path
    # every node's operands are defined before use
    body = code[code.index("_elem("):code.index("extern")]
    for name in ("v_ta", "v_si", "v_sf", "v_so", "v_m1", "v_m2", "v_c_next", "v_tc", "v_h"):
        assert body.index("const T %s =" % name) < body.rindex(name)
    for dtype, store in (("float16", "__half"), ("float64", "double")):
        assert "typedef %s S;" % store in build_program(nodes, 1, g[0].inputs, g[0].outputs, dtype)


def test_codegen_rejects_bad_groups(pkg):
    from chainer_compiler_b200 import _lib
    from chainer_compiler_b200.fusion import Node, build_program
    with pytest.raises(_lib.ChxqError):
        build_program([Node("Relu", ["x"], ["y"])], 1, ["x"], ["y"])  # op outside the generator's set (nvrtc_builder.cc:84-86)
    with pytest.raises(_lib.ChxqError):
        build_program([Node("Tanh", ["y2"], ["y"]), Node("Exp", ["y"], ["y2"])], 1, ["x"], ["y"])  # cyclic / input not in group
    code = build_program([Node("Constant", [], ["k"], np.float32(0.1)), Node("Mul", ["x", "k"], ["y"]), Node("Tanh", ["y"], ["z"])], 3, ["x"], ["z"])
    assert "0.100000001" in code  # constants keep full fp32 precision


def _nvrtc_compile(code, name):
    """Compiles CUDA source for sm_100a with NVRTC (needs no GPU); returns (ok, log)."""
    nv = None
    for path in ("libnvrtc.so.12", "/usr/local/cuda/lib64/libnvrtc.so.12"):
        try:
            nv = ctypes.CDLL(path)
            break
        except OSError:
            continue
    if nv is None:
        pytest.skip("libnvrtc is not installed on this host")
    prog = ctypes.c_void_p()
    assert nv.nvrtcCreateProgram(ctypes.byref(prog), code.encode(), (name + ".cu").encode(), 0, None, None) == 0
    opts = (ctypes.c_char_p * 3)(b"--gpu-architecture=sm_100a", b"--std=c++17", b"-I/usr/local/cuda/include")
    rc = nv.nvrtcCompileProgram(prog, 3, opts)
    n = ctypes.c_size_t()
    nv.nvrtcGetProgramLogSize(prog, ctypes.byref(n))
    log = ctypes.create_string_buffer(n.value + 1)
    nv.nvrtcGetProgramLog(prog, log)
    nv.nvrtcDestroyProgram(ctypes.byref(prog))
    return rc == 0, log.value.decode(errors="replace")


@pytest.mark.parametrize("dtype", ["float32", "float64", "float16"])
def test_generated_source_compiles_for_sm100a(pkg, dtype):
    from chainer_compiler_b200.fusion import Node, build_program, lstm_cell_group
    nodes = lstm_cell_group()
    ok, log = _nvrtc_compile(build_program(nodes, 4, ["a", "c_prev", "f", "i", "o"], ["c_next", "h"], dtype), "fusion4")
    assert ok, log
    nodes = [Node("Constant", [], ["k"], np.float32(1.5)), Node("Div", ["x", "k"], ["d"]), Node("Exp", ["d"], ["e"]), Node("Sub", ["e", "x"], ["y"]),
             Node("Identity", ["y"], ["z"])]
    ok, log = _nvrtc_compile(build_program(nodes, 5, ["x"], ["z", "e"], dtype), "fusion5")
    assert ok, log
