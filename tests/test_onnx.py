"""ONNX ingestion and the `--quantize` rewrite (CPU): the wire-format reader / writer, the test-directory format, the
instruction sequence of the dynamic IntegerOps pass, and the oracle's evaluation of the quantized MNIST graph against the
expected outputs the reference ships with that fixture (tests/golden/mnist, written by tests/golden/make_mnist_golden.py)."""
import os

import numpy as np
import pytest

import __graft_entry__ as entry

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "mnist")


@pytest.fixture(scope="module")
def mods():
    entry.load_package()
    from chainer_compiler_b200 import onnx_io, run_onnx
    return onnx_io, run_onnx


def test_tensor_round_trip_and_payload_rules(mods):
    onnx_io, _ = mods
    rng = np.random.default_rng(0)
    for dt in (np.float32, np.float64, np.int64, np.int32, np.int16, np.int8, np.uint8, np.float16, np.bool_):
        a = (rng.standard_normal((3, 4, 5)) * 50).astype(dt)
        name, b = onnx_io.parse_tensor(onnx_io.serialize_tensor(a, "t"))
        assert name == "t" and b.dtype == a.dtype and np.array_equal(a, b)
    name, s = onnx_io.parse_tensor(onnx_io.serialize_tensor(np.float32(2.5)))
    assert s.shape == () and s == np.float32(2.5)
    # raw_data: field 9; raw together with typed data is refused (compiler/tensor.cc:95-103)
    raw = onnx_io._enc_field(1, 0, 2) + onnx_io._enc_field(2, 0, onnx_io.INT32) + onnx_io._enc_field(9, 2, np.array([7, -9], "<i4").tobytes())
    assert np.array_equal(onnx_io.parse_tensor(raw)[1], np.array([7, -9], np.int32))
    with pytest.raises(onnx_io.OnnxError):
        onnx_io.parse_tensor(raw + onnx_io._enc_field(5, 2, b"\x01"))
    with pytest.raises(onnx_io.OnnxError):
        onnx_io.parse_tensor(onnx_io._enc_field(1, 0, 3) + onnx_io._enc_field(2, 0, onnx_io.FLOAT) + onnx_io._enc_field(4, 2, b"\0\0\0\0"))


def test_mnist_directory_loads(mods):
    onnx_io, _ = mods
    model, cases = onnx_io.load_test_dir(GOLDEN)
    assert [n.op_type for n in model.nodes] == ["Reshape", "Conv", "Add", "Relu", "MaxPool", "Conv", "Add", "Relu", "MaxPool", "Reshape", "MatMul", "Add"]
    assert model.inputs == ["Input3"] and model.outputs == ["Plus214_Output_0"] and model.opset == 8
    assert model.nodes[1].attrs["auto_pad"] == "SAME_UPPER" and model.nodes[1].attrs["kernel_shape"] == [5, 5]
    assert model.initializers["Parameter87"].shape == (16, 8, 5, 5)
    assert len(cases) == 3 and cases[0][0]["Input3"].shape == (1, 1, 28, 28) and cases[0][1][0][1].shape == (1, 10)
    again = onnx_io.parse_model(onnx_io.serialize_model(model))
    assert [repr(n) for n in again.nodes] == [repr(n) for n in model.nodes]


def test_quantize_pass_emits_the_reference_sequence(mods):
    onnx_io, run_onnx = mods
    model, _ = onnx_io.load_test_dir(GOLDEN)
    prog = run_onnx.compile_model(model, quantize=True)
    ops = [i.op for i in prog.insts]
    conv_seq = ["ReduceMinMax", "DynamicQuantParamsU8", "QuantizeLinear", "ConvInteger", "Cast", "ScaleProduct", "Mul"]
    assert ops[:7] == conv_seq and ops[7:10] == ["Add", "Relu", "MaxPool"] and ops[10:17] == conv_seq
    assert ops[-8:] == ["ReduceMinMax", "DynamicQuantParamsU8", "QuantizeLinear", "MatMulInteger", "Cast", "ScaleProduct", "Mul", "Add"]
    assert "MatMulInteger" in ops and "Conv" not in ops and "MatMul" not in ops
    ci = prog.insts[3]
    wq, wz = prog.constants[ci.inputs[1]], prog.constants[ci.inputs[3]]
    assert wq.dtype == np.uint8 and wz.dtype == np.uint8 and wz.shape == (8,)   # uint8 weights, per output channel (compiler/quantize.cc:392-400)
    per_tensor = run_onnx.compile_model(model, quantize=True, per_channel=False)
    assert per_tensor.constants[per_tensor.insts[3].inputs[3]].size == 1
    # without --quantize the float graph is kept as it is (and has no kernel here)
    assert [i.op for i in run_onnx.compile_model(model).insts][:2] == ["Conv", "Add"]


def test_oracle_runs_the_quantized_mnist_graph_close_to_the_shipped_outputs(mods):
    """The expected outputs in the fixture are the float model's; the dynamically quantized graph (8-bit activations and
    weights) must classify the same digit and stay within a few per cent of them."""
    onnx_io, run_onnx = mods
    entry.load_oracle()
    from oracle import networks
    model, cases = onnx_io.load_test_dir(GOLDEN)
    prog = run_onnx.compile_model(model, quantize=True)
    for ins, expected in cases:
        (name, got), = networks.run_program(prog, ins)
        want = expected[0][1]
        assert name == expected[0][0] and got.shape == want.shape
        assert int(np.argmax(got)) == int(np.argmax(want))
        rel = float(np.linalg.norm(got - want) / np.linalg.norm(want))
        print("quantized MNIST vs shipped float output: relative L2 distance %.4f" % rel)
        assert rel < 0.05


QOPS = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "qops")


@pytest.mark.parametrize("name", sorted(os.listdir(QOPS)))
def test_operator_directories_load_and_match_the_oracle(mods, name):
    """tests/golden/qops (written by tests/golden/make_qop_dirs.py): one quantized operator per directory, every operand a
    graph input; the oracle's evaluation of the loaded program reproduces the stored outputs bit for bit."""
    onnx_io, run_onnx = mods
    entry.load_oracle()
    from oracle import networks
    model, cases = onnx_io.load_test_dir(os.path.join(QOPS, name))
    prog = run_onnx.compile_model(model)
    assert len(cases) == 1
    for ins, expected in cases:
        got = dict(networks.run_program(prog, ins))
        for oname, want in expected:
            assert got[oname].dtype == want.dtype and np.array_equal(got[oname], want), name


def _conv_bn_model(onnx_io, rng, with_bias):
    N = onnx_io.Node
    f32 = np.float32
    inits = {"w": (rng.standard_normal((6, 3, 3, 3)) * 0.2).astype(f32), "gamma": rng.uniform(0.5, 1.5, 6).astype(f32),
             "beta": (rng.standard_normal(6) * 0.1).astype(f32), "mean": (rng.standard_normal(6) * 0.1).astype(f32), "var": rng.uniform(0.5, 1.5, 6).astype(f32)}
    conv_in = ["x", "w"]
    if with_bias:
        inits["b"] = (rng.standard_normal(6) * 0.1).astype(f32)
        conv_in.append("b")
    nodes = [N("Conv", conv_in, ["c"], {"kernel_shape": [3, 3], "pads": [1, 1, 1, 1]}),
             N("BatchNormalization", ["c", "gamma", "beta", "mean", "var"], ["bn"], {"epsilon": 2e-5}),
             N("Relu", ["bn"], ["y"], {})]
    return onnx_io.Model(nodes, inits, ["x"], ["y"], ir_version=5, opset=10)


def test_merge_conv_bn_pass_and_its_order_against_quantize(mods):
    """compiler/merge.cc:142-215 and the pass order of compiler/passes.cc:121-128."""
    import torch
    onnx_io, run_onnx = mods
    rng = np.random.default_rng(5)
    for with_bias in (False, True):
        model = _conv_bn_model(onnx_io, rng, with_bias)
        prog = run_onnx.compile_model(model)
        assert [i.op for i in prog.insts] == ["Conv", "Relu"] and len(prog.insts[0].inputs) == 3
        w2, b2 = prog.constants[prog.insts[0].inputs[1]], prog.constants[prog.insts[0].inputs[2]]
        i = model.initializers
        x = torch.from_numpy(rng.standard_normal((2, 3, 8, 8)).astype(np.float32))
        c = torch.nn.functional.conv2d(x, torch.from_numpy(i["w"]), torch.from_numpy(i["b"]) if with_bias else None, 1, 1)
        sh = (1, -1, 1, 1)
        bn = (c - torch.from_numpy(i["mean"]).reshape(sh)) / torch.sqrt(torch.from_numpy(i["var"]).reshape(sh) + 2e-5) * torch.from_numpy(i["gamma"]).reshape(sh) \
            + torch.from_numpy(i["beta"]).reshape(sh)
        merged = torch.nn.functional.conv2d(x, torch.from_numpy(w2), torch.from_numpy(b2), 1, 1)
        assert torch.allclose(bn, merged, rtol=1e-4, atol=1e-5)
        assert w2.dtype == np.float32 and b2.dtype == np.float32
        # reference order: the quantizer takes the bias-free Conv first, the BatchNormalization stays a float node; a Conv with
        # bias is not quantized (compiler/quantize.cc:366-369) and is merged
        ops = [k.op for k in run_onnx.compile_model(model, quantize=True).insts]
        if with_bias:
            assert ops == ["Conv", "Relu"]
        else:
            assert ops == ["ReduceMinMax", "DynamicQuantParamsU8", "QuantizeLinear", "ConvInteger", "Cast", "ScaleProduct", "Mul", "BatchNormalization", "Relu"]
        # merge first: one quantized convolution, the merged bias added after the scale-back
        ops = [k.op for k in run_onnx.compile_model(model, quantize=True, fold_bn_first=True).insts]
        assert ops == ["ReduceMinMax", "DynamicQuantParamsU8", "QuantizeLinear", "ConvInteger", "Cast", "ScaleProduct", "Mul", "Add", "Relu"]
    # a Conv with a second user, or one that is a graph output, is left alone
    model = _conv_bn_model(onnx_io, rng, False)
    model.outputs = ["y", "c"]
    assert [k.op for k in run_onnx.compile_model(model).insts] == ["Conv", "BatchNormalization", "Relu"]


def test_fused_program_equals_the_unfused_one_on_the_oracle(mods):
    onnx_io, run_onnx = mods
    entry.load_oracle()
    from oracle import networks
    model, cases = onnx_io.load_test_dir(GOLDEN)
    plain = run_onnx.compile_model(model, quantize=True)
    fused = run_onnx.compile_model(model, quantize=True, fuse=True)
    groups = [i for i in fused.insts if i.op == "ElementWiseNvrtc"]
    # Mul (scale-back) + Add (bias) after each of the two convolutions and after the MatMul; Relu is not in the reference's
    # fusable set (compiler/fusion_elementwise.cc:12-24)
    assert len(groups) == 3 and all([m[0] for m in g.attrs["members"]] == ["Mul", "Add"] for g in groups)
    assert all("fusion%d" % g.attrs["fusion_id"] in g.attrs["code"] for g in groups)
    assert len(fused.insts) == len(plain.insts) - 3
    for ins, _ in cases[:2]:
        (_, a), = networks.run_program(plain, ins)
        (_, b), = networks.run_program(fused, ins)
        assert np.array_equal(a, b)


def test_exported_onnx_graph_round_trips(mods, tmp_path):
    """--out_onnx: the quantized program written as standard ONNX nodes, read back and evaluated, gives the same bits."""
    onnx_io, run_onnx = mods
    entry.load_oracle()
    from oracle import networks
    model, cases = onnx_io.load_test_dir(GOLDEN)
    prog = run_onnx.compile_model(model, quantize=True)
    exported = run_onnx.program_to_onnx(prog)
    kinds = [n.op_type for n in exported.nodes]
    assert kinds[:12] == ["ReduceMin", "ReduceMax", "Sub", "Div", "Sub", "Div", "Floor", "Cast", "QuantizeLinear", "ConvInteger", "Cast", "Mul"]
    assert not any(k in kinds for k in ("ReduceMinMax", "DynamicQuantParamsU8", "ScaleProduct"))
    path = tmp_path / "q.onnx"
    path.write_bytes(onnx_io.serialize_model(exported))
    again = run_onnx.compile_model(onnx_io.load_model(str(path)))
    for ins, _ in cases[:2]:
        (_, a), = networks.run_program(prog, ins)
        (_, b), = networks.run_program(again, ins)
        assert np.array_equal(a, b)
    assert run_onnx.run_onnx([str(path), "--compile_only", "--quiet"]) == 0
    args = run_onnx.parse_args(["--test", "d", "--chrome_tracing", "t.json", "-t", "--backend", "chxvm", "--fuse_operations", "--use_nvrtc", "--skip_inference"])
    assert args.chrome_tracing == "t.json" and args.trace and args.fuse_operations and args.use_nvrtc and args.skip_inference


def test_compare_dump_dirs(mods, tmp_path):
    import io
    entry.load_package()
    from chainer_compiler_b200 import compare_dump_dirs
    a, b = tmp_path / "a", tmp_path / "b"
    a.mkdir()
    b.mkdir()
    x = np.arange(12, dtype=np.float32).reshape(3, 4)
    np.save(a / "00000_x.npy", x)
    np.save(a / "00001_y.npy", x.astype(np.uint8))
    np.save(a / "00002_only_here.npy", x)
    np.save(b / "00000_y.npy", x.astype(np.uint8))       # numbered differently: matched by name
    y = x.copy()
    y[1, 2] += 0.5
    np.save(b / "00005_x.npy", y)
    log = io.StringIO()
    assert compare_dump_dirs.compare(str(a), str(b), out=log) == 1
    text = log.getvalue()
    assert "y: OK" in text and "x: 1 of 12 elements differ" in text and "only_here" not in text
    assert compare_dump_dirs.compare(str(a), str(b), atol=1.0, out=io.StringIO()) == 0


def _residual_join_model(onnx_io, rng):
    N, f32, u8, i8 = onnx_io.Node, np.float32, np.uint8, np.int8
    inits = {"s_in": f32(1 / 64.0).reshape(()), "z0": u8(0).reshape(()), "z9": u8(9).reshape(()),
             "w1": rng.integers(-127, 128, (16, 16, 3, 3), dtype=i8), "ws1": rng.uniform(0.001, 0.003, 16).astype(f32), "wz1": np.zeros(16, i8),
             "w2": rng.integers(-127, 128, (16, 16, 1, 1), dtype=i8), "ws2": rng.uniform(0.001, 0.003, 16).astype(f32), "wz2": np.zeros(16, i8),
             "b2": rng.integers(-500, 500, 16).astype(np.int32),
             "s1": f32(0.02).reshape(()), "s2": f32(0.03).reshape(()), "s_out": f32(0.05).reshape(())}
    nodes = [N("QuantizeLinear", ["x", "s_in", "z0"], ["xq"], {}),
             N("QLinearConv", ["xq", "s_in", "z0", "w1", "ws1", "wz1", "s1", "z0"], ["h1"], {"kernel_shape": [3, 3], "pads": [1, 1, 1, 1]}),
             N("QLinearConv", ["h1", "s1", "z0", "w2", "ws2", "wz2", "s2", "z9", "b2"], ["h2"], {"kernel_shape": [1, 1]}),
             N("DequantizeLinear", ["h2", "s2", "z9"], ["f2"], {}),
             N("DequantizeLinear", ["xq", "s_in", "z0"], ["fx"], {}),
             N("Add", ["f2", "fx"], ["sum"], {}),
             N("Relu", ["sum"], ["r"], {}),
             N("QuantizeLinear", ["r", "s_out", "z0"], ["yq"], {}),
             N("DequantizeLinear", ["yq", "s_out", "z0"], ["y"], {})]
    return onnx_io.Model(nodes, inits, ["x"], ["y"], ir_version=5, opset=10)


def test_residual_join_peephole_keeps_every_bit(mods):
    onnx_io, run_onnx = mods
    entry.load_oracle()
    from oracle import networks
    rng = np.random.default_rng(12)
    model = _residual_join_model(onnx_io, rng)
    plain = run_onnx.compile_model(model, peephole=False)
    fused = run_onnx.compile_model(model, peephole="join")
    both = run_onnx.compile_model(model)
    assert [i.op for i in fused.insts] == ["QuantizeLinear", "QLinearConv", "QLinearConv", "QAddU8", "DequantizeLinear"]
    assert fused.insts[3].attrs["relu"] == 1 and fused.insts[3].inputs[0] == "h2" and fused.insts[3].inputs[3] == "xq"
    # the convolution whose only reader is the join takes it into its epilogue
    assert [i.op for i in both.insts] == ["QuantizeLinear", "QLinearConv", "QLinearConv", "DequantizeLinear"]
    assert both.insts[2].attrs["residual"] == 1 and both.insts[2].inputs[9:] == ["xq", "s_in", "z0", "s_out", "z0"] and both.insts[2].outputs == ["yq"]
    x = rng.uniform(0, 3.9, (2, 16, 9, 9)).astype(np.float32)
    for mode in ("emulate", "exact"):
        ta, tb, tc = {}, {}, {}
        (_, a), = networks.run_program(plain, {"x": x}, trace=ta, conv_mode=mode)
        (_, b), = networks.run_program(fused, {"x": x}, trace=tb, conv_mode=mode)
        (_, c), = networks.run_program(both, {"x": x}, trace=tc, conv_mode=mode)
        assert np.array_equal(ta["yq"], tb["yq"]) and np.array_equal(a, b) and ta["yq"].max() > 0
        assert np.array_equal(ta["yq"], tc["yq"]) and np.array_equal(a, c)
    # the export writes the join back as the five standard nodes
    for prog in (fused, both):
        kinds = [n.op_type for n in run_onnx.program_to_onnx(prog).nodes]
        assert kinds == [n.op_type for n in model.nodes]
    # a second reader of an intermediate value, or a non-constant scale, blocks the rewrite
    model.outputs = ["y", "sum"]
    assert "QAddU8" not in [i.op for i in run_onnx.compile_model(model).insts]


def test_stem_peephole(mods):
    """QuantizeLinear -> QLinearConv -> MaxPool(3, 2) at the head of a network becomes one instruction; the oracle's evaluation
    and the exported graph are unchanged."""
    onnx_io, run_onnx = mods
    entry.load_oracle()
    from oracle import networks
    N, f32, u8, i8 = onnx_io.Node, np.float32, np.uint8, np.int8
    rng = np.random.default_rng(17)
    inits = {"s_in": f32(1 / 255.0).reshape(()), "z0": u8(0).reshape(()), "w": rng.integers(-127, 128, (16, 3, 7, 7), dtype=i8),
             "ws": rng.uniform(0.0005, 0.002, 16).astype(f32), "wz": np.zeros(16, i8), "b": rng.integers(-500, 500, 16).astype(np.int32),
             "s1": f32(0.05).reshape(())}
    nodes = [N("QuantizeLinear", ["x", "s_in", "z0"], ["xq"], {}),
             N("QLinearConv", ["xq", "s_in", "z0", "w", "ws", "wz", "s1", "z0", "b"], ["c"], {"kernel_shape": [7, 7], "strides": [2, 2], "pads": [3, 3, 3, 3]}),
             N("MaxPool", ["c"], ["p"], {"kernel_shape": [3, 3], "strides": [2, 2], "ceil_mode": 1}),
             N("DequantizeLinear", ["p", "s1", "z0"], ["y"], {})]
    model = onnx_io.Model(nodes, inits, ["x"], ["y"], ir_version=5, opset=12)
    plain, fused = run_onnx.compile_model(model, peephole=False), run_onnx.compile_model(model)
    assert [i.op for i in fused.insts] == ["QLinearConv", "DequantizeLinear"]
    st = fused.insts[0]
    assert st.inputs[0] == "x" and st.outputs == ["p"] and st.attrs["quantize_input"] == 1 and st.attrs["pool"] == 2
    x = rng.uniform(0, 1, (1, 3, 30, 34)).astype(f32)
    (_, a), = networks.run_program(plain, {"x": x})
    (_, b), = networks.run_program(fused, {"x": x})
    assert a.shape == (1, 16, 7, 8) and np.array_equal(a, b)
    assert [n.op_type for n in run_onnx.program_to_onnx(fused).nodes] == [n.op_type for n in nodes]
    # a second reader of the quantized image or of the convolution's output keeps the nodes apart
    model.outputs = ["y", "c"]
    st = run_onnx.compile_model(model).insts[0]
    assert st.op == "QLinearConv" and st.attrs.get("quantize_input") == 1 and not st.attrs.get("pool")
