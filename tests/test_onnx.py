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
