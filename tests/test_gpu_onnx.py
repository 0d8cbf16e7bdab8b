"""`run_onnx --quantize` on the GPU against the oracle's evaluation of the same program: quantized tensors and int32
accumulators bit-exact, float outputs equal up to the order of fp32 glue operations; and the command-line entry."""
import json
import os

import numpy as np
import pytest

import __graft_entry__ as entry

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "mnist")


def test_quantized_mnist_matches_oracle(pkg, orc):
    from chainer_compiler_b200 import onnx_io, run_onnx
    entry.load_oracle()
    from oracle import networks
    model, cases = onnx_io.load_test_dir(GOLDEN)
    for per_channel in (True, False):
        prog = run_onnx.compile_model(model, quantize=True, per_channel=per_channel)
        ex = run_onnx.Executor(prog, "cuda:0")
        for ins, expected in cases:
            gt, ot = {}, {}
            (name, got), = ex.run(ins, trace=gt)
            (_, want), = networks.run_program(prog, ins, trace=ot)
            for inst in prog.insts:
                for o in inst.outputs:
                    g = gt[o].cpu().numpy() if hasattr(gt[o], "cpu") else np.asarray(gt[o])
                    if inst.op in ("QuantizeLinear", "ConvInteger", "MatMulInteger", "ReduceMinMax", "DynamicQuantParamsU8"):
                        assert np.array_equal(g, np.asarray(ot[o])), (inst.op, o)
                    else:
                        assert np.allclose(g, ot[o], rtol=1e-6, atol=1e-4), (inst.op, o)
            ref = expected[0][1]
            assert int(np.argmax(got.cpu().numpy())) == int(np.argmax(ref))


def test_run_onnx_command_line(pkg, tmp_path):
    from chainer_compiler_b200 import run_onnx
    report = str(tmp_path / "report.json")
    rc = run_onnx.run_onnx(["--test", GOLDEN, "--quantize", "-d", "cuda:0", "-I", "2", "--rtol", "0.05", "--atol", "50", "--report_json", report, "-q"])
    assert rc == 0
    rep = json.load(open(report))
    assert rep["failures"] == 0 and rep["quantize"] and len(rep["outputs"]) == 3
    # at the reference's default tolerances the 8-bit graph is (rightly) out of tolerance against the float outputs
    assert run_onnx.run_onnx([GOLDEN, "--quantize", "-q"]) == 1
    assert run_onnx.run_onnx([GOLDEN, "--quantize", "--no_check_values", "-q"]) == 0
    with pytest.raises(SystemExit):
        run_onnx.run_onnx([GOLDEN, "-q"])  # float Conv / MatMul: no kernel in this package
    # the float graph as torch expressions reproduces the shipped outputs (library convolutions may use TF32: loose tolerance)
    assert run_onnx.run_onnx([GOLDEN, "--float_ops_via_torch", "--rtol", "1e-2", "--atol", "1", "-q"]) == 0
