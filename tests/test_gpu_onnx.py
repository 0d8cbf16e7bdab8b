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
                        assert np.array_equal(g.reshape(-1) if g.size == 1 else g, np.asarray(ot[o]).reshape(-1) if g.size == 1 else np.asarray(ot[o])), (inst.op, o)
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


QOPS = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "qops")


@pytest.mark.parametrize("name", sorted(os.listdir(QOPS)))
def test_operator_directories_run_exactly(pkg, name):
    """One quantized operator per directory, scalars as graph inputs (tests/golden/make_qop_dirs.py): integer outputs are
    compared with zero tolerance, float outputs (DequantizeLinear) at one fp32 rounding."""
    from chainer_compiler_b200 import run_onnx
    assert run_onnx.run_onnx(["--test", os.path.join(QOPS, name), "--rtol", "1e-7", "--atol", "0", "-q"]) == 0


def test_fused_groups_tracing_and_dumps(pkg, tmp_path):
    from chainer_compiler_b200 import onnx_io, run_onnx
    model, cases = onnx_io.load_test_dir(GOLDEN)
    plain = run_onnx.Executor(run_onnx.compile_model(model, quantize=True), "cuda:0")
    fused_prog = run_onnx.compile_model(model, quantize=True, fuse=True)
    assert sum(i.op == "ElementWiseNvrtc" for i in fused_prog.insts) == 3
    fused = run_onnx.Executor(fused_prog, "cuda:0")
    for ins, _ in cases:
        (_, a), = plain.run(ins)
        (_, b), = fused.run(ins)
        # the generated kernel may contract the Mul and the Add into one fused multiply-add
        assert np.allclose(a.cpu().numpy(), b.cpu().numpy(), rtol=1e-5, atol=1e-4)
    trace, dumps = str(tmp_path / "trace.json"), str(tmp_path / "dumps")
    rc = run_onnx.run_onnx(["--test", GOLDEN, "--quantize", "--fuse_operations", "--use_nvrtc", "--chrome_tracing", trace, "--dump_outputs_dir", dumps,
                            "--no_check_values", "-q"])
    assert rc == 0
    events = json.load(open(trace))
    assert len(events) == 3 * len(fused_prog.insts)
    assert all(e["ph"] == "X" and e["cat"] == "ChxVM" and e["pid"] == 1 and e["tid"] == 1 and e["dur"] >= 0 for e in events)
    assert [e["name"] for e in events[:len(fused_prog.insts)]] == [i.op for i in fused_prog.insts]
    assert [e["args"]["pc"] for e in events[:4]] == [0, 1, 2, 3] and all(events[k]["ts"] <= events[k + 1]["ts"] for k in range(len(events) - 1))
    files = sorted(os.listdir(dumps))
    assert files[0].startswith("00000_") and all(f[:5].isdigit() and f[5] == "_" and f.endswith(".npy") for f in files)
    last = fused_prog.insts[-1]
    y = np.load(os.path.join(dumps, "%05d_%s.npy" % (len(fused_prog.insts) - 1, last.outputs[0])))
    assert y.shape == (1, 10)


def test_exported_graph_and_bn_folding_on_the_device(pkg, tmp_path):
    import torch
    from chainer_compiler_b200 import onnx_io, run_onnx
    model, cases = onnx_io.load_test_dir(GOLDEN)
    out = str(tmp_path / "quantized.onnx")
    assert run_onnx.run_onnx(["--test", GOLDEN, "--quantize", "--out_onnx", out, "--skip_inference", "-q"]) == 0
    prog = run_onnx.compile_model(model, quantize=True)
    again = run_onnx.compile_model(onnx_io.load_model(out))
    assert any(i.op == "ReduceMin" for i in again.insts) and any(i.op == "ConvInteger" for i in again.insts)
    e1, e2 = run_onnx.Executor(prog, "cuda:0"), run_onnx.Executor(again, "cuda:0")
    for ins, _ in cases:
        (_, a), = e1.run(ins)
        (_, b), = e2.run(ins)
        assert torch.equal(a, b)
    # Conv + BatchNormalization: merged first and quantized as one convolution, against the float pair
    rng = np.random.default_rng(8)
    N, f32 = onnx_io.Node, np.float32
    inits = {"w": (rng.standard_normal((16, 8, 3, 3)) * 0.2).astype(f32), "gamma": rng.uniform(0.5, 1.5, 16).astype(f32),
             "beta": (rng.standard_normal(16) * 0.1).astype(f32), "mean": (rng.standard_normal(16) * 0.1).astype(f32), "var": rng.uniform(0.5, 1.5, 16).astype(f32)}
    nodes = [N("Conv", ["x", "w"], ["c"], {"kernel_shape": [3, 3], "pads": [1, 1, 1, 1]}),
             N("BatchNormalization", ["c", "gamma", "beta", "mean", "var"], ["y"], {"epsilon": 2e-5})]
    m = onnx_io.Model(nodes, inits, ["x"], ["y"], ir_version=5, opset=10)
    x = rng.standard_normal((2, 8, 12, 12)).astype(f32)
    t = lambda k: torch.from_numpy(inits[k])  # noqa: E731
    sh = (1, -1, 1, 1)
    want = (torch.nn.functional.conv2d(torch.from_numpy(x), t("w"), None, 1, 1) - t("mean").reshape(sh)) / torch.sqrt(t("var").reshape(sh) + 2e-5) \
        * t("gamma").reshape(sh) + t("beta").reshape(sh)
    for first in (False, True):
        p = run_onnx.compile_model(m, quantize=True, fold_bn_first=first)
        assert ("BatchNormalization" in [i.op for i in p.insts]) == (not first)
        (_, y), = run_onnx.Executor(p, "cuda:0").run({"x": x})
        err = (y.cpu() - want).abs().max().item()
        assert err < 0.05 * want.abs().max().item(), (first, err)


def test_statically_quantized_resnet_file_runs_on_the_tensor_core_kernels(pkg, ops, orc, tmp_path):
    """models.ResNet50Int8.to_onnx(): the calibrated network as a standard ONNX file, executed by run_onnx (packed weights,
    channels_last activations, residual joins as one kernel) against the oracle's evaluation of the same file."""
    import torch
    from chainer_compiler_b200 import models, onnx_io, run_onnx
    from oracle import networks
    dev = torch.device("cuda:0")
    net = models.ResNet50Int8(2, dev, seed=3, image=64, width_mult=0.25)
    x = torch.rand((2, 3, 64, 64), generator=torch.Generator().manual_seed(4))
    net.calibrate(x.to(dev))
    want = net.forward(x.to(dev), fused=False).cpu().numpy()
    model = net.to_onnx()
    d = str(tmp_path / "resnet")
    onnx_io.write_test_dir(d, model, [({"x": x.numpy()}, [("logits", want)])])
    # the hand-built forward() pools the uint8 map and dequantizes the mean; the file dequantizes, then pools: fp32 rounding only
    atol = "%g" % (1e-5 * float(np.abs(want).max()))
    assert run_onnx.run_onnx(["--test", d, "--rtol", "1e-4", "--atol", atol, "-q"]) == 0
    launches = pkg._lib.lib().chxq_launch_count()
    model2, cases = onnx_io.load_test_dir(d)
    prog = run_onnx.compile_model(model2)
    # all 16 residual joins moved into the epilogue of the block's last convolution
    assert sum(i.op == "QAddU8" for i in prog.insts) == 0 and sum(i.op == "QLinearConv" for i in prog.insts) == 53
    assert sum(bool(i.attrs.get("residual")) for i in prog.insts) == 16
    assert sum(i.op == "QAddU8" for i in run_onnx.compile_model(model2, peephole="join").insts) == 16
    ex = run_onnx.Executor(prog, "cuda:0")
    gt, ot = {}, {}
    (_, got), = ex.run(cases[0][0], trace=gt)
    assert all(p.eligible for p in ex.packed.values()) and len(ex.packed) == 53     # every convolution ran from packed weights
    assert pkg._lib.lib().chxq_launch_count() > launches
    (_, ref), = networks.run_program(prog, cases[0][0], trace=ot, conv_mode="exact")
    for inst in prog.insts:
        o = inst.outputs[0]
        g = gt[o].cpu().numpy()
        if g.dtype == np.uint8:
            assert np.array_equal(g, ot[o]), (inst.op, o)
        else:
            assert np.allclose(g, ot[o], rtol=1e-5, atol=1e-5 * float(np.abs(ot[o]).max())), (inst.op, o)
    assert np.allclose(got.cpu().numpy(), ref, rtol=1e-5, atol=1e-5 * float(np.abs(ref).max()))
    # without the peepholes (five-node joins), and with the join as its own kernel, the same bits
    for level in (False, "join"):
        ex2 = run_onnx.Executor(run_onnx.compile_model(model2, peephole=level), "cuda:0")
        (_, got2), = ex2.run(cases[0][0])
        assert torch.equal(got, got2), level
    # a captured graph replays to the same bits, also on new input values
    assert ex.is_static()
    ex.capture(cases[0][0])
    (_, got3), = ex.replay(cases[0][0])
    assert torch.equal(got, got3)
    x2 = torch.rand((2, 3, 64, 64), generator=torch.Generator().manual_seed(5)).numpy()
    (_, eager), = run_onnx.Executor(prog, "cuda:0").run({"x": x2})
    (_, replayed), = ex.replay({"x": x2})
    assert torch.equal(eager, replayed)
    assert run_onnx.run_onnx(["--test", d, "--rtol", "1e-4", "--atol", atol, "-q", "-I", "3", "--cuda_graph"]) == 0
    # single-multiplier requantization: the quantized maps of the hand-built folded forward, bit for bit
    taps, gt = {}, {}
    net.forward(x.to(dev), fused=True, fold=True, taps=taps)
    run_onnx.Executor(prog, "cuda:0", fold_scales=True).run(cases[0][0], trace=gt)
    assert prog.insts[0].attrs.get("quantize_input") and prog.insts[0].attrs.get("pool") == 2 and prog.insts[0].outputs == ["pool"]
    assert torch.equal(gt["pool"], ops.MaxPoolU8(taps["stem"], 3, 2, 0, cover_all=True)) and all(torch.equal(gt["b%d_out" % i], taps["block%d" % i]) for i in range(16))
    # the dynamically quantized graph is static only while its scales and zero points stay on the device
    dyn = run_onnx.compile_model(onnx_io.load_test_dir(GOLDEN)[0], quantize=True)
    assert run_onnx.Executor(dyn, "cuda:0").is_static() and not run_onnx.Executor(dyn, "cuda:0", device_scalars=False).is_static()


def test_dynamic_quantization_scalars_stay_on_device(pkg, ops, orc, dev):
    """ReduceMin / ReduceMax -> scale, zero point -> QuantizeLinear -> ConvInteger with every scalar read by the kernels from
    device memory: bit-exact against the oracle's dynamic parameters (compiler/quantize.cc:172-207, including the range that is
    not widened to include zero) and against the host-scalar path."""
    import torch
    rng = np.random.default_rng(4)
    for lo, hi in ((-1.7, 2.9), (0.25, 3.0), (-4.0, -0.5), (0.0, 0.0)):
        x = rng.uniform(lo, hi, (2, 3, 9, 11)).astype(np.float32)
        xt = torch.from_numpy(x).to(dev)
        mm = ops.MinMax(xt)
        scale, zp = ops.DynamicQuantParamsU8(mm[0:1], mm[1:2])
        want_scale, want_zp = orc.dynamic_params_u8(x) if lo != hi else (np.float32(1.0), 0.0)
        want_zp = int(np.clip(want_zp, 0, 255))
        assert np.float32(scale.item()) == np.float32(want_scale) and int(zp.item()) == want_zp, (lo, hi)
        q_dev = ops.QuantizeLinear(xt, scale, zp)
        q_host = ops.QuantizeLinear(xt, np.float32(want_scale), np.uint8(want_zp))
        assert torch.equal(q_dev, q_host)
        assert np.array_equal(q_dev.cpu().numpy(), orc.quantize_linear(x, want_scale, want_zp))
        w = rng.integers(0, 256, (5, 3, 3, 3), dtype=np.uint8)
        wz = rng.integers(100, 140, 5).astype(np.uint8)
        y = ops.ConvInteger(q_dev, torch.from_numpy(w).to(dev), zp, torch.from_numpy(wz).to(dev), (1, 1), (1, 1), 1)
        assert np.array_equal(y.cpu().numpy(), orc.conv_integer(q_dev.cpu().numpy(), w, want_zp, wz.astype(np.int32), (1, 1), (1, 1)))
    ops.device_status()


def test_quantized_mnist_runs_without_host_reads_and_in_a_graph(pkg, orc):
    """The `--quantize` program keeps its dynamic scales and zero points on the device: it is static (no device-to-host read), it
    can be captured in a CUDA graph, and the captured replay, the eager device-scalar run and the host-scalar run agree bit for bit."""
    import torch
    from chainer_compiler_b200 import onnx_io, run_onnx
    model, cases = onnx_io.load_test_dir(GOLDEN)
    prog = run_onnx.compile_model(model, quantize=True)
    ex_dev = run_onnx.Executor(prog, "cuda:0")
    ex_host = run_onnx.Executor(prog, "cuda:0", device_scalars=False)
    assert ex_dev.is_static() and not ex_host.is_static()
    ins0 = cases[0][0]
    ex_dev.capture(ins0)
    for ins, expected in cases:
        (_, a), = ex_dev.run(ins)
        (_, b), = ex_host.run(ins)
        (_, c), = ex_dev.replay(ins)
        torch.cuda.synchronize()
        assert torch.equal(a, b) and torch.equal(a, c)
        assert int(np.argmax(a.cpu().numpy())) == int(np.argmax(expected[0][1]))
    rc = run_onnx.run_onnx(["--test", GOLDEN, "--quantize", "-I", "20", "--cuda_graph", "--rtol", "0.05", "--atol", "50", "-q"])
    assert rc == 0
