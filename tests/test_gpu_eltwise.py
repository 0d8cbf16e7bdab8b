"""Fused elementwise groups: generated kernels against the CPU oracle (fp32 per-op evaluation and fp64 truth)."""
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "hotpath_vectors.npz")
RTOL = 1e-5  # the bound the path is specified to: 1e-5 relative for fp32 fused elementwise
ATOL = 1e-6  # absolute floor where the value itself is within 1e-1 of zero (the reference's own comparison uses atol 1e-6)


def _lstm(fusion):
    nodes = fusion.lstm_cell_group()
    g = fusion.fuse_elementwise(nodes, {}, ["c_next", "h"])[0]
    return nodes, g


def _oracle_nodes(nodes, inputs):
    order = list(inputs) + [n.outputs[0] for n in nodes]
    out = []
    for n in nodes:
        if n.op_type == "Constant":
            out.append(("Constant", [], float(np.asarray(n.value).reshape(-1)[0])))
        else:
            out.append((n.op_type, [order.index(v) for v in n.inputs]))
    return out, order


@pytest.mark.parametrize("shape", [(1,), (7,), (64, 33), (4096, 512), (3, 5, 17)])
def test_lstm_group_fp32(pkg, ops, orc, dev, shape):
    from chainer_compiler_b200 import fusion
    nodes, g = _lstm(fusion)
    code = fusion.build_program(nodes, 11, g.inputs, g.outputs)
    rng = np.random.default_rng(len(shape))
    ins = [rng.standard_normal(shape).astype(np.float32) for _ in g.inputs]
    outs = ops.ElementWiseNvrtc([torch.from_numpy(v).to(dev) for v in ins], 2, code, 11)
    onodes, order = _oracle_nodes(nodes, g.inputs)
    ids = [order.index(v) for v in g.outputs]
    truth = orc.eltwise(onodes, ins, ids, fp64=True)
    cpu32 = orc.eltwise(onodes, ins, ids)
    for o, t, c in zip(outs, truth, cpu32):
        o = o.cpu().numpy()
        assert o.shape == tuple(shape)
        assert np.allclose(o, t, rtol=RTOL, atol=ATOL)
        assert np.allclose(o, c, rtol=RTOL, atol=ATOL)
        rel = np.abs(o - t) / np.maximum(np.abs(t), 0.1)
        assert rel.max() < RTOL


def test_broadcast_unaligned_and_cache(pkg, ops, orc, dev):
    from chainer_compiler_b200 import fusion
    N = fusion.Node
    nodes = [N("Constant", [], ["k"], np.float32(0.3)), N("Mul", ["x", "k"], ["m"]), N("Add", ["m", "b"], ["s"]), N("Exp", ["s"], ["e"]),
             N("Sub", ["e", "x"], ["y"]), N("Identity", ["y"], ["z"])]
    g = fusion.fuse_elementwise(nodes, {}, ["z"])[0]
    assert g.inputs == ["b", "x"] and g.outputs == ["z"]
    code = fusion.build_program([nodes[i] for i in g.node_indices], 3, g.inputs, g.outputs)
    rng = np.random.default_rng(2)
    x = rng.standard_normal((6, 1031)).astype(np.float32)
    b = rng.standard_normal((1031,)).astype(np.float32)  # broadcast against x (runtime/ops/nvrtc.cc:103-110)
    xt = torch.from_numpy(np.concatenate([np.zeros(1, np.float32), x.reshape(-1)])).to(dev)[1:].reshape(6, 1031)  # 4-byte offset
    for _ in range(2):  # second call hits the compile cache
        (z,) = ops.ElementWiseNvrtc([torch.from_numpy(b).to(dev), xt], 1, code, 3)
    want = np.exp(x.astype(np.float64) * np.float64(np.float32(0.3)) + b) - x
    assert z.shape == (6, 1031) and np.allclose(z.cpu().numpy(), want, rtol=RTOL, atol=ATOL)


def test_sigmoid_tail_accuracy(pkg, ops, dev):
    """1/(1+exp(-x)) keeps its relative accuracy for very negative x, where tanh(x/2)/2+1/2 loses it."""
    from chainer_compiler_b200 import fusion
    nodes = [fusion.Node("Sigmoid", ["x"], ["s"]), fusion.Node("Mul", ["s", "s"], ["y"])]
    code = fusion.build_program(nodes, 5, ["x"], ["y"])
    x = np.linspace(-30, 30, 20001).astype(np.float32)
    (y,) = ops.ElementWiseNvrtc([torch.from_numpy(x).to(dev)], 1, code, 5)
    want = (1.0 / (1.0 + np.exp(-x.astype(np.float64)))) ** 2
    assert (np.abs(y.cpu().numpy() - want) / want).max() < RTOL


@pytest.mark.parametrize("dtype,tol", [("float64", 1e-12), ("float16", 2e-3)])
def test_other_float_types(pkg, ops, orc, dev, dtype, tol):
    from chainer_compiler_b200 import fusion
    nodes, g = _lstm(fusion)
    code = fusion.build_program(nodes, 21, g.inputs, g.outputs, dtype)
    rng = np.random.default_rng(9)
    ins = [rng.standard_normal(1000 + 3).astype(np.float32).astype(dtype) for _ in g.inputs]  # fp32-representable values
    outs = ops.ElementWiseNvrtc([torch.from_numpy(v).to(dev) for v in ins], 2, code, 21)
    onodes, order = _oracle_nodes(nodes, g.inputs)
    truth = orc.eltwise(onodes, [v.astype(np.float32) for v in ins], [order.index(v) for v in g.outputs], fp64=True)
    if dtype == "float16":  # the inputs the kernel sees are the fp16-rounded ones
        truth = orc.eltwise(onodes, [v.astype(np.float32) for v in ins], [order.index(v) for v in g.outputs], fp64=True)
    for o, t in zip(outs, truth):
        assert str(o.dtype).endswith(dtype) and np.allclose(o.cpu().numpy().astype(np.float64), t, rtol=tol, atol=tol)


def test_rejects(pkg, ops, dev):
    from chainer_compiler_b200 import fusion
    nodes, g = _lstm(fusion)
    code = fusion.build_program(nodes, 1, g.inputs, g.outputs)
    with pytest.raises(ops.ChxqError):
        ops.ElementWiseNvrtc([], 2, code, 1)
    a = torch.zeros(4, device=dev)
    with pytest.raises(ops.ChxqError):  # mixed dtypes (runtime/ops/nvrtc.cc:102)
        ops.ElementWiseNvrtc([a, a, a, a, a.double()], 2, code, 1)
    with pytest.raises(ops.ChxqError) as e:  # code that does not compile reports the NVRTC log
        ops.ElementWiseNvrtc([a], 1, 'extern "C" __global__ void fusion9(size_t n, float* a, float* b) { this is not CUDA }', 9)
    assert e.value.code == 4


def test_golden_eltwise(pkg, ops, dev):
    from chainer_compiler_b200 import fusion
    g = np.load(GOLDEN)
    nodes, grp = _lstm(fusion)
    code = fusion.build_program(nodes, 2, grp.inputs, grp.outputs)
    c_next, h = ops.ElementWiseNvrtc([torch.from_numpy(g["ew_" + n]).to(dev) for n in grp.inputs], 2, code, 2)
    assert np.allclose(c_next.cpu().numpy(), g["ew_c_next"], rtol=RTOL, atol=ATOL) and np.allclose(h.cpu().numpy(), g["ew_h"], rtol=RTOL, atol=ATOL)


def test_lstm_group_full_size(pkg, ops, orc, dev):
    """4096 x 4096 x 5 inputs: a 1/64 sample of rows against the fp64 oracle plus a conservation property on the whole
    output (h is bounded by |tanh(c')|, c' by |c| + 1)."""
    from chainer_compiler_b200 import fusion
    nodes, g = _lstm(fusion)
    code = fusion.build_program(nodes, 31, g.inputs, g.outputs)
    gen = torch.Generator(device=dev).manual_seed(0)
    ins = [torch.randn((4096, 4096), device=dev, generator=gen) for _ in g.inputs]
    c_next, h = ops.ElementWiseNvrtc(ins, 2, code, 31)
    c_prev = ins[g.inputs.index("c_prev")]
    assert bool((c_next.abs() <= c_prev.abs() + 1.0 + 1e-6).all()) and bool((h.abs() <= torch.tanh(c_next).abs() + 1e-6).all())
    rows = slice(0, 4096, 64)
    onodes, order = _oracle_nodes(nodes, g.inputs)
    truth = orc.eltwise(onodes, [t[rows].cpu().numpy() for t in ins], [order.index(v) for v in g.outputs], fp64=True)
    assert np.allclose(c_next[rows].cpu().numpy(), truth[0], rtol=RTOL, atol=ATOL) and np.allclose(h[rows].cpu().numpy(), truth[1], rtol=RTOL, atol=ATOL)
