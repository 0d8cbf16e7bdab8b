"""Whole-network parity: the int8 ResNet-50 and the quantized MLP against the oracle's op chains."""
import numpy as np
import pytest
import torch

from helpers import lsb_report

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def small_resnet(pkg, dev):
    from chainer_compiler_b200 import models
    torch.manual_seed(0)
    net = models.ResNet50Int8(batch=4, device=dev, seed=1, image=64, num_classes=40, width_mult=0.25)
    rng = np.random.default_rng(0)
    x = rng.uniform(0, 1, (4, 3, 64, 64)).astype(np.float32)
    xt = torch.from_numpy(x).to(dev)
    net.calibrate(xt)
    return net, x, xt


def test_resnet_fused_unfused_graph_agree(small_resnet, ops):
    net, x, xt = small_resnet
    taps_f, taps_u = {}, {}
    lf = net.forward(xt, fused=True, taps=taps_f)
    lu = net.forward(xt, fused=False, taps=taps_u)
    ops.device_status()
    for k in taps_f:
        assert torch.equal(taps_f[k], taps_u[k]), k
    assert torch.equal(lf, lu)
    graph, lg = net.capture(xt)
    lg.zero_()
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(lg, lf)


def test_resnet_matches_oracle(small_resnet, orc, ops):
    import __graft_entry__ as entry
    entry.load_oracle()
    from oracle import networks
    net, x, xt = small_resnet
    params = net.export_numpy()
    taps = {}
    logits = net.forward(xt, taps=taps).cpu().numpy()
    ops.device_status()
    otaps = {}
    want = networks.resnet50_forward(params, x, mode="exact", taps=otaps)
    for k, v in otaps.items():
        got = taps[k].cpu().numpy()
        assert np.array_equal(got, v), "tap %s differs from the integer-domain oracle" % k
    assert np.array_equal(logits, want)
    # against the reference's fp32-emulating chain: per layer the mismatch is at most one step; end to end the steps compound,
    # so the whole-network check is on the logits (they stay close) with the per-tap mismatch counts reported.
    etaps = {}
    emul = networks.resnet50_forward(params, x, mode="emulate", taps=etaps)
    mx, cnt, tot = lsb_report(taps["stem"].cpu().numpy(), etaps["stem"])
    print("stem: %d of %d bytes differ from the fp32-emulating chain (max %d LSB)" % (cnt, tot, mx))
    assert mx <= 1
    worst = 0
    for k in otaps:
        if k.startswith("block"):
            m, c, t = lsb_report(taps[k].cpu().numpy(), etaps[k])
            worst = max(worst, m)
    print("blocks: worst compounded difference %d LSB; logits max abs diff %.3g" % (worst, np.abs(logits - emul).max()))
    assert np.abs(logits - emul).max() <= 0.05 * max(1.0, np.abs(emul).max())


def test_resnet_folded_requantization(small_resnet, orc, ops):
    """forward(fold=True) -- what the benchmark runs -- is bit-exact against the oracle chain restating the folded arithmetic,
    and its logits stay close to the reference-order network's."""
    import __graft_entry__ as entry
    entry.load_oracle()
    from oracle import networks
    net, x, xt = small_resnet
    taps = {}
    logits = net.forward(xt, taps=taps, fold=True).cpu().numpy()
    ops.device_status()
    otaps = {}
    want = networks.resnet50_forward(net.export_numpy(), x, mode="fold", taps=otaps)
    for k, v in otaps.items():
        assert np.array_equal(taps[k].cpu().numpy(), v), k
    assert np.array_equal(logits, want)
    exact = net.forward(xt).cpu().numpy()
    ex_taps = {}
    net.forward(xt, taps=ex_taps)
    mx, cnt, tot = lsb_report(taps["stem"].cpu().numpy(), ex_taps["stem"].cpu().numpy())
    print("stem, folded vs reference-order requantization: %d of %d bytes differ (max %d LSB)" % (cnt, tot, mx))
    assert mx <= 1
    assert np.abs(logits - exact).max() <= 0.05 * max(1.0, np.abs(exact).max())
    graph, lg = net.capture(xt, fold=True)
    graph.replay()
    torch.cuda.synchronize()
    assert np.array_equal(lg.cpu().numpy(), logits)


def test_resnet_layer_outputs_within_one_step_of_reference_chain(small_resnet, orc, ops):
    """Each QLinearConv of the network, fed the SAME input bytes on both sides, is at most 1 LSB from the reference's
    dequantize -> fp32 conv -> quantize result; the mismatch count is reported."""
    net, x, xt = small_resnet
    xq = ops.QuantizeLinear(xt, net.in_scale, np.uint8(0))
    h = net._run_conv(net.stem, xq)
    h = ops.MaxPoolU8(h, 3, 2, 0, cover_all=True)
    total = diff = 0
    for b in net.blocks[:4]:
        for name in ("conv1", "conv2", "conv3"):
            c = b[name]
            inp = h if name == "conv1" else prev
            out = net._run_conv(c, inp)
            ref = orc.qlinear_conv(inp.cpu().numpy(), c.x_scale, 0, c.w_q, c.w_scale, c.w_zp.astype(np.int32), c.y_scale, c.y_zp, b=c.bias_q,
                                   strides=(c.stride, c.stride), pads=(c.pad, c.pad))
            mx, cnt, tot = lsb_report(out.cpu().numpy(), ref)
            assert mx <= 1, c.name
            total += tot
            diff += cnt
            prev = out
        sc = net._run_conv(b["proj"], h) if b["proj"] is not None else h
        h = ops.QAddU8(prev, b["conv3"].y_scale, b["conv3"].y_zp, sc, b["res"][0], b["res"][1], b["out_scale"], 0, relu=True)
    print("QLinearConv layers: %d of %d output bytes differ by 1 LSB from the fp32-emulating reference chain" % (diff, total))
    ops.device_status()


def test_mlp_matches_oracle(pkg, ops, orc, dev):
    import __graft_entry__ as entry
    entry.load_oracle()
    from oracle import networks
    from chainer_compiler_b200 import models
    mlp = models.QuantizedMLP(dev, seed=0)
    rng = np.random.default_rng(0)
    x = rng.uniform(0, 1, (64, 784)).astype(np.float32)
    layers = [dict(w_q=l["w_q"], w_scale=l["w_scale"]) for l in mlp.layers]
    exact = networks.mlp_forward(layers, mlp.act_scale, x, mode="exact")
    emul = networks.mlp_forward(layers, mlp.act_scale, x, mode="emulate")
    for path in (1, 0):
        y = mlp.forward(torch.from_numpy(x).to(dev), path=path).cpu().numpy()
        assert y.shape == (64, 10) and np.array_equal(y, exact)
        assert np.abs(y - emul).max() <= 3 * float(mlp.act_scale)  # three requantizing layers, one step each at most... compounded
    # constant weights packed once (each MatMul as a packed 1x1 convolution): the same bits
    assert np.array_equal(mlp.forward_packed(torch.from_numpy(x).to(dev)).cpu().numpy(), exact)
    ops.device_status()


@pytest.fixture(scope="module")
def small_mobilenet(pkg, dev):
    from chainer_compiler_b200 import models
    net = models.MobileNetV2Int8(batch=2, device=dev, seed=3, image=64, num_classes=24)
    rng = np.random.default_rng(5)
    x = rng.uniform(0, 1, (2, 3, 64, 64)).astype(np.float32)
    xt = torch.from_numpy(x).to(dev)
    net.calibrate(xt)
    return net, x, xt


def test_mobilenet_fused_unfused_agree(small_mobilenet, ops):
    net, x, xt = small_mobilenet
    tf, tu = {}, {}
    lf = net.forward(xt, fused=True, taps=tf)
    lu = net.forward(xt, fused=False, taps=tu)
    ops.device_status()
    for k in tf:
        assert torch.equal(tf[k], tu[k]), k
    assert torch.equal(lf, lu)


@pytest.mark.parametrize("mode", ["exact", "fold"])
def test_mobilenet_matches_oracle(small_mobilenet, orc, ops, mode):
    """MobileNetV2 (1x1 tensor-core layers with asymmetric activation zero points, depthwise 3x3 stride 1 and 2, ReLU6 clamps,
    residual joins without Relu) against the oracle's chain, every block output bit-exact."""
    import __graft_entry__ as entry
    entry.load_oracle()
    from oracle import networks
    net, x, xt = small_mobilenet
    taps = {}
    logits = net.forward(xt, taps=taps, fold=(mode == "fold")).cpu().numpy()
    ops.device_status()
    otaps = {}
    want = networks.mobilenetv2_forward(net.export_numpy(), x, mode=mode, taps=otaps)
    for k, v in otaps.items():
        assert np.array_equal(taps[k].cpu().numpy(), v), "tap %s differs" % k
    assert np.array_equal(logits, want)
    if mode == "exact":
        etaps = {}
        emul = networks.mobilenetv2_forward(net.export_numpy(), x, mode="emulate", taps=etaps)
        mx, cnt, tot = lsb_report(taps["stem"].cpu().numpy(), etaps["stem"])
        print("mobilenet stem: %d of %d bytes differ from the fp32-emulating chain (max %d LSB)" % (cnt, tot, mx))
        assert mx <= 1
        # 52 quantized layers compound their 1-LSB differences: the whole-network bound is on the relative L2 distance
        rel = float(np.linalg.norm(logits - emul) / np.linalg.norm(emul))
        print("mobilenet logits: relative L2 distance to the fp32-emulating chain %.3g" % rel)
        assert rel <= 0.1


def test_engine_stream_matches_single_calls(pkg, dev):
    """InferenceEngine.run_stream (double-buffered copies around the captured graph) returns, batch by batch, what the
    synchronous run_host returns."""
    from chainer_compiler_b200 import models, dataparallel as dp
    net = models.ResNet50Int8(batch=2, device=dev, seed=2, image=64, num_classes=16, width_mult=0.25)
    eng = dp.InferenceEngine(net, 1, fold=True)
    gen = torch.Generator().manual_seed(3)
    eng.prepare(torch.rand((2, 3, 64, 64), generator=gen).to(dev))
    batches = [torch.rand((2, 3, 64, 64), generator=gen).pin_memory() for _ in range(5)]
    want = [eng.run_host(b).clone() for b in batches]
    got = [h.clone() for h in eng.run_stream(batches)]
    assert len(got) == 5
    for g, w in zip(got, want):
        assert torch.equal(g, w)
    got2 = [h.clone() for h in eng.run_stream(batches[:1])]
    assert torch.equal(got2[0], want[0])
    # the device-resident step alternates between the two captured graphs: both give the same logits
    eng.set_resident_input(batches[0])
    for _ in range(3):
        out = eng.step_device()
        eng.drain()
        torch.cuda.synchronize()
        assert torch.equal(out.cpu(), want[0])


def test_engine_uint8_host_batches_give_the_same_logits(pkg, ops, dev):
    """An engine fed batches the host has already quantized (QuantizeLinear with the network's input scale) returns the logits of
    the fp32-input engine bit for bit: the stem reads the uint8 NCHW map directly instead of quantizing on the fly."""
    from chainer_compiler_b200 import models, dataparallel as dp
    net = models.ResNet50Int8(batch=2, device=dev, seed=2, image=64, num_classes=16, width_mult=0.25)
    gen = torch.Generator().manual_seed(4)
    calib = torch.rand((2, 3, 64, 64), generator=gen)
    eng = dp.InferenceEngine(net, 1, fold=True)
    eng.prepare(calib.to(dev))
    eng8 = dp.InferenceEngine(net, 1, fold=True, input_dtype=torch.uint8)
    eng8.prepare(calib)
    batches = [torch.rand((2, 3, 64, 64), generator=gen).pin_memory() for _ in range(3)]
    qbatches = [ops.QuantizeLinear(b.to(dev), net.in_scale, np.uint8(0)).cpu().pin_memory() for b in batches]
    want = [eng.run_host(b).clone() for b in batches]
    got = [h.clone() for h in eng8.run_stream(qbatches)]
    for g, w in zip(got, want):
        assert torch.equal(g, w)
    ops.device_status()
