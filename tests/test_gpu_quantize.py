"""QuantizeLinear / DequantizeLinear / one-pass glue kernels against the CPU oracle: bit-exact."""
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "hotpath_vectors.npz")


def _t(a, dev):
    return torch.from_numpy(np.ascontiguousarray(a)).to(dev)


@pytest.mark.parametrize("n", [0, 1, 15, 16, 17, 1000, 65536 + 5])
@pytest.mark.parametrize("zp,dtype", [(0, np.uint8), (131, np.uint8), (0, np.int8), (-17, np.int8)])
@pytest.mark.parametrize("mode", [0, 1])
def test_quantize_linear_bit_exact(ops, orc, dev, n, zp, dtype, mode):
    rng = np.random.default_rng(n + 1)
    x = np.concatenate([rng.uniform(-4, 4, n), (np.arange(n) - n // 2 + 0.5) * 0.013])[:n].astype(np.float32)
    y = ops.QuantizeLinear(_t(x, dev), 0.013, dtype(zp), round_mode=mode).cpu().numpy()
    want = orc.quantize_linear(x, 0.013, zp, dtype, mode)
    assert y.dtype == want.dtype and np.array_equal(y, want)


def test_quantize_linear_ties_and_mode_difference(ops, orc, dev):
    """Exact .5 ties: the reference rounds half up (quantize.cc:33-34), ONNX rounds half to even; both are offered and the
    number of elements on which they differ is what the oracle counts."""
    x = ((np.arange(0, 255) + 0.5) * 0.25).astype(np.float32)  # exactly representable ties at scale 0.25
    ref = ops.QuantizeLinear(_t(x, dev), 0.25, np.uint8(0), round_mode=ops.ROUND_REF).cpu().numpy()
    rne = ops.QuantizeLinear(_t(x, dev), 0.25, np.uint8(0), round_mode=ops.ROUND_RNE).cpu().numpy()
    assert np.array_equal(ref, orc.quantize_linear(x, 0.25, 0)) and np.array_equal(rne, orc.quantize_linear(x, 0.25, 0, round_mode=1))
    assert int((ref != rne).sum()) == orc.quantize_mode_diff(x, 0.25, 0) == 128


def test_quantize_unaligned_and_default_zero_point(ops, orc, dev):
    rng = np.random.default_rng(3)
    x = rng.uniform(0, 1, 4099).astype(np.float32)
    xt = _t(x, dev)[3:]  # 12-byte offset: the scalar kernel must take over
    y = ops.QuantizeLinear(xt, 1.0 / 255.0).cpu().numpy()  # absent zero point -> uint8 0 (quantize.cc:50-51)
    assert y.dtype == np.uint8 and np.array_equal(y, orc.quantize_linear(x[3:], 1.0 / 255.0, 0))


def test_quantize_preserves_layout(ops, orc, dev):
    rng = np.random.default_rng(4)
    x = rng.uniform(-1, 1, (2, 5, 4, 3)).astype(np.float32)
    xt = _t(x, dev).contiguous(memory_format=torch.channels_last)
    y = ops.QuantizeLinear(xt, 0.01, np.uint8(128))
    assert y.is_contiguous(memory_format=torch.channels_last)
    assert np.array_equal(y.cpu().numpy(), orc.quantize_linear(x, 0.01, 128))


@pytest.mark.parametrize("n", [0, 1, 16, 33, 100003])
@pytest.mark.parametrize("zp,dtype", [(0, np.uint8), (3, np.uint8), (-5, np.int8)])
def test_dequantize_linear_bit_exact(ops, orc, dev, n, zp, dtype):
    rng = np.random.default_rng(n + 7)
    q = rng.integers(np.iinfo(dtype).min, np.iinfo(dtype).max + 1, n).astype(dtype)
    y = ops.DequantizeLinear(_t(q, dev), 0.037, dtype(zp)).cpu().numpy()
    assert np.array_equal(y, orc.dequantize_linear(q, 0.037, zp))


def test_quantize_rejects(ops, dev):
    with pytest.raises(ops.ChxqError):
        ops.QuantizeLinear(torch.zeros(4, device=dev), 1.0, np.int16(0))  # zero point dtype decides the output dtype
    with pytest.raises(ops.ChxqError):
        ops.QuantizeLinear(torch.zeros(4, device=dev, dtype=torch.float64), 1.0)
    with pytest.raises(ops.ChxqError):
        ops.DequantizeLinear(torch.zeros(4, device=dev), 1.0)


def test_golden_quantize(ops, dev):
    g = np.load(GOLDEN)
    x = _t(g["q_x"], dev)
    assert np.array_equal(ops.QuantizeLinear(x, 0.02, np.uint8(3)).cpu().numpy(), g["q_u8_ref"])
    assert np.array_equal(ops.QuantizeLinear(x, 0.02, np.uint8(3), round_mode=1).cpu().numpy(), g["q_u8_rne"])
    assert np.array_equal(ops.QuantizeLinear(x, 0.02, np.int8(-5)).cpu().numpy(), g["q_i8_ref"])
    assert np.array_equal(ops.QuantizeLinear(x, 0.02, np.int8(-5), round_mode=1).cpu().numpy(), g["q_i8_rne"])
    assert np.array_equal(ops.DequantizeLinear(_t(g["q_u8_ref"], dev), 0.02, np.uint8(3)).cpu().numpy(), g["dq_u8"])
    assert np.array_equal(ops.DequantizeLinear(_t(g["q_i8_ref"], dev), 0.031, np.int8(-5)).cpu().numpy(), g["dq_i8"])


def test_quantize_dequantize_round_trip_full_size(ops, dev):
    """ResNet-50 input size (256 x 3 x 224 x 224): Q(DQ(q)) == q for every byte value pattern, and the output histogram of a
    uniform input is flat -- properties that need no CPU pass over 38.5 M elements."""
    n = 256 * 3 * 224 * 224
    q = (torch.arange(n, device=dev, dtype=torch.int64) * 2654435761 >> 7).to(torch.uint8)
    x = ops.DequantizeLinear(q, 1.0 / 255.0, np.uint8(0))
    q2 = ops.QuantizeLinear(x, 1.0 / 255.0, np.uint8(0))
    assert torch.equal(q, q2)
    q3 = ops.QuantizeLinear(ops.DequantizeLinear(q, 0.05, np.uint8(77)), 0.05, np.uint8(77), round_mode=1)
    assert torch.equal(q, q3)


def test_glue_kernels(ops, orc, dev):
    rng = np.random.default_rng(11)
    x = rng.integers(0, 256, (3, 32, 13, 13), dtype=np.uint8)
    xt = _t(x, dev).contiguous(memory_format=torch.channels_last)
    for cover in (False, True):
        y = ops.MaxPoolU8(xt, 3, 2, 0, cover_all=cover)
        assert np.array_equal(y.cpu().numpy(), orc.maxpool_u8(x, 3, 2, 0, cover_all=cover))
    x2 = rng.integers(0, 256, (2, 24, 5, 5), dtype=np.uint8)  # 24 channels: scalar path
    y = ops.MaxPoolU8(_t(x2, dev).contiguous(memory_format=torch.channels_last), 3, 1, 1)
    assert np.array_equal(y.cpu().numpy(), orc.maxpool_u8(x2, 3, 1, 1))
    p = ops.GlobalAveragePoolDequant(xt, 0.031, 4)
    assert np.array_equal(p.cpu().numpy(), orc.global_avgpool_dq(x, 0.031, 4))
    w = rng.standard_normal((10, 32)).astype(np.float32)
    b = rng.standard_normal(10).astype(np.float32)
    pf = p.cpu().numpy()
    assert np.array_equal(ops.Linear(p, _t(w, dev), _t(b, dev)).cpu().numpy(), orc.linear_f32(pf, w, b))
    a = rng.integers(0, 256, (2, 16, 7, 7), dtype=np.uint8)
    c = rng.integers(0, 256, (2, 16, 7, 7), dtype=np.uint8)
    for relu in (True, False):
        y = ops.QAddU8(_t(a, dev), 0.02, 131, _t(c, dev), 0.05, 7, 0.04, 0 if relu else 99, relu=relu)
        assert np.array_equal(y.cpu().numpy(), orc.qadd_relu(a, 0.02, 131, c, 0.05, 7, 0.04, 0 if relu else 99, relu=relu))
    f = rng.standard_normal(100003).astype(np.float32)
    mm = ops.MinMax(_t(f, dev)).cpu().numpy()
    assert mm[0] == f.min() and mm[1] == f.max()
    nchw = _t(x, dev)
    assert torch.equal(ops.to_contiguous_nchw(ops.to_channels_last(nchw)), nchw)
    assert torch.equal(ops.to_channels_last(nchw), xt)
    ops.device_status()


def test_quantize_division_is_correctly_rounded(ops, orc, dev):
    """The uint8 round-half-up kernel divides by the (constant) scale with a reciprocal and two residual corrections instead
    of an IEEE division per element.  Values sitting one or two ulps either side of every rounding boundary, over ordinary,
    power-of-two, nearly-power-of-two, tiny and huge scales, must still quantize exactly as x / scale does."""
    rng = np.random.default_rng(123)
    scales = [1.0 / 255.0, 0.02, 0.25, 3.0, 1e-3, 0.0123456, np.float32(1.9999999), np.float32(1.0000001), 7e-9, 3.3e7, 1e-20, 1e20,
              float(np.nextafter(np.float32(0.5), np.float32(0)))] + list(rng.uniform(1e-4, 10.0, 12).astype(np.float32))
    k = np.arange(-4, 262, dtype=np.float64)
    for s in scales:
        s32 = np.float32(s)
        base = ((k + 0.5) * np.float64(s32)).astype(np.float32)  # boundaries of the half-up rounding
        xs = [base]
        for ulps in (1, 2, 3):
            up, dn = base.copy(), base.copy()
            for _ in range(ulps):
                up = np.nextafter(up, np.float32(np.inf))
                dn = np.nextafter(dn, np.float32(-np.inf))
            xs += [up, dn]
        xs.append((rng.uniform(-5, 300, 200000) * np.float64(s32)).astype(np.float32))
        xs.append(np.array([0.0, -0.0, np.inf, -np.inf, 1e38, -1e38, 1e-45, 1e-38], np.float32))
        x = np.concatenate(xs).astype(np.float32)
        x = np.concatenate([x, x[: (-len(x)) % 4]])
        for zp in (0, 7):
            got = ops.QuantizeLinear(torch.from_numpy(x).to(dev), float(s32), np.uint8(zp)).cpu().numpy()
            want = orc.quantize_linear(x, s32, zp)
            assert np.array_equal(got, want), "scale %r zero point %d: %d mismatches" % (s, zp, int((got != want).sum()))


@pytest.mark.parametrize("to_int8", [True, False])
@pytest.mark.parametrize("per_channel", [True, False])
def test_prepare_weights_matches_host_quantizer_and_merge(pkg, ops, orc, dev, to_int8, per_channel):
    """Device model preparation (Conv + BatchNormalization merge, then the weight quantizer) against the oracle's merge
    (compiler/merge.cc:166-189) followed by its quantizer (compiler/quantize.cc:70-129): every output bit for bit."""
    rng = np.random.default_rng(31 + 2 * int(to_int8) + int(per_channel))
    for shape in ((64, 16, 3, 3), (10, 1000), (7, 3, 1, 1), (300, 5, 5, 5)):
        w = (rng.standard_normal(shape) * 0.1).astype(np.float32)
        w[0].reshape(-1)[:3] = [0.0, 0.05, -0.05]
        if shape[0] > 8:
            w[3] = np.abs(w[3])       # a channel with no negative weight (range widened to include zero)
            w[5] = 0.0                # an all-zero channel: uint8 scale 1; int8 scale 0 is left out below
        M = shape[0]
        gamma, beta = rng.uniform(0.5, 1.5, M).astype(np.float32), (rng.standard_normal(M) * 0.1).astype(np.float32)
        mean, var = (rng.standard_normal(M) * 0.1).astype(np.float32), rng.uniform(0.5, 1.5, M).astype(np.float32)
        bias = (rng.standard_normal(M) * 0.1).astype(np.float32)
        if to_int8 and per_channel and shape[0] > 8:
            w[5].reshape(-1)[0] = 0.01    # int8 with scale 0 divides 0 by 0 in the reference: not a defined case
        for bn, cb in ((None, None), ((gamma, beta, mean, var), None), ((gamma, beta, mean, var), bias)):
            if bn is None:
                wf, bf = w, None
            else:
                wf, bf = orc.merge_conv_bn(w, gamma, beta, mean, var, 2e-5, cb)
            if per_channel:
                qo, so, zo = orc.quantize_weight_per_channel(wf, to_int8)
            else:
                qo, so, zo = orc.quantize_data(wf, to_int8)
                so, zo = np.array([so], np.float32), np.array([zo], np.int32)
            tb = None if bn is None else tuple(torch.from_numpy(v).to(dev) for v in bn)
            q, s, z, fb, fw = ops.PrepareWeights(torch.from_numpy(w).to(dev), tb, None if cb is None else torch.from_numpy(cb).to(dev), 2e-5,
                                                 to_int8, per_channel, return_folded=True)
            ops.device_status()
            assert np.array_equal(fw.cpu().numpy(), wf), (shape, "folded weights")
            assert np.array_equal(s.cpu().numpy(), so) and np.array_equal(z.cpu().numpy(), zo), (shape, "scales / zero points")
            assert np.array_equal(q.cpu().numpy(), qo), (shape, "quantized weights")
            if bn is not None:
                assert np.array_equal(fb.cpu().numpy(), bf), (shape, "folded bias")
            else:
                assert fb is None
    from chainer_compiler_b200 import _lib
    with pytest.raises(_lib.ChxqError):
        ops.PrepareWeights(torch.zeros((4, 3), device=dev), (torch.ones(3, device=dev),) * 4)
