"""QLinearConv -> 1x1 QLinearConv (+ residual join) as one kernel (chxq_qlinear_conv_chain_packed), at the widths of the ResNet-50
bottlenecks: bit-identical to the two packed calls in sequence and to the integer-domain oracle of the two ops."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _t(a, dev, cl=False):
    t = torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    return t.contiguous(memory_format=torch.channels_last) if cl else t


def _layer(rng, cin, cout, k):
    w = rng.integers(-127, 128, (cout, cin, k, k)).astype(np.int8)
    ws = rng.uniform(0.5, 1.5, cout).astype(np.float32) * np.float32(2.0 / (127.0 * np.sqrt(cin * k * k)))
    bias = rng.integers(-2000, 2000, cout).astype(np.int32)
    return w, ws, bias


# (name, N, cin, mid, cout, H, k, stride, pad, residual)
CASES = [
    ("res2_tail", 4, 64, 64, 256, 56, 3, 1, 1, True),
    ("res3_tail", 4, 128, 128, 512, 28, 3, 1, 1, True),
    ("res4_tail", 8, 256, 256, 1024, 14, 3, 1, 1, True),
    ("res3_no_join", 2, 128, 128, 512, 28, 3, 1, 1, False),
    ("ragged_cols_and_rows", 3, 64, 64, 208, 13, 3, 1, 1, True),   # 208 output channels: the last pass is clipped; 13 x 13 maps: ragged tiles
    ("first_1x1_strided", 2, 256, 128, 384, 28, 1, 2, 0, False),   # a strided 1x1 in front instead of a 3x3
    ("many_tiles_per_cta", 16, 64, 64, 128, 56, 3, 1, 1, True),    # more tiles than SMs x 2: the ring and the accumulator buffers wrap
]


@pytest.mark.parametrize("name,N,cin,mid,cout,H,k,stride,pad,res", CASES, ids=[c[0] for c in CASES])
def test_conv_chain_matches_two_calls_and_oracle(ops, orc, dev, name, N, cin, mid, cout, H, k, stride, pad, res):
    rng = np.random.default_rng(mid * 3 + cout + N)
    x = rng.integers(0, 256, (N, cin, H, H), dtype=np.uint8)
    w1, ws1, b1 = _layer(rng, cin, mid, k)
    w2, ws2, b2 = _layer(rng, mid, cout, 1)
    z1, z2 = np.zeros(mid, np.int8), np.zeros(cout, np.int8)
    sx, s1, s2, zy2 = np.float32(0.02), np.float32(0.05), np.float32(0.04), (117 if res else 0)
    Ho = (H + 2 * pad - k) // stride + 1
    pk1 = ops.PackedConv(_t(w1, dev), _t(z1, dev), x.shape, strides=(stride, stride), pads=(pad, pad))
    pk2 = ops.PackedConv(_t(w2, dev), _t(z2, dev), (N, mid, Ho, Ho))
    assert pk1.eligible and pk2.eligible
    c1 = dict(x_scale=sx, x_zero_point=np.uint8(0), w_scale=_t(ws1, dev), w_zero_point=_t(z1, dev), y_scale=s1, y_zero_point=np.uint8(0), b=_t(b1, dev),
              fold_scales=True)
    c2 = dict(x_scale=s1, x_zero_point=np.uint8(0), w_scale=_t(ws2, dev), w_zero_point=_t(z2, dev), y_scale=s2, y_zero_point=np.uint8(zy2), b=_t(b2, dev),
              fold_scales=True)
    r = None
    if res:
        r = rng.integers(0, 256, (N, cout, Ho, Ho), dtype=np.uint8)
        c2.update(residual=_t(r, dev, True), res_scale=0.04, res_zero_point=0, res_relu=True, out_scale=0.06, out_zero_point=0)
    xd = _t(x, dev, True)
    y = ops.QLinearConvChainPacked(xd, pk1, c1, pk2, c2)
    ops.device_status()
    y = y.cpu().numpy()
    # the two calls in sequence
    h = ops.QLinearConvPacked(xd, pk1, **{k_: v for k_, v in c1.items()})
    y2 = ops.QLinearConvPacked(h, pk2, **{k_: v for k_, v in c2.items()}).cpu().numpy()
    assert np.array_equal(y, y2), "%s: %d of %d bytes differ from the two calls" % (name, int((y != y2).sum()), y.size)
    # the integer-domain oracle of the two ops
    if N * Ho * Ho * cout <= 8 * 14 * 14 * 1024 * 4:
        acc1 = orc.conv_integer(x, w1, 0, None, strides=(stride, stride), pads=(pad, pad))
        hq = orc.requantize(acc1, sx, ws1, s1, 0, bias=b1, channel_axis=1, fold=True)
        acc2 = orc.conv_integer(hq, w2, 0, None)
        want = orc.requantize(acc2, s1, ws2, s2, zy2, bias=b2, channel_axis=1, fold=True)
        if res:
            want = orc.qadd_relu(want, s2, zy2, r, 0.04, 0, 0.06, 0, relu=True, fold=True)
        assert np.array_equal(y, want), "%s: %d of %d bytes differ from the oracle" % (name, int((y != want).sum()), y.size)


def test_conv_chain_refuses_what_it_cannot_run(ops, dev):
    """Pairs without a fused kernel answer ERR_UNSUPPORTED (the caller then makes two calls); inconsistent pairs are invalid."""
    rng = np.random.default_rng(5)
    N, cin, mid, cout, H = 2, 64, 96, 256, 8   # 96 channels between the layers: no kernel
    w1, ws1, b1 = _layer(rng, cin, mid, 3)
    w2, ws2, b2 = _layer(rng, mid, cout, 1)
    z1, z2 = np.zeros(mid, np.int8), np.zeros(cout, np.int8)
    x = _t(rng.integers(0, 256, (N, cin, H, H), dtype=np.uint8), dev, True)
    pk1 = ops.PackedConv(_t(w1, dev), _t(z1, dev), x.shape, strides=(1, 1), pads=(1, 1))
    pk2 = ops.PackedConv(_t(w2, dev), _t(z2, dev), (N, mid, H, H))
    c1 = dict(x_scale=0.02, x_zero_point=np.uint8(0), w_scale=_t(ws1, dev), w_zero_point=_t(z1, dev), y_scale=0.05, y_zero_point=np.uint8(0), b=_t(b1, dev),
              fold_scales=True)
    c2 = dict(x_scale=0.05, x_zero_point=np.uint8(0), w_scale=_t(ws2, dev), w_zero_point=_t(z2, dev), y_scale=0.04, y_zero_point=np.uint8(0), b=_t(b2, dev),
              fold_scales=True)
    with pytest.raises(ops.ChxqError) as ei:
        ops.QLinearConvChainPacked(x, pk1, c1, pk2, c2)
    assert ei.value.code == ops._lib.ERR_UNSUPPORTED
    with pytest.raises(ops.ChxqError) as ei:   # reference-order requantization: no fused kernel
        ops.QLinearConvChainPacked(x, pk1, dict(c1, fold_scales=False), pk2, c2)
    assert ei.value.code == ops._lib.ERR_UNSUPPORTED
    with pytest.raises(ops.ChxqError) as ei:   # the second layer's input scale is not the first one's output scale
        ops.QLinearConvChainPacked(x, pk1, c1, pk2, dict(c2, x_scale=0.07))
    assert ei.value.code == ops._lib.ERR_INVALID_ARGUMENT
    ops.device_status()
