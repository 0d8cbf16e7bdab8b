"""ConvInteger / QLinearConv: CUDA-core, depthwise and tcgen05 kernels against the CPU oracle.
int32 accumulators bit-exact; requantized outputs bit-exact against the integer-domain oracle and at most one step from the
fp32-emulating oracle (the reference's dequantize -> fp32 conv -> quantize), mismatch counts printed."""
import os

import numpy as np
import pytest
import torch

from helpers import lsb_report

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "hotpath_vectors.npz")
SIMT, TENSOR, AUTO = 1, 2, 0


def _t(a, dev, cl=False):
    if a is None:
        return None
    t = torch.from_numpy(np.array(a)).to(dev)  # np.array keeps 0-d arrays 0-d
    return t.contiguous(memory_format=torch.channels_last) if cl else t


def _rand(rng, shape, dtype, lo=None, hi=None):
    lo = np.iinfo(dtype).min if lo is None else lo
    hi = np.iinfo(dtype).max if hi is None else hi
    return rng.integers(lo, hi + 1, shape).astype(dtype)


@pytest.mark.parametrize("N,C,H,W,M,k,stride,pad,group,auto_pad", [
    (2, 8, 9, 11, 12, 3, (2, 1), (1, 1), 2, ""),
    (1, 3, 16, 16, 8, 7, (2, 2), (3, 3), 1, ""),
    (2, 6, 7, 7, 6, 3, (1, 1), (1, 1), 6, ""),
    (1, 4, 10, 10, 5, 5, (), (), 1, "SAME_UPPER"),
    (2, 4, 9, 9, 4, 2, (2, 2), (), 1, "SAME_UPPER"),
    (1, 16, 5, 5, 32, 1, (), (), 1, ""),
])
@pytest.mark.parametrize("cl", [False, True])
def test_conv_integer_simt(ops, orc, dev, N, C, H, W, M, k, stride, pad, group, auto_pad, cl):
    rng = np.random.default_rng(C * 100 + M)
    x = _rand(rng, (N, C, H, W), np.uint8)
    w = _rand(rng, (M, C // group, k, k), np.int8)
    for zx, zw in ((None, None), (7, _rand(rng, M, np.int8, -9, 9)), (128, np.array([3], np.int8))):
        y = ops.ConvInteger(_t(x, dev, cl), _t(w, dev), None if zx is None else np.uint8(zx), _t(zw, dev), stride, pad, group, auto_pad, path=SIMT)
        want = orc.conv_integer(x, w, zx, zw, stride, pad, group, auto_pad)
        assert y.shape == want.shape and np.array_equal(y.cpu().numpy(), want)


# (N, C, H, W, M, k, stride, pad): direct TMA path when stride 1, im2col path otherwise
TC_CASES = [
    (2, 64, 8, 8, 64, 1, 1, 0),      # 1x1, flattened positions
    (3, 128, 7, 7, 256, 1, 1, 0),    # odd map, ragged position tile, BN 256
    (2, 64, 8, 8, 64, 3, 1, 1),      # 3x3, box 8x8x2
    (5, 32, 7, 7, 48, 3, 1, 1),      # odd map: box 1x1x128 over 5 images, bk 32, ragged N tile
    (2, 48, 12, 12, 80, 3, 1, 1),    # C = 48 -> bk 32 + zero-filled chunk? (48 = 32 + 16), box 4x4x8
    (2, 144, 6, 6, 32, 1, 1, 0),     # C = 144 -> ragged last K chunk filled by TMA
    (2, 256, 14, 14, 128, 3, 1, 1),  # box 2x2x32, bk 128
    (4, 64, 16, 16, 128, 1, 2, 0),   # stride 2 1x1: TMA box with element strides
    (2, 16, 9, 9, 24, 3, 2, 1),      # stride 2 3x3 with padding (strided box, shifted per tap), M = 24 (ragged column tile, scalar stores)
    (1, 64, 10, 10, 64, 5, 1, 2),    # 5x5
]


@pytest.mark.parametrize("N,C,H,W,M,k,stride,pad", TC_CASES)
def test_conv_integer_tensor(ops, orc, dev, N, C, H, W, M, k, stride, pad):
    rng = np.random.default_rng(C + M + H)
    x = _rand(rng, (N, C, H, W), np.uint8)
    w = _rand(rng, (M, C, k, k), np.int8)
    y = ops.ConvInteger(_t(x, dev, True), _t(w, dev), None, None, (stride, stride), (pad, pad), path=TENSOR)
    ops.device_status()
    assert y.is_contiguous(memory_format=torch.channels_last)
    want = orc.conv_integer(x, w, None, None, (stride, stride), (pad, pad))
    assert np.array_equal(y.cpu().numpy(), want)
    # the reference's own signature, NCHW in and NCHW out, on the tensor-core kernels (transposes through the workspace)
    y2 = ops.ConvInteger(_t(x, dev, False), _t(w, dev), None, None, (stride, stride), (pad, pad), path=TENSOR)
    ops.device_status()
    assert y2.is_contiguous() and np.array_equal(y2.cpu().numpy(), want)


@pytest.mark.parametrize("N,C,H,W,M,k,stride,pad", [TC_CASES[2], TC_CASES[4], TC_CASES[8], TC_CASES[0]])
@pytest.mark.parametrize("zx,zwmode,wdt", [(128, None, np.int8), (0, "vec", np.uint8), (9, "vec", np.int8), (200, "scalar", np.uint8)])
def test_conv_integer_tensor_zero_points(ops, orc, dev, N, C, H, W, M, k, stride, pad, zx, zwmode, wdt):
    """Zero points on the tensor-core path: x_zp with padding needs the explicit pad value (im2col); w_zp needs the
    per-position input sums."""
    rng = np.random.default_rng(zx + M)
    x = _rand(rng, (N, C, H, W), np.uint8)
    w = _rand(rng, (M, C, k, k), wdt)
    zw = None if zwmode is None else (_rand(rng, M, wdt, 0, 20) if zwmode == "vec" else _rand(rng, 1, wdt, 1, 20))
    y = ops.ConvInteger(_t(x, dev, True), _t(w, dev), np.uint8(zx), _t(zw, dev), (stride, stride), (pad, pad), path=TENSOR)
    ops.device_status()
    want = orc.conv_integer(x, w, zx, zw, (stride, stride), (pad, pad))
    assert np.array_equal(y.cpu().numpy(), want)


@pytest.mark.parametrize("shape,M,k,pad,nchw", [
    ((3, 3, 30, 30), 64, 7, 3, True),    # ResNet stem: 4 x 4 blocks per window
    ((2, 3, 17, 21), 32, 3, 1, True),    # MobileNet stem, odd map
    ((2, 1, 16, 16), 16, 5, 2, True),    # one channel, 5x5
    ((2, 4, 13, 12), 24, 4, 0, False),   # NHWC input with four channels, no padding, even window
    ((1, 2, 9, 9), 8, 2, 0, True),       # 2x2 / 2: a single block per window
])
def test_conv_stride2_small_channel_space_to_depth(ops, orc, dev, pkg, shape, M, k, pad, nchw):
    """Stride-2 convolutions over at most four channels (network stems) run as a stride-1 convolution over 2x2 pixel blocks
    read through a TMA map with overlapping rows; packed entry, NHWC output.  Accumulators against the oracle with and
    without zero points (the block map's halo holds the activation zero point), and the requantizing entry on top."""
    import ctypes
    from chainer_compiler_b200 import _lib
    rng = np.random.default_rng(k * 10 + M)
    x = _rand(rng, shape, np.uint8)
    w = _rand(rng, (M, shape[1], k, k), np.int8)
    xt = _t(x, dev) if nchw else _t(x, dev, True)
    for zx, wz in ((0, None), (77, None), (5, _rand(rng, M, np.int8, -9, 9))):
        pk = ops.PackedConv(_t(w, dev), _t(wz, dev), x.shape, (2, 2), (pad, pad), x_layout=_lib.NCHW if nchw else _lib.NHWC)
        assert pk.eligible
        g = pk.g
        y = torch.empty((g.N, g.M, g.Ho, g.Wo), dtype=torch.int32, device=dev, memory_format=torch.channels_last)
        nb = pkg.lib().chxq_conv_packed_workspace(ctypes.byref(g), zx, pk.flags)
        ws = ops.workspace(nb, dev)
        _lib.check(pkg.lib().chxq_conv_integer_packed(ops._ptr(xt), ops._ptr(pk.blob), ctypes.byref(g), 1, zx, pk.flags, ops._ptr(y), ops._ptr(ws),
                                                      nb, ops._stream()))
        ops.device_status()
        assert np.array_equal(y.cpu().numpy(), orc.conv_integer(x, w, zx, wz, (2, 2), (pad, pad))), (zx, wz is not None)
    pk = ops.PackedConv(_t(w, dev), None, x.shape, (2, 2), (pad, pad), x_layout=_lib.NCHW if nchw else _lib.NHWC)
    ws_ = rng.uniform(0.0005, 0.002, M).astype(np.float32)
    bias = _rand(rng, M, np.int32, -3000, 3000)
    wz0 = np.zeros(M, np.int8)
    for fold in (False, True):
        yq = ops.QLinearConvPacked(xt, pk, 0.02, np.uint8(3), _t(ws_, dev), _t(wz0, dev), 0.05, np.uint8(20), b=_t(bias, dev), fold_scales=fold)
        ops.device_status()
        acc = orc.conv_integer(x, w, 3, wz0, (2, 2), (pad, pad))
        assert np.array_equal(yq.cpu().numpy(), orc.requantize(acc, 0.02, ws_, 0.05, 20, bias=bias, channel_axis=1, fold=fold)), fold


@pytest.mark.parametrize("path,cl", [(SIMT, False), (SIMT, True), (TENSOR, True), (TENSOR, False)])  # (TENSOR, False): NCHW in and out, as the reference's op
@pytest.mark.parametrize("N,C,H,W,M,k,stride,pad", [TC_CASES[2], TC_CASES[3], TC_CASES[8], TC_CASES[1]])
def test_qlinear_conv(ops, orc, dev, path, cl, N, C, H, W, M, k, stride, pad):
    rng = np.random.default_rng(M * 7 + k)
    x = _rand(rng, (N, C, H, W), np.uint8)
    w = _rand(rng, (M, C, k, k), np.int8, -127, 127)
    ws = rng.uniform(0.0005, 0.002, M).astype(np.float32)
    wz = np.zeros(M, np.int8)
    bias = _rand(rng, M, np.int32, -3000, 3000)
    sx, sy = 0.02, 0.09
    for zx, zy, mode in ((0, 0, 0), (0, 17, 1), (5, 3, 0)):
        y = ops.QLinearConv(_t(x, dev, cl), sx, np.uint8(zx), _t(w, dev), _t(ws, dev), _t(wz, dev), sy, np.uint8(zy), _t(bias, dev),
                            (stride, stride), (pad, pad), round_mode=mode, path=path)
        ops.device_status()
        y = y.cpu().numpy()
        acc = orc.conv_integer(x, w, zx, wz, (stride, stride), (pad, pad))
        exact = orc.requantize(acc, sx, ws, sy, zy, bias=bias, channel_axis=1, round_mode=mode)
        assert np.array_equal(y, exact), "integer-domain requantization must be bit-exact"
        emul = orc.qlinear_conv(x, sx, zx, w, ws, wz, sy, zy, b=bias, strides=(stride, stride), pads=(pad, pad), round_mode=mode)
        mx, cnt, tot = lsb_report(y, emul)
        print("QLinearConv C%d M%d k%d: %d of %d differ from the fp32-emulating chain, max %d LSB" % (C, M, k, cnt, tot, mx))
        assert mx <= 1


def test_qlinear_conv_per_tensor_weights_int8_output_and_nonzero_wzp(ops, orc, dev):
    rng = np.random.default_rng(12)
    x = _rand(rng, (2, 32, 6, 6), np.int8)  # int8 activations
    w = _rand(rng, (32, 32, 3, 3), np.uint8)  # asymmetric uint8 weights, per-tensor
    ws, wz = np.array(0.003, np.float32), np.array(120, np.uint8)
    for path, cl in ((SIMT, False), (TENSOR, True)):
        y = ops.QLinearConv(_t(x, dev, cl), 0.05, np.int8(-4), _t(w, dev), _t(ws, dev), _t(wz, dev), 0.4, np.int8(-9), None, (1, 1), (1, 1), path=path)
        ops.device_status()
        assert y.dtype == torch.int8
        acc = orc.conv_integer(x, w, -4, wz.reshape(1), (1, 1), (1, 1))
        exact = orc.requantize(acc, 0.05, ws.reshape(1), 0.4, -9, channel_axis=1, y_dtype=np.int8)
        assert np.array_equal(y.cpu().numpy(), exact)
        emul = orc.qlinear_conv(x, 0.05, -4, w, ws, wz, 0.4, -9, strides=(1, 1), pads=(1, 1), y_dtype=np.int8)
        assert lsb_report(y.cpu().numpy(), emul)[0] <= 1


def test_qlinear_conv_rejects(ops, dev):
    x = torch.zeros((1, 8, 4, 4), dtype=torch.uint8, device=dev)
    w = torch.zeros((8, 8, 3, 3), dtype=torch.int8, device=dev)
    s8, z8 = torch.ones(8, device=dev), torch.zeros(8, dtype=torch.int8, device=dev)
    with pytest.raises(ops.ChxqError):  # per-channel length != M (quantize.cc:79)
        ops.QLinearConv(x, 1.0, np.uint8(0), w, torch.ones(5, device=dev), torch.zeros(5, dtype=torch.int8, device=dev), 1.0, np.uint8(0))
    with pytest.raises(ops.ChxqError):  # scale / zero point ranks differ (quantize.cc:76-77)
        ops.QLinearConv(x, 1.0, np.uint8(0), w, s8, torch.zeros((), dtype=torch.int8, device=dev), 1.0, np.uint8(0))
    with pytest.raises(ops.ChxqError):  # group does not divide the channels
        ops.QLinearConv(x, 1.0, np.uint8(0), w, s8, z8, 1.0, np.uint8(0), group=3)
    with pytest.raises(ops.ChxqError):
        ops.QLinearConv(x, 1.0, np.uint8(0), w, s8, z8, 1.0, np.uint8(0), auto_pad="VALID")
    with pytest.raises(ops.ChxqError):  # kernel larger than the padded input
        ops.QLinearConv(x, 1.0, np.uint8(0), torch.zeros((8, 8, 7, 7), dtype=torch.int8, device=dev), s8, z8, 1.0, np.uint8(0))
    y = ops.QLinearConv(torch.zeros((0, 8, 4, 4), dtype=torch.uint8, device=dev), 1.0, np.uint8(0), w, s8, z8, 1.0, np.uint8(0), pads=(1, 1))
    assert y.shape == (0, 8, 4, 4)


@pytest.mark.parametrize("path", [SIMT, TENSOR])
def test_qlinear_conv_fused_residual_and_clamp(ops, orc, dev, path):
    """The epilogue fusions equal the separate ops bit for bit: QLinearConv, then DequantizeLinear x2 + Add + Relu +
    QuantizeLinear (residual tail); and the ReLU6 clamp in the quantized domain."""
    rng = np.random.default_rng(13)
    x = _rand(rng, (2, 64, 8, 8), np.uint8)
    w = _rand(rng, (128, 64, 1, 1), np.int8)
    ws = rng.uniform(0.0005, 0.002, 128).astype(np.float32)
    wz = np.zeros(128, np.int8)
    r = _rand(rng, (2, 128, 8, 8), np.uint8)
    xt, wt, wst, wzt, rt = _t(x, dev, True), _t(w, dev), _t(ws, dev), _t(wz, dev), _t(r, dev, True)
    plain = ops.QLinearConv(xt, 0.02, np.uint8(0), wt, wst, wzt, 0.05, np.uint8(121), path=path)
    tail = ops.QAddU8(plain, 0.05, 121, rt, 0.03, 14, 0.04, 0, relu=True)
    fused = ops.QLinearConv(xt, 0.02, np.uint8(0), wt, wst, wzt, 0.05, np.uint8(121), path=path, residual=rt, res_scale=0.03, res_zero_point=14,
                            out_scale=0.04, out_zero_point=0)
    ops.device_status()
    assert torch.equal(fused, tail)
    acc = orc.conv_integer(x, w, 0, wz)
    y1 = orc.requantize(acc, 0.02, ws, 0.05, 121, channel_axis=1)
    assert np.array_equal(fused.cpu().numpy(), orc.qadd_relu(y1, 0.05, 121, r, 0.03, 14, 0.04, 0, relu=True))
    clamped = ops.QLinearConv(xt, 0.02, np.uint8(0), wt, wst, wzt, 0.05, np.uint8(0), path=path, clamp_hi_q=120)
    want = orc.requantize(acc, 0.02, ws, 0.05, 0, channel_axis=1, clamp_hi_q=120)
    assert np.array_equal(clamped.cpu().numpy(), want) and want.max() == 120


@pytest.mark.parametrize("C,H,W,k,stride,pad", [(32, 14, 14, 3, 1, 1), (96, 15, 13, 3, 2, 1), (144, 7, 7, 3, 1, 1), (16, 9, 9, 5, 1, 2)])
def test_depthwise_qlinear_conv(ops, orc, dev, C, H, W, k, stride, pad):
    rng = np.random.default_rng(C + k)
    x = _rand(rng, (3, C, H, W), np.uint8)
    w = _rand(rng, (C, 1, k, k), np.int8, -127, 127)
    ws = rng.uniform(0.001, 0.004, C).astype(np.float32)
    wz = np.zeros(C, np.int8)
    bias = _rand(rng, C, np.int32, -500, 500)
    for zx, clamp in ((0, -1), (6, 150)):
        args = (0.02, np.uint8(zx), _t(w, dev), _t(ws, dev), _t(wz, dev), 0.03, np.uint8(0), _t(bias, dev), (stride, stride), (pad, pad), C)
        fast = ops.QLinearConv(_t(x, dev, True), *args, path=AUTO, clamp_hi_q=None if clamp < 0 else clamp)  # depthwise kernel
        slow = ops.QLinearConv(_t(x, dev, False), *args, path=SIMT, clamp_hi_q=None if clamp < 0 else clamp)  # generic kernel, NCHW
        acc = orc.conv_integer(x, w, zx, wz, (stride, stride), (pad, pad), C)
        exact = orc.requantize(acc, 0.02, ws, 0.03, 0, bias=bias, channel_axis=1, clamp_hi_q=clamp)
        assert np.array_equal(fast.cpu().numpy(), exact) and np.array_equal(slow.cpu().numpy(), exact)
        emul = orc.qlinear_conv(x, 0.02, zx, w, ws, wz, 0.03, 0, b=bias, strides=(stride, stride), pads=(pad, pad), group=C, clamp_hi_q=clamp)
        assert lsb_report(exact, emul)[0] <= 1


def test_depthwise_uint8_weights_with_zero_points(ops, orc, dev):
    """uint8 depthwise weights: (w - w_zp) fits int8 for one channel set (dot-product path) and needs nine bits for another
    (scalar path); int8 activations; folded scales; residual tail."""
    rng = np.random.default_rng(31)
    C = 64
    for x_dtype, zx, wlo, whi, zlo, zhi in ((np.uint8, 3, 100, 160, 110, 150), (np.uint8, 0, 0, 255, 0, 255), (np.int8, -5, 90, 170, 120, 140)):
        x = _rand(rng, (2, C, 11, 9), x_dtype)
        w = _rand(rng, (C, 1, 3, 3), np.uint8, wlo, whi)
        wz = _rand(rng, C, np.uint8, zlo, zhi)
        ws = rng.uniform(0.001, 0.004, C).astype(np.float32)
        r = _rand(rng, (2, C, 11, 9), np.uint8)
        for fold in (False, True):
            y = ops.QLinearConv(_t(x, dev, True), 0.02, x_dtype(zx), _t(w, dev), _t(ws, dev), _t(wz, dev), 0.03, np.uint8(20), None, (1, 1), (1, 1), C,
                                fold_scales=fold, residual=_t(r, dev, True), res_scale=0.04, res_zero_point=3, out_scale=0.05, out_zero_point=0)
            acc = orc.conv_integer(x, w, zx, wz, (1, 1), (1, 1), C)
            y1 = orc.requantize(acc, 0.02, ws, 0.03, 20, channel_axis=1, fold=fold)
            want = orc.qadd_relu(y1, 0.03, 20, r, 0.04, 3, 0.05, 0, relu=True, fold=fold)
            assert np.array_equal(y.cpu().numpy(), want)
    ops.device_status()


def test_golden_conv(ops, dev):
    g = np.load(GOLDEN)
    x, w, zw = g["cv_x"], g["cv_w"], g["cv_zw"]
    for cl in (False, True):
        y = ops.ConvInteger(_t(x, dev, cl), _t(w, dev), np.uint8(7), _t(zw, dev), (2, 1), (1, 1), 2, path=SIMT)
        assert np.array_equal(y.cpu().numpy(), g["cv_y"])
        y = ops.ConvInteger(_t(x, dev, cl), _t(w, dev), np.uint8(7), None, (2, 2), (), 2, "SAME_UPPER", path=SIMT)
        assert np.array_equal(y.cpu().numpy(), g["cv_y_same"])
        y = ops.QLinearConv(_t(x, dev, cl), 0.02, np.uint8(7), _t(w, dev), _t(g["qc_ws"], dev), _t(zw, dev), 0.04, np.uint8(9), _t(g["qc_bias"], dev),
                            (1, 1), (1, 1), 2, path=SIMT).cpu().numpy()
        assert np.array_equal(y, g["qc_y_exact"]) and np.abs(y.astype(int) - g["qc_y"].astype(int)).max() <= 1


def test_conv_full_size_layer_properties(ops, dev):
    """One ResNet-50 layer at benchmark size (256 x 64 x 56 x 56, 3x3 -> 64): linearity in the weights
    (conv(x, w1) + conv(x, w2) == conv(x, w1 + w2) on int32 accumulators) and agreement of a strided sample of output
    positions with the CUDA-core kernel run on the same data."""
    gen = torch.Generator(device=dev).manual_seed(3)
    x = torch.randint(0, 256, (256, 64, 56, 56), dtype=torch.uint8, device=dev, generator=gen).contiguous(memory_format=torch.channels_last)
    w1 = torch.randint(-60, 61, (64, 64, 3, 3), dtype=torch.int8, device=dev, generator=gen)
    w2 = torch.randint(-60, 61, (64, 64, 3, 3), dtype=torch.int8, device=dev, generator=gen)
    y1 = ops.ConvInteger(x, w1, None, None, (1, 1), (1, 1), path=TENSOR)
    y2 = ops.ConvInteger(x, w2, None, None, (1, 1), (1, 1), path=TENSOR)
    y12 = ops.ConvInteger(x, (w1 + w2), None, None, (1, 1), (1, 1), path=TENSOR)
    ops.device_status()
    assert torch.equal(y1 + y2, y12)
    xs = x[:2].contiguous(memory_format=torch.channels_last)
    ref = ops.ConvInteger(xs, w1, None, None, (1, 1), (1, 1), path=SIMT)
    assert torch.equal(y1[:2], ref)
    xs = x[254:].contiguous(memory_format=torch.channels_last)
    assert torch.equal(y1[254:], ops.ConvInteger(xs, w1, None, None, (1, 1), (1, 1), path=SIMT))


@pytest.mark.parametrize("path,cl", [(SIMT, False), (TENSOR, True)])
@pytest.mark.parametrize("N,C,H,W,M,k,stride,pad", [TC_CASES[2], TC_CASES[6], TC_CASES[8]])
def test_qlinear_conv_folded_scales(ops, orc, dev, path, cl, N, C, H, W, M, k, stride, pad):
    """fold_scales: one multiplier per channel.  Bit-exact against the oracle's restatement of that arithmetic; at most one
    step from both the reference-order kernel and the fp32-emulating chain, with the mismatch counts printed."""
    rng = np.random.default_rng(M + 3 * k)
    x = _rand(rng, (N, C, H, W), np.uint8)
    w = _rand(rng, (M, C, k, k), np.int8, -127, 127)
    ws = rng.uniform(0.0005, 0.002, M).astype(np.float32)
    wz = np.zeros(M, np.int8)
    bias = _rand(rng, M, np.int32, -3000, 3000)
    r = _rand(rng, (N, M, (H + 2 * pad - k) // stride + 1, (W + 2 * pad - k) // stride + 1), np.uint8)
    sx, sy = 0.02, 0.09
    for zy, mode in ((0, 0), (17, 1), (131, 0)):
        args = (_t(x, dev, cl), sx, np.uint8(0), _t(w, dev), _t(ws, dev), _t(wz, dev), sy, np.uint8(zy), _t(bias, dev), (stride, stride), (pad, pad))
        y = ops.QLinearConv(*args, round_mode=mode, path=path, fold_scales=True).cpu().numpy()
        y_ref_order = ops.QLinearConv(*args, round_mode=mode, path=path).cpu().numpy()
        acc = orc.conv_integer(x, w, 0, wz, (stride, stride), (pad, pad))
        want = orc.requantize(acc, sx, ws, sy, zy, bias=bias, channel_axis=1, round_mode=mode, fold=True)
        assert np.array_equal(y, want)
        emul = orc.qlinear_conv(x, sx, 0, w, ws, wz, sy, zy, b=bias, strides=(stride, stride), pads=(pad, pad), round_mode=mode)
        m1, c1, tot = lsb_report(y, y_ref_order)
        m2, c2, _ = lsb_report(y, emul)
        print("folded vs reference-order kernel: %d of %d differ; vs fp32-emulating chain: %d differ" % (c1, tot, c2))
        assert m1 <= 1 and m2 <= 1
        # folded residual tail
        yr = ops.QLinearConv(*args, round_mode=mode, path=path, fold_scales=True, residual=_t(r, dev, cl), res_scale=0.05, res_zero_point=9,
                             out_scale=0.11, out_zero_point=0).cpu().numpy()
        want_r = orc.qadd_relu(want, sy, zy, r, 0.05, 9, 0.11, 0, relu=True, round_mode=mode, fold=True)
        assert np.array_equal(yr, want_r)
        chain = orc.qadd_relu(emul, sy, zy, r, 0.05, 9, 0.11, 0, relu=True, round_mode=mode)
        assert lsb_report(yr, chain)[0] <= 2  # one step from the convolution, one from the folded tail
    ops.device_status()


@pytest.fixture
def grouped_kernel(pkg):
    """Forces the grouped-tile tensor-core kernel wherever a problem is eligible; restores the default choice afterwards."""
    assert pkg.lib().chxq_tc_variant(2) == 0
    yield
    assert pkg.lib().chxq_tc_variant(0) == 0


GROUPED_CASES = [
    (2, 64, 8, 8, 64, 1, 1, 0),      # one position tile in a group of four, 64-channel block
    (3, 128, 7, 7, 256, 1, 1, 0),    # ragged positions, two channel blocks
    (9, 64, 8, 8, 64, 3, 1, 1),      # 3x3 boxes, groups of four with a ragged last group
    (2, 48, 12, 12, 80, 3, 1, 1),    # ragged channel block (80 of 128), K tile 64 with TMA zero fill
    (2, 256, 14, 14, 128, 3, 1, 1),  # K tile 128
    (1, 64, 10, 10, 64, 5, 1, 2),    # 5x5
    (4, 64, 16, 16, 128, 1, 2, 0),   # stride 2: TMA box with element strides
    (2, 144, 6, 6, 32, 1, 1, 0),     # ragged last K chunk, 32 output channels
    (3, 64, 20, 13, 64, 3, 1, 1),    # halo tiles: ragged in both directions (13 = 8 + 5 columns, 20 = 16 + 4 rows)
    (2, 128, 16, 16, 192, 3, 1, 1),  # halo tiles, two channel chunks of 64, 128-channel blocks with a ragged last block
    (2, 64, 9, 12, 64, 2, 1, 0),     # halo tiles, 2 x 2 window without padding
    (5, 32, 20, 20, 16, 1, 1, 0),    # 16 output channels: one chunk per tile, dealt out tile by tile (folded form); ragged last group
    (3, 96, 15, 15, 32, 1, 1, 0),    # 32 output channels, K tile 128
    (2, 144, 17, 9, 32, 3, 1, 1),    # 32 output channels, 3 x 3 window
]


@pytest.mark.parametrize("N,C,H,W,M,k,stride,pad", GROUPED_CASES)
def test_grouped_tensor_core_kernel(pkg, ops, orc, dev, grouped_kernel, N, C, H, W, M, k, stride, pad):
    """The grouped-tile kernel (outputs staged in shared memory, TMA store, residual by TMA load) against the oracle and,
    bit for bit, against the one-tile-per-step kernel: reference-order and folded requantization, activation zero point,
    ReLU6 clamp, residual tails with and without Relu."""
    rng = np.random.default_rng(N * 1000 + C + M + k)
    x = _rand(rng, (N, C, H, W), np.uint8)
    w = _rand(rng, (M, C, k, k), np.int8, -127, 127)
    ws = rng.uniform(0.0005, 0.002, M).astype(np.float32)
    wz = np.zeros(M, np.int8)
    bias = _rand(rng, M, np.int32, -3000, 3000)
    Ho, Wo = (H + 2 * pad - k) // stride + 1, (W + 2 * pad - k) // stride + 1
    r = _rand(rng, (N, M, Ho, Wo), np.uint8)
    sx, sy = 0.02, 0.09
    xt, wt, wst, wzt, bt, rt = _t(x, dev, True), _t(w, dev), _t(ws, dev), _t(wz, dev), _t(bias, dev), _t(r, dev, True)

    def run(variant, zx, zy, **kw):
        assert pkg.lib().chxq_tc_variant(variant) == 0
        y = ops.QLinearConv(xt, sx, np.uint8(zx), wt, wst, wzt, sy, np.uint8(zy), bt, (stride, stride), (pad, pad), path=TENSOR, **kw)
        ops.device_status()
        return y

    cases = [
        dict(zx=0, zy=0, kw={}),
        dict(zx=5, zy=17, kw={}),
        dict(zx=0, zy=131, kw=dict(fold_scales=True)),
        dict(zx=7, zy=131, kw=dict(fold_scales=True)),  # folded epilogue with the activation zero-point term
        dict(zx=0, zy=0, kw=dict(clamp_hi_q=77)),
        dict(zx=0, zy=121, kw=dict(residual=rt, res_scale=0.05, res_zero_point=9, out_scale=0.11, out_zero_point=0)),
        dict(zx=0, zy=121, kw=dict(residual=rt, res_scale=0.05, res_zero_point=9, out_scale=0.11, out_zero_point=0, fold_scales=True)),
        dict(zx=0, zy=121, kw=dict(residual=rt, res_scale=0.05, res_zero_point=9, out_scale=0.11, out_zero_point=100, res_relu=False)),
        dict(zx=0, zy=121, kw=dict(residual=rt, res_scale=0.05, res_zero_point=9, out_scale=0.11, out_zero_point=100, res_relu=False,
                                   fold_scales=True)),
    ]
    for c in cases:
        ref = run(1, c["zx"], c["zy"], **c["kw"])
        for variant in (2, 3, 4, 7, 6):  # 3, 4: halo tiles where the geometry allows them (3x3 and smaller, stride 1): planes, swizzled; 7: CTA pairs where eligible; 6: as the default choice but never CTA pairs
            got = run(variant, c["zx"], c["zy"], **c["kw"])
            assert torch.equal(got, ref), (variant, c)
    acc = orc.conv_integer(x, w, 0, wz, (stride, stride), (pad, pad))
    want = orc.requantize(acc, sx, ws, sy, 131, bias=bias, channel_axis=1, fold=True)
    assert np.array_equal(run(2, 0, 131, fold_scales=True).cpu().numpy(), want)
    acc7 = orc.conv_integer(x, w, 7, wz, (stride, stride), (pad, pad))
    want7 = orc.requantize(acc7, sx, ws, sy, 131, bias=bias, channel_axis=1, fold=True)
    assert np.array_equal(run(2, 7, 131, fold_scales=True).cpu().numpy(), want7)
    want = orc.requantize(acc, sx, ws, sy, 121, bias=bias, channel_axis=1)
    want_r = orc.qadd_relu(want, sy, 121, r, 0.05, 9, 0.11, 100, relu=False)
    got = run(2, 0, 121, residual=rt, res_scale=0.05, res_zero_point=9, out_scale=0.11, out_zero_point=100, res_relu=False)
    assert np.array_equal(got.cpu().numpy(), want_r)


def test_grouped_kernel_networks(pkg, ops, dev, grouped_kernel):
    """ResNet-50 (reduced width) through the grouped kernel equals the same network through the one-tile kernel."""
    from chainer_compiler_b200 import models
    net = models.ResNet50Int8(batch=8, device=dev, seed=4, image=64, num_classes=32, width_mult=0.5)
    xt = torch.rand((8, 3, 64, 64), generator=torch.Generator().manual_seed(1)).to(dev)
    net.calibrate(xt)
    for fold in (False, True):
        assert pkg.lib().chxq_tc_variant(2) == 0
        t2 = {}
        l2 = net.forward(xt, fold=fold, taps=t2)
        ops.device_status()
        assert pkg.lib().chxq_tc_variant(1) == 0
        t1 = {}
        l1 = net.forward(xt, fold=fold, taps=t1)
        for k in t1:
            assert torch.equal(t1[k], t2[k]), (fold, k)
        assert torch.equal(l1, l2)


@pytest.mark.parametrize("N,C,H,W,M,group,k,stride,pad", [
    (2, 32, 14, 14, 32, 32, 3, 1, 1),     # depthwise, one ragged block of 64
    (3, 96, 15, 13, 96, 96, 3, 2, 1),     # depthwise stride 2, odd map, two blocks (64 + 32)
    (2, 144, 8, 8, 144, 144, 3, 1, 1),    # depthwise, 144 = 2 x 64 + 16
    (2, 16, 9, 9, 16, 16, 5, 1, 2),       # depthwise 5x5
    (2, 64, 8, 8, 128, 2, 3, 1, 1),       # two groups of 32 -> 64 channels
    (1, 48, 10, 10, 192, 3, 1, 1, 0),     # three groups of 16 -> 64, 1x1
])
def test_grouped_conv_tensor_core_packed(pkg, ops, orc, dev, N, C, H, W, M, group, k, stride, pad):
    """Grouped and depthwise convolutions on the tensor-core path (packed entry): a column tile reads its group's input
    channels only; depthwise weights become diagonal 64 x 64 blocks.  Accumulators and requantized outputs against the
    oracle, with and without an activation zero point where the geometry allows it."""
    import ctypes
    from chainer_compiler_b200 import _lib
    rng = np.random.default_rng(C + M + k)
    x = _rand(rng, (N, C, H, W), np.uint8)
    w = _rand(rng, (M, C // group, k, k), np.int8)
    xt = _t(x, dev, True)
    pk = ops.PackedConv(_t(w, dev), None, x.shape, (stride, stride), (pad, pad), group=group)
    assert pk.eligible and (pk.flags & 2)
    g = pk.g
    for zx in ((0,) if pad else (0, 9)):
        y = torch.empty((g.N, g.M, g.Ho, g.Wo), dtype=torch.int32, device=dev, memory_format=torch.channels_last)
        nb = pkg.lib().chxq_conv_packed_workspace(ctypes.byref(g), zx, pk.flags)
        ws = ops.workspace(nb, dev)
        _lib.check(pkg.lib().chxq_conv_integer_packed(ops._ptr(xt), ops._ptr(pk.blob), ctypes.byref(g), 1, zx, pk.flags, ops._ptr(y), ops._ptr(ws),
                                                      nb, ops._stream()))
        ops.device_status()
        assert np.array_equal(y.cpu().numpy(), orc.conv_integer(x, w, zx, None, (stride, stride), (pad, pad), group)), zx
    ws_ = rng.uniform(0.0005, 0.002, M).astype(np.float32)
    bias = _rand(rng, M, np.int32, -3000, 3000)
    wz0 = np.zeros(M, np.int8)
    acc = orc.conv_integer(x, w, 0, wz0, (stride, stride), (pad, pad), group)
    for fold in (False, True):
        for variant in (0, 1, 2, 3, 4):  # 1: 3x3 depthwise layers run on the row-dp4a CUDA-core kernel; the others keep the diagonal blocks on the tensor cores
            assert pkg.lib().chxq_tc_variant(variant) == 0
            yq = ops.QLinearConvPacked(xt, pk, 0.02, np.uint8(0), _t(ws_, dev), _t(wz0, dev), 0.05, np.uint8(20), b=_t(bias, dev), fold_scales=fold,
                                       clamp_hi_q=200)
            ops.device_status()
            want = orc.requantize(acc, 0.02, ws_, 0.05, 20, bias=bias, channel_axis=1, fold=fold, clamp_hi_q=200)
            assert np.array_equal(yq.cpu().numpy(), want), (fold, variant)
    assert pkg.lib().chxq_tc_variant(0) == 0


def test_quantize_fused_into_stem_conv(pkg, ops, orc, dev):
    """QuantizeLinear fused into the stem convolution's repack pass equals the two ops in sequence, in both rounding modes and
    with a zero point; geometries that are not on the space-to-depth path are refused."""
    from chainer_compiler_b200 import _lib
    rng = np.random.default_rng(21)
    xf = rng.uniform(-0.2, 1.2, (3, 3, 30, 26)).astype(np.float32)
    xf[0, 0, 0, :4] = [0.5 / 255, 1.5 / 255, 2.5 / 255, -1.0]  # exact ties and a negative
    w = _rand(rng, (32, 3, 7, 7), np.int8)
    ws = rng.uniform(0.0005, 0.002, 32).astype(np.float32)
    wz = np.zeros(32, np.int8)
    bias = _rand(rng, 32, np.int32, -3000, 3000)
    pk = ops.PackedConv(_t(w, dev), _t(wz, dev), xf.shape, (2, 2), (3, 3), x_layout=_lib.NCHW)
    xt = _t(xf, dev)
    for zx, qmode in ((0, 0), (9, 0), (0, 1), (9, 1)):
        xq = ops.QuantizeLinear(xt, 1 / 255.0, np.uint8(zx), round_mode=qmode)
        assert np.array_equal(xq.cpu().numpy(), orc.quantize_linear(xf, 1 / 255.0, zx, round_mode=qmode))
        two = ops.QLinearConvPacked(xq, pk, 1 / 255.0, np.uint8(zx), _t(ws, dev), _t(wz, dev), 0.05, np.uint8(3), b=_t(bias, dev), fold_scales=True)
        one = ops.QuantizeLinearConvPacked(xt, pk, 1 / 255.0, np.uint8(zx), _t(ws, dev), _t(wz, dev), 0.05, np.uint8(3), b=_t(bias, dev), fold_scales=True,
                                           quant_round_mode=qmode)
        ops.device_status()
        assert torch.equal(one, two), (zx, qmode)
    w1 = _rand(rng, (32, 16, 1, 1), np.int8)
    pk1 = ops.PackedConv(_t(w1, dev), _t(wz, dev), (2, 16, 8, 8))
    with pytest.raises(_lib.ChxqError):
        ops.QuantizeLinearConvPacked(torch.zeros((2, 16, 8, 8), device=dev).contiguous(memory_format=torch.channels_last), pk1, 0.1, np.uint8(0),
                                     _t(ws, dev), _t(wz, dev), 0.05, np.uint8(3))


@pytest.mark.parametrize("case", ["stem64", "stem_odd", "stem224", "c64_1x1", "c64_3x3_m128", "c64_m32"])
def test_conv_with_fused_max_pooling(pkg, ops, orc, dev, case):
    """QLinearConv + MaxPool(3, 2, 0) as one kernel (pooling on the staged output tiles, overlapping tile groups) against the
    two ops run one after the other, and against the oracle's convolution and pooling."""
    from chainer_compiler_b200 import _lib
    rng = np.random.default_rng(sum(map(ord, case)))
    if case.startswith("stem"):
        N, H, W = {"stem64": (2, 64, 64), "stem_odd": (3, 62, 90), "stem224": (8, 224, 224)}[case]
        M = 64
        xf = rng.uniform(-0.1, 1.1, (N, 3, H, W)).astype(np.float32)
        w = _rand(rng, (M, 3, 7, 7), np.int8)
        geom = dict(strides=(2, 2), pads=(3, 3), x_layout=_lib.NCHW)
        xt, x_scale = _t(xf, dev), 1 / 255.0
        xq_np = orc.quantize_linear(xf, x_scale, 0)
    else:
        N, C, H, W, M, k = {"c64_1x1": (2, 64, 20, 36, 64, 1), "c64_3x3_m128": (2, 64, 21, 19, 128, 3), "c64_m32": (1, 64, 9, 40, 32, 1)}[case]
        xq_np = _rand(rng, (N, C, H, W), np.uint8)
        w = _rand(rng, (M, C, k, k), np.int8)
        geom = dict(strides=(1, 1), pads=(k // 2, k // 2))
        xt, x_scale = _t(xq_np, dev, True), 0.02
    ws = rng.uniform(0.0005, 0.002, M).astype(np.float32) / (1 if case.startswith("stem") else 8)
    wz = np.zeros(M, np.int8)
    bias = _rand(rng, M, np.int32, -3000, 3000)
    pk = ops.PackedConv(_t(w, dev), _t(wz, dev), xt.shape, **geom)
    assert pk.eligible
    args = (pk, x_scale, np.uint8(0), _t(ws, dev), _t(wz, dev), 0.05, np.uint8(2))
    for fold in (False, True):
        for cover_all in (True, False):
            if xt.dtype == torch.float32:
                conv = ops.QuantizeLinearConvPacked(xt, *args, b=_t(bias, dev), fold_scales=fold)
            else:
                conv = ops.QLinearConvPacked(xt, *args, b=_t(bias, dev), fold_scales=fold)
            two = ops.MaxPoolU8(conv, 3, 2, 0, cover_all=cover_all)
            one = ops.QLinearConvMaxPoolPacked(xt, *args, b=_t(bias, dev), cover_all=cover_all, fold_scales=fold)
            ops.device_status()
            assert one.shape == two.shape and torch.equal(one, two), (case, fold, cover_all)
            assert int(one.max()) > 2
    if case != "stem224":
        acc = orc.conv_integer(xq_np, w, 0, wz.astype(np.int32), strides=geom["strides"], pads=geom["pads"])
        want = orc.maxpool_u8(orc.requantize(acc, x_scale, ws, 0.05, 2, bias=bias, channel_axis=1), 3, 2, 0, cover_all=True)
        got = ops.QLinearConvMaxPoolPacked(xt, *args, b=_t(bias, dev), cover_all=True)
        assert np.array_equal(got.cpu().numpy(), want)
    # refused: other pooling windows; convolutions whose K tile is 128 bytes
    with pytest.raises(_lib.ChxqError):
        ops.QLinearConvMaxPoolPacked(xt, *args, b=_t(bias, dev), pool_kernel=2)
    w128 = _rand(rng, (64, 128, 1, 1), np.int8)
    x128 = _t(_rand(rng, (1, 128, 16, 16), np.uint8), dev, True)
    wz64, ws64 = np.zeros(64, np.int8), np.full(64, 1e-4, np.float32)
    pk128 = ops.PackedConv(_t(w128, dev), _t(wz64, dev), x128.shape)
    with pytest.raises(_lib.ChxqError):
        ops.QLinearConvMaxPoolPacked(x128, pk128, 0.02, np.uint8(0), _t(ws64, dev), _t(wz64, dev), 0.05, np.uint8(2))


@pytest.mark.parametrize("N,C,H,W,stride,pad,wdtype", [
    (2, 20, 13, 11, 1, 1, np.int8),      # 20 channels: five words per position; odd, non-square map
    (3, 96, 17, 15, 2, 1, np.int8),      # stride 2, odd map
    (1, 36, 30, 30, 1, 1, np.int8),      # more than one strip of rows
    (2, 144, 56, 56, 2, 1, np.int8),     # a MobileNetV2 shape
    (2, 32, 9, 9, 1, 0, np.int8),        # no padding
    (2, 16, 8, 12, 1, 1, np.uint8),      # uint8 weights with zero point 0
    (520, 960, 7, 7, 1, 1, np.int8),     # staged kernel: a CTA walks two images; seven channel blocks, the last one partly beyond the map
    (260, 576, 14, 14, 2, 1, np.int8),   # staged kernel, stride 2, several images per CTA
    (3, 144, 56, 56, 1, 1, np.int8),     # staged kernel: ten stages per image, column tiles with halo columns from their neighbours
    (2, 32, 112, 112, 1, 1, np.int8),    # staged kernel: 32-byte channel blocks, nineteen stages (the ring wraps four times)
    (2, 48, 11, 70, 2, 0, np.uint8),     # staged kernel: wide map, ragged last column tile, no padding, uint8 weights
])
def test_depthwise3x3_row_kernel_through_the_op_signature(ops, orc, dev, N, C, H, W, stride, pad, wdtype):
    """3x3 depthwise QLinearConv with symmetric weights over a zero-point-0 map (the row-dp4a kernels: rows staged by TMA where the
    channel count is a multiple of 16, plain loads elsewhere), called through the op's own signature on NHWC maps: bit-exact against
    the integer-domain oracle in both requantization forms, with a ReLU6-style clamp."""
    rng = np.random.default_rng(C * 3 + H)
    x = _rand(rng, (N, C, H, W), np.uint8)
    w = _rand(rng, (C, 1, 3, 3), wdtype) if wdtype == np.int8 else rng.integers(0, 256, (C, 1, 3, 3)).astype(np.uint8)
    ws_ = rng.uniform(0.0005, 0.002, C).astype(np.float32)
    bias = _rand(rng, C, np.int32, -3000, 3000)
    wz = np.zeros(C, wdtype)
    acc = orc.conv_integer(x, w, 0, wz, (stride, stride), (pad, pad), C)
    for fold in (False, True):
        want = orc.requantize(acc, 0.02, ws_, 0.05, 7, bias=bias, channel_axis=1, fold=fold, clamp_hi_q=180)
        y = ops.QLinearConv(_t(x, dev, True), 0.02, np.uint8(0), _t(w, dev), _t(ws_, dev), _t(wz, dev), 0.05, np.uint8(7), _t(bias, dev), (stride, stride),
                            (pad, pad), C, fold_scales=fold, clamp_hi_q=180)
        ops.device_status()
        assert np.array_equal(y.cpu().numpy(), want), (fold, int((y.cpu().numpy() != want).sum()))
