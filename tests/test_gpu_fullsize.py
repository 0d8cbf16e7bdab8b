"""Parity at the benchmark configurations' own layer shapes (full channel width, 224-derived maps), not shrunken networks.

Every case compares the CUDA path with the oracle on seeded inputs: the exact int32 accumulator path bit for bit (the
integer-domain oracle), and the reference's arithmetic (runtime/ops/quantize.cc:62-94: dequantize, fp32 convolution, quantize)
within one output step, mismatch counts printed.  Batches are small so that the CPU oracle finishes in seconds; the kernels,
tile shapes and K loops are those of the full batch (a position tile never depends on the batch size beyond its count).
"""
import numpy as np
import pytest
import torch

from helpers import lsb_report

pytestmark = pytest.mark.gpu


def _t(a, dev, cl=False):
    t = torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    return t.contiguous(memory_format=torch.channels_last) if cl else t


def _layer(rng, cin, cout, k):
    w = rng.integers(-127, 128, (cout, cin, k, k)).astype(np.int8)
    ws = rng.uniform(0.5, 1.5, cout).astype(np.float32) * np.float32(2.0 / (127.0 * np.sqrt(cin * k * k)))
    bias = rng.integers(-2000, 2000, cout).astype(np.int32)
    return w, ws, bias


# (name, N, cin, cout, H, k, stride, pad, residual): one layer of every ResNet-50 stage family at full width
RESNET_LAYERS = [
    ("res2_conv2", 4, 64, 64, 56, 3, 1, 1, False),
    ("res2_conv3+join", 4, 64, 256, 56, 1, 1, 0, True),
    ("res3_conv1_s2", 4, 256, 128, 56, 1, 2, 0, False),
    ("res4_conv2", 8, 256, 256, 14, 3, 1, 1, False),
    ("res4_conv3+join", 8, 256, 1024, 14, 1, 1, 0, True),
    ("res5_conv2", 8, 512, 512, 7, 3, 1, 1, False),
    ("res5_conv3+join", 8, 512, 2048, 7, 1, 1, 0, True),
    ("res5_proj_s2", 8, 1024, 2048, 14, 1, 2, 0, False),
]


@pytest.mark.parametrize("name,N,cin,cout,H,k,stride,pad,res", RESNET_LAYERS, ids=[c[0] for c in RESNET_LAYERS])
@pytest.mark.parametrize("fold", [False, True], ids=["reforder", "folded"])
def test_resnet50_layer_full_width(ops, orc, dev, name, N, cin, cout, H, k, stride, pad, res, fold):
    rng = np.random.default_rng(cin * 7 + cout)
    x = rng.integers(0, 256, (N, cin, H, H), dtype=np.uint8)
    w, ws, bias = _layer(rng, cin, cout, k)
    wz = np.zeros(cout, np.int8)
    sx, sy, zy = np.float32(0.02), np.float32(0.05), (117 if res else 0)
    pk = ops.PackedConv(_t(w, dev), _t(wz, dev), x.shape, strides=(stride, stride), pads=(pad, pad))
    assert pk.eligible
    Ho = (H + 2 * pad - k) // stride + 1
    kw = {}
    r = None
    if res:
        r = rng.integers(0, 256, (N, cout, Ho, Ho), dtype=np.uint8)
        kw = dict(residual=_t(r, dev, True), res_scale=0.04, res_zero_point=0, res_relu=True, out_scale=0.06, out_zero_point=0)
    y = ops.QLinearConvPacked(_t(x, dev, True), pk, sx, np.uint8(0), _t(ws, dev), _t(wz, dev), sy, np.uint8(zy), b=_t(bias, dev),
                              fold_scales=fold, **kw).cpu().numpy()
    ops.device_status()
    # bit-exact against the integer-domain oracle (the kernels' own arithmetic restated on the CPU)
    acc = orc.conv_integer(x, w, 0, None, strides=(stride, stride), pads=(pad, pad))
    want = orc.requantize(acc, sx, ws, sy, zy, bias=bias, channel_axis=1, fold=fold)
    if res:
        want = orc.qadd_relu(want, sy, zy, r, 0.04, 0, 0.06, 0, relu=True, fold=fold)
    assert np.array_equal(y, want), "%s: %d of %d bytes differ from the integer-domain oracle" % (name, int((y != want).sum()), y.size)
    # the reference's arithmetic on the same input bytes: at most one output step per operator
    conv_ref = orc.qlinear_conv(x, sx, 0, w, ws, wz.astype(np.int32), sy, zy, b=bias, strides=(stride, stride), pads=(pad, pad))
    if res:
        y_conv = ops.QLinearConvPacked(_t(x, dev, True), pk, sx, np.uint8(0), _t(ws, dev), _t(wz, dev), sy, np.uint8(zy), b=_t(bias, dev),
                                       fold_scales=fold).cpu().numpy()
        mx, cnt, tot = lsb_report(y_conv, conv_ref)
        join_ref = orc.qadd_relu(y_conv, sy, zy, r, 0.04, 0, 0.06, 0, relu=True)  # reference-order join fed the kernel's own conv bytes
        mx2, cnt2, tot2 = lsb_report(y, join_ref)
        print("%s (%s): conv %d of %d bytes one step from the reference chain; join %d of %d" % (name, "folded" if fold else "reference order",
                                                                                                  cnt, tot, cnt2, tot2))
        assert mx <= 1 and mx2 <= 1
    else:
        mx, cnt, tot = lsb_report(y, conv_ref)
        print("%s (%s): %d of %d bytes one step from the reference chain" % (name, "folded" if fold else "reference order", cnt, tot))
        assert mx <= 1


def test_resnet50_stem_224_with_pool(ops, orc, dev):
    """The 7x7 / 2 stem on 224 x 224 images with its QuantizeLinear in front and the 3x3 / 2 max pooling behind, as one
    call, against the oracle's three ops."""
    rng = np.random.default_rng(3)
    N = 2
    xf = rng.uniform(0, 1, (N, 3, 224, 224)).astype(np.float32)
    w, ws, bias = _layer(rng, 3, 64, 7)
    wz = np.zeros(64, np.int8)
    sx, sy = np.float32(1.0 / 255.0), np.float32(0.03)
    pk = ops.PackedConv(_t(w, dev), _t(wz, dev), xf.shape, strides=(2, 2), pads=(3, 3), x_layout=ops.NCHW)
    assert pk.eligible
    xq = orc.quantize_linear(xf, sx, 0)
    acc = orc.conv_integer(xq, w, 0, None, strides=(2, 2), pads=(3, 3))
    conv_ref = orc.qlinear_conv(xq, sx, 0, w, ws, wz.astype(np.int32), sy, 0, b=bias, strides=(2, 2), pads=(3, 3))
    for fold in (False, True):
        want = orc.requantize(acc, sx, ws, sy, 0, bias=bias, channel_axis=1, fold=fold)
        y = ops.QuantizeLinearConvPacked(_t(xf, dev), pk, sx, np.uint8(0), _t(ws, dev), _t(wz, dev), sy, np.uint8(0), b=_t(bias, dev), fold_scales=fold)
        assert np.array_equal(y.cpu().numpy(), want), fold
        mx, cnt, tot = lsb_report(want, conv_ref)
        print("stem 224 (%s): %d of %d bytes one step from the reference chain" % ("folded" if fold else "reference order", cnt, tot))
        assert mx <= 1
        pooled = ops.QLinearConvMaxPoolPacked(_t(xf, dev), pk, sx, np.uint8(0), _t(ws, dev), _t(wz, dev), sy, np.uint8(0), b=_t(bias, dev), cover_all=True,
                                              fold_scales=fold)
        assert np.array_equal(pooled.cpu().numpy(), orc.maxpool_u8(want, 3, 2, 0, cover_all=True)), fold
    ops.device_status()


@pytest.mark.parametrize("S", [8192])
def test_matmul_integer_large_sampled(ops, dev, S):
    """MatMulInteger at the sweep's large sizes: exact dot products on sampled rows and columns (int64 on the host), plus the
    checksum identity sum_n Y[m, n] = (A[m, :] - za) . sum_n B[:, n] on every row."""
    gen = torch.Generator(device=dev).manual_seed(S)
    a = torch.randint(0, 256, (S, S), dtype=torch.uint8, device=dev, generator=gen)
    b = torch.randint(-127, 128, (S, S), dtype=torch.int8, device=dev, generator=gen)
    za = torch.tensor([128], dtype=torch.uint8, device=dev)
    y = ops.MatMulInteger(a, b, za, None, path=ops.PATH_TENSOR)
    ops.device_status()
    rng = np.random.default_rng(0)
    rows = np.unique(np.concatenate([rng.integers(0, S, 24), [0, 127, 128, S - 1]]))
    cols = np.unique(np.concatenate([rng.integers(0, S, 24), [0, 63, 64, S - 1]]))
    A = a[torch.from_numpy(rows).to(dev)].cpu().numpy().astype(np.int64) - 128
    B = b[:, torch.from_numpy(cols).to(dev)].cpu().numpy().astype(np.int64)
    got = y[torch.from_numpy(rows).to(dev)][:, torch.from_numpy(cols).to(dev)].cpu().numpy().astype(np.int64)
    assert np.array_equal(got, A @ B)
    # checksum of every row; fp64 holds these integers exactly (every partial sum is below 2^53)
    bsum = b.to(torch.float64).sum(dim=1)                     # [K]
    want_rows = (a.to(torch.float64) - 128.0) @ bsum          # [M]
    assert torch.equal(y.to(torch.float64).sum(dim=1), want_rows)


def test_mobilenetv2_block_224_shapes(ops, orc, dev):
    """One inverted-residual block at MobileNetV2's 56 x 56 stage (24 -> 144 -> depthwise 3x3 -> 24, stored as 32 channels):
    expansion with ReLU6 clamp, depthwise on the tensor-core path, linear projection with the residual join."""
    rng = np.random.default_rng(11)
    N, H = 2, 56
    x = rng.integers(0, 256, (N, 32, H, H), dtype=np.uint8)
    x[:, 24:] = 0
    sx = np.float32(0.03)
    # expansion 1x1 (ReLU6 as the upper clamp)
    w1, ws1, b1 = _layer(rng, 32, 144, 1)
    w1[:, 24:] = 0
    wz1 = np.zeros(144, np.int8)
    s1, clamp1 = np.float32(6.0 / 240.0), 240
    # depthwise 3x3
    w2 = rng.integers(-127, 128, (144, 1, 3, 3)).astype(np.int8)
    ws2 = rng.uniform(0.5, 1.5, 144).astype(np.float32) * np.float32(0.004)
    b2 = rng.integers(-500, 500, 144).astype(np.int32)
    wz2 = np.zeros(144, np.int8)
    s2, clamp2 = np.float32(6.0 / 250.0), 250
    # projection 1x1 (linear, asymmetric) + residual join without Relu
    w3, ws3, b3 = _layer(rng, 144, 32, 1)
    wz3 = np.zeros(32, np.int8)
    s3, z3, so, zo = np.float32(0.05), 120, np.float32(0.07), 110
    for fold in (False, True):
        pk1 = ops.PackedConv(_t(w1, dev), _t(wz1, dev), x.shape)
        h1 = ops.QLinearConvPacked(_t(x, dev, True), pk1, sx, np.uint8(0), _t(ws1, dev), _t(wz1, dev), s1, np.uint8(0), b=_t(b1, dev), clamp_hi_q=clamp1,
                                   fold_scales=fold)
        a1 = orc.conv_integer(x, w1, 0, None)
        want1 = orc.requantize(a1, sx, ws1, s1, 0, bias=b1, channel_axis=1, clamp_hi_q=clamp1, fold=fold)
        assert np.array_equal(h1.cpu().numpy(), want1), ("expand", fold)
        pk2 = ops.PackedConv(_t(w2, dev), _t(wz2, dev), want1.shape, strides=(1, 1), pads=(1, 1), group=144)
        assert pk2.eligible
        h2 = ops.QLinearConvPacked(h1, pk2, s1, np.uint8(0), _t(ws2, dev), _t(wz2, dev), s2, np.uint8(0), b=_t(b2, dev), clamp_hi_q=clamp2, fold_scales=fold)
        a2 = orc.conv_integer(want1, w2, 0, None, strides=(1, 1), pads=(1, 1), group=144)
        want2 = orc.requantize(a2, s1, ws2, s2, 0, bias=b2, channel_axis=1, clamp_hi_q=clamp2, fold=fold)
        assert np.array_equal(h2.cpu().numpy(), want2), ("depthwise", fold)
        ref2 = orc.qlinear_conv(want1, s1, 0, w2, ws2, wz2.astype(np.int32), s2, 0, b=b2, strides=(1, 1), pads=(1, 1), group=144, clamp_hi_q=clamp2)
        assert lsb_report(want2, ref2)[0] <= 1
        pk3 = ops.PackedConv(_t(w3, dev), _t(wz3, dev), want2.shape)
        h3 = ops.QLinearConvPacked(h2, pk3, s2, np.uint8(0), _t(ws3, dev), _t(wz3, dev), s3, np.uint8(z3), b=_t(b3, dev), fold_scales=fold,
                                   residual=_t(x, dev, True), res_scale=float(sx), res_zero_point=0, res_relu=False, out_scale=float(so), out_zero_point=zo)
        a3 = orc.conv_integer(want2, w3, 0, None)
        want3 = orc.requantize(a3, s2, ws3, s3, z3, bias=b3, channel_axis=1, fold=fold)
        want3 = orc.qadd_relu(want3, s3, z3, x, sx, 0, so, zo, relu=False, fold=fold)
        assert np.array_equal(h3.cpu().numpy(), want3), ("project+join", fold)
    ops.device_status()


def test_workspace_growth_keeps_captured_graphs_valid(ops, dev):
    """A graph captured around an op that uses scratch keeps working after a later, larger op made the scratch buffer grow:
    the superseded buffer stays owned by the op layer instead of going back to the allocator."""
    gen = torch.Generator(device=dev).manual_seed(1)
    a = torch.randint(0, 256, (256, 512), dtype=torch.uint8, device=dev, generator=gen)
    b = torch.randint(-127, 128, (512, 384), dtype=torch.int8, device=dev, generator=gen)
    za = torch.tensor([7], dtype=torch.uint8, device=dev)
    want = ops.MatMulInteger(a, b, za, None, path=ops.PATH_TENSOR).clone()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        y = ops.MatMulInteger(a, b, za, None, path=ops.PATH_TENSOR)
    # a much larger problem: the scratch buffer grows
    a2 = torch.randint(0, 256, (512, 4096), dtype=torch.uint8, device=dev, generator=gen)
    b2 = torch.randint(-127, 128, (4096, 4096), dtype=torch.int8, device=dev, generator=gen)
    big = ops.MatMulInteger(a2, b2, None, None, path=ops.PATH_TENSOR)
    junk = [torch.full((1 << 20,), 0x5A, dtype=torch.uint8, device=dev) for _ in range(8)]  # would land in a freed block
    y.zero_()
    g.replay()
    torch.cuda.synchronize()
    assert torch.equal(y, want)
    del big, junk
    ops.device_status()


def test_packed_conv_rejects_bad_residual(ops, dev):
    """Host-side rejection only: a residual of the wrong shape, dtype or layout never reaches a kernel."""
    w = torch.zeros((64, 64, 1, 1), dtype=torch.int8, device=dev)
    wz = torch.zeros(64, dtype=torch.int8, device=dev)
    ws = torch.ones(64, device=dev)
    x = torch.zeros((2, 64, 8, 8), dtype=torch.uint8, device=dev).contiguous(memory_format=torch.channels_last)
    pk = ops.PackedConv(w, wz, x.shape)
    good = torch.zeros((2, 64, 8, 8), dtype=torch.uint8, device=dev).contiguous(memory_format=torch.channels_last)
    ops.QLinearConvPacked(x, pk, 0.1, np.uint8(0), ws, wz, 0.1, np.uint8(0), residual=good, res_scale=0.1, out_scale=0.1)
    for bad in (torch.zeros((2, 64, 8, 8), dtype=torch.uint8, device=dev),                   # NCHW-contiguous
                good[:1],                                                                    # fewer images
                good.to(torch.int8),                                                         # wrong dtype
                torch.zeros((2, 32, 8, 8), dtype=torch.uint8, device=dev).contiguous(memory_format=torch.channels_last)):
        with pytest.raises(ops.ChxqError) as e:
            ops.QLinearConvPacked(x, pk, 0.1, np.uint8(0), ws, wz, 0.1, np.uint8(0), residual=bad, res_scale=0.1, out_scale=0.1)
        assert e.value.code == 1  # CHXQ_ERR_INVALID_ARGUMENT
    ops.device_status()


# (N, cin, cout, H, k, stride, pad, residual, x_zp): dense layers the CTA-pair kernel (tcgen05.mma.cta_group::2) takes
PAIR_CASES = [
    (8, 256, 256, 14, 3, 1, 1, False, 0),     # res4 conv2: 13 position tiles (odd: the last pair has one real tile)
    (8, 256, 1024, 14, 1, 1, 0, True, 0),     # res4 conv3 + join: four 256-channel blocks
    (8, 1024, 512, 14, 1, 2, 0, False, 0),    # res5 conv1: stride 2, K = 8 x 128
    (8, 512, 512, 7, 3, 1, 1, False, 5),      # res5 conv2 on 7 x 7 maps (tiles of 128 images) with an activation zero point... no padding value issue: see below
    (3, 128, 320, 28, 1, 1, 0, True, 0),      # ragged channel block (256 + 64), K = one 128-byte tile
    (2, 384, 256, 10, 1, 1, 0, False, 9),     # 200 positions: ragged position tile; activation zero point term
]


@pytest.mark.parametrize("N,cin,cout,H,k,stride,pad,res,zx", PAIR_CASES)
def test_cta_pair_kernel(pkg, ops, orc, dev, N, cin, cout, H, k, stride, pad, res, zx):
    """The CTA-pair kernel, forced on (it is chosen by itself only for problems that fill the GPU), against the integer-domain
    oracle bit for bit and against the grouped-tile kernel."""
    from chainer_compiler_b200 import _lib
    if pad and zx:
        zx = 0  # padding with a non-zero activation zero point takes the explicit im2col path, not this kernel
    rng = np.random.default_rng(cin + cout + H)
    x = rng.integers(0, 256, (N, cin, H, H), dtype=np.uint8)
    w, ws, bias = _layer(rng, cin, cout, k)
    wz = np.zeros(cout, np.int8)
    sx, sy, zy = np.float32(0.02), np.float32(0.05), (117 if res else 3)
    pk = ops.PackedConv(_t(w, dev), _t(wz, dev), x.shape, strides=(stride, stride), pads=(pad, pad))
    Ho = (H + 2 * pad - k) // stride + 1
    kw = {}
    r = None
    if res:
        r = rng.integers(0, 256, (N, cout, Ho, Ho), dtype=np.uint8)
        kw = dict(residual=_t(r, dev, True), res_scale=0.04, res_zero_point=7, res_relu=True, out_scale=0.06, out_zero_point=0)
    acc = orc.conv_integer(x, w, zx, None, strides=(stride, stride), pads=(pad, pad))
    L = pkg.lib()
    try:
        for fold in (False, True):
            want = orc.requantize(acc, sx, ws, sy, zy, bias=bias, channel_axis=1, fold=fold)
            if res:
                want = orc.qadd_relu(want, sy, zy, r, 0.04, 7, 0.06, 0, relu=True, fold=fold)
            got = {}
            for variant in (7, 6):
                _lib.check(L.chxq_tc_variant(variant))
                got[variant] = ops.QLinearConvPacked(_t(x, dev, True), pk, sx, np.uint8(zx), _t(ws, dev), _t(wz, dev), sy, np.uint8(zy), b=_t(bias, dev),
                                                     fold_scales=fold, **kw).cpu().numpy()
                ops.device_status()
            assert np.array_equal(got[7], want), "CTA-pair kernel: %d of %d bytes differ from the oracle (fold=%s)" % (
                int((got[7] != want).sum()), want.size, fold)
            assert np.array_equal(got[6], want)
    finally:
        _lib.check(L.chxq_tc_variant(0))


@pytest.mark.parametrize("M,N,K,a_dt,b_dt,za_mode,zb_mode", [
    (300, 512, 384, np.uint8, np.int8, "scalar", None),     # ragged rows (3 position tiles: the last pair has one real tile)
    (256, 320, 128, np.uint8, np.int8, "vec", "vec"),       # ragged 256-column block, vector zero points on both sides, one K tile
    (1024, 256, 1024, np.int8, np.uint8, None, "scalar"),   # signed left operand, unsigned right operand with a zero point
    (130, 1000, 256, np.uint8, np.uint8, "vec", None),      # N not a multiple of 16: scalar stores
])
def test_matmul_integer_on_cta_pairs(pkg, ops, orc, dev, M, N, K, a_dt, b_dt, za_mode, zb_mode):
    """MatMulInteger on the CTA-pair kernel (int32 accumulators stored from registers), forced on, bit-exact against the oracle
    and equal to the one-tile kernel."""
    from chainer_compiler_b200 import _lib
    rng = np.random.default_rng(M + N + K)
    ia, ib = np.iinfo(a_dt), np.iinfo(b_dt)
    a = rng.integers(ia.min, ia.max + 1, (M, K)).astype(a_dt)
    b = rng.integers(ib.min, ib.max + 1, (K, N)).astype(b_dt)
    za = None if za_mode is None else (rng.integers(ia.min, ia.max + 1, K).astype(a_dt) if za_mode == "vec" else np.array([ia.min + 128], a_dt))
    zb = None if zb_mode is None else (rng.integers(ib.min, ib.max + 1, N).astype(b_dt) if zb_mode == "vec" else np.array([ib.min + 100], b_dt))
    want = orc.matmul_integer(a, b, za, zb)
    L = pkg.lib()
    tt = lambda v: None if v is None else torch.from_numpy(v).to(dev)  # noqa: E731
    try:
        for variant in (7, 6):
            _lib.check(L.chxq_tc_variant(variant))
            y = ops.MatMulInteger(tt(a), tt(b), tt(za), tt(zb), path=ops.PATH_TENSOR)
            ops.device_status()
            assert np.array_equal(y.cpu().numpy(), want), variant
    finally:
        _lib.check(L.chxq_tc_variant(0))


def test_conv_integer_on_cta_pairs(pkg, ops, orc, dev):
    """ConvInteger with packed weights on the CTA-pair kernel: 3 x 3 with padding and an activation zero point of zero, and a
    1 x 1 with an activation zero point (the column-correction term)."""
    from chainer_compiler_b200 import _lib
    rng = np.random.default_rng(8)
    L = pkg.lib()
    try:
        _lib.check(L.chxq_tc_variant(7))
        for (N, C, H, M, k, pad, zx) in ((4, 128, 14, 256, 3, 1, 0), (3, 256, 10, 512, 1, 0, 131)):
            x = rng.integers(0, 256, (N, C, H, H), dtype=np.uint8)
            w = rng.integers(-127, 128, (M, C, k, k)).astype(np.int8)
            pk = ops.PackedConv(_t(w, dev), None, x.shape, strides=(1, 1), pads=(pad, pad))
            y = ops.ConvIntegerPacked(_t(x, dev, True), pk, np.uint8(zx))
            ops.device_status()
            assert np.array_equal(y.cpu().numpy(), orc.conv_integer(x, w, zx, None, (1, 1), (pad, pad)))
    finally:
        _lib.check(L.chxq_tc_variant(0))
