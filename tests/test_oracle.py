"""The CPU oracle against (a) known answers read off the reference's source, (b) independent int64 / fp32 numpy
formulations, (c) the committed golden vectors.  No GPU involved."""
import os

import numpy as np
import pytest

from helpers import np_conv_integer, np_matmul_integer, np_quantize_ref, np_quantize_rne

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "hotpath_vectors.npz")


def test_quantize_known_answers(orc):
    # runtime/ops/quantize.cc:29-34: (x / s + zp) clamped, + 0.5f, truncated.
    s = np.float32(1.0)
    x = np.array([0.4, 0.5, 1.5, 2.5, 254.6, 300.0, -7.0, 0.49999997], np.float32)
    assert orc.quantize_linear(x, s, 0).tolist() == [0, 1, 2, 3, 255, 255, 0, 1]  # ties go up; 0.49999997 + 0.5 rounds to 1.0 in fp32
    assert orc.quantize_linear(x, s, 0, round_mode=orc.ROUND_RNE).tolist() == [0, 0, 2, 2, 255, 255, 0, 0]  # half-to-even
    # int8 output: truncation toward zero after +0.5 mis-rounds negatives (-3.2 -> -2.7 -> -2), as the reference does.
    xi = np.array([-3.2, -3.7, -128.4, 126.5, 3.2], np.float32)
    assert orc.quantize_linear(xi, s, 0, np.int8).tolist() == [-2, -3, -127, 127, 3]
    assert orc.quantize_linear(xi, s, 0, np.int8, orc.ROUND_RNE).tolist() == [-3, -4, -128, 126, 3]
    # zero point is added before the clamp
    assert orc.quantize_linear(np.array([-5.0, 0.0, 5.0], np.float32), s, 3).tolist() == [0, 3, 8]
    assert orc.quantize_mode_diff(x, s, 0) == 3


def test_dequantize_known_answers(orc):
    q = np.array([0, 3, 255], np.uint8)
    assert np.array_equal(orc.dequantize_linear(q, 0.5, 3), np.array([-1.5, 0.0, 126.0], np.float32))
    assert np.array_equal(orc.dequantize_linear(np.array([-128, 127], np.int8), 2.0, 0), np.array([-256.0, 254.0], np.float32))


@pytest.mark.parametrize("signed,zp", [(False, 0), (False, 131), (True, 0), (True, -17)])
def test_quantize_vs_numpy(orc, signed, zp):
    rng = np.random.default_rng(1)
    x = np.concatenate([rng.uniform(-4, 4, 4000), (np.arange(-300, 300) + 0.5) * 0.013]).astype(np.float32)
    dt = np.int8 if signed else np.uint8
    assert np.array_equal(orc.quantize_linear(x, 0.013, zp, dt), np_quantize_ref(x, 0.013, zp, signed))
    assert np.array_equal(orc.quantize_linear(x, 0.013, zp, dt, orc.ROUND_RNE), np_quantize_rne(x, 0.013, zp, signed))


@pytest.mark.parametrize("za,zb", [(None, None), ([128], None), ([7], [3]), ("vec", "vec")])
def test_matmul_integer_vs_int64(orc, za, zb):
    rng = np.random.default_rng(2)
    a = rng.integers(0, 256, (19, 33), dtype=np.uint8)
    b = rng.integers(-128, 128, (33, 21)).astype(np.int8)
    if za == "vec":
        za = rng.integers(0, 256, 33, dtype=np.uint8)
    if zb == "vec":
        zb = rng.integers(-128, 128, 21).astype(np.int8)
    assert np.array_equal(orc.matmul_integer(a, b, za, zb), np_matmul_integer(a, b, za, zb))


def test_matmul_integer_batched_and_wraparound(orc):
    rng = np.random.default_rng(3)
    a = rng.integers(0, 256, (2, 3, 5, 8), dtype=np.uint8)
    b = rng.integers(0, 256, (2, 3, 8, 4), dtype=np.uint8)
    assert np.array_equal(orc.matmul_integer(a, b), np_matmul_integer(a, b))
    # int32 wrap-around: 255*255*K exceeds 2^31 for K = 40000
    a = np.full((1, 40000), 255, np.uint8)
    b = np.full((40000, 1), 255, np.uint8)
    assert orc.matmul_integer(a, b)[0, 0] == np_matmul_integer(a, b)[0, 0]
    assert int(orc.matmul_integer(a, b)[0, 0]) != 255 * 255 * 40000


@pytest.mark.parametrize("group,stride,pad,zx,zwmode", [(1, (1, 1), (1, 1), 0, None), (2, (2, 1), (1, 2), 9, "vec"), (8, (1, 1), (1, 1), 3, "scalar"),
                                                       (1, (2, 2), (3, 3), 128, None)])
def test_conv_integer_vs_int64(orc, group, stride, pad, zx, zwmode):
    rng = np.random.default_rng(4)
    C, M = 8, 8 * (2 if group < 8 else 1)
    k = 7 if pad == (3, 3) else 3
    x = rng.integers(0, 256, (2, C, 10, 9), dtype=np.uint8)
    w = rng.integers(-127, 128, (M, C // group, k, k)).astype(np.int8)
    zw = None if zwmode is None else (rng.integers(-9, 9, M).astype(np.int8) if zwmode == "vec" else np.array([5], np.int8))
    got = orc.conv_integer(x, w, zx, zw, strides=stride, pads=pad, group=group)
    assert np.array_equal(got, np_conv_integer(x, w, zx, zw, stride, pad, group))


def test_conv_geometry_follows_reference(orc):
    # CalculateAutoPad (runtime/chainerx_util.cc:291-302): SAME_UPPER puts the odd pad at the end
    g = orc.conv_geometry(28, 28, 5, 5, auto_pad="SAME_UPPER")
    assert (g["pt"], g["pb"], g["Ho"]) == (2, 2, 28)
    g = orc.conv_geometry(7, 7, 2, 2, strides=[1, 1], auto_pad="SAME_UPPER")
    assert (g["pt"], g["pb"], g["pl"], g["pr"], g["Ho"], g["Wo"]) == (0, 1, 0, 1, 7, 7)
    g = orc.conv_geometry(10, 10, 3, 3, strides=[2, 2], auto_pad="SAME_UPPER")
    assert (g["pt"], g["pb"], g["Ho"]) == (0, 1, 5)
    # ComplementStride / ComplementPad: empty -> 1 / 0 (runtime/chainerx_util.cc:180-200)
    g = orc.conv_geometry(10, 12, 3, 3)
    assert (g["sh"], g["sw"], g["pt"], g["pl"], g["Ho"], g["Wo"]) == (1, 1, 0, 0, 8, 10)
    with pytest.raises(ValueError):
        orc.conv_geometry(10, 10, 3, 3, auto_pad="SAME_LOWER")


def test_qlinear_conv_is_dequant_conv_quant(orc):
    """orc_qlinear_conv against a numpy fp32 restatement of runtime/ops/quantize.cc:62-94 (accumulation order differs,
    so equality is asked only within one step) and against the integer-domain requantization."""
    rng = np.random.default_rng(5)
    x = rng.integers(0, 256, (2, 6, 8, 8), dtype=np.uint8)
    w = rng.integers(-127, 128, (10, 6, 3, 3)).astype(np.int8)
    ws = rng.uniform(0.002, 0.005, 10).astype(np.float32)
    wz = rng.integers(-3, 3, 10).astype(np.int8)
    y = orc.qlinear_conv(x, 0.03, 5, w, ws, wz, 0.08, 11, strides=(1, 1), pads=(1, 1))
    xf = (x.astype(np.float32) - np.float32(5)) * np.float32(0.03)
    wf = (w.astype(np.float32) - wz.astype(np.float32)[:, None, None, None]) * ws[:, None, None, None]
    import torch
    yf = torch.nn.functional.conv2d(torch.from_numpy(xf), torch.from_numpy(wf), padding=1).numpy()
    want = np_quantize_ref(yf, 0.08, 11)
    assert np.abs(y.astype(int) - want.astype(int)).max() <= 1
    acc = orc.conv_integer(x, w, 5, wz, strides=(1, 1), pads=(1, 1))
    y2 = orc.requantize(acc, 0.03, ws, 0.08, 11, channel_axis=1)
    assert np.abs(y.astype(int) - y2.astype(int)).max() <= 1


def test_weight_quantizer_known_answers(orc):
    # compiler/quantize.cc:77-81: int8 scale = 2 * max|w| / 254, q = rint(w / scale); range includes 0 (:71-72)
    w = np.array([[0.5, -1.27, 1.0, 0.004]], np.float32)
    q, s, z = orc.quantize_weight_per_channel(w, True)
    assert np.isclose(s[0], np.float32(1.27) * 2 / 254) and z[0] == 0
    assert q.tolist() == [[50, -127, 100, 0]]
    # uint8: scale = (max - min) / 255, zp = rint(-min / scale)
    qu, su, zu = orc.quantize_data(np.array([-1.0, 0.0, 4.0, 2.0], np.float32), False)
    assert np.isclose(su, 5.0 / 255) and zu == 51
    assert qu.tolist() == [0, 51, 255, 153]
    # all-positive tensor still includes 0 in its range
    qu, su, zu = orc.quantize_data(np.array([1.0, 2.0], np.float32), False)
    assert zu == 0 and np.isclose(su, 2.0 / 255)


def test_dynamic_params_reference_quirk(orc):
    # compiler/quantize.cc:190-197: min/max are NOT widened to include 0, so an all-positive tensor gives a negative zero point
    s, z = orc.dynamic_params_u8(np.array([0.5, 1.0, 3.05], np.float32))
    assert np.isclose(s, 0.01) and z == -50.0


def test_eltwise_fp32_vs_fp64(orc):
    rng = np.random.default_rng(6)
    ins = [rng.standard_normal(5000).astype(np.float32) for _ in range(5)]
    nodes = [("Tanh", [0]), ("Sigmoid", [3]), ("Sigmoid", [2]), ("Sigmoid", [4]), ("Mul", [5, 6]), ("Mul", [7, 1]), ("Add", [9, 10]),
             ("Tanh", [11]), ("Mul", [8, 12])]
    f32 = orc.eltwise(nodes, ins, [11, 13])
    f64 = orc.eltwise(nodes, ins, [11, 13], fp64=True)
    a, c, f, i, o = [v.astype(np.float64) for v in ins]
    sig = lambda v: 1.0 / (1.0 + np.exp(-v))  # noqa: E731
    cn = np.tanh(a) * sig(i) + sig(f) * c
    assert np.allclose(f64[0], cn, rtol=1e-12) and np.allclose(f64[1], sig(o) * np.tanh(cn), rtol=1e-12)
    for got, want in zip(f32, f64):
        assert np.allclose(got, want, rtol=1e-5, atol=1e-6)
    # constants and the remaining ops
    out = orc.eltwise([("Constant", [], 2.5), ("Mul", [0, 1]), ("Exp", [2]), ("Sub", [3, 0]), ("Identity", [4]), ("Div", [5, 1])],
                      [np.array([0.5, 1.0], np.float32)], [6])
    assert np.allclose(out[0], (np.exp(np.array([1.25, 2.5])) - np.array([0.5, 1.0])) / 2.5, rtol=1e-6)


def test_golden_vectors(orc):
    g = np.load(GOLDEN)
    x = g["q_x"]
    assert np.array_equal(orc.quantize_linear(x, 0.02, 3, np.uint8, orc.ROUND_REF), g["q_u8_ref"])
    assert np.array_equal(orc.quantize_linear(x, 0.02, 3, np.uint8, orc.ROUND_RNE), g["q_u8_rne"])
    assert np.array_equal(orc.quantize_linear(x, 0.02, -5, np.int8, orc.ROUND_REF), g["q_i8_ref"])
    assert np.array_equal(orc.quantize_linear(x, 0.02, -5, np.int8, orc.ROUND_RNE), g["q_i8_rne"])
    assert np.array_equal(orc.dequantize_linear(g["q_u8_ref"], 0.02, 3), g["dq_u8"])
    assert np.array_equal(orc.dequantize_linear(g["q_i8_ref"], 0.031, -5), g["dq_i8"])
    assert np.array_equal(orc.matmul_integer(g["mm_a"], g["mm_b"]), g["mm_y_plain"])
    assert np.array_equal(orc.matmul_integer(g["mm_a"], g["mm_b"], [128], [3]), g["mm_y_scalar_zp"])
    assert np.array_equal(orc.matmul_integer(g["mm_a"], g["mm_b"], g["mm_za"], g["mm_zb"]), g["mm_y_vector_zp"])
    assert np.array_equal(orc.qlinear_matmul(g["mm_a"], 0.01, 128, g["mm_b"], 0.02, 0, 0.05, 7), g["qmm_y"])
    assert np.array_equal(orc.conv_integer(g["cv_x"], g["cv_w"], 7, g["cv_zw"], strides=[2, 1], pads=[1, 1], group=2), g["cv_y"])
    assert np.array_equal(orc.conv_integer(g["cv_x"], g["cv_w"], 7, None, strides=[2, 2], group=2, auto_pad="SAME_UPPER"), g["cv_y_same"])
    assert np.array_equal(orc.qlinear_conv(g["cv_x"], 0.02, 7, g["cv_w"], g["qc_ws"], g["cv_zw"], 0.04, 9, b=g["qc_bias"], strides=[1, 1],
                                           pads=[1, 1], group=2), g["qc_y"])
    q, s, z = orc.quantize_weight_per_channel(g["wq_w"], True)
    assert np.array_equal(q, g["wq_q"]) and np.array_equal(s, g["wq_s"])
    # golden int32 results also agree with the independent int64 formulation
    assert np.array_equal(g["mm_y_vector_zp"], np_matmul_integer(g["mm_a"], g["mm_b"], g["mm_za"], g["mm_zb"]))
    assert np.array_equal(g["cv_y"], np_conv_integer(g["cv_x"], g["cv_w"], 7, g["cv_zw"], (2, 1), (1, 1), 2))
