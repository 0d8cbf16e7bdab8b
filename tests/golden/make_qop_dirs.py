"""Writes tests/golden/qops/<name>/ -- `run_onnx` test directories (model.onnx + test_data_set_0/{input,output}_*.pb) with one
quantized operator each, in the layout of the ONNX backend node tests the reference runs for these operators
(scripts/runtests.py:556-582): every operand, the scale and zero-point scalars included, is a graph input.  Shapes and values
are this repository's own (seeded); the expected outputs are the CPU oracle's.  A last directory chains the operators with
their parameters as initializers.

    python tests/golden/make_qop_dirs.py
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
import __graft_entry__ as entry  # noqa: E402


def main():
    entry.load_package()
    entry.load_oracle()
    from chainer_compiler_b200 import onnx_io
    from oracle import oracle as orc
    N = onnx_io.Node
    rng = np.random.default_rng(2024)
    f32, u8, i8 = np.float32, np.uint8, np.int8
    out = os.path.join(HERE, "qops")

    def emit(name, nodes, inputs, outputs, initializers=None):
        model = onnx_io.Model(nodes, initializers or {}, list(inputs), [k for k, _ in outputs], ir_version=5, opset=10, name=name)
        onnx_io.write_test_dir(os.path.join(out, name), model, [(inputs, outputs)])

    # QuantizeLinear: ties and out-of-range values included
    x = (rng.standard_normal((3, 5, 7)) * 40).astype(f32)
    x.reshape(-1)[:6] = [0.5 * 0.25, 1.5 * 0.25, -300.0, 300.0, 2.5 * 0.25, -0.5 * 0.25]
    s, zp = f32(0.25), u8(121)
    emit("quantizelinear_u8", [N("QuantizeLinear", ["x", "y_scale", "y_zero_point"], ["y"], {})],
         {"x": x, "y_scale": s.reshape(()), "y_zero_point": zp.reshape(())}, [("y", orc.quantize_linear(x, s, int(zp)))])
    xp = np.abs(x)
    emit("quantizelinear_i8", [N("QuantizeLinear", ["x", "y_scale", "y_zero_point"], ["y"], {})],
         {"x": xp, "y_scale": f32(1.5).reshape(()), "y_zero_point": i8(-5).reshape(())}, [("y", orc.quantize_linear(xp, f32(1.5), -5, out_dtype=i8))])

    # DequantizeLinear
    q = rng.integers(0, 256, (4, 6, 5), dtype=u8)
    emit("dequantizelinear_u8", [N("DequantizeLinear", ["x", "x_scale", "x_zero_point"], ["y"], {})],
         {"x": q, "x_scale": f32(0.031).reshape(()), "x_zero_point": u8(77).reshape(())}, [("y", orc.dequantize_linear(q, f32(0.031), 77))])
    qi = rng.integers(-128, 128, (33,), dtype=i8)
    emit("dequantizelinear_i8_no_zero_point", [N("DequantizeLinear", ["x", "x_scale"], ["y"], {})],
         {"x": qi, "x_scale": f32(2.0).reshape(())}, [("y", orc.dequantize_linear(qi, f32(2.0), 0))])

    # MatMulInteger: scalar zero points, and a per-column zero point for b
    a = rng.integers(0, 256, (5, 19), dtype=u8)
    b = rng.integers(0, 256, (19, 7), dtype=u8)
    za, zb = np.array([12], u8), np.array([3], u8)
    emit("matmulinteger", [N("MatMulInteger", ["a", "b", "a_zero_point", "b_zero_point"], ["y"], {})],
         {"a": a, "b": b, "a_zero_point": za, "b_zero_point": zb}, [("y", orc.matmul_integer(a, b, za, zb))])
    bs = rng.integers(-128, 128, (19, 7), dtype=i8)
    zbv = rng.integers(-5, 6, (7,), dtype=i8)
    emit("matmulinteger_per_column", [N("MatMulInteger", ["a", "b", "a_zero_point", "b_zero_point"], ["y"], {})],
         {"a": a, "b": bs, "a_zero_point": za, "b_zero_point": zbv}, [("y", orc.matmul_integer(a, bs, za, zbv))])

    # QLinearMatMul
    sa, sb, sy = f32(0.02), f32(0.004), f32(0.05)
    emit("qlinearmatmul", [N("QLinearMatMul", ["a", "a_scale", "a_zero_point", "b", "b_scale", "b_zero_point", "y_scale", "y_zero_point"], ["y"], {})],
         {"a": a, "a_scale": sa.reshape(()), "a_zero_point": u8(113).reshape(()), "b": b, "b_scale": sb.reshape(()), "b_zero_point": u8(114).reshape(()),
          "y_scale": sy.reshape(()), "y_zero_point": u8(118).reshape(())},
         [("y", orc.qlinear_matmul(a, sa, 113, b, sb, 114, sy, 118))])

    # ConvInteger: padding, stride, per-output-channel weight zero points
    cx = rng.integers(0, 256, (2, 3, 9, 8), dtype=u8)
    cw = rng.integers(0, 256, (4, 3, 3, 3), dtype=u8)
    czw = rng.integers(100, 150, (4,), dtype=u8)
    attrs = {"kernel_shape": [3, 3], "pads": [1, 1, 1, 1], "strides": [2, 1]}
    emit("convinteger_with_padding", [N("ConvInteger", ["x", "w", "x_zero_point", "w_zero_point"], ["y"], attrs)],
         {"x": cx, "w": cw, "x_zero_point": u8(9).reshape(()), "w_zero_point": czw},
         [("y", orc.conv_integer(cx, cw, 9, czw.astype(np.int32), (2, 1), (1, 1)))])
    emit("convinteger_same_upper", [N("ConvInteger", ["x", "w", "x_zero_point"], ["y"], {"kernel_shape": [3, 3], "auto_pad": "SAME_UPPER", "strides": [2, 2]})],
         {"x": cx, "w": cw, "x_zero_point": u8(9).reshape(())}, [("y", orc.conv_integer(cx, cw, 9, None, (2, 2), (), 1, "SAME_UPPER"))])

    # QLinearConv: per-channel and per-tensor weights, groups
    qw = rng.integers(-127, 128, (6, 2, 3, 3), dtype=i8)
    qx = rng.integers(0, 256, (2, 4, 7, 7), dtype=u8)
    ws = rng.uniform(0.001, 0.004, 6).astype(f32)
    wz = np.zeros(6, i8)
    ins = ["x", "x_scale", "x_zero_point", "w", "w_scale", "w_zero_point", "y_scale", "y_zero_point"]
    emit("qlinearconv_per_channel_groups", [N("QLinearConv", ins, ["y"], {"kernel_shape": [3, 3], "pads": [1, 1, 1, 1], "group": 2})],
         {"x": qx, "x_scale": f32(0.02).reshape(()), "x_zero_point": u8(128).reshape(()), "w": qw, "w_scale": ws, "w_zero_point": wz,
          "y_scale": f32(0.03).reshape(()), "y_zero_point": u8(120).reshape(())},
         [("y", orc.qlinear_conv(qx, f32(0.02), 128, qw, ws, wz, f32(0.03), u8(120), None, (), (1, 1), 2))])
    pw = rng.integers(0, 256, (5, 4, 1, 1), dtype=u8)
    emit("qlinearconv_per_tensor", [N("QLinearConv", ins, ["y"], {})],
         {"x": qx, "x_scale": f32(0.02).reshape(()), "x_zero_point": u8(128).reshape(()), "w": pw, "w_scale": f32(0.002).reshape(()),
          "w_zero_point": u8(131).reshape(()), "y_scale": f32(0.04).reshape(()), "y_zero_point": u8(100).reshape(())},
         [("y", orc.qlinear_conv(qx, f32(0.02), 128, pw, f32(0.002).reshape(()), u8(131).reshape(()), f32(0.04), u8(100)))])

    # chain with the parameters as initializers: Q -> QLinearConv -> DQ
    fx = rng.uniform(-1, 1, (2, 4, 7, 7)).astype(f32)
    inits = {"sx": f32(1 / 127.0).reshape(()), "zx": u8(128).reshape(()), "w": qw, "ws": ws, "wz": wz, "sy": f32(0.03).reshape(()), "zy": u8(120).reshape(())}
    xq = orc.quantize_linear(fx, inits["sx"][()], 128)
    yq = orc.qlinear_conv(xq, inits["sx"][()], 128, qw, ws, wz, f32(0.03), u8(120), None, (), (1, 1), 2)
    emit("chain_initializers",
         [N("QuantizeLinear", ["x", "sx", "zx"], ["xq"], {}),
          N("QLinearConv", ["xq", "sx", "zx", "w", "ws", "wz", "sy", "zy"], ["yq"], {"kernel_shape": [3, 3], "pads": [1, 1, 1, 1], "group": 2}),
          N("DequantizeLinear", ["yq", "sy", "zy"], ["y"], {})],
         {"x": fx}, [("y", orc.dequantize_linear(yq, f32(0.03), 120))], inits)
    print("wrote", sorted(os.listdir(out)))


if __name__ == "__main__":
    main()
