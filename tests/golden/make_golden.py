"""Generates tests/golden/hotpath_vectors.npz from the CPU oracle (oracle/chxq_oracle.c).

The reference checkout holds no golden vectors for these ops (its ONNX node-test data directory is an
empty submodule) and cannot be built or imported here, so the vectors below are outputs of the
by-specification oracle on seeded inputs.  They freeze the oracle's behaviour: a later change to the
oracle that alters any of them is caught by tests/test_oracle.py.  Run from the repository root:

    python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import oracle as orc  # noqa: E402


def main():
    rng = np.random.default_rng(20240607)
    out = {}
    x = np.concatenate([rng.uniform(-3, 3, 500), (np.arange(-20, 280) + 0.5) * 0.02, [0.0, -0.0, 1e9, -1e9]]).astype(np.float32)
    out["q_x"] = x
    out["q_u8_ref"] = orc.quantize_linear(x, 0.02, 3, np.uint8, orc.ROUND_REF)
    out["q_u8_rne"] = orc.quantize_linear(x, 0.02, 3, np.uint8, orc.ROUND_RNE)
    out["q_i8_ref"] = orc.quantize_linear(x, 0.02, -5, np.int8, orc.ROUND_REF)
    out["q_i8_rne"] = orc.quantize_linear(x, 0.02, -5, np.int8, orc.ROUND_RNE)
    out["dq_u8"] = orc.dequantize_linear(out["q_u8_ref"], 0.02, 3)
    out["dq_i8"] = orc.dequantize_linear(out["q_i8_ref"], 0.031, -5)

    a = rng.integers(0, 256, (37, 48), dtype=np.uint8)
    b = rng.integers(-127, 128, (48, 29)).astype(np.int8)
    out["mm_a"], out["mm_b"] = a, b
    out["mm_za"] = rng.integers(0, 256, 48, dtype=np.uint8)
    out["mm_zb"] = rng.integers(-20, 20, 29).astype(np.int8)
    out["mm_y_plain"] = orc.matmul_integer(a, b)
    out["mm_y_scalar_zp"] = orc.matmul_integer(a, b, [128], [3])
    out["mm_y_vector_zp"] = orc.matmul_integer(a, b, out["mm_za"], out["mm_zb"])
    out["qmm_y"] = orc.qlinear_matmul(a, 0.01, 128, b, 0.02, 0, 0.05, 7)

    xc = rng.integers(0, 256, (2, 8, 9, 11), dtype=np.uint8)
    wc = rng.integers(-127, 128, (12, 4, 3, 3)).astype(np.int8)
    out["cv_x"], out["cv_w"] = xc, wc
    out["cv_zw"] = rng.integers(-5, 5, 12).astype(np.int8)
    out["cv_y"] = orc.conv_integer(xc, wc, 7, out["cv_zw"], strides=[2, 1], pads=[1, 1], group=2)
    out["cv_y_same"] = orc.conv_integer(xc, wc, 7, None, strides=[2, 2], group=2, auto_pad="SAME_UPPER")
    ws = rng.uniform(0.001, 0.004, 12).astype(np.float32)
    bias = rng.integers(-2000, 2000, 12).astype(np.int32)
    out["qc_ws"], out["qc_bias"] = ws, bias
    out["qc_y"] = orc.qlinear_conv(xc, 0.02, 7, wc, ws, out["cv_zw"], 0.04, 9, b=bias, strides=[1, 1], pads=[1, 1], group=2)
    acc = orc.conv_integer(xc, wc, 7, out["cv_zw"], strides=[1, 1], pads=[1, 1], group=2)
    out["qc_y_exact"] = orc.requantize(acc, 0.02, ws, 0.04, 9, bias=bias, channel_axis=1)

    w = (rng.standard_normal((6, 20)) * 0.05).astype(np.float32)
    q, s, z = orc.quantize_weight_per_channel(w, True)
    out["wq_w"], out["wq_q"], out["wq_s"] = w, q, s
    qu, su, zu = orc.quantize_data(w, False)
    out["wq_qu"], out["wq_su"], out["wq_zu"] = qu, np.float32(su), np.int32(zu)

    ins = [rng.standard_normal(300).astype(np.float32) for _ in range(5)]
    names = ["a", "c_prev", "f", "i", "o"]
    nodes = [("Tanh", [0]), ("Sigmoid", [3]), ("Sigmoid", [2]), ("Sigmoid", [4]), ("Mul", [5, 6]), ("Mul", [7, 1]), ("Add", [9, 10]),
             ("Tanh", [11]), ("Mul", [8, 12])]
    c_next, h = orc.eltwise(nodes, ins, [11, 13])
    for n, v in zip(names, ins):
        out["ew_" + n] = v
    out["ew_c_next"], out["ew_h"] = c_next, h
    np.savez_compressed(os.path.join(os.path.dirname(os.path.abspath(__file__)), "hotpath_vectors.npz"), **out)
    print("wrote %d arrays" % len(out))


if __name__ == "__main__":
    main()
