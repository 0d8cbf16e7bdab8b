"""Writes tests/golden/mnist/ -- a `run_onnx` test directory (model.onnx + test_data_set_{0,1,2}/{input,output}_0.pb) -- from
the MNIST fixture the reference ships in data/mnist/ (model and three input / expected-output pairs).  The files are read
with this repository's own ONNX reader and written back with its writer (typed tensor fields, as the reference's writer
does), so the directory also pins the reader / writer pair.  Run from a checkout that has the reference next to it:

    python tests/golden/make_mnist_golden.py /path/to/reference/data/mnist
"""
import importlib.util
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))


def main():
    src = sys.argv[1]
    spec = importlib.util.spec_from_file_location("onnx_io", os.path.join(ROOT, "chainer-compiler_b200", "onnx_io.py"))
    onnx_io = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(onnx_io)
    model, cases = onnx_io.load_test_dir(src)
    dst = os.path.join(HERE, "mnist")
    onnx_io.write_test_dir(dst, model, cases)
    model2, cases2 = onnx_io.load_test_dir(dst)
    assert [repr(n) for n in model2.nodes] == [repr(n) for n in model.nodes]
    for k, v in model.initializers.items():
        assert np.array_equal(v, model2.initializers[k])
    for (i1, o1), (i2, o2) in zip(cases, cases2):
        for k in i1:
            assert np.array_equal(i1[k], i2[k])
        for (n1, a1), (n2, a2) in zip(o1, o2):
            assert n1 == n2 and np.array_equal(a1, a2)
    print("wrote", dst, "with", len(cases), "data sets")


if __name__ == "__main__":
    main()
