"""Compares two directories written by `run_onnx --dump_outputs_dir` (reference tool: tools/compare_dump_dirs.py).

    python chainer-compiler_b200/compare_dump_dirs.py DIR1 DIR2 [--rtol 1e-7] [--atol 0]

Files are `<instruction id>_<value name>.npy`; values are matched by name, so the two runs may number their instructions
differently (for instance with and without --fuse_operations).  Prints one line per value present in both directories and
returns the number of values that differ."""
import argparse
import os
import re
import sys

import numpy as np


def read_dump_dir(d):
    """[(value name, path)] in instruction order."""
    found = []
    for f in sorted(os.listdir(d)):
        m = re.match(r"(\d+)_(.*)\.npy$", f)
        if m:
            found.append((m.group(2), os.path.join(d, f)))
    return found


def compare(dir1, dir2, rtol=1e-7, atol=0.0, out=sys.stderr):
    second = dict(read_dump_dir(dir2))
    differing = 0
    for name, path1 in read_dump_dir(dir1):
        path2 = second.get(name)
        if path2 is None:
            continue
        a, b = np.load(path1), np.load(path2)
        if a.shape != b.shape or a.dtype != b.dtype:
            out.write("%s: %s %s against %s %s\n" % (name, a.dtype, a.shape, b.dtype, b.shape))
            differing += 1
            continue
        af, bf = a.astype(np.float64), b.astype(np.float64)
        if np.allclose(af, bf, rtol=rtol, atol=atol, equal_nan=True):
            out.write("%s: OK\n" % name)
        else:
            d = np.abs(af - bf)
            k = int(np.argmax(d))
            out.write("%s: %d of %d elements differ, largest |a - b| = %.6g at flat index %d (%r against %r)\n"
                      % (name, int((d > atol + rtol * np.abs(bf)).sum()), a.size, d.reshape(-1)[k], k, a.reshape(-1)[k], b.reshape(-1)[k]))
            differing += 1
    return differing


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("dir1")
    ap.add_argument("dir2")
    ap.add_argument("--rtol", type=float, default=1e-7)
    ap.add_argument("--atol", type=float, default=0.0)
    args = ap.parse_args(argv)
    return compare(args.dir1, args.dir2, args.rtol, args.atol)


if __name__ == "__main__":
    sys.exit(1 if main() else 0)
