"""B200-native kernels for chainer-compiler's quantized-inference VM ops.

``ops`` mirrors the reference's op bodies (QuantizeLinear, DequantizeLinear, QLinearConv, QLinearMatMul,
ConvInteger, MatMulInteger, ElementWiseNvrtc) over the C ABI of ``libchxq.so``; ``fusion`` is the
elementwise grouping and source generator; ``models`` builds the synthetic int8 networks the benchmarks
run; ``dataparallel`` shards batches over the GPUs of one node.
"""
from . import _lib  # noqa: F401
from ._lib import ChxqError, ChxqLibraryError, build, lib  # noqa: F401

__all__ = ["ChxqError", "ChxqLibraryError", "build", "lib"]
