"""The allocation-free MatMulInteger entry (chxq_matmul_integer_noalloc) through the C ABI.

Some callers of the library cannot allocate device memory at the moment they call it: a memory pool's allocation hook
(it runs with the pool locked), or a serving process that gave all of its device memory away at start-up and must not
pay the device-wide synchronisation of a driver allocation.  For them the tensor-core path's scratch lives in a fixed
array inside the library.  The test calls the entry twice in a row -- the second call smaller and with other zero
points, so that bytes left in the shared array by the first call would show -- and asks for exactly the output of the
ordinary entry (int32 accumulators: bit-exact).  This file sorts last so that a run stopping at the first failure has
already run every other test; it does not depend on them.
"""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def _both(pkg, ops, a, b, za, zb):
    from chainer_compiler_b200 import _lib
    L = pkg.lib()
    M, K = a.shape
    N = b.shape[1]
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    code = {torch.uint8: _lib.UINT8, torch.int8: _lib.INT8}
    y_new = torch.full((M, N), -7, dtype=torch.int32, device=a.device)
    _lib.check(L.chxq_matmul_integer_noalloc(_ptr(a), code[a.dtype], _ptr(b), code[b.dtype], M, N, K, _ptr(za), 0 if za is None else za.numel(),
                                             _ptr(zb), 0 if zb is None else zb.numel(), _ptr(y_new), stream))
    y_old = ops.MatMulInteger(a, b, za, zb, path=ops.PATH_TENSOR if K % 16 == 0 else ops.PATH_AUTO)
    ops.device_status()
    return y_new, y_old


def test_noalloc_matches_ordinary_entry_twice(pkg, ops, orc, dev):
    gen = torch.Generator(device=dev).manual_seed(5)
    # first call: near the scratch limit (N * K = 4 MiB of repacked B), vector zero points on both sides
    a = torch.randint(0, 256, (777, 2048), dtype=torch.uint8, device=dev, generator=gen)
    b = torch.randint(-128, 128, (2048, 2048), dtype=torch.int8, device=dev, generator=gen)
    za = torch.randint(0, 256, (2048,), dtype=torch.uint8, device=dev, generator=gen)
    zb = torch.randint(-128, 128, (2048,), dtype=torch.int8, device=dev, generator=gen)
    y_new, y_old = _both(pkg, ops, a, b, za, zb)
    assert torch.equal(y_new, y_old)
    # second call, straight after: smaller, ragged, scalar / absent zero points -- stale scratch must not matter
    a2 = torch.randint(0, 256, (130, 272), dtype=torch.uint8, device=dev, generator=gen)
    b2 = torch.randint(-128, 128, (272, 72), dtype=torch.int8, device=dev, generator=gen)
    za2 = torch.tensor([128], dtype=torch.uint8, device=dev)
    y_new2, y_old2 = _both(pkg, ops, a2, b2, za2, None)
    assert torch.equal(y_new2, y_old2)
    assert np.array_equal(y_new2.cpu().numpy(), orc.matmul_integer(a2.cpu().numpy(), b2.cpu().numpy(), [128], None))
    # the first problem once more gives the first answer again
    y_new3, _ = _both(pkg, ops, a, b, za, zb)
    assert torch.equal(y_new3, y_old)


def test_noalloc_rejects_oversize_and_takes_unaligned_k(pkg, ops, orc, dev):
    from chainer_compiler_b200 import _lib
    L = pkg.lib()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    a = torch.zeros((64, 4096), dtype=torch.uint8, device=dev)
    b = torch.zeros((4096, 4096), dtype=torch.int8, device=dev)
    y = torch.empty((64, 4096), dtype=torch.int32, device=dev)
    rc = L.chxq_matmul_integer_noalloc(_ptr(a), _lib.UINT8, _ptr(b), _lib.INT8, 64, 4096, 4096, None, 0, None, 0, _ptr(y), stream)
    assert rc == _lib.ERR_WORKSPACE and b"fixed array" in L.chxq_last_error()
    # K = 50 is not a tensor-core shape: the CUDA-core kernel answers, still without scratch
    rng = np.random.default_rng(1)
    a2 = rng.integers(0, 256, (40, 50), dtype=np.uint8)
    b2 = rng.integers(-128, 128, (50, 24)).astype(np.int8)
    y_new, y_old = _both(pkg, ops, torch.from_numpy(a2).to(dev), torch.from_numpy(b2).to(dev), None, None)
    assert torch.equal(y_new, y_old) and np.array_equal(y_new.cpu().numpy(), orc.matmul_integer(a2, b2))


def test_noalloc_int8_a_and_unaligned_a(pkg, ops, orc, dev):
    """A signed left operand on the tensor-core path, and a left operand that starts one byte off a 16-byte boundary (the
    tensor-core kernel cannot read it, so the CUDA-core kernel answers -- still without scratch)."""
    rng = np.random.default_rng(2)
    a = rng.integers(-128, 128, (200, 320)).astype(np.int8)
    b = rng.integers(0, 256, (320, 96), dtype=np.uint8)
    za = rng.integers(-128, 128, 320).astype(np.int8)
    zb = rng.integers(0, 256, 96, dtype=np.uint8)
    y_new, y_old = _both(pkg, ops, torch.from_numpy(a).to(dev), torch.from_numpy(b).to(dev), torch.from_numpy(za).to(dev), torch.from_numpy(zb).to(dev))
    assert torch.equal(y_new, y_old) and np.array_equal(y_new.cpu().numpy(), orc.matmul_integer(a, b, za, zb))
    from chainer_compiler_b200 import _lib
    L = pkg.lib()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    a2 = rng.integers(0, 256, (64, 128), dtype=np.uint8)
    b2 = rng.integers(-128, 128, (128, 48)).astype(np.int8)
    buf = torch.zeros(64 * 128 + 16, dtype=torch.uint8, device=dev)
    off = (16 - buf.data_ptr() % 16) % 16 + 1
    a_dev = buf[off:off + 64 * 128].view(64, 128)
    a_dev.copy_(torch.from_numpy(a2))
    assert a_dev.data_ptr() % 16 == 1
    b_dev = torch.from_numpy(b2).to(dev)
    y = torch.full((64, 48), -7, dtype=torch.int32, device=dev)
    _lib.check(L.chxq_matmul_integer_noalloc(_ptr(a_dev), _lib.UINT8, _ptr(b_dev), _lib.INT8, 64, 48, 128, None, 0, None, 0, _ptr(y), stream))
    ops.device_status()
    assert np.array_equal(y.cpu().numpy(), orc.matmul_integer(a2, b2))
