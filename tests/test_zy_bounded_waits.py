"""The bounded device-side waits of the tensor-core kernels, made to run out once in the allowed way: a wait on a barrier
that nothing completes.  A test hook makes the one-tile kernel's producer leave out one weight load, so that the stage never
fills; with the wait limit shortened to 5 ms the MMA warp's wait expires, the CTA raises its abort flag, every role leaves
its loop, the CTA waits out its copies in flight, frees its tensor memory and RETURNS.  Nothing traps, faults or spins on: the
context stays usable, the status word reports the timeout, and the next ordinary launch is bit-exact."""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_expired_wait_reports_timeout_and_context_survives(pkg, ops, orc, dev):
    from chainer_compiler_b200 import _lib
    L = pkg.lib()
    rng = np.random.default_rng(0)
    a = rng.integers(0, 256, (128, 256), dtype=np.uint8)   # one 128-row tile, two 128-byte K blocks
    b = rng.integers(-127, 128, (256, 64)).astype(np.int8)
    at, bt = torch.from_numpy(a).to(dev), torch.from_numpy(b).to(dev)
    want = orc.matmul_integer(a, b)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    ops.device_status()
    try:
        _lib.check(L.chxq_tc_variant(1))                       # the one-tile kernel
        _lib.check(L.chxq_tc_test_hooks(5_000_000, 1))         # 5 ms limit; the weight load of K block 1 is left out
        ops.MatMulInteger(at, bt, None, None, path=ops.PATH_TENSOR)
        rc = L.chxq_device_status(stream)                      # synchronizes; the kernel has returned by itself
        assert rc == _lib.ERR_DEVICE_TIMEOUT, rc
        assert L.chxq_device_status(stream) == _lib.OK         # reading the status cleared it
    finally:
        _lib.check(L.chxq_tc_test_hooks(2_000_000_000, -1))
        _lib.check(L.chxq_tc_variant(0))
    # the context is intact: the same problem, ordinary launch, exact result; and a launch of the grouped kernel family
    y = ops.MatMulInteger(at, bt, None, None, path=ops.PATH_TENSOR)
    ops.device_status()
    assert np.array_equal(y.cpu().numpy(), want)
    y8 = ops.QLinearMatMul(at, 0.01, np.uint8(0), bt, 0.002, np.int8(0), 0.5, np.uint8(3), path=ops.PATH_TENSOR)
    ops.device_status()
    assert np.array_equal(y8.cpu().numpy(), orc.requantize(want, 0.01, np.array([0.002], np.float32), 0.5, 3))
