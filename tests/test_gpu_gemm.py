"""MatMulInteger / QLinearMatMul: CUDA-core and tcgen05 kernels against the CPU oracle.
int32 accumulators are bit-exact; requantized outputs are bit-exact against the integer-domain oracle and within one
step of the fp32-emulating oracle, with the mismatch count printed."""
import os

import numpy as np
import pytest
import torch

from helpers import lsb_report

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "hotpath_vectors.npz")
SIMT, TENSOR, AUTO = 1, 2, 0


def _t(a, dev):
    return None if a is None else torch.from_numpy(np.ascontiguousarray(a)).to(dev)


def _rand(rng, shape, dtype):
    return rng.integers(np.iinfo(dtype).min, np.iinfo(dtype).max + 1, shape).astype(dtype)


@pytest.mark.parametrize("M,N,K", [(1, 1, 1), (5, 7, 3), (33, 65, 47), (128, 64, 64), (200, 100, 130)])
@pytest.mark.parametrize("adt,bdt", [(np.uint8, np.int8), (np.uint8, np.uint8), (np.int8, np.int8)])
@pytest.mark.parametrize("zpmode", ["none", "scalar", "vector"])
def test_matmul_integer_simt(ops, orc, dev, M, N, K, adt, bdt, zpmode):
    rng = np.random.default_rng(M * 1000 + N)
    a, b = _rand(rng, (M, K), adt), _rand(rng, (K, N), bdt)
    za = zb = None
    if zpmode == "scalar":
        za, zb = _rand(rng, 1, adt), _rand(rng, 1, bdt)
    elif zpmode == "vector":
        za, zb = _rand(rng, K, adt), _rand(rng, N, bdt)
    y = ops.MatMulInteger(_t(a, dev), _t(b, dev), _t(za, dev), _t(zb, dev), path=SIMT).cpu().numpy()
    assert np.array_equal(y, orc.matmul_integer(a, b, za, zb))


@pytest.mark.parametrize("M,N,K", [(128, 64, 32), (128, 256, 128), (200, 80, 96), (1, 16, 16), (300, 1000, 784), (257, 48, 272), (512, 512, 512)])
@pytest.mark.parametrize("adt,bdt", [(np.uint8, np.int8), (np.uint8, np.uint8), (np.int8, np.int8), (np.int8, np.uint8)])
def test_matmul_integer_tensor_plain(ops, orc, dev, M, N, K, adt, bdt):
    rng = np.random.default_rng(M + N + K)
    a, b = _rand(rng, (M, K), adt), _rand(rng, (K, N), bdt)
    y = ops.MatMulInteger(_t(a, dev), _t(b, dev), path=TENSOR)
    ops.device_status()
    assert np.array_equal(y.cpu().numpy(), orc.matmul_integer(a, b))


@pytest.mark.parametrize("M,N,K", [(130, 72, 80), (256, 256, 256)])
@pytest.mark.parametrize("zpmode", ["a_scalar", "b_scalar", "both_scalar", "both_vector"])
def test_matmul_integer_tensor_zero_points(ops, orc, dev, M, N, K, zpmode):
    rng = np.random.default_rng(K)
    a, b = _rand(rng, (M, K), np.uint8), _rand(rng, (K, N), np.int8)
    za = zb = None
    if zpmode in ("a_scalar", "both_scalar"):
        za = np.array([128], np.uint8)
    if zpmode in ("b_scalar", "both_scalar"):
        zb = np.array([-3], np.int8)
    if zpmode == "both_vector":
        za, zb = _rand(rng, K, np.uint8), _rand(rng, N, np.int8)
    y = ops.MatMulInteger(_t(a, dev), _t(b, dev), _t(za, dev), _t(zb, dev), path=TENSOR)
    ops.device_status()
    assert np.array_equal(y.cpu().numpy(), orc.matmul_integer(a, b, za, zb))


def test_matmul_integer_batched_and_auto(ops, orc, dev):
    rng = np.random.default_rng(5)
    a, b = _rand(rng, (2, 3, 64, 48), np.uint8), _rand(rng, (2, 3, 48, 32), np.int8)
    for path in (SIMT, TENSOR, AUTO):
        y = ops.MatMulInteger(_t(a, dev), _t(b, dev), path=path)
        assert np.array_equal(y.cpu().numpy(), orc.matmul_integer(a, b))
    # K not a multiple of 16: AUTO falls to the CUDA-core kernel, TENSOR refuses
    a, b = _rand(rng, (40, 50), np.uint8), _rand(rng, (50, 24), np.int8)
    assert np.array_equal(ops.MatMulInteger(_t(a, dev), _t(b, dev)).cpu().numpy(), orc.matmul_integer(a, b))
    with pytest.raises(ops.ChxqError) as e:
        ops.MatMulInteger(_t(a, dev), _t(b, dev), path=TENSOR)
    assert e.value.code == 2
    ops.device_status()


def test_matmul_integer_rejects(ops, dev):
    a = torch.zeros((4, 8), dtype=torch.uint8, device=dev)
    b = torch.zeros((8, 4), dtype=torch.int8, device=dev)
    with pytest.raises(ops.ChxqError):
        ops.MatMulInteger(a, b, torch.zeros((2, 2), dtype=torch.uint8, device=dev))  # zero point rank > 1 (quantize.cc:105)
    with pytest.raises(ops.ChxqError):
        ops.MatMulInteger(a, b, torch.zeros(3, dtype=torch.uint8, device=dev))  # length neither 1 nor K
    with pytest.raises(ops.ChxqError):
        ops.MatMulInteger(a, torch.zeros((7, 4), dtype=torch.int8, device=dev))
    with pytest.raises(ops.ChxqError):
        ops.MatMulInteger(a.float(), b)
    assert ops.MatMulInteger(torch.zeros((0, 8), dtype=torch.uint8, device=dev), b).shape == (0, 4)


@pytest.mark.parametrize("path", [SIMT, TENSOR])
@pytest.mark.parametrize("M,N,K,zy,ydt", [(64, 1000, 784, 0, np.uint8), (130, 48, 96, 7, np.uint8), (128, 128, 128, -3, np.int8)])
def test_qlinear_matmul(ops, orc, dev, path, M, N, K, zy, ydt):
    rng = np.random.default_rng(N)
    a, b = _rand(rng, (M, K), np.uint8), _rand(rng, (K, N), np.int8)
    sa, sb, sy = 0.01, 0.002, 0.03
    for mode in (0, 1):
        y = ops.QLinearMatMul(_t(a, dev), sa, np.uint8(128), _t(b, dev), sb, np.int8(0), sy, ydt(zy), round_mode=mode, path=path)
        ops.device_status()
        y = y.cpu().numpy()
        acc = orc.matmul_integer(a, b, [128], None)
        exact = orc.requantize(acc, sa, np.array([sb], np.float32), sy, zy, y_dtype=ydt, round_mode=mode)
        assert np.array_equal(y, exact), "integer-domain requantization must be bit-exact"
        emul = orc.qlinear_matmul(a, sa, 128, b, sb, 0, sy, zy, ydt, mode)
        mx, cnt, tot = lsb_report(y, emul)
        print("QLinearMatMul %dx%dx%d mode %d: %d of %d differ from the fp32-emulating chain, max %d LSB" % (M, N, K, mode, cnt, tot, mx))
        assert mx <= 1


def test_golden_matmul(ops, dev):
    g = np.load(GOLDEN)
    a, b = _t(g["mm_a"], dev), _t(g["mm_b"], dev)
    for path in (SIMT, TENSOR):
        assert np.array_equal(ops.MatMulInteger(a, b, path=path).cpu().numpy(), g["mm_y_plain"])
        assert np.array_equal(ops.MatMulInteger(a, b, _t(g["mm_za"], dev), _t(g["mm_zb"], dev), path=path).cpu().numpy(), g["mm_y_vector_zp"])
        y = ops.QLinearMatMul(a, 0.01, np.uint8(128), b, 0.02, np.int8(0), 0.05, np.uint8(7), path=path).cpu().numpy()
        assert np.abs(y.astype(int) - g["qmm_y"].astype(int)).max() <= 1
    ops.device_status()


@pytest.mark.parametrize("S", [1024, 4096])
def test_matmul_integer_sweep_checksum(ops, dev, S):
    """Sweep sizes (A uint8 zero point 128, B int8): row and column checksums of the full result against int64 sums of the
    operands -- sum_n y[m,n] = sum_k a'[m,k] * (sum_n b[k,n]) -- and a random sample of entries against exact dot products."""
    gen = torch.Generator(device=dev).manual_seed(S)
    a = torch.randint(0, 256, (S, S), dtype=torch.uint8, device=dev, generator=gen)
    b = torch.randint(-127, 128, (S, S), dtype=torch.int8, device=dev, generator=gen)
    za = torch.tensor([128], dtype=torch.uint8, device=dev)
    y = ops.MatMulInteger(a, b, za, None, path=TENSOR)
    ops.device_status()
    an, bn, yn = a.cpu().numpy().astype(np.int64) - 128, b.cpu().numpy().astype(np.int64), y.cpu().numpy().astype(np.int64)
    assert np.array_equal(yn.sum(axis=1), an @ bn.sum(axis=1))
    assert np.array_equal(yn.sum(axis=0), an.sum(axis=0) @ bn)
    rng = np.random.default_rng(S)
    for m, n in zip(rng.integers(0, S, 64), rng.integers(0, S, 64)):
        assert yn[m, n] == int(an[m] @ bn[:, n])
    y2 = ops.MatMulInteger(a, b, za, None, path=SIMT) if S <= 1024 else None
    if y2 is not None:
        assert torch.equal(y, y2)
