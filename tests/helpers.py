"""Shared helpers of the parity tests: independent numpy formulations and comparison utilities."""
import numpy as np


def np_quantize_ref(x, scale, zp, signed=False):
    """Reference rounding, independent formulation: floor(clamp(x/s + zp) + 0.5) for values >= -0.5, truncation toward zero otherwise."""
    lo, hi = (-128.0, 127.0) if signed else (0.0, 255.0)
    t = x.astype(np.float32) / np.float32(scale)
    if zp != 0:
        t = t + np.float32(zp)
    t = np.minimum(t, np.float32(hi))
    t = np.maximum(np.float32(lo), t)
    t = t + np.float32(0.5)
    return np.trunc(t).astype(np.int8 if signed else np.uint8)


def np_quantize_rne(x, scale, zp, signed=False):
    lo, hi = (-128.0, 127.0) if signed else (0.0, 255.0)
    r = np.rint(x.astype(np.float32) / np.float32(scale)) + np.float32(zp)
    return np.clip(r, lo, hi).astype(np.int8 if signed else np.uint8)


def np_matmul_integer(a, b, za=None, zb=None):
    A = a.astype(np.int64)
    B = b.astype(np.int64)
    if za is not None:
        A = A - np.asarray(za).astype(np.int64)
    if zb is not None:
        B = B - np.asarray(zb).astype(np.int64)
    y = np.matmul(A, B)
    return ((y + 2**31) % 2**32 - 2**31).astype(np.int32)


def np_conv_integer(x, w, zx, zw, stride, pad, group):
    """Direct int64 convolution, NCHW/OIHW, symmetric padding (pad_h, pad_w)."""
    N, C, H, W = x.shape
    M, Cg, KH, KW = w.shape
    X = x.astype(np.int64) - (zx or 0)
    Wt = w.astype(np.int64)
    if zw is not None:
        z = np.asarray(zw).astype(np.int64).reshape(-1)
        Wt = Wt - (z.reshape(-1, 1, 1, 1) if z.size > 1 else z[0])
    Xp = np.zeros((N, C, H + 2 * pad[0], W + 2 * pad[1]), np.int64)
    Xp[:, :, pad[0]:pad[0] + H, pad[1]:pad[1] + W] = X
    Ho = (H + 2 * pad[0] - KH) // stride[0] + 1
    Wo = (W + 2 * pad[1] - KW) // stride[1] + 1
    y = np.zeros((N, M, Ho, Wo), np.int64)
    Mg = M // group
    for g in range(group):
        xs = Xp[:, g * Cg:(g + 1) * Cg]
        ws = Wt[g * Mg:(g + 1) * Mg]
        for kh in range(KH):
            for kw in range(KW):
                patch = xs[:, :, kh:kh + stride[0] * (Ho - 1) + 1:stride[0], kw:kw + stride[1] * (Wo - 1) + 1:stride[1]]
                y[:, g * Mg:(g + 1) * Mg] += np.einsum("nchw,mc->nmhw", patch, ws[:, :, kh, kw])
    return ((y + 2**31) % 2**32 - 2**31).astype(np.int32)


def lsb_report(got, want):
    d = np.abs(got.astype(np.int32) - want.astype(np.int32))
    return int(d.max()) if d.size else 0, int((d > 0).sum()), int(d.size)


def nhwc(t):
    import torch
    return t.contiguous(memory_format=torch.channels_last)
