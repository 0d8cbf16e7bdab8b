"""Host-side mirror of the reference's VM op bodies for the quantized hot path.

Each function has the name, argument order and argument meaning of the corresponding entry of
the reference's op table (``runtime/chxvm_defs.py:431-434,451-469``) and does what the reference's
``XxxOp::RunImpl`` does around the arithmetic: validate, allocate a fresh output, call the kernel.
The arithmetic itself runs in ``libchxq.so`` through the C ABI; PyTorch supplies device memory and
the current stream only.  There is no fallback: without a CUDA device or without the built
library every op raises.

Array arguments are ``torch`` CUDA tensors, logically NCHW / row-major as in the reference.
Activation maps that are ``channels_last`` in memory take the NHWC kernels (tensor cores,
depthwise kernel) and yield ``channels_last`` outputs; plain contiguous NCHW maps take the general
CUDA-core kernels.  ``Scalar`` arguments are Python / numpy scalars; a zero point carries its dtype
as a numpy scalar (``np.uint8(3)``, ``np.int8(-1)``) the way ``StrictScalar`` does in the reference
(``runtime/strict_scalar.h:8-34``).
"""
import ctypes

import numpy as np
import torch

from . import _lib
from ._lib import (FLOAT16, FLOAT32, FLOAT64, INT8, NCHW, NHWC, PATH_AUTO, PATH_SIMT, PATH_TENSOR, ROUND_REF, ROUND_RNE, UINT8,  # noqa: F401
                   ChxqError, ConvGeom, QConvParams, check, lib)

_TORCH_Q = {torch.uint8: UINT8, torch.int8: INT8}
_TORCH_F = {torch.float16: FLOAT16, torch.float32: FLOAT32, torch.float64: FLOAT64}
_workspaces = {}
_zero_zp_cache = {}  # (data_ptr, numel, dtype) -> (version, all zero?) of weight zero-point tensors seen by QLinearConv
_retired_workspaces = []  # superseded scratch buffers: kept alive because captured CUDA graphs hold their raw addresses


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def _require_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise ChxqError(_lib.ERR_INVALID_ARGUMENT, "chxq ops run on CUDA tensors only (no CPU path exists)")


def _qcode(t, what):
    if t.dtype not in _TORCH_Q:
        raise ChxqError(_lib.ERR_INVALID_ARGUMENT, "%s must be uint8 or int8, got %s" % (what, t.dtype))
    return _TORCH_Q[t.dtype]


def workspace(nbytes, device):
    """Grow-only scratch buffer per device, 256-byte aligned (the op body owns scratch, as it owns outputs).

    A CUDA graph captured around these ops bakes the buffer's address into its kernel nodes.  When a later call needs more
    scratch a larger buffer is allocated, and the superseded one is never handed back to the allocator: a graph captured
    earlier keeps writing its im2col data and row sums into memory that still belongs to this module, not into a block the
    allocator may have given to a live tensor.  Growth is geometric (at least 1.5x), so the retained buffers sum to less than
    three times the largest request."""
    if nbytes == 0:
        return None
    key = (device.index if device.index is not None else torch.cuda.current_device())
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        if ws is not None:
            _retired_workspaces.append(ws)
            nbytes = max(int(nbytes), ws.numel() + ws.numel() // 2)
        ws = torch.empty(int(nbytes), dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


def _weight_zero_points_are_zero(wz):
    """Whether a weight zero-point tensor holds only zeros, learned by ONE device-to-host read per tensor (and again only after
    an in-place change, which bumps the tensor's version): weight zero points are graph constants, and symmetric int8 weights,
    the common case, have none.  The C ABI treats a zero point that is present as non-zero, because it never reads device
    memory back; this op body is the place that may know better, as the reference's VM knows its constants at Init."""
    if torch.cuda.is_current_stream_capturing():
        return False  # no synchronization during a capture: the general form
    key = (wz.data_ptr(), wz.numel(), wz.dtype)
    hit = _zero_zp_cache.get(key)
    if hit is not None and hit[0] == wz._version:
        return hit[1]
    zero = not bool(torch.any(wz != 0).item())
    if len(_zero_zp_cache) > 4096:
        _zero_zp_cache.clear()
    _zero_zp_cache[key] = (wz._version, zero)
    return zero


def _check_residual(op, residual, y_shape, channels_last):
    """A fused residual is read with the output's indexing: it must be a uint8 map of the output's shape and layout, and the
    tensor-core kernels read it 16 bytes at a time."""
    if residual is None:
        return
    if tuple(residual.shape) != tuple(y_shape) or residual.dtype != torch.uint8 or _is_channels_last(residual) != bool(channels_last):
        raise ChxqError(_lib.ERR_INVALID_ARGUMENT, "%s: residual must be a uint8 map with the output's shape and layout" % op)
    if channels_last and residual.data_ptr() % 16:
        raise ChxqError(_lib.ERR_INVALID_ARGUMENT, "%s: residual must start on a 16-byte boundary" % op)


def _zp_scalar(zp, default_dtype=np.uint8):
    """(value, chxq dtype code) of an OptionalScalar zero point."""
    if zp is None:
        return 0, (UINT8 if default_dtype == np.uint8 else INT8)
    if isinstance(zp, torch.Tensor):
        if zp.numel() != 1:
            raise ChxqError(_lib.ERR_INVALID_ARGUMENT, "a Scalar zero point must have one element")
        return int(zp.item()), _qcode(zp, "zero point")
    if isinstance(zp, (np.generic, np.ndarray)):
        dt = np.asarray(zp).dtype
        if dt == np.int8:
            return int(zp), INT8
        if dt == np.uint8:
            return int(zp), UINT8
        # runtime/ops/quantize.cc:19-25: the zero point's dtype is uint8 or int8, anything else CHECK-fails
        raise ChxqError(_lib.ERR_INVALID_ARGUMENT, "a zero point must be uint8 or int8, got %s" % dt)
    # plain Python ints carry no dtype: the reference's default is uint8 (runtime/ops/quantize.cc:50-51)
    return int(zp), (UINT8 if default_dtype == np.uint8 else INT8)


def _is_channels_last(t):
    return t.dim() == 4 and t.is_contiguous(memory_format=torch.channels_last) and not (t.is_contiguous() and t.shape[1] != 1)


def _is_device_scalar(v):
    return isinstance(v, torch.Tensor) and v.is_cuda and v.numel() == 1


def QuantizeLinear(x, y_scale, y_zero_point=None, round_mode=ROUND_REF):
    """runtime/chxvm_defs.py:451-453; body runtime/ops/quantize.cc:16-35,48-53.

    y_scale (and y_zero_point) may be one-element CUDA tensors: the scalars are then read by the kernel on the device, without
    the device-to-host read the reference's VM does per Scalar argument (runtime/chxvm_var.cc:70-76)."""
    _require_cuda(x)
    if x.dtype != torch.float32:
        raise ChxqError(_lib.ERR_INVALID_ARGUMENT, "QuantizeLinear: x must be float32, got %s" % x.dtype)
    if _is_device_scalar(y_scale):
        if y_scale.dtype != torch.float32:
            raise ChxqError(_lib.ERR_INVALID_ARGUMENT, "QuantizeLinear: a device y_scale must be float32")
        if y_zero_point is not None and not _is_device_scalar(y_zero_point):
            zp_h, code_h = _zp_scalar(y_zero_point)
            y_zero_point = torch.tensor([zp_h], dtype=torch.uint8 if code_h == UINT8 else torch.int8, device=x.device)
        code = UINT8 if y_zero_point is None else _qcode(y_zero_point, "QuantizeLinear: y_zero_point")
        if not (x.is_contiguous() or _is_channels_last(x)):
            x = x.contiguous()
        y = torch.empty_like(x, dtype=torch.uint8 if code == UINT8 else torch.int8)
        check(lib().chxq_quantize_linear_dev(_ptr(x), x.numel(), _ptr(y_scale), _ptr(y_zero_point), code, round_mode, _ptr(y), _stream()))
        return y
    zp, code = _zp_scalar(y_zero_point)
    if not (x.is_contiguous() or _is_channels_last(x)):
        x = x.contiguous()
    y = torch.empty_like(x, dtype=torch.uint8 if code == UINT8 else torch.int8)
    check(lib().chxq_quantize_linear(_ptr(x), x.numel(), float(y_scale), zp, code, round_mode, _ptr(y), _stream()))
    return y


def DequantizeLinear(x, x_scale, x_zero_point=None):
    """runtime/chxvm_defs.py:454-456; body runtime/ops/quantize.cc:37-44,55-60."""
    _require_cuda(x)
    code = _qcode(x, "DequantizeLinear: x")
    zp, _ = _zp_scalar(x_zero_point)
    if not (x.is_contiguous() or _is_channels_last(x)):
        x = x.contiguous()
    y = torch.empty_like(x, dtype=torch.float32)
    check(lib().chxq_dequantize_linear(_ptr(x), code, x.numel(), float(x_scale), zp, _ptr(y), _stream()))
    return y


def _zp_array(zp, like, what):
    """OptionalArray zero point: device tensor of the operand's dtype with ndim <= 1."""
    if zp is None:
        return None, 0
    if not isinstance(zp, torch.Tensor):
        zp = torch.as_tensor(np.asarray(zp), device=like.device)
    _require_cuda(zp)
    if zp.dim() > 1:
        raise ChxqError(_lib.ERR_INVALID_ARGUMENT, "%s must have at most one dimension" % what)  # runtime/ops/quantize.cc:105,109
    if zp.dtype != like.dtype:
        raise ChxqError(_lib.ERR_INVALID_ARGUMENT, "%s must have the operand's dtype %s, got %s" % (what, like.dtype, zp.dtype))
    zp = zp.contiguous().reshape(-1)
    return zp, zp.numel()


def MatMulInteger(a, b, a_zero_point=None, b_zero_point=None, path=PATH_AUTO):
    """runtime/chxvm_defs.py:462-465; body runtime/ops/quantize.cc:96-114."""
    _require_cuda(a, b)
    ca, cb = _qcode(a, "MatMulInteger: a"), _qcode(b, "MatMulInteger: b")
    if a.dim() < 2 or b.dim() < 2:
        raise ChxqError(_lib.ERR_INVALID_ARGUMENT, "MatMulInteger: operands need at least two dimensions")
    if a.dim() > 2 and a.shape[:-2] != b.shape[:-2]:
        raise ChxqError(_lib.ERR_UNSUPPORTED, "MatMulInteger: batched operands need equal leading dimensions")
    if a.dim() != b.dim():
        raise ChxqError(_lib.ERR_UNSUPPORTED, "MatMulInteger: operands need the same number of dimensions")
    M, K = a.shape[-2], a.shape[-1]
    K2, N = b.shape[-2], b.shape[-1]
    if K != K2:
        raise ChxqError(_lib.ERR_INVALID_ARGUMENT, "MatMulInteger: inner dimensions differ (%d vs %d)" % (K, K2))
    batch = 1
    for d in a.shape[:-2]:
        batch *= d
    a, b = a.contiguous(), b.contiguous()
    za, za_len = _zp_array(a_zero_point, a, "a_zero_point")
    zb, zb_len = _zp_array(b_zero_point, b, "b_zero_point")
    y = torch.empty(tuple(a.shape[:-2]) + (M, N), dtype=torch.int32, device=a.device)
    ws_bytes = lib().chxq_matmul_integer_workspace(batch, M, N, K) if path != PATH_SIMT else 0
    ws = workspace(ws_bytes, a.device)
    check(lib().chxq_matmul_integer(_ptr(a), ca, _ptr(b), cb, batch, M, N, K, _ptr(za), za_len, _ptr(zb), zb_len, _ptr(y), _ptr(ws), ws_bytes,
                                    path, _stream()))
    return y


def QLinearMatMul(a, a_scale, a_zero_point, b, b_scale, b_zero_point, y_scale, y_zero_point, round_mode=ROUND_REF, path=PATH_AUTO):
    """ONNX QLinearMatMul.  The reference has no VM op for it: compiler/simplifier.cc:675-694 rewrites the
    node into DequantizeLinear, DequantizeLinear, MatMul, QuantizeLinear with scalar parameters; this is
    that chain as one kernel."""
    _require_cuda(a, b)
    ca, cb = _qcode(a, "QLinearMatMul: a"), _qcode(b, "QLinearMatMul: b")
    if a.dim() != 2 or b.dim() != 2 or a.shape[1] != b.shape[0]:
        raise ChxqError(_lib.ERR_INVALID_ARGUMENT, "QLinearMatMul: expected [M,K] x [K,N]")
    M, K = a.shape
    N = b.shape[1]
    za, _ = _zp_scalar(a_zero_point)
    zb, _ = _zp_scalar(b_zero_point)
    zy, cy = _zp_scalar(y_zero_point)
    a, b = a.contiguous(), b.contiguous()
    y = torch.empty((M, N), dtype=torch.uint8 if cy == UINT8 else torch.int8, device=a.device)
    ws_bytes = lib().chxq_matmul_integer_workspace(1, M, N, K) if path != PATH_SIMT else 0
    ws = workspace(ws_bytes, a.device)
    check(lib().chxq_qlinear_matmul(_ptr(a), ca, float(a_scale), za, _ptr(b), cb, float(b_scale), zb, float(y_scale), zy, cy, M, N, K, round_mode,
                                    _ptr(y), _ptr(ws), ws_bytes, path, _stream()))
    return y


def conv_geometry(x, w, strides, pads, group, auto_pad):
    """Geometry of a convolution the way the reference resolves it (runtime/chainerx_util.cc:180-200,276-311)."""
    return conv_geometry_from_shapes(tuple(x.shape), _qcode(x, "x"), tuple(w.shape), _qcode(w, "w"), strides, pads, group, auto_pad)


def conv_geometry_from_shapes(x_shape, x_code, w_shape, w_code, strides, pads, group, auto_pad):
    if len(x_shape) != 4 or len(w_shape) != 4:
        raise ChxqError(_lib.ERR_UNSUPPORTED, "convolutions over 2 spatial dimensions only")
    N, C, H, W = x_shape
    M, Cg, KH, KW = w_shape
    g = ConvGeom()
    s = (ctypes.c_int64 * 2)(*(list(strides) + [1, 1])[:2])
    p = (ctypes.c_int64 * 2)(*(list(pads) + [0, 0])[:2])
    check(lib().chxq_conv_resolve_geometry(N, C, H, W, M, Cg, KH, KW, s, len(strides), p, len(pads), group, (auto_pad or "").encode(),
                                           ctypes.byref(g)))
    g.x_dtype = x_code
    g.w_dtype = w_code
    return g


def _conv_io(x, g, out_dtype):
    """Pick layouts: channels_last maps use the NHWC kernels."""
    if _is_channels_last(x):
        g.x_layout = g.y_layout = NHWC
        y = torch.empty((g.N, g.M, g.Ho, g.Wo), dtype=out_dtype, device=x.device, memory_format=torch.channels_last)
    else:
        x = x.contiguous()
        g.x_layout = g.y_layout = NCHW
        y = torch.empty((g.N, g.M, g.Ho, g.Wo), dtype=out_dtype, device=x.device)
    return x, y


def ConvInteger(x, w, x_zero_point=None, w_zero_point=None, strides=(), pads=(), group=1, auto_pad="", path=PATH_AUTO):
    """runtime/chxvm_defs.py:466-469; body runtime/ops/quantize.cc:116-146.

    x_zero_point may be a one-element CUDA tensor of x's dtype (a zero point computed on the device): it is then read by the
    kernel, not by the host (general CUDA-core kernel)."""
    _require_cuda(x, w)
    g = conv_geometry(x, w, strides, pads, group, auto_pad)
    x, y = _conv_io(x, g, torch.int32)
    w = w.contiguous()
    if _is_device_scalar(x_zero_point):
        if x_zero_point.dtype != x.dtype:
            raise ChxqError(_lib.ERR_INVALID_ARGUMENT, "ConvInteger: a device x_zero_point must have x's dtype")
        zw, zw_len = _zp_array(w_zero_point, w, "w_zero_point")
        check(lib().chxq_conv_integer_dev(_ptr(x), _ptr(w), ctypes.byref(g), _ptr(x_zero_point), _ptr(zw), zw_len, _ptr(y), _stream()))
        return y
    zx, _ = _zp_scalar(x_zero_point)
    zw, zw_len = _zp_array(w_zero_point, w, "w_zero_point")
    ws_bytes = lib().chxq_conv_workspace(ctypes.byref(g)) if path != PATH_SIMT else 0
    ws = workspace(ws_bytes, x.device)
    check(lib().chxq_conv_integer(_ptr(x), _ptr(w), ctypes.byref(g), int(x_zero_point is not None), zx, _ptr(zw), zw_len, _ptr(y), _ptr(ws),
                                  ws_bytes, path, _stream()))
    return y


def _qconv_params(x, w, x_scale, x_zero_point, w_scale, w_zero_point, y_scale, y_zero_point, b, round_mode, clamp_hi_q, residual, res_scale,
                  res_zero_point, res_relu, out_scale, out_zero_point, keep, fold_scales=False):
    p = QConvParams()
    p.fold_scales = int(bool(fold_scales))
    zx, _ = _zp_scalar(x_zero_point)
    zy, cy = _zp_scalar(y_zero_point)
    if not isinstance(w_scale, torch.Tensor):
        w_scale = torch.as_tensor(np.asarray(w_scale, np.float32), device=x.device)
    if not isinstance(w_zero_point, torch.Tensor):
        w_zero_point = torch.as_tensor(np.asarray(w_zero_point), device=x.device)
    _require_cuda(w_scale, w_zero_point)
    # runtime/ops/quantize.cc:76-77: scale and zero point agree in size and rank; rank is 0 or 1.
    if w_scale.numel() != w_zero_point.numel() or w_scale.dim() != w_zero_point.dim() or w_scale.dim() > 1:
        raise ChxqError(_lib.ERR_INVALID_ARGUMENT, "QLinearConv: w_scale and w_zero_point must both be 0-d or both be 1-d of equal length")
    if w_scale.dim() == 1 and w_scale.shape[0] != w.shape[0]:
        raise ChxqError(_lib.ERR_INVALID_ARGUMENT, "QLinearConv: per-channel w_scale needs one entry per output channel")  # :79
    if w_scale.dtype != torch.float32 or w_zero_point.dtype != w.dtype:
        raise ChxqError(_lib.ERR_INVALID_ARGUMENT, "QLinearConv: w_scale must be float32 and w_zero_point must have w's dtype")
    w_scale, w_zero_point = w_scale.contiguous(), w_zero_point.contiguous()
    keep.extend([w_scale, w_zero_point])
    p.x_scale, p.x_zero_point = float(x_scale), zx
    p.w_scale, p.w_zero_point, p.w_params_len = w_scale.data_ptr(), w_zero_point.data_ptr(), w_scale.numel()
    if _weight_zero_points_are_zero(w_zero_point):
        p.w_zero_point = None  # symmetric weights: the kernels skip the weight zero-point term (and its input sums)
    p.y_scale, p.y_zero_point, p.y_dtype = float(y_scale), zy, cy
    if b is not None:
        _require_cuda(b)
        if b.dtype != torch.int32 or b.numel() != w.shape[0]:
            raise ChxqError(_lib.ERR_INVALID_ARGUMENT, "QLinearConv: bias must be int32 with one entry per output channel")
        b = b.contiguous()
        keep.append(b)
        p.bias = b.data_ptr()
    p.round_mode = round_mode
    p.clamp_hi_q = -1 if clamp_hi_q is None else int(clamp_hi_q)
    if residual is not None:
        _require_cuda(residual)
        p.residual = residual.data_ptr()
        p.res_scale, p.res_zero_point, p.res_relu = float(res_scale), int(res_zero_point), int(bool(res_relu))
        p.out_scale, p.out_zero_point = float(out_scale), int(out_zero_point)
    return p, cy


def QLinearConv(x, x_scale, x_zero_point, w, w_scale, w_zero_point, y_scale, y_zero_point, b=None, strides=(), pads=(), group=1,
                auto_pad="", round_mode=ROUND_REF, path=PATH_AUTO, clamp_hi_q=None, residual=None, res_scale=1.0, res_zero_point=0,
                res_relu=True, out_scale=1.0, out_zero_point=0, fold_scales=False):
    """runtime/chxvm_defs.py:457-461; body runtime/ops/quantize.cc:62-94.

    The keyword arguments after ``auto_pad`` have no counterpart in the reference: ``clamp_hi_q`` folds a
    ReLU6 into the output range, ``residual`` (+ scales) fuses the DequantizeLinear, DequantizeLinear, Add,
    Relu, QuantizeLinear nodes that follow the convolution of a residual block into the epilogue,
    ``fold_scales`` requantizes with one multiplier per channel instead of a multiply and a divide.
    """
    _require_cuda(x, w)
    g = conv_geometry(x, w, strides, pads, group, auto_pad)
    keep = []
    p, cy = _qconv_params(x, w, x_scale, x_zero_point, w_scale, w_zero_point, y_scale, y_zero_point, b, round_mode, clamp_hi_q, residual,
                          res_scale, res_zero_point, res_relu, out_scale, out_zero_point, keep, fold_scales)
    x, y = _conv_io(x, g, torch.uint8 if cy == UINT8 else torch.int8)
    if residual is not None:
        if residual.shape != y.shape or residual.dtype != torch.uint8 or _is_channels_last(residual) != (g.y_layout == NHWC):
            raise ChxqError(_lib.ERR_INVALID_ARGUMENT, "QLinearConv: residual must be a uint8 map with the output's shape and layout")
    w = w.contiguous()
    ws_bytes = lib().chxq_conv_workspace(ctypes.byref(g)) if path != PATH_SIMT else 0
    ws = workspace(ws_bytes, x.device)
    check(lib().chxq_qlinear_conv(_ptr(x), _ptr(w), ctypes.byref(g), ctypes.byref(p), _ptr(y), _ptr(ws), ws_bytes, path, _stream()))
    return y


class PackedConv:
    """Constant weights of one QLinearConv / ConvInteger, packed once for the tensor-core path."""

    def __init__(self, w, w_zero_point, x_shape, strides=(), pads=(), group=1, auto_pad="", x_dtype=torch.uint8, x_layout=NHWC):
        _require_cuda(w)
        self.w = w.contiguous()
        self.g = conv_geometry_from_shapes(tuple(x_shape), _TORCH_Q[x_dtype], tuple(self.w.shape), _qcode(self.w, "w"), strides, pads, group,
                                           auto_pad)
        self.g.x_layout, self.g.y_layout = x_layout, NHWC
        self.zw, self.zw_len = _zp_array(w_zero_point, self.w, "w_zero_point")
        nbytes = lib().chxq_conv_prepack_bytes(ctypes.byref(self.g))
        self.flags = 0
        self.blob = None
        if nbytes:
            self.blob = torch.empty(int(nbytes), dtype=torch.uint8, device=w.device)
            flags = ctypes.c_int32(0)
            check(lib().chxq_conv_prepack(_ptr(self.w), ctypes.byref(self.g), _ptr(self.zw), self.zw_len, _ptr(self.blob), nbytes,
                                          ctypes.byref(flags), _stream()))
            self.flags = flags.value

    @property
    def eligible(self):
        return bool(self.flags & 1)


def QLinearConvPacked(x, packed, x_scale, x_zero_point, w_scale, w_zero_point, y_scale, y_zero_point, b=None, round_mode=ROUND_REF,
                      clamp_hi_q=None, residual=None, res_scale=1.0, res_zero_point=0, res_relu=True, out_scale=1.0, out_zero_point=0,
                      out=None, fold_scales=False):
    """QLinearConv with weights packed by PackedConv; x must be a channels_last map of the packed geometry."""
    _require_cuda(x)
    g = packed.g
    layout_ok = _is_channels_last(x) if g.x_layout == NHWC else x.is_contiguous()
    if tuple(x.shape) != (g.N, g.C, g.H, g.W) or not layout_ok:
        raise ChxqError(_lib.ERR_INVALID_ARGUMENT, "QLinearConvPacked: x does not match the packed geometry / layout")
    keep = []
    _check_residual("QLinearConvPacked", residual, (g.N, g.M, g.Ho, g.Wo), True)
    p, cy = _qconv_params(x, packed.w, x_scale, x_zero_point, w_scale, w_zero_point, y_scale, y_zero_point, b, round_mode, clamp_hi_q, residual,
                          res_scale, res_zero_point, res_relu, out_scale, out_zero_point, keep, fold_scales)
    if out is not None and (tuple(out.shape) != (g.N, g.M, g.Ho, g.Wo) or not _is_channels_last(out) or out.dtype != (torch.uint8 if cy == UINT8 else torch.int8)):
        raise ChxqError(_lib.ERR_INVALID_ARGUMENT, "QLinearConvPacked: out must be a channels_last map of the output's shape and dtype")
    y = out if out is not None else torch.empty((g.N, g.M, g.Ho, g.Wo), dtype=torch.uint8 if cy == UINT8 else torch.int8, device=x.device,
                                                 memory_format=torch.channels_last)
    if not packed.eligible:
        raise ChxqError(_lib.ERR_UNSUPPORTED, "QLinearConvPacked: this geometry is not eligible for the packed tensor-core path")
    ws_bytes = lib().chxq_conv_packed_workspace(ctypes.byref(g), p.x_zero_point, packed.flags)
    ws = workspace(ws_bytes, x.device)
    check(lib().chxq_qlinear_conv_packed(_ptr(x), _ptr(packed.blob), ctypes.byref(g), ctypes.byref(p), packed.flags, _ptr(y), _ptr(ws),
                                         ws_bytes, _stream()))
    return y


def QLinearConvChainPacked(x, packed1, conv1, packed2, conv2, out=None):
    """Two QLinearConvPacked calls as one kernel: `packed1` / `conv1` describe a convolution with 64, 128 or 256 output channels,
    `packed2` / `conv2` the 1x1, stride-1 convolution that is its only reader.  conv1 and conv2 are dicts of the keyword arguments
    QLinearConvPacked takes after `packed` (x_scale, x_zero_point, w_scale, w_zero_point, y_scale, y_zero_point, b, clamp_hi_q,
    fold_scales, and for conv2 the residual tail's residual, res_scale, res_zero_point, res_relu, out_scale, out_zero_point).  The
    map between the two convolutions is never written.  Bit-identical to the two calls in sequence; raises
    ChxqError(ERR_UNSUPPORTED) when the pair has no fused kernel (the caller then makes the two calls)."""
    _require_cuda(x)
    g1, g2 = packed1.g, packed2.g
    if tuple(x.shape) != (g1.N, g1.C, g1.H, g1.W) or not _is_channels_last(x):
        raise ChxqError(_lib.ERR_INVALID_ARGUMENT, "QLinearConvChainPacked: x does not match the packed geometry / layout")
    if not (packed1.eligible and packed2.eligible):
        raise ChxqError(_lib.ERR_UNSUPPORTED, "QLinearConvChainPacked: a geometry is not eligible for the packed tensor-core path")
    keep = []
    c1, c2 = dict(conv1), dict(conv2)
    if c1.get("residual") is not None:
        raise ChxqError(_lib.ERR_INVALID_ARGUMENT, "QLinearConvChainPacked: only the second convolution may carry a residual tail")
    residual = c2.get("residual")
    _check_residual("QLinearConvChainPacked", residual, (g2.N, g2.M, g2.Ho, g2.Wo), True)

    def params(pk, c, res):
        return _qconv_params(x, pk.w, c["x_scale"], c["x_zero_point"], c["w_scale"], c.get("w_zero_point"), c["y_scale"], c["y_zero_point"], c.get("b"),
                             c.get("round_mode", ROUND_REF), c.get("clamp_hi_q"), res, c.get("res_scale", 1.0), c.get("res_zero_point", 0),
                             c.get("res_relu", True), c.get("out_scale", 1.0), c.get("out_zero_point", 0), keep, c.get("fold_scales", False))

    p1, cy1 = params(packed1, c1, None)
    p2, cy2 = params(packed2, c2, residual)
    if cy1 != UINT8 or cy2 != UINT8:
        raise ChxqError(_lib.ERR_UNSUPPORTED, "QLinearConvChainPacked: both outputs must be uint8")
    shape = (g2.N, g2.M, g2.Ho, g2.Wo)
    if out is not None and (tuple(out.shape) != shape or not _is_channels_last(out) or out.dtype != torch.uint8):
        raise ChxqError(_lib.ERR_INVALID_ARGUMENT, "QLinearConvChainPacked: out must be a channels_last uint8 map of the output's shape")
    y = out if out is not None else torch.empty(shape, dtype=torch.uint8, device=x.device, memory_format=torch.channels_last)
    check(lib().chxq_qlinear_conv_chain_packed(_ptr(x), _ptr(packed1.blob), ctypes.byref(g1), ctypes.byref(p1), packed1.flags, _ptr(packed2.blob),
                                               ctypes.byref(g2), ctypes.byref(p2), packed2.flags, _ptr(y), _stream()))
    return y


def QLinearConvMaxPoolPacked(x, packed, x_scale, x_zero_point, w_scale, w_zero_point, y_scale, y_zero_point, b=None, pool_kernel=3, pool_stride=2,
                             pool_pad=0, cover_all=False, round_mode=ROUND_REF, quant_round_mode=ROUND_REF, clamp_hi_q=None, out=None,
                             fold_scales=False):
    """QLinearConvPacked followed by MaxPoolU8(pool_kernel, pool_stride, pool_pad, cover_all) as one kernel; bit-identical to the
    two ops.  x: the uint8 map, or the fp32 tensor in front of a QuantizeLinear(x_scale, x_zero_point) (as
    QuantizeLinearConvPacked).  Only kernel 3 / stride 2 / pad 0 pooling behind a convolution whose packed K tile is 64 bytes
    (network stems); raises ChxqError(ERR_UNSUPPORTED) otherwise."""
    _require_cuda(x)
    g = packed.g
    layout_ok = _is_channels_last(x) if g.x_layout == NHWC else x.is_contiguous()
    if tuple(x.shape) != (g.N, g.C, g.H, g.W) or not layout_ok or x.dtype not in (torch.float32, torch.uint8):
        raise ChxqError(_lib.ERR_INVALID_ARGUMENT, "QLinearConvMaxPoolPacked: x does not match the packed geometry / layout")
    if not packed.eligible:
        raise ChxqError(_lib.ERR_UNSUPPORTED, "QLinearConvMaxPoolPacked: this geometry is not eligible for the packed tensor-core path")
    keep = []
    p, cy = _qconv_params(x, packed.w, x_scale, x_zero_point, w_scale, w_zero_point, y_scale, y_zero_point, b, round_mode, clamp_hi_q, None, 1.0, 0,
                          True, 1.0, 0, keep, fold_scales)
    if cy != UINT8:
        raise ChxqError(_lib.ERR_UNSUPPORTED, "QLinearConvMaxPoolPacked: the output must be uint8")
    extra = pool_stride - 1 if cover_all else 0
    Hp, Wp = (g.Ho + 2 * pool_pad - pool_kernel + extra) // pool_stride + 1, (g.Wo + 2 * pool_pad - pool_kernel + extra) // pool_stride + 1
    y = out if out is not None else torch.empty((g.N, g.M, Hp, Wp), dtype=torch.uint8, device=x.device, memory_format=torch.channels_last)
    ws_bytes = lib().chxq_conv_packed_workspace(ctypes.byref(g), p.x_zero_point, packed.flags)
    ws = workspace(ws_bytes, x.device)
    check(lib().chxq_qlinear_conv_maxpool_packed(_ptr(x), int(x.dtype == torch.float32), quant_round_mode, _ptr(packed.blob), ctypes.byref(g),
                                                 ctypes.byref(p), packed.flags, pool_kernel, pool_stride, pool_pad, int(bool(cover_all)), _ptr(y), _ptr(ws),
                                                 ws_bytes, _stream()))
    return y


def ConvIntegerPacked(x, packed, x_zero_point=None):
    """ConvInteger with weights packed by PackedConv; x must be a channels_last map of the packed geometry."""
    _require_cuda(x)
    g = packed.g
    layout_ok = _is_channels_last(x) if g.x_layout == NHWC else x.is_contiguous()
    if tuple(x.shape) != (g.N, g.C, g.H, g.W) or not layout_ok:
        raise ChxqError(_lib.ERR_INVALID_ARGUMENT, "ConvIntegerPacked: x does not match the packed geometry / layout")
    if not packed.eligible:
        raise ChxqError(_lib.ERR_UNSUPPORTED, "ConvIntegerPacked: this geometry is not eligible for the packed tensor-core path")
    zx, _ = _zp_scalar(x_zero_point)
    y = torch.empty((g.N, g.M, g.Ho, g.Wo), dtype=torch.int32, device=x.device, memory_format=torch.channels_last)
    ws_bytes = lib().chxq_conv_packed_workspace(ctypes.byref(g), zx, packed.flags)
    ws = workspace(ws_bytes, x.device)
    check(lib().chxq_conv_integer_packed(_ptr(x), _ptr(packed.blob), ctypes.byref(g), int(x_zero_point is not None), zx, packed.flags, _ptr(y),
                                         _ptr(ws), ws_bytes, _stream()))
    return y


def QuantizeLinearConvPacked(x, packed, x_scale, x_zero_point, w_scale, w_zero_point, y_scale, y_zero_point, b=None, round_mode=ROUND_REF,
                             quant_round_mode=ROUND_REF, clamp_hi_q=None, out=None, fold_scales=False):
    """QuantizeLinear(x, x_scale, x_zero_point) fused into the packed QLinearConv that consumes it: x is the fp32 tensor (same
    layout as the packed geometry expects of the quantized map).  Only for stride-2 convolutions over at most 4 channels
    (network stems); bit-identical to the two ops run one after the other."""
    _require_cuda(x)
    g = packed.g
    layout_ok = _is_channels_last(x) if g.x_layout == NHWC else x.is_contiguous()
    if tuple(x.shape) != (g.N, g.C, g.H, g.W) or not layout_ok or x.dtype != torch.float32:
        raise ChxqError(_lib.ERR_INVALID_ARGUMENT, "QuantizeLinearConvPacked: x must be the fp32 tensor of the packed geometry / layout")
    keep = []
    xq_like = torch.empty(0, dtype=torch.uint8, device=x.device)
    p, cy = _qconv_params(xq_like, packed.w, x_scale, x_zero_point, w_scale, w_zero_point, y_scale, y_zero_point, b, round_mode, clamp_hi_q, None, 1.0, 0,
                          True, 1.0, 0, keep, fold_scales)
    y = out if out is not None else torch.empty((g.N, g.M, g.Ho, g.Wo), dtype=torch.uint8 if cy == UINT8 else torch.int8, device=x.device,
                                                 memory_format=torch.channels_last)
    if not packed.eligible:
        raise ChxqError(_lib.ERR_UNSUPPORTED, "QuantizeLinearConvPacked: this geometry is not eligible for the packed tensor-core path")
    ws_bytes = lib().chxq_conv_packed_workspace(ctypes.byref(g), p.x_zero_point, packed.flags)
    ws = workspace(ws_bytes, x.device)
    check(lib().chxq_quantize_qlinear_conv_packed(_ptr(x), quant_round_mode, _ptr(packed.blob), ctypes.byref(g), ctypes.byref(p), packed.flags, _ptr(y),
                                                  _ptr(ws), ws_bytes, _stream()))
    return y


def ElementWiseNvrtc(inputs, num_outputs, code, fusion_id):
    """runtime/chxvm_defs.py:431-434; body runtime/ops/nvrtc.cc:90-161: broadcast every input to the common
    shape, make it contiguous, allocate num_outputs arrays of that shape and dtype, run the generated kernel."""
    if not inputs:
        raise ChxqError(_lib.ERR_INVALID_ARGUMENT, "ElementWiseNvrtc: no inputs")
    _require_cuda(*inputs)
    dtype = inputs[0].dtype
    if dtype not in _TORCH_F:
        raise ChxqError(_lib.ERR_INVALID_ARGUMENT, "ElementWiseNvrtc: dtype %s is not a float type" % dtype)
    for t in inputs:
        if t.dtype != dtype:
            raise ChxqError(_lib.ERR_INVALID_ARGUMENT, "ElementWiseNvrtc: all inputs must share one dtype")  # runtime/ops/nvrtc.cc:102
    shape = torch.broadcast_shapes(*[tuple(t.shape) for t in inputs])
    ins = [(t if tuple(t.shape) == tuple(shape) else t.broadcast_to(shape)).contiguous() for t in inputs]
    outs = [torch.empty(shape, dtype=dtype, device=ins[0].device) for _ in range(num_outputs)]
    n = ins[0].numel()
    in_ptrs = (ctypes.c_void_p * len(ins))(*[t.data_ptr() for t in ins])
    out_ptrs = (ctypes.c_void_p * len(outs))(*[t.data_ptr() for t in outs])
    check(lib().chxq_eltwise_run(code.encode() if isinstance(code, str) else code, fusion_id, in_ptrs, len(ins), out_ptrs, len(outs), n,
                                 _TORCH_F[dtype], _stream()))
    return outs


# ---- glue ops of a quantized CNN graph -------------------------------------------------------------

def MaxPoolU8(x, kernel, stride, pad=0, cover_all=False):
    """MaxPool (runtime/ops/pooling.cc:47-60) on a uint8 channels_last map."""
    _require_cuda(x)
    if x.dtype != torch.uint8 or not _is_channels_last(x):
        raise ChxqError(_lib.ERR_INVALID_ARGUMENT, "MaxPoolU8: expected a uint8 channels_last map")
    N, C, H, W = x.shape

    def osz(i):
        return (i + 2 * pad - kernel + (stride - 1 if cover_all else 0)) // stride + 1

    Ho, Wo = osz(H), osz(W)
    y = torch.empty((N, C, Ho, Wo), dtype=torch.uint8, device=x.device, memory_format=torch.channels_last)
    check(lib().chxq_maxpool_u8_nhwc(_ptr(x), N, H, W, C, kernel, stride, pad, Ho, Wo, _ptr(y), _stream()))
    return y


def GlobalAveragePoolDequant(x, x_scale, x_zero_point=0):
    """DequantizeLinear followed by a global AveragePool (runtime/ops/pooling.cc:62-75) of a uint8 channels_last map -> [N, C] fp32."""
    _require_cuda(x)
    if x.dtype != torch.uint8 or not _is_channels_last(x):
        raise ChxqError(_lib.ERR_INVALID_ARGUMENT, "GlobalAveragePoolDequant: expected a uint8 channels_last map")
    N, C, H, W = x.shape
    y = torch.empty((N, C), dtype=torch.float32, device=x.device)
    check(lib().chxq_global_avgpool_dq_nhwc(_ptr(x), N, H * W, C, float(x_scale), int(x_zero_point), _ptr(y), _stream()))
    return y


def Linear(x, w, b=None):
    """runtime/ops/connection.cc:12-15 (fp32): y = x w^T + b."""
    _require_cuda(x, w, b)
    x, w = x.contiguous(), w.contiguous()
    y = torch.empty((x.shape[0], w.shape[0]), dtype=torch.float32, device=x.device)
    check(lib().chxq_linear_f32(_ptr(x), _ptr(w), _ptr(b.contiguous()) if b is not None else None, x.shape[0], x.shape[1], w.shape[0], _ptr(y),
                                _stream()))
    return y


def QAddU8(a, a_scale, a_zero_point, b, b_scale, b_zero_point, y_scale, y_zero_point=0, relu=True, round_mode=ROUND_REF):
    """DequantizeLinear(a), DequantizeLinear(b), Add, Relu, QuantizeLinear in one pass (same memory layout in and out)."""
    _require_cuda(a, b)
    if a.shape != b.shape or a.dtype != torch.uint8 or b.dtype != torch.uint8 or a.stride() != b.stride():
        raise ChxqError(_lib.ERR_INVALID_ARGUMENT, "QAddU8: operands must be uint8 maps of equal shape and layout")
    y = torch.empty_like(a)
    check(lib().chxq_qadd_u8(_ptr(a), float(a_scale), int(a_zero_point), _ptr(b), float(b_scale), int(b_zero_point), a.numel(), float(y_scale),
                             int(y_zero_point), int(bool(relu)), round_mode, _ptr(y), _stream()))
    return y


def to_channels_last(x):
    """NCHW -> NHWC copy of a 1- or 4-byte map through the library's transpose kernel."""
    _require_cuda(x)
    if _is_channels_last(x):
        return x
    x = x.contiguous()
    N, C, H, W = x.shape
    y = torch.empty_like(x, memory_format=torch.channels_last)
    check(lib().chxq_nchw_to_nhwc(_ptr(x), x.element_size(), N, C, H, W, 0, _ptr(y), _stream()))
    return y


def to_contiguous_nchw(x):
    _require_cuda(x)
    if x.is_contiguous():
        return x
    if not _is_channels_last(x):
        return x.contiguous()
    N, C, H, W = x.shape
    y = torch.empty((N, C, H, W), dtype=x.dtype, device=x.device)
    check(lib().chxq_nhwc_to_nchw(_ptr(x), x.element_size(), N, C, H, W, 0, _ptr(y), _stream()))
    return y


def PrepareWeights(w, bn=None, conv_bias=None, epsilon=1e-5, to_int8=True, per_channel=True, return_folded=False):
    """Model preparation on the device: the Conv + BatchNormalization merge (compiler/merge.cc:142-215) followed by the weight
    quantizer (compiler/quantize.cc:70-129).  w: fp32 [M, ...]; bn: None or (scale, bias, mean, var), fp32 [M] each.
    Returns (q, scales, zero_points, folded_bias or None[, folded_w]); zero_points are int32."""
    _require_cuda(w)
    if w.dtype != torch.float32:
        raise ChxqError(_lib.ERR_INVALID_ARGUMENT, "PrepareWeights: w must be float32")
    w = w.contiguous()
    M = w.shape[0]
    inner = w.numel() // M
    vec = lambda t: None if t is None else t.to(device=w.device, dtype=torch.float32).contiguous()  # noqa: E731
    gamma, beta, mean, var = (vec(t) for t in bn) if bn is not None else (None, None, None, None)
    conv_bias = vec(conv_bias)
    for t in (gamma, beta, mean, var, conv_bias):
        if t is not None and t.numel() != M:
            raise ChxqError(_lib.ERR_INVALID_ARGUMENT, "PrepareWeights: per-channel vectors need one entry per output channel")
    n = M if per_channel else 1
    q = torch.empty(w.shape, dtype=torch.int8 if to_int8 else torch.uint8, device=w.device)
    scales = torch.empty(n, dtype=torch.float32, device=w.device)
    zps = torch.empty(n, dtype=torch.int32, device=w.device)
    folded_bias = torch.empty(M, dtype=torch.float32, device=w.device) if bn is not None else None
    folded_w = torch.empty_like(w) if return_folded else None
    ws_bytes = lib().chxq_prepare_weights_workspace(M)
    ws = workspace(ws_bytes, w.device)
    p = lambda t: None if t is None else _ptr(t)  # noqa: E731
    check(lib().chxq_prepare_weights(_ptr(w), M, inner, p(gamma), p(beta), p(mean), p(var), float(epsilon), p(conv_bias), int(to_int8), int(per_channel),
                                     _ptr(q), _ptr(scales), _ptr(zps), p(folded_w), p(folded_bias), _ptr(ws), ws_bytes, _stream()))
    return (q, scales, zps, folded_bias, folded_w) if return_folded else (q, scales, zps, folded_bias)


def DynamicQuantParamsU8(rmin, rmax):
    """scale, zero point of the dynamic uint8 quantization of an activation from its ReduceMin / ReduceMax, as the Sub, Div,
    Floor, Cast nodes of compiler/quantize.cc:196-207 compute them, on the device: returns (float32[1], uint8[1]) CUDA tensors."""
    _require_cuda(rmin, rmax)
    if rmin.dtype != torch.float32 or rmax.dtype != torch.float32 or rmin.numel() != 1 or rmax.numel() != 1:
        raise ChxqError(_lib.ERR_INVALID_ARGUMENT, "DynamicQuantParamsU8: rmin and rmax must be one-element float32 tensors")
    scale = torch.empty(1, dtype=torch.float32, device=rmin.device)
    zp = torch.empty(1, dtype=torch.uint8, device=rmin.device)
    check(lib().chxq_dynamic_quant_params_u8(_ptr(rmin), _ptr(rmax), _ptr(scale), _ptr(zp), _stream()))
    return scale, zp


def MinMax(x):
    """ReduceMin and ReduceMax of an fp32 tensor in one pass -> device tensor [min, max]."""
    _require_cuda(x)
    x = x.contiguous()
    out = torch.empty(2, dtype=torch.float32, device=x.device)
    check(lib().chxq_minmax_f32(_ptr(x), x.numel(), _ptr(out), _stream()))
    return out


def device_status():
    """Raises if a bounded device-side wait expired since the last call (synchronises the stream)."""
    check(lib().chxq_device_status(_stream()))
