"""ctypes front-end of the CPU oracle (``chxq_oracle.c``).

TEST INFRASTRUCTURE ONLY: imported by the test suite, the smoke check and the bench's
CPU-baseline leg, never by the product package.  PARITY UNPINNED: the reference holds no
golden vectors for these ops in its checkout (its ONNX node-test data directory is an empty
submodule), so this is a by-specification restatement; see the header of ``chxq_oracle.c``.

Every function takes and returns numpy arrays in the reference's layouts (NCHW activations,
OIHW weights, row-major matrices).
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libchxq_oracle.so")
_lib = None

ROUND_REF = 0  # (t + 0.5f) then truncation, runtime/ops/quantize.cc:33-34
ROUND_RNE = 1  # round-half-to-even, saturating (ONNX)

BIAS_NONE, BIAS_ONNX, BIAS_RAW = 0, 1, 2

EW_OPS = {"Identity": 0, "Tanh": 1, "Exp": 2, "Sigmoid": 3, "Add": 4, "Sub": 5, "Mul": 6, "Div": 7, "Constant": 8}


class _EwNode(ctypes.Structure):
    _fields_ = [("op", ctypes.c_int32), ("in0", ctypes.c_int32), ("in1", ctypes.c_int32), ("cval", ctypes.c_float)]


def build(force=False):
    """Compile the oracle with the Makefile beside it (gcc + OpenMP)."""
    src = os.path.join(_HERE, "chxq_oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-s", "-B", "libchxq_oracle.so"])
    return _LIB_PATH


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(_LIB_PATH)
        _lib.orc_quantize_mode_diff.restype = ctypes.c_int64
        _lib.orc_num_threads.restype = ctypes.c_int
    return _lib


def num_threads():
    return lib().orc_num_threads()


def set_num_threads(n):
    lib().orc_set_num_threads(ctypes.c_int(int(n)))


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def _c(a, dtype=None):
    return np.ascontiguousarray(a, dtype=dtype)


def _signed(a):
    if a.dtype == np.int8:
        return 1
    if a.dtype == np.uint8:
        return 0
    raise TypeError("expected int8 or uint8, got %s" % a.dtype)


def _i64(v):
    return ctypes.c_int64(int(v))


def _f(v):
    return ctypes.c_float(float(np.float32(v)))


def quantize_linear(x, y_scale, y_zero_point=0, out_dtype=np.uint8, round_mode=ROUND_REF):
    x = _c(x, np.float32)
    out_dtype = np.dtype(out_dtype)
    y = np.empty(x.shape, out_dtype)
    lib().orc_quantize_linear(_p(x), _i64(x.size), _f(y_scale), ctypes.c_int(int(y_zero_point)),
                              ctypes.c_int(int(out_dtype == np.int8)), ctypes.c_int(round_mode), _p(y))
    return y


def quantize_mode_diff(x, y_scale, y_zero_point=0, out_dtype=np.uint8):
    x = _c(x, np.float32)
    return int(lib().orc_quantize_mode_diff(_p(x), _i64(x.size), _f(y_scale), ctypes.c_int(int(y_zero_point)),
                                            ctypes.c_int(int(np.dtype(out_dtype) == np.int8))))


def dequantize_linear(x, x_scale, x_zero_point=0):
    x = _c(x)
    y = np.empty(x.shape, np.float32)
    lib().orc_dequantize_linear(_p(x), ctypes.c_int(_signed(x)), _i64(x.size), _f(x_scale), ctypes.c_int(int(x_zero_point)), _p(y))
    return y


def _zp_arr(zp):
    if zp is None:
        return np.zeros(0, np.int32)
    return _c(np.asarray(zp).reshape(-1), np.int32)


def matmul_integer(a, b, a_zero_point=None, b_zero_point=None):
    a, b = _c(a), _c(b)
    if a.ndim == 2:
        batch, (M, K), N = 1, a.shape, b.shape[-1]
        out_shape = (M, N)
    else:
        assert a.shape[:-2] == b.shape[:-2], "oracle covers equal leading dims only"
        batch = int(np.prod(a.shape[:-2]))
        M, K, N = a.shape[-2], a.shape[-1], b.shape[-1]
        out_shape = a.shape[:-2] + (M, N)
    assert b.shape[-2] == K
    za, zb = _zp_arr(a_zero_point), _zp_arr(b_zero_point)
    assert za.size in (0, 1, K) and zb.size in (0, 1, N)
    y = np.empty(out_shape, np.int32)
    lib().orc_matmul_integer(_p(a), ctypes.c_int(_signed(a)), _p(b), ctypes.c_int(_signed(b)), _i64(batch), _i64(M), _i64(N), _i64(K),
                             _p(za), _i64(za.size), _p(zb), _i64(zb.size), _p(y))
    return y


def conv_geometry(H, W, KH, KW, strides=(), pads=(), auto_pad=""):
    """Returns dict(sh, sw, pt, pl, pb, pr, Ho, Wo) following runtime/chainerx_util.cc:180-200,276-311."""
    s = (ctypes.c_int64 * 2)(*(list(strides) + [0, 0])[:2])
    p = (ctypes.c_int64 * 2)(*(list(pads) + [0, 0])[:2])
    out = (ctypes.c_int64 * 8)()
    rc = lib().orc_conv_geometry(_i64(H), _i64(W), _i64(KH), _i64(KW), s, ctypes.c_int(len(strides)), p, ctypes.c_int(len(pads)),
                                 ctypes.c_char_p(auto_pad.encode()), out)
    if rc != 0:
        raise ValueError("unsupported convolution geometry")
    return dict(zip(("sh", "sw", "pt", "pl", "pb", "pr", "Ho", "Wo"), [int(v) for v in out]))


def conv_integer(x, w, x_zero_point=None, w_zero_point=None, strides=(), pads=(), group=1, auto_pad=""):
    x, w = _c(x), _c(w)
    N, C, H, W = x.shape
    M, Cg, KH, KW = w.shape
    assert Cg * group == C and M % group == 0
    g = conv_geometry(H, W, KH, KW, strides, pads, auto_pad)
    zw = _zp_arr(w_zero_point)
    assert zw.size in (0, 1, M)
    y = np.empty((N, M, g["Ho"], g["Wo"]), np.int32)
    lib().orc_conv_integer(_p(x), ctypes.c_int(_signed(x)), _p(w), ctypes.c_int(_signed(w)), _i64(N), _i64(C), _i64(H), _i64(W), _i64(M),
                           _i64(KH), _i64(KW), _i64(g["sh"]), _i64(g["sw"]), _i64(g["pt"]), _i64(g["pl"]), _i64(g["Ho"]), _i64(g["Wo"]),
                           _i64(group), ctypes.c_int(int(x_zero_point is not None)), ctypes.c_int32(int(x_zero_point or 0)), _p(zw),
                           _i64(zw.size), _p(y))
    return y


def qlinear_conv(x, x_scale, x_zero_point, w, w_scale, w_zero_point, y_scale, y_zero_point, b=None, strides=(), pads=(), group=1,
                 auto_pad="", y_dtype=np.uint8, round_mode=ROUND_REF, bias_mode=BIAS_ONNX, clamp_hi_q=-1):
    x, w = _c(x), _c(w)
    N, C, H, W = x.shape
    M, Cg, KH, KW = w.shape
    assert Cg * group == C and M % group == 0
    g = conv_geometry(H, W, KH, KW, strides, pads, auto_pad)
    ws = _c(np.asarray(w_scale, np.float32).reshape(-1))
    wz = _c(np.asarray(w_zero_point).reshape(-1), np.int32)
    assert ws.size == wz.size and ws.size in (1, M)
    y_dtype = np.dtype(y_dtype)
    y = np.empty((N, M, g["Ho"], g["Wo"]), y_dtype)
    bias = None if b is None else _c(b, np.int32)
    lib().orc_qlinear_conv(_p(x), ctypes.c_int(_signed(x)), _f(x_scale), ctypes.c_int(int(x_zero_point)), _p(w), ctypes.c_int(_signed(w)),
                           _p(ws), _p(wz), _i64(ws.size), _f(y_scale), ctypes.c_int(int(y_zero_point)), ctypes.c_int(int(y_dtype == np.int8)),
                           None if bias is None else _p(bias), ctypes.c_int(bias_mode if bias is not None else BIAS_NONE), _i64(N), _i64(C),
                           _i64(H), _i64(W), _i64(M), _i64(KH), _i64(KW), _i64(g["sh"]), _i64(g["sw"]), _i64(g["pt"]), _i64(g["pl"]),
                           _i64(g["Ho"]), _i64(g["Wo"]), _i64(group), ctypes.c_int(round_mode), ctypes.c_int(int(clamp_hi_q)), _p(y))
    return y


def requantize(acc, x_scale, w_scale, y_scale, y_zero_point, bias=None, channel_axis=-1, y_dtype=np.uint8, round_mode=ROUND_REF,
               clamp_hi_q=-1, fold=False):
    """Integer-domain requantization of an exact int32 accumulator (see orc_requantize)."""
    acc = _c(acc, np.int32)
    axis = channel_axis % acc.ndim
    M = acc.shape[axis]
    chan_stride = int(np.prod(acc.shape[axis + 1:])) if axis + 1 < acc.ndim else 1
    ws = _c(np.asarray(w_scale, np.float32).reshape(-1))
    assert ws.size in (1, M)
    y_dtype = np.dtype(y_dtype)
    y = np.empty(acc.shape, y_dtype)
    b = None if bias is None else _c(bias, np.int32)
    lib().orc_requantize(_p(acc), _i64(acc.size), _i64(M), _i64(chan_stride), _f(x_scale), _p(ws), _i64(ws.size),
                         None if b is None else _p(b), _f(y_scale), ctypes.c_int(int(y_zero_point)), ctypes.c_int(int(y_dtype == np.int8)),
                         ctypes.c_int(round_mode), ctypes.c_int(int(clamp_hi_q)), ctypes.c_int(int(fold)), _p(y))
    return y


def qlinear_matmul(a, a_scale, a_zero_point, b, b_scale, b_zero_point, y_scale, y_zero_point, y_dtype=np.uint8, round_mode=ROUND_REF):
    a, b = _c(a), _c(b)
    M, K = a.shape
    N = b.shape[1]
    y_dtype = np.dtype(y_dtype)
    y = np.empty((M, N), y_dtype)
    lib().orc_qlinear_matmul(_p(a), ctypes.c_int(_signed(a)), _f(a_scale), ctypes.c_int(int(a_zero_point)), _p(b), ctypes.c_int(_signed(b)),
                             _f(b_scale), ctypes.c_int(int(b_zero_point)), _f(y_scale), ctypes.c_int(int(y_zero_point)),
                             ctypes.c_int(int(y_dtype == np.int8)), _i64(M), _i64(N), _i64(K), ctypes.c_int(round_mode), _p(y))
    return y


def quantize_data(w, to_int8=True):
    """compiler/quantize.cc:70-89 on a whole tensor.  Returns (q, scale, zero_point)."""
    w = _c(w, np.float32)
    q = np.empty(w.shape, np.int8 if to_int8 else np.uint8)
    s = ctypes.c_float()
    z = ctypes.c_int32()
    lib().orc_quantize_data(_p(w), _i64(w.size), ctypes.c_int(int(to_int8)), _p(q), ctypes.byref(s), ctypes.byref(z))
    return q, np.float32(s.value), int(z.value)


def quantize_weight_per_channel(w, to_int8=True):
    """compiler/quantize.cc:98-129.  Returns (q, scales[M], zero_points[M])."""
    w = _c(w, np.float32)
    M = w.shape[0]
    q = np.empty(w.shape, np.int8 if to_int8 else np.uint8)
    s = np.empty(M, np.float32)
    z = np.empty(M, np.int32)
    lib().orc_quantize_weight_per_channel(_p(w), _i64(M), _i64(w.size // M), ctypes.c_int(int(to_int8)), _p(q), _p(s), _p(z))
    return q, s, z


def merge_conv_bn(w, bn_scale, bn_bias, bn_mean, bn_var, epsilon, conv_bias=None):
    """MergeConvBN, compiler/merge.cc:166-189, every step a single-rounded fp32 array operation as ChainerX evaluates it:
    s = scale / sqrt(var + eps); w'[m] = w[m] * s[m]; b' = (b - mean) * s + bn_bias.  Returns (w', b')."""
    f = np.float32
    w, bn_scale, bn_bias, bn_mean, bn_var = (np.asarray(v, f) for v in (w, bn_scale, bn_bias, bn_mean, bn_var))
    bc = np.zeros(bn_scale.shape[0], f) if conv_bias is None else np.asarray(conv_bias, f)
    s = (bn_scale / np.sqrt(bn_var + f(epsilon))).astype(f)
    new_w = (w * s.reshape((-1,) + (1,) * (w.ndim - 1))).astype(f)
    t = ((bc - bn_mean).astype(f) * s).astype(f)
    return new_w, (t + bn_bias).astype(f)


def dynamic_params_u8(x):
    x = _c(x, np.float32)
    s = ctypes.c_float()
    z = ctypes.c_float()
    lib().orc_dynamic_params_u8(_p(x), _i64(x.size), ctypes.byref(s), ctypes.byref(z))
    return np.float32(s.value), float(z.value)


def _ew_pack(nodes, n_inputs):
    arr = (_EwNode * len(nodes))()
    for j, nd in enumerate(nodes):
        op, ins = nd[0], nd[1]
        arr[j].op = EW_OPS[op]
        arr[j].in0 = ins[0] if len(ins) > 0 else 0
        arr[j].in1 = ins[1] if len(ins) > 1 else 0
        arr[j].cval = float(nd[2]) if len(nd) > 2 else 0.0
        for i in ins:
            assert 0 <= i < n_inputs + j, "nodes must be in topological order"
    return arr


def eltwise(nodes, inputs, out_ids, fp64=False):
    """Evaluate a fused elementwise group.

    nodes: list of (op_name, [input value ids], [constant]) in topological order; value ids
    0..len(inputs)-1 are the inputs, node j defines value len(inputs)+j.  fp64=False: one
    fp32 pass per node (the reference's CPU path); fp64=True: the DAG in double precision.
    """
    ins = [_c(np.broadcast_to(np.asarray(i, np.float32), np.broadcast_shapes(*[np.shape(k) for k in inputs]))) for i in inputs]
    shape = ins[0].shape
    n = ins[0].size
    arr = _ew_pack(nodes, len(ins))
    in_ptrs = (ctypes.c_void_p * len(ins))(*[i.ctypes.data for i in ins])
    outs = [np.empty(shape, np.float64 if fp64 else np.float32) for _ in out_ids]
    out_ptrs = (ctypes.c_void_p * len(outs))(*[o.ctypes.data for o in outs])
    ids = (ctypes.c_int32 * len(out_ids))(*out_ids)
    fn = lib().orc_eltwise_f64 if fp64 else lib().orc_eltwise_f32
    fn(arr, ctypes.c_int(len(nodes)), in_ptrs, ctypes.c_int(len(ins)), _i64(n), ids, ctypes.c_int(len(outs)), out_ptrs)
    return outs


def maxpool_u8(x, k, s, p=0, cover_all=False):
    x = _c(x, np.uint8)
    N, C, H, W = x.shape

    def osz(i):
        if cover_all:
            return (i + 2 * p - k + s - 1) // s + 1
        return (i + 2 * p - k) // s + 1

    Ho, Wo = osz(H), osz(W)
    y = np.empty((N, C, Ho, Wo), np.uint8)
    lib().orc_maxpool_u8(_p(x), _i64(N), _i64(C), _i64(H), _i64(W), _i64(k), _i64(s), _i64(p), _i64(Ho), _i64(Wo), _p(y))
    return y


def global_avgpool_dq(x, scale, zp=0):
    x = _c(x, np.uint8)
    N, C, H, W = x.shape
    y = np.empty((N, C), np.float32)
    lib().orc_global_avgpool_dq(_p(x), _i64(N), _i64(C), _i64(H * W), _f(scale), ctypes.c_int(int(zp)), _p(y))
    return y


def linear_f32(x, w, b=None):
    x, w = _c(x, np.float32), _c(w, np.float32)
    N, K = x.shape
    O = w.shape[0]
    y = np.empty((N, O), np.float32)
    bb = None if b is None else _c(b, np.float32)
    lib().orc_linear_f32(_p(x), _p(w), None if bb is None else _p(bb), _i64(N), _i64(K), _i64(O), _p(y))
    return y


def qadd_relu(a, a_scale, a_zp, b, b_scale, b_zp, y_scale, y_zp=0, relu=True, round_mode=ROUND_REF, fold=False):
    a, b = _c(a, np.uint8), _c(b, np.uint8)
    y = np.empty(a.shape, np.uint8)
    fn = lib().orc_qadd_relu_fold if fold else lib().orc_qadd_relu
    fn(_p(a), _f(a_scale), ctypes.c_int(int(a_zp)), _p(b), _f(b_scale), ctypes.c_int(int(b_zp)), _i64(a.size), _f(y_scale),
                        ctypes.c_int(int(y_zp)), ctypes.c_int(int(relu)), ctypes.c_int(round_mode), _p(y))
    return y
