"""ctypes binding of ``libchxq.so`` (the C ABI declared in ``include/chxq.h``).

The library is the only compute path of this package: there is no CPU or PyTorch fallback.
Importing this module loads the shared object and raises ``ChxqLibraryError`` if it is missing.
"""
import ctypes
import os
import subprocess

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libchxq.so")
CSRC = os.path.join(_HERE, "csrc")

# status codes
OK, ERR_INVALID_ARGUMENT, ERR_UNSUPPORTED, ERR_CUDA, ERR_JIT, ERR_DEVICE_TIMEOUT, ERR_WORKSPACE = range(7)
# dtype codes (compiler/dtype.h:14-26 of the reference)
BOOL, INT8, INT16, INT32, INT64, UINT8, FLOAT16, FLOAT32, FLOAT64 = range(1, 10)
ROUND_REF, ROUND_RNE = 0, 1
NCHW, NHWC = 0, 1
PATH_AUTO, PATH_SIMT, PATH_TENSOR = 0, 1, 2

DTYPE_BY_NAME = {"float16": FLOAT16, "float32": FLOAT32, "float64": FLOAT64}
EW_OPS = {"Identity": 0, "Tanh": 1, "Exp": 2, "Sigmoid": 3, "Add": 4, "Sub": 5, "Mul": 6, "Div": 7, "Constant": 8}


class ChxqLibraryError(RuntimeError):
    pass


class ChxqError(RuntimeError):
    """A non-zero status from the C ABI (the reference CHECK-fails or throws on the same conditions)."""

    def __init__(self, code, message):
        super().__init__("chxq error %d: %s" % (code, message))
        self.code = code


class ConvGeom(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int32) for n in (
        "N", "C", "H", "W", "M", "KH", "KW", "stride_h", "stride_w", "pad_top", "pad_left", "pad_bottom", "pad_right", "group", "Ho", "Wo",
        "x_dtype", "w_dtype", "x_layout", "y_layout", "x_cstride", "y_cstride")]


class QConvParams(ctypes.Structure):
    _fields_ = [
        ("x_scale", ctypes.c_float), ("x_zero_point", ctypes.c_int32),
        ("w_scale", ctypes.c_void_p), ("w_zero_point", ctypes.c_void_p), ("w_params_len", ctypes.c_int64),
        ("y_scale", ctypes.c_float), ("y_zero_point", ctypes.c_int32), ("y_dtype", ctypes.c_int32),
        ("bias", ctypes.c_void_p), ("round_mode", ctypes.c_int32), ("clamp_hi_q", ctypes.c_int32),
        ("residual", ctypes.c_void_p), ("res_scale", ctypes.c_float), ("res_zero_point", ctypes.c_int32), ("res_relu", ctypes.c_int32),
        ("out_scale", ctypes.c_float), ("out_zero_point", ctypes.c_int32), ("fold_scales", ctypes.c_int32),
    ]


class EwNode(ctypes.Structure):
    _fields_ = [("op", ctypes.c_int32), ("inputs", ctypes.c_int32 * 2), ("output", ctypes.c_int32), ("constant", ctypes.c_double)]


class GraphNode(ctypes.Structure):
    _fields_ = [
        ("op_type", ctypes.c_char_p), ("inputs", ctypes.POINTER(ctypes.c_int32)), ("n_inputs", ctypes.c_int32),
        ("outputs", ctypes.POINTER(ctypes.c_int32)), ("n_outputs", ctypes.c_int32), ("is_grad", ctypes.c_int32),
        ("const_is_float", ctypes.c_int32), ("const_num_elements", ctypes.c_int64),
    ]


class GraphValue(ctypes.Structure):
    _fields_ = [("dtype", ctypes.c_int32), ("is_graph_output", ctypes.c_int32)]


# Every symbol include/chxq.h declares, with its restype (argtypes are given where a wrong implicit
# conversion would be silent: floats, 64-bit integers and pointers).
_c = ctypes
_vp, _i32, _i64, _f32, _sz = _c.c_void_p, _c.c_int32, _c.c_int64, _c.c_float, _c.c_size_t
SIGNATURES = {
    "chxq_last_error": (_c.c_char_p, []),
    "chxq_version": (_c.c_int, []),
    "chxq_device_status": (_c.c_int, [_vp]),
    "chxq_launch_count": (_i64, []),
    "chxq_tc_variant": (_c.c_int, [_i32]),
    "chxq_tc_pair_slots": (_c.c_int, [_c.POINTER(_c.c_int32)]),
    "chxq_tc_test_hooks": (_c.c_int, [_i64, _i32]),
    "chxq_tc_profile": (_c.c_int, [_i32]),
    "chxq_tc_profile_read": (_c.c_int, [_c.POINTER(_c.c_double), _c.POINTER(_i64), _c.POINTER(_c.c_double)]),
    "chxq_quantize_linear": (_c.c_int, [_vp, _i64, _f32, _i32, _i32, _i32, _vp, _vp]),
    "chxq_dequantize_linear": (_c.c_int, [_vp, _i32, _i64, _f32, _i32, _vp, _vp]),
    "chxq_matmul_integer_workspace": (_sz, [_i64, _i64, _i64, _i64]),
    "chxq_matmul_integer": (_c.c_int, [_vp, _i32, _vp, _i32, _i64, _i64, _i64, _i64, _vp, _i64, _vp, _i64, _vp, _vp, _sz, _i32, _vp]),
    "chxq_matmul_integer_noalloc": (_c.c_int, [_vp, _i32, _vp, _i32, _i64, _i64, _i64, _vp, _i64, _vp, _i64, _vp, _vp]),
    "chxq_qlinear_matmul": (_c.c_int, [_vp, _i32, _f32, _i32, _vp, _i32, _f32, _i32, _f32, _i32, _i32, _i64, _i64, _i64, _i32, _vp, _vp, _sz,
                                       _i32, _vp]),
    "chxq_conv_resolve_geometry": (_c.c_int, [_i32] * 8 + [_c.POINTER(_i64), _i32, _c.POINTER(_i64), _i32, _i32, _c.c_char_p,
                                                        _c.POINTER(ConvGeom)]),
    "chxq_conv_workspace": (_sz, [_c.POINTER(ConvGeom)]),
    "chxq_conv_packed_workspace": (_sz, [_c.POINTER(ConvGeom), _i32, _i32]),
    "chxq_conv_integer": (_c.c_int, [_vp, _vp, _c.POINTER(ConvGeom), _i32, _i32, _vp, _i64, _vp, _vp, _sz, _i32, _vp]),
    "chxq_qlinear_conv": (_c.c_int, [_vp, _vp, _c.POINTER(ConvGeom), _c.POINTER(QConvParams), _vp, _vp, _sz, _i32, _vp]),
    "chxq_conv_prepack_bytes": (_sz, [_c.POINTER(ConvGeom)]),
    "chxq_conv_prepack": (_c.c_int, [_vp, _c.POINTER(ConvGeom), _vp, _i64, _vp, _sz, _c.POINTER(_i32), _vp]),
    "chxq_qlinear_conv_packed": (_c.c_int, [_vp, _vp, _c.POINTER(ConvGeom), _c.POINTER(QConvParams), _i32, _vp, _vp, _sz, _vp]),
    "chxq_qlinear_conv_chain_packed": (_c.c_int, [_vp, _vp, _c.POINTER(ConvGeom), _c.POINTER(QConvParams), _i32, _vp, _c.POINTER(ConvGeom),
                                                 _c.POINTER(QConvParams), _i32, _vp, _vp]),
    "chxq_quantize_qlinear_conv_packed": (_c.c_int, [_vp, _i32, _vp, _c.POINTER(ConvGeom), _c.POINTER(QConvParams), _i32, _vp, _vp, _sz, _vp]),
    "chxq_qlinear_conv_maxpool_packed": (_c.c_int, [_vp, _i32, _i32, _vp, _c.POINTER(ConvGeom), _c.POINTER(QConvParams), _i32, _i32, _i32, _i32, _i32, _vp,
                                                   _vp, _sz, _vp]),
    "chxq_conv_integer_packed": (_c.c_int, [_vp, _vp, _c.POINTER(ConvGeom), _i32, _i32, _i32, _vp, _vp, _sz, _vp]),
    "chxq_eltwise_codegen": (_c.c_int, [_c.POINTER(EwNode), _i32, _c.POINTER(_i32), _i32, _c.POINTER(_i32), _i32, _c.POINTER(_c.c_char_p), _i32,
                                        _i32, _i32, _c.c_char_p, _sz, _c.POINTER(_sz)]),
    "chxq_eltwise_run": (_c.c_int, [_c.c_char_p, _i32, _c.POINTER(_vp), _i32, _c.POINTER(_vp), _i32, _i64, _i32, _vp]),
    "chxq_fuse_elementwise": (_c.c_int, [_c.POINTER(GraphNode), _i32, _c.POINTER(GraphValue), _i32, _c.POINTER(_i32), _c.POINTER(_i32)]),
    "chxq_quantize_weights_host": (_c.c_int, [_vp, _i64, _i64, _i32, _i32, _vp, _vp, _vp]),
    "chxq_prepare_weights_workspace": (_sz, [_i64]),
    "chxq_prepare_weights": (_c.c_int, [_vp, _i64, _i64, _vp, _vp, _vp, _vp, _f32, _vp, _i32, _i32, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _vp]),
    "chxq_maxpool_u8_nhwc": (_c.c_int, [_vp] + [_i32] * 9 + [_vp, _vp]),
    "chxq_global_avgpool_dq_nhwc": (_c.c_int, [_vp, _i32, _i32, _i32, _f32, _i32, _vp, _vp]),
    "chxq_linear_f32": (_c.c_int, [_vp, _vp, _vp, _i32, _i32, _i32, _vp, _vp]),
    "chxq_qadd_u8": (_c.c_int, [_vp, _f32, _i32, _vp, _f32, _i32, _i64, _f32, _i32, _i32, _i32, _vp, _vp]),
    "chxq_nchw_to_nhwc": (_c.c_int, [_vp, _i32, _i32, _i32, _i32, _i32, _i32, _vp, _vp]),
    "chxq_nhwc_to_nchw": (_c.c_int, [_vp, _i32, _i32, _i32, _i32, _i32, _i32, _vp, _vp]),
    "chxq_minmax_f32": (_c.c_int, [_vp, _i64, _vp, _vp]),
    "chxq_dynamic_quant_params_u8": (_c.c_int, [_vp, _vp, _vp, _vp, _vp]),
    "chxq_quantize_linear_dev": (_c.c_int, [_vp, _i64, _vp, _vp, _i32, _i32, _vp, _vp]),
    "chxq_conv_integer_dev": (_c.c_int, [_vp, _vp, _vp, _vp, _vp, _i64, _vp, _vp]),
}

_lib = None


def build(verbose=False):
    """Compile libchxq.so in-tree with nvcc for sm_100a (needs no GPU)."""
    out = subprocess.run(["make", "-C", CSRC, "-j", "8"], capture_output=True, text=True)
    if out.returncode != 0:
        raise ChxqLibraryError("building libchxq.so failed:\n" + out.stdout[-4000:] + out.stderr[-4000:])
    if verbose:
        print(out.stdout[-2000:])
    return LIB_PATH


def lib():
    """The loaded library.  Fails loudly when the CUDA extension has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ChxqLibraryError(
                "libchxq.so is missing at %s; build it with `make -C %s` (this package has no fallback path)" % (LIB_PATH, CSRC))
        try:
            l = ctypes.CDLL(LIB_PATH)
        except OSError as e:
            raise ChxqLibraryError("libchxq.so failed to load: %s" % e)
        for name, (res, args) in SIGNATURES.items():
            try:
                fn = getattr(l, name)
            except AttributeError:
                raise ChxqLibraryError("libchxq.so does not export %s; rebuild it" % name)
            fn.restype = res
            fn.argtypes = args
        _lib = l
    return _lib


def check(code):
    if code != OK:
        raise ChxqError(code, lib().chxq_last_error().decode("utf-8", "replace"))
