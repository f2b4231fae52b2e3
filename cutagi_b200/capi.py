"""ctypes binding of include/tagi_b200.h. Device pointers are passed as integers (e.g. ``tensor.data_ptr()``)."""
import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libtagi_b200.so")

TAGI_OK = 0
IMPL_AUTO, IMPL_FFMA, IMPL_TF32X3 = 0, 1, 2
ACT_RELU, ACT_MIXTURE_RELU = 1, 2   # tagi_linear_fwd_act / tagi_conv2d_fwd_act


class TagiError(RuntimeError):
    def __init__(self, code, msg):
        super().__init__(f"tagi_b200 status {code}: {msg}")
        self.code = code


class ConvGeom(C.Structure):
    """Mirror of ``tagi_conv2d_geom``."""
    _fields_ = [(n, C.c_int) for n in
                ("B", "fi", "hi", "wi", "fo", "ho", "wo", "k", "stride", "pad", "pad_type", "has_bias")]


_p = C.c_void_p
_i = C.c_int
_SIGNATURES = {
    "tagi_set_impl": [_i],
    "tagi_get_impl": [],
    "tagi_version": [],
    "tagi_tc_status": [C.POINTER(_i), _i],
    "tagi_reserve_scratch": [C.c_size_t],
    "tagi_release_scratch": [],
    "tagi_tc_set_chunked": [_i],
    "tagi_tc_set_sm_budget": [_i],
    "tagi_tc_set_variant": [_i],
    "tagi_linear_fwd": [_p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _p, _p, _p],
    "tagi_linear_bwd_state": [_p, _p, _p, _p, _i, _i, _i, _p, _p, _p],
    "tagi_linear_bwd_param": [_p, _p, _p, _p, _p, _i, _i, _i, _i, _p, _p, _p, _p, _p],
    "tagi_linear_bwd_param_rows": [_p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _p, _p, _p, _p, _p],
    "tagi_conv2d_out_size": [_i, _i, _i, _i, _i, _i, C.POINTER(_i), C.POINTER(_i)],
    "tagi_conv2d_fwd": [C.POINTER(ConvGeom), _p, _p, _p, _p, _p, _p, _p, _p, _p],
    "tagi_conv2d_bwd_state": [C.POINTER(ConvGeom), _p, _p, _p, _p, _p, _p, _p],
    "tagi_conv2d_bwd_param": [C.POINTER(ConvGeom), _p, _p, _p, _p, _p, _p, _p, _p, _p, _p],
    "tagi_relu_fwd": [_p, _p, C.c_size_t, _p, _p, _p, _p],
    "tagi_linear_fwd_relu": [_p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _p, _p, _p, _p],
    "tagi_conv2d_fwd_relu": [C.POINTER(ConvGeom), _p, _p, _p, _p, _p, _p, _p, _p, _p, _p],
    "tagi_linear_fwd_act": [_p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _p, _p, _p, _p],
    "tagi_conv2d_fwd_act": [C.POINTER(ConvGeom), _p, _p, _p, _p, _p, _p, _i, _p, _p, _p, _p],
    "tagi_mixture_relu_fwd": [_p, _p, C.c_size_t, _p, _p, _p, _p],
    "tagi_output_delta": [_p, _p, _p, _p, _p, C.c_size_t, _p, _p, _p],
    "tagi_output_delta_selected": [_p, _p, _p, _p, _p, _p, _i, _i, _i, _p, _p, _p],
    "tagi_param_update": [_i, C.c_size_t, _p, _p, _p, _p, _p, _p],
    "tagi_param_update_multi": [_i, _i, _p, _p, _p],
    "tagi_conv2d_bwd_param_noalloc": [C.POINTER(ConvGeom), _p, _p, _p, _p, _p, _p, _p, _p, _p, _p],
    "tagi_bn2d_fwd": [_i, _i, _i, _i, _i, C.c_float, C.c_float] + [_p] * 13,
    "tagi_bn2d_bwd": [_i, _i, _i, _i, _i, C.c_float] + [_p] * 16,
    "tagi_avgpool2d_fwd": [C.POINTER(ConvGeom), _p, _p, _p, _p, _p],
    "tagi_avgpool2d_bwd_state": [C.POINTER(ConvGeom), _p, _p, _p, _p, _p, _p],
    "tagi_add_shortcut": [_p, _p, _p, C.c_size_t, _p, _p, _p],
    "tagi_io_create": [C.c_size_t, C.c_size_t, C.c_size_t, C.c_size_t, _i, C.POINTER(_p)],
    "tagi_io_destroy": [_p],
    "tagi_io_host_buffers": [_p, _i, C.POINTER(_p), C.POINTER(_p), C.POINTER(_p)],
    "tagi_io_device_buffers": [_p, _i, C.POINTER(_p), C.POINTER(_p), C.POINTER(_p)],
    "tagi_io_upload": [_p, _i, _p],
    "tagi_io_consumed": [_p, _i, _p],
    "tagi_io_download": [_p, _i, _p, _p, C.c_size_t, _p],
    "tagi_io_wait_output": [_p, _i, C.POINTER(_p), C.POINTER(_p)],
}

_lib = None


def load():
    """Load libtagi_b200.so; raises if it is missing (there is no fallback path)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} not found: build the CUDA library first (python -m cutagi_b200.build); "
                "cutagi_b200 has no CPU or PyTorch fallback")
        _lib = C.CDLL(LIB_PATH)
        _lib.tagi_last_error_string.restype = C.c_char_p
        _lib.tagi_conv2d_workspace_bytes.restype = C.c_size_t
        _lib.tagi_conv2d_workspace_bytes.argtypes = [C.POINTER(ConvGeom)]
        _lib.tagi_scratch_bytes.restype = C.c_size_t
        _lib.tagi_scratch_bytes.argtypes = []
        for name, args in _SIGNATURES.items():
            fn = getattr(_lib, name)
            fn.argtypes = args
            fn.restype = _i
    return _lib


class _Lib:
    """Attribute access to the entry points with status checking: ``lib.tagi_linear_fwd(...)`` raises TagiError."""

    def __getattr__(self, name):
        fn = getattr(load(), name)
        if name in ("tagi_get_impl", "tagi_version", "tagi_last_error_string", "tagi_conv2d_workspace_bytes",
                    "tagi_scratch_bytes"):
            return fn

        def checked(*args):
            rc = fn(*args)
            if rc != TAGI_OK:
                raise TagiError(rc, load().tagi_last_error_string().decode())
            return rc

        checked.__name__ = name
        return checked


lib = _Lib()


def tc_status(reset=True):
    """Status word of the TF32X3 kernels on the current device (0 = no bounded wait ever ran out)."""
    s = _i(0)
    lib.tagi_tc_status(C.byref(s), int(reset))
    return s.value


def conv_out_size(k, stride, wi, hi, pad, pad_type):
    wo, ho = _i(0), _i(0)
    lib.tagi_conv2d_out_size(k, stride, wi, hi, pad, pad_type, C.byref(wo), C.byref(ho))
    return wo.value, ho.value
