"""ctypes binding of the C-ABI library (include/kdw.h).

The library is the only implementation of the operators: if it is missing or a symbol cannot be
resolved, importing fails with an error - there is no fallback path.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, 'csrc', 'libkdw.so')

_i64 = ctypes.c_int64
_int = ctypes.c_int
_ptr = ctypes.c_void_p

# name -> (restype, argtypes); one entry per function declared in include/kdw.h
SIGNATURES = {
    'kdw_version': (_int, []),
    'kdw_last_error': (ctypes.c_char_p, []),
    'kdw_device_status': (_int, [ctypes.POINTER(_int)]),
    'kdw_test_wait_limits': (_int, [_i64, _int]),
    'kdw_fprop_f16': (_int, [_ptr, _ptr, _ptr] + [_i64] * 5 + [_i64] * 6 + [_int, _int, _ptr]),
    'kdw_fprop_f16_range': (
        _int,
        [_ptr, _ptr, _ptr] + [_i64] * 5 + [_i64] * 3 + [_i64] * 4 + [_i64] * 3 + [_int, _int, _ptr],
    ),
    'kdw_fprop_variants': (_int, []),
    'kdw_fprop_variant_channels': (_int, [_int]),
    'kdw_fprop_auto_variant': (_int, [_i64, _i64, _i64]),
    'kdw_wgrad_workspace_bytes': (_i64, [_i64] * 5),
    'kdw_wgrad_f16': (_int, [_ptr, _ptr, _ptr, _i64, _ptr, _ptr] + [_i64] * 5 + [_i64] * 6 + [_int, _ptr]),
    'kdw_wgrad_f16_range': (
        _int,
        [_ptr, _ptr, _ptr, _i64, _ptr, _ptr] + [_i64] * 5 + [_i64] * 3 + [_i64] * 4 + [_i64] * 3 + [_int, _ptr],
    ),
    'kdw_wgrad_f16_static': (_int, [_ptr, _ptr, _ptr, _ptr] + [_i64] * 5 + [_i64] * 6 + [_ptr]),
    'kdw_wgrad_variants': (_int, []),
    'kdw_wgrad_variant_channels': (_int, [_int]),
    'kdw_wgrad_auto_variant': (_int, [_i64, _i64, _i64]),
    'kdw_fprop_addstats_workspace_bytes': (_i64, [_i64] * 5),
    'kdw_fprop_addstats_variants': (_int, []),
    'kdw_fprop_addstats_f16': (_int, [_ptr] * 5 + [_i64] + [_ptr] * 2 + [_i64] * 5 + [_i64] * 9 + [_int, _ptr]),
    'kdw_fprop_bnrelu_variants': (_int, []),
    'kdw_fprop_bnrelu_f16': (_int, [_ptr] * 5 + [_i64] * 5 + [_i64] * 6 + [_int, _int, _ptr]),
    'kdw_allreduce_buffer_bytes': (_i64, [_i64, _int]),
    'kdw_allreduce_push_f32': (_int, [_ptr, _ptr, _ptr, _ptr, _i64, _i64, _int, _int, ctypes.c_uint32, _i64, _ptr]),
}

_lib = None


class KdwError(RuntimeError):
    """A C-ABI call returned a non-zero status."""

    def __init__(self, code, message):
        super().__init__(f'kdw error {code}: {message}')
        self.code = code


def load():
    """Loads libkdw.so once and declares every prototype."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f'{LIB_PATH} is missing: build the CUDA library first (python -m kerops_b200.build). '
            'kerops_b200 has no non-CUDA implementation.'
        )
    lib = ctypes.CDLL(LIB_PATH)
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is not exported
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib


def check(code):
    if code != 0:
        msg = load().kdw_last_error()
        raise KdwError(code, msg.decode() if msg else '')


def device_status():
    """Reads and clears the device status word of the current CUDA device (synchronises)."""
    v = _int(0)
    check(load().kdw_device_status(ctypes.byref(v)))
    return v.value
