"""ctypes binding of libtkquant.so.  There is no fallback: a missing library is an error."""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# TKQ_LIB_PATH points at another build of the library (e.g. one installed outside the package)
LIB_PATH = os.environ.get('TKQ_LIB_PATH') or os.path.join(_HERE, 'lib', 'libtkquant.so')

# enums of include/tkquant.h
DT_BF16, DT_FP32 = 0, 1
FMT_E4M3, FMT_E2M1, FMT_E5M6 = 0, 1, 2
ROUND_SF, SF_COL_MAJOR, SF_UE8M0, SF_ONLY, CAST_ONLY, EXACT_CODES = 1, 2, 4, 8, 16, 32

_vp, _i64, _int, _uint, _f32 = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_uint, ctypes.c_float

# name -> argument types, in the order of include/tkquant.h
SIGNATURES = {
    'tkq_version': [],
    'tkq_device_error': [],
    'tkq_selftest_bounded_wait': [_vp, _uint, _vp, _vp],
    'tkq_per_token_cast': [_vp, _int, _i64, _i64, _i64, _int, _i64, _uint, _vp, _vp, _i64, _vp],
    'tkq_per_token_cast_quantized': [_vp, _int, _vp, _uint, _i64, _int, _int, _i64, _i64, _i64, _int, _i64, _uint, _vp, _vp, _i64,
                                     _vp],
    'tkq_per_token_cast_e5m6': [_vp, _int, _i64, _i64, _i64, _uint, _vp, _vp, _i64, _vp],
    'tkq_per_block_cast': [_vp, _int, _i64, _i64, _int, _int, _int, _uint, _vp, _vp, _i64, _vp],
    'tkq_per_channel_cast': [_vp, _int, _i64, _i64, _uint, _vp, _vp, _vp],
    'tkq_per_channel_cast_fused': [_vp, _int, _vp, _vp, _i64, _i64, _i64, _uint, _vp, _vp, _vp],
    'tkq_per_channel_cast_and_transpose': [_vp, _i64, _i64, _int, _uint, _vp, _vp, _vp],
    'tkq_swiglu_forward_and_per_channel_cast': [_vp, _i64, _i64, _int, _int, _f32, _uint, _vp, _vp, _vp],
    'tkq_per_block_cast_lossless': [_vp, _vp, _uint, _i64, _int, _int, _i64, _i64, _i64, _int, _int, _uint, _vp, _vp, _i64, _vp],
    'tkq_cast_back': [_vp, _int, _vp, _uint, _i64, _int, _int, _i64, _i64, _int, _vp, _vp],
    'tkq_swiglu_forward_and_per_token_cast': [_vp, _int, _i64, _i64, _i64, _vp, _vp, _vp, _f32, _vp, _f32, _int, _uint,
                                              _vp, _vp, _i64, _vp],
    'tkq_swiglu_backward_and_per_token_cast': [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _f32, _uint,
                                               _vp, _vp, _vp, _vp, _vp, _vp],
    'tkq_expand_to_fused': [_vp, _i64, _i64, _vp, _i64, _vp, _i64, _vp, _i64, _uint, _vp, _vp, _i64, _vp],
}

_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f'{LIB_PATH} is missing: build it with `python -m tilekernels_b200.build` (nvcc, sm_100a). '
                'tilekernels_b200 has no other backend.')
        handle = ctypes.CDLL(LIB_PATH)
        for name, argtypes in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.argtypes = argtypes
            fn.restype = _int
        handle.tkq_last_error_string.restype = ctypes.c_char_p
        handle.tkq_last_error_string.argtypes = []
        _lib = handle
    return _lib


def check(rc: int, what: str) -> None:
    """Turn a non-zero return of the C ABI into RuntimeError (the asserts of the wrappers run before any launch)."""
    if rc != 0:
        raise RuntimeError(f'{what} failed with code {rc}: {lib().tkq_last_error_string().decode()}')
