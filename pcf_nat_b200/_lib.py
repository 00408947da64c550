"""ctypes binding of the C ABI declared in include/na1d_b200.h.

There is no CPU or eager fallback: if the shared library is missing, importing this module
raises, and every wrapper raises ``Na1dError`` on a non-zero status.
"""
import ctypes
import os
import re

from ._build import LIB

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "na1d_b200.h")

NA1D_BF16 = 0
NA1D_FP16 = 1


class Na1dError(RuntimeError):
    def __init__(self, status, where):
        self.status = status
        msg = _lib.na1d_status_string(status).decode() if _lib is not None else "?"
        if status == -7 and _lib is not None:
            msg += " [cudaError %d]" % _lib.na1d_last_cuda_error()
        super().__init__("%s failed with status %d: %s" % (where, status, msg))


def declared_symbols(header=HEADER):
    """Names of all functions the public header declares."""
    src = open(header).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(na1d_[a-z0-9_]+)\s*\(", src)))


def _load():
    if not os.path.exists(LIB):
        raise ImportError(
            "pcf_nat_b200: %s is missing. Build it with `python -m pcf_nat_b200._build` "
            "(needs nvcc); there is no fallback implementation." % LIB)
    return ctypes.CDLL(LIB)


_lib = None
_lib = _load()

_i64, _i32, _f32, _ptr = ctypes.c_int64, ctypes.c_int, ctypes.c_float, ctypes.c_void_p

_lib.na1d_status_string.restype = ctypes.c_char_p
_lib.na1d_status_string.argtypes = [_i32]
_lib.na1d_last_cuda_error.restype = _i32
_lib.na1d_version.restype = _i32
for _name in ("na1d_qk_forward", "na1d_q_backward", "na1d_k_backward", "na1d_av_forward",
              "na1d_a_backward", "na1d_v_backward"):
    _f = getattr(_lib, _name)
    _f.restype = _i32
    _f.argtypes = [_ptr, _ptr, _ptr, _i64, _i64, _i64, _i64, _i64, _i64, _i32, _ptr]
_lib.na1d_fused_forward.restype = _i32
_lib.na1d_fused_forward.argtypes = [_ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr,
                                    _i64, _i64, _i64, _i64, _i64, _i64, _i64, _f32, _i32, _ptr]
_lib.na1d_fused_backward.restype = _i32
_lib.na1d_fused_backward.argtypes = [_ptr] * 13 + [_i64] * 7 + [_f32, _i32, _ptr]
_lib.na1d_fused_backward_static.restype = _i32
_lib.na1d_fused_backward_static.argtypes = [_ptr] * 12 + [_i64] * 7 + [_f32, _i32, _ptr]
_lib.na1d_window_index.restype = _i32
_lib.na1d_window_index.argtypes = [_ptr, _ptr, _i64, _i64, _i64, _i64, _ptr]
_lib.na1d_fused_kernel_family.restype = _i32
_lib.na1d_fused_kernel_family.argtypes = [_i64, _i64, _i64, _i64, _i64, _i64, _i32, _i32]
_lib.na1d_fused_kernel_tiling.restype = _i32
_lib.na1d_fused_kernel_tiling.argtypes = [_i64, _i64, _i64, _i64, _i64, _i64, _i32, _i32]
_u64 = ctypes.c_uint64
_lib.na1d_dropout_keep_mask.restype = _i32
_lib.na1d_dropout_keep_mask.argtypes = [_ptr, _i64, _i64, _f32, _u64]
_lib.na1d_fused_forward_dropout.restype = _i32
_lib.na1d_fused_forward_dropout.argtypes = [_ptr] * 7 + [_i64] * 7 + [_f32, _f32, _u64, _i32, _ptr]
_lib.na1d_fused_backward_dropout.restype = _i32
_lib.na1d_fused_backward_dropout.argtypes = [_ptr] * 12 + [_i64] + [_i64] * 7 + [_f32, _f32, _u64, _i32, _ptr]
_lib.na1d_fused_strided_supported.restype = _i32
_lib.na1d_fused_strided_supported.argtypes = [_i64, _i64, _i64, _i64, _i64, _i64, _i32, _i32, _i32]
_lib.na1d_fused_forward_strided.restype = _i32
_lib.na1d_fused_forward_strided.argtypes = [_ptr] * 7 + [_ptr] * 4 + [_i64] * 7 + [_f32, _i32, _ptr]
_lib.na1d_fused_backward_strided.restype = _i32
_lib.na1d_fused_backward_strided.argtypes = [_ptr] * 12 + [_i64] + [_ptr] * 7 + [_i64] * 7 + [_f32, _i32, _ptr]
_lib.na1d_tensor_map_cache_stats.restype = _i32
_lib.na1d_tensor_map_cache_stats.argtypes = [_ptr, _ptr]
_lib.na1d_set_kernel_family.restype = _i32
_lib.na1d_set_kernel_family.argtypes = [_i32]
_lib.na1d_device_status.restype = _i32
_lib.na1d_device_status.argtypes = []


def lib():
    return _lib


def check(status, where):
    if status != 0:
        raise Na1dError(status, where)
