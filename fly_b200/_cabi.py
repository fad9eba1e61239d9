"""ctypes binding of the C ABI in include/sblocal_b200.h.

The library is loaded from fly_b200/lib (built in-tree by fly_b200.build).
There is no fallback: if the library is missing or a call fails, an exception
is raised.
"""
import ctypes
import os
import threading

from . import build as _build

SBL_DTYPE_F32 = 0
SBL_DTYPE_BF16 = 1
SBL_FLAG_GENERIC_PATH = 1

SBL_OK = 0
SBL_ERR_INVALID_ARGUMENT = -1
SBL_ERR_UNSUPPORTED = -2
SBL_ERR_WORKSPACE = -3
SBL_ERR_CUDA = -4
SBL_ERR_DEVICE_STATUS = -5

ABI_VERSION = 1

EXPORTS = ('sbl_version', 'sbl_last_error', 'sbl_has_tensor_path', 'sbl_workspace_bytes', 'sbl_forward',
           'sbl_key_logscale', 'sbl_key_summary', 'sbl_band_forward', 'sbl_query_features',
           'sbl_key_features', 'sbl_attention_weights', 'sbl_check_status', 'sbl_selftest_wait_timeout',
           'sbl_key_logscale_static', 'sbl_static_last_error', 'sbl_status_words')


class SblParams(ctypes.Structure):
    """Mirror of `struct SblParams`."""
    _fields_ = [
        ('dtype', ctypes.c_int32),
        ('B', ctypes.c_int32), ('H', ctypes.c_int32), ('T', ctypes.c_int32), ('S', ctypes.c_int32),
        ('E', ctypes.c_int32), ('D', ctypes.c_int32),
        ('r', ctypes.c_int32),
        ('w', ctypes.c_int32),
        ('softmax_temp', ctypes.c_float),
        ('softmax_eps', ctypes.c_float),
        ('q', ctypes.c_void_p), ('q_stride_b', ctypes.c_int64), ('q_stride_t', ctypes.c_int64),
        ('q_stride_h', ctypes.c_int64),
        ('k', ctypes.c_void_p), ('k_stride_b', ctypes.c_int64), ('k_stride_s', ctypes.c_int64),
        ('k_stride_h', ctypes.c_int64),
        ('v', ctypes.c_void_p), ('v_stride_b', ctypes.c_int64), ('v_stride_s', ctypes.c_int64),
        ('v_stride_h', ctypes.c_int64),
        ('out', ctypes.c_void_p), ('o_stride_b', ctypes.c_int64), ('o_stride_t', ctypes.c_int64),
        ('o_stride_h', ctypes.c_int64),
        ('W', ctypes.c_void_p),
        ('key_lengths', ctypes.c_void_p),
        ('q_pos0', ctypes.c_int64), ('k_pos0', ctypes.c_int64),
        ('S_total', ctypes.c_int64),
        ('sum_lo', ctypes.c_int32), ('sum_hi', ctypes.c_int32),
        ('flags', ctypes.c_int32),
        ('reserved', ctypes.c_int32 * 3),
    ]


class SblError(RuntimeError):
    """A C-ABI call returned a non-zero status."""
    def __init__(self, status, message):
        super().__init__(f'sblocal_b200 status {status}: {message}')
        self.status = status


_lock = threading.Lock()
_lib = None


def library_path():
    """In-tree library, or the file named by SBLOCAL_B200_LIB (debug builds)."""
    return os.environ.get('SBLOCAL_B200_LIB') or _build.LIB_PATH


def load():
    """Loads (once) and returns the ctypes library handle."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        path = library_path()
        if not os.path.exists(path):
            raise ImportError(
                f'{path} is missing: build it with `python -m fly_b200.build` (needs nvcc). '
                'sblocal_b200 has no fallback path.')
        lib = ctypes.CDLL(path)
        P = ctypes.POINTER(SblParams)
        vp, sz = ctypes.c_void_p, ctypes.c_size_t
        lib.sbl_version.restype = ctypes.c_int
        lib.sbl_version.argtypes = []
        lib.sbl_last_error.restype = ctypes.c_char_p
        lib.sbl_last_error.argtypes = []
        lib.sbl_has_tensor_path.restype = ctypes.c_int
        lib.sbl_has_tensor_path.argtypes = []
        lib.sbl_workspace_bytes.restype = ctypes.c_int
        lib.sbl_workspace_bytes.argtypes = [P, ctypes.POINTER(sz)]
        lib.sbl_forward.restype = ctypes.c_int
        lib.sbl_forward.argtypes = [P, vp, sz, vp]
        lib.sbl_key_logscale.restype = ctypes.c_int
        lib.sbl_key_logscale.argtypes = [P, vp, sz, vp, vp]
        lib.sbl_key_summary.restype = ctypes.c_int
        lib.sbl_key_summary.argtypes = [P, vp, sz, vp, vp, vp, vp]
        lib.sbl_band_forward.restype = ctypes.c_int
        lib.sbl_band_forward.argtypes = [P, vp, sz, vp, vp, vp, vp]
        lib.sbl_query_features.restype = ctypes.c_int
        lib.sbl_query_features.argtypes = [P, vp, sz, vp, vp, vp]
        lib.sbl_key_features.restype = ctypes.c_int
        lib.sbl_key_features.argtypes = [P, vp, sz, vp, vp, vp]
        lib.sbl_attention_weights.restype = ctypes.c_int
        lib.sbl_attention_weights.argtypes = [P, vp, sz, vp, vp, vp, vp]
        lib.sbl_check_status.restype = ctypes.c_int
        lib.sbl_check_status.argtypes = [P, vp, sz, vp]
        lib.sbl_status_words.restype = ctypes.c_int
        lib.sbl_status_words.argtypes = [P, ctypes.POINTER(sz)]
        lib.sbl_selftest_wait_timeout.restype = ctypes.c_int
        lib.sbl_selftest_wait_timeout.argtypes = [vp, sz, vp]
        lib.sbl_key_logscale_static.restype = ctypes.c_int
        lib.sbl_key_logscale_static.argtypes = [P, vp, vp]
        lib.sbl_static_last_error.restype = ctypes.c_char_p
        lib.sbl_static_last_error.argtypes = []
        if lib.sbl_version() != ABI_VERSION:
            raise ImportError(f'{path} has ABI version {lib.sbl_version()}, expected {ABI_VERSION}: rebuild')
        _lib = lib
    return _lib


def check(status):
    """Raises the Python exception that corresponds to a C status."""
    if status == SBL_OK:
        return
    msg = load().sbl_last_error().decode('utf-8', 'replace')
    if status == SBL_ERR_INVALID_ARGUMENT:
        raise ValueError(f'sblocal_b200: {msg}')
    if status == SBL_ERR_UNSUPPORTED:
        raise NotImplementedError(f'sblocal_b200: {msg}')
    raise SblError(status, msg)
