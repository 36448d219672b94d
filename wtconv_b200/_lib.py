"""ctypes binding of ``libwtconv_b200.so`` (the C ABI in ``include/wtconv_b200.h``).

The shared library holds the hand-written sm_100a kernels; there is no other
implementation behind this module.  If the library has not been built the import
of the symbols fails loudly with the build command -- nothing falls back to
PyTorch ops or to the CPU.
"""
from __future__ import annotations

import ctypes
import os
import threading

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libwtconv_b200.so")

F32, BF16, F16 = 0, 1, 2

_lock = threading.Lock()
_lib = None

# every symbol include/wtconv_b200.h declares: (name, restype, argtypes)
_VP, _I, _LLP = ctypes.c_void_p, ctypes.c_int, ctypes.POINTER(ctypes.c_longlong)
SYMBOLS = {
    "wtconv_query": (_I, [_I]),
    "wtconv_status_string": (ctypes.c_char_p, [_I]),
    "wtconv_device_status": (_I, [_VP]),
    "wtconv_packed_param_floats": (ctypes.c_size_t, [_I, _I, _I, _I]),
    "wtconv_pack_params": (_I, [_I, _I, _I, _I, _I, ctypes.c_double, ctypes.c_double, _VP, _VP, _VP,
                                ctypes.POINTER(_VP), ctypes.POINTER(_VP), _VP, _VP]),
    "wtconv_pack_params_adjoint": (_I, [_I, _I, _I, _I, _I, ctypes.c_double, ctypes.c_double, _VP, _VP, _VP,
                                        ctypes.POINTER(_VP), ctypes.POINTER(_VP), _VP, _VP]),
    "wtconv_param_grads": (_I, [_I, _I, _I, _I, _I, ctypes.c_double, ctypes.c_double, _VP, _VP, _VP, _VP,
                                ctypes.POINTER(_VP), ctypes.POINTER(_VP), _VP, _VP, _VP, ctypes.POINTER(_VP),
                                ctypes.POINTER(_VP), _VP]),
    "wtconv2d_pyramid_floats": (ctypes.c_size_t, [_I, _I, _I, _I, _I]),
    "wtconv2d_pyramid": (_I, [_VP, _VP, _I, _I, _I, _I, _I, _I, _LLP, _VP]),
    "wtconv2d_weight_grad_stat_floats": (ctypes.c_size_t, [_I, _I, _I]),
    "wtconv2d_weight_grad_stats": (_I, [_VP, _VP, _VP, _VP, _VP, _I, _I, _I, _I, _I, _I, _I, _LLP, _LLP, _VP]),
    "wtconv2d_workspace_bytes": (_I, [_I, _I, _I, _I, _I, _I, _I, _LLP, _LLP, ctypes.POINTER(ctypes.c_size_t)]),
    "wtconv2d_launch_count": (_I, [_I, _I, _I, _I, _I, _I, _I, _I, _LLP, _LLP, ctypes.POINTER(_I)]),
    "wtconv2d_forward": (_I, [_VP, _VP, _VP, _VP, ctypes.c_size_t, _I, _I, _I, _I, _I, _I, _I, _I, _LLP, _LLP, _VP]),
    "wtconv2d_forward_noalloc": (_I, [_VP, _VP, _VP, _I, _I, _I, _I, _I, _I, _I, _I, _LLP, _LLP, _VP]),
    "wtconv1d_forward": (_I, [_VP, _VP, _VP, _I, _I, _I, _I, _I, _I, _I, _LLP, _LLP, _VP]),
}


class WTConvLibraryError(RuntimeError):
    pass


def load():
    """Returns the loaded library; raises WTConvLibraryError when it is not built."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None:
            if not os.path.exists(LIB_PATH):
                raise WTConvLibraryError(
                    f"{LIB_PATH} is missing: build the sm_100a kernels first "
                    "(python -m wtconv_b200.build, or __graft_entry__.build()). "
                    "There is no fallback implementation.")
            lib = ctypes.CDLL(LIB_PATH)
            for name, (res, args) in SYMBOLS.items():
                fn = getattr(lib, name)          # AttributeError if the export is missing
                fn.restype = res
                fn.argtypes = args
            _lib = lib
    return _lib


def status_string(status: int) -> str:
    return load().wtconv_status_string(int(status)).decode()


def check(status: int, what: str):
    """Maps a non-zero status to the exception a PyTorch user expects."""
    if status == 0:
        return
    msg = f"{what}: {status_string(status)} (status {status})"
    if status in (-2, -3):
        raise ValueError(msg)
    raise RuntimeError(msg)
