"""ctypes loader of the C part of the oracle (oracle/nm24_oracle.c). Test infrastructure only."""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_build", "libnm24_oracle.so")


def _lib():
    if not os.path.exists(_SO):
        subprocess.run(["make", "-s", "-C", _HERE], check=True)
    lib = ctypes.CDLL(_SO)
    lib.nm24_project.restype = None
    lib.nm24_project.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64, ctypes.c_void_p, ctypes.c_void_p]
    return lib


def project(soft: np.ndarray):
    """(hard float32 [rows, cols], meta uint8 [rows, ceil(cols/8)]) of a float32 matrix."""
    soft = np.ascontiguousarray(soft, dtype=np.float32)
    rows, cols = soft.shape
    hard = np.empty_like(soft)
    meta = np.zeros((rows, (cols + 7) // 8), dtype=np.uint8)
    _lib().nm24_project(soft.ctypes.data, rows, cols, hard.ctypes.data, meta.ctypes.data)
    return hard, meta
