"""ctypes access to the C restatement of the NVFP4 quantiser (oracle/nvfp4_ref.c). Test-side only."""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None


def build() -> str:
    """Compile libpkv_oracle.so next to its source (gcc; a second or so)."""
    subprocess.run(["make", "-s", "-C", _HERE, "libpkv_oracle.so"], check=True)
    return os.path.join(_HERE, "libpkv_oracle.so")


def lib():
    global _LIB
    if _LIB is None:
        path = os.path.join(_HERE, "libpkv_oracle.so")
        src = os.path.join(_HERE, "nvfp4_ref.c")
        if not os.path.exists(path) or os.path.getmtime(path) < os.path.getmtime(src):
            build()
        _LIB = ctypes.CDLL(path)
    return _LIB


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def nvfp4_quantize(x: np.ndarray, second: float, scale_up: bool = False):
    x = np.ascontiguousarray(x, dtype=np.float32)
    rows, width = x.shape
    codes = np.empty((rows, width), np.uint8)
    scales = np.empty((rows, width // 16), np.uint8)
    xhat = np.empty((rows, width), np.float32)
    fn = lib().pkv_ref_nvfp4_quantize_scale_up if scale_up else lib().pkv_ref_nvfp4_quantize
    fn(_p(x), ctypes.c_long(rows), ctypes.c_long(width), ctypes.c_float(second), _p(codes), _p(scales), _p(xhat))
    return codes, scales, xhat


def nvfp4_dequantize(codes: np.ndarray, scales: np.ndarray, second: float):
    codes = np.ascontiguousarray(codes, dtype=np.uint8)
    scales = np.ascontiguousarray(scales, dtype=np.uint8)
    rows, width = codes.shape
    out = np.empty((rows, width), np.float32)
    lib().pkv_ref_nvfp4_dequantize(_p(codes), _p(scales), ctypes.c_long(rows), ctypes.c_long(width),
                                   ctypes.c_float(second), _p(out))
    return out
