"""Loader for libsalt_gpu_b200.so.  There is no fallback of any kind: if the
shared library has not been built, loading raises."""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libsalt_gpu_b200.so")
_lib = None


def library_path() -> str:
    """Absolute path of the built shared library (for hosts that link it directly)."""
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(f"{LIB_PATH} is missing: build it with `python salt-core_b200/build.py`")
    return LIB_PATH


def load_library() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python salt-core_b200/build.py` "
                "(there is no CPU or PyTorch fallback for this path)")
        _lib = C.CDLL(LIB_PATH)
    return _lib
