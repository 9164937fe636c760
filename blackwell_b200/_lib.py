"""ctypes loader for libblackwell_kernels.so.  Fails loudly when the library is
missing or does not export a symbol that ``include/blackwell_b200.h`` declares."""
from __future__ import annotations

import ctypes as C
import os
import re

HERE = os.path.dirname(os.path.abspath(__file__))
SO_PATH = os.path.join(HERE, "lib", "libblackwell_kernels.so")
HEADER = os.path.join(HERE, "..", "include", "blackwell_b200.h")

_lib = None


def declared_symbols(header: str = HEADER) -> list[str]:
    """Names of every function the C header declares."""
    text = open(header).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(bw_[a-z0-9_]+)\s*\(", text)))


def load() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(SO_PATH):
            raise ImportError(
                f"{SO_PATH} is missing: build it with `python -m blackwell_b200._build` "
                "(nvcc, sm_100a). There is no fallback path.")
        lib = C.CDLL(SO_PATH)
        missing = [s for s in declared_symbols() if not hasattr(lib, s)]
        if missing:
            raise ImportError(f"libblackwell_kernels.so does not export: {missing}")
        lib.bw_launch_count.restype = C.c_longlong
        _lib = lib
    return _lib
