"""ctypes binding of ``libgguftrain_cuda.so``.

The prototypes are read from ``include/gguftrain.h`` so the binding cannot drift from the declared
ABI. There is no fallback: when the shared library is missing or fails to load, importing the
backend raises.
"""
from __future__ import annotations

import ctypes as C
import os
import re

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "csrc", "libgguftrain_cuda.so")
HEADER_PATH = os.path.join(os.path.dirname(_PKG), "include", "gguftrain.h")

_TYPES = {
    "gt_ctx*": C.c_void_p, "gt_ctx**": C.POINTER(C.c_void_p), "gt_buf": C.c_uint64, "gt_buf*": C.POINTER(C.c_uint64),
    "const gt_buf*": C.POINTER(C.c_uint64), "int32_t": C.c_int32, "int32_t*": C.POINTER(C.c_int32),
    "const int32_t*": C.POINTER(C.c_int32), "uint64_t": C.c_uint64, "uint64_t*": C.POINTER(C.c_uint64),
    "const uint64_t*": C.POINTER(C.c_uint64), "float": C.c_float, "float*": C.POINTER(C.c_float), "double": C.c_double,
    "const void*": C.c_void_p, "void*": C.c_void_p, "char*": C.c_char_p, "const uint8_t*": C.c_void_p,
    "uint8_t*": C.c_void_p, "uint32_t*": C.POINTER(C.c_uint32),
}


def declared_functions(header_path: str = HEADER_PATH):
    """[(name, restype_str, [argtype_str...])] for every function the header declares."""
    text = open(header_path).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    out = []
    for m in re.finditer(r"(gt_status|const char\*)\s+(gt_\w+)\s*\(([^)]*)\)\s*;", text):
        ret, name, args = m.group(1), m.group(2), m.group(3)
        types = []
        for a in args.split(","):
            a = a.strip()
            if not a or a == "void":
                continue
            mm = re.match(r"(.*?)(\w+)$", a)
            t = mm.group(1).strip().replace(" *", "*")
            types.append(t)
        out.append((name, ret, types))
    return out


class GtError(RuntimeError):
    def __init__(self, code, msg):
        super().__init__(msg)
        self.code = code


_lib = None


def load():
    """Load the shared library and attach prototypes. Raises if it is absent."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python {os.path.join(_PKG, 'csrc', 'build.py')}` "
            "(needs nvcc). There is no CPU fallback.")
    lib = C.CDLL(LIB_PATH)
    for name, ret, types in declared_functions():
        fn = getattr(lib, name)
        fn.restype = C.c_char_p if ret.startswith("const char") else C.c_int32
        fn.argtypes = [_TYPES[t] for t in types]
    _lib = lib
    return lib
