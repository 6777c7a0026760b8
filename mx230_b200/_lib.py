"""ctypes binding of libmx230_attn.so: one prototype per symbol of include/mx230_attn.h.

The library is mandatory: loading fails loudly when it has not been built, and every
call raises on a non-zero status (the reference panics on a failed launch,
02-flash-attention/src/main.rs:50,87).  There is no CPU or PyTorch fallback.
"""
from __future__ import annotations

import ctypes as C
import os
import re

PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG, "libmx230_attn.so")
HEADER = os.path.join(os.path.dirname(PKG), "include", "mx230_attn.h")

OK = 0
ERR_INVALID_ARG, ERR_UNSUPPORTED, ERR_WORKSPACE, ERR_CUDA, ERR_DEVICE_STATUS, ERR_NO_DEVICE = range(1, 7)
Q8_SCORE_REF, Q8_SCORE_EXACT = 0, 1
OPT_Q8_SCORE_MODE, OPT_DECODE_CHUNK, OPT_DECODE_TENSOR, OPT_BWD_TWO_PASS = 1, 2, 3, 4
OPT_BWD_REUSE_STAGED, OPT_WAIT_LIMIT, OPT_TEST_DROP_TILE = 5, 6, 7
K_COUNT = 14


class Mx230Error(RuntimeError):
    def __init__(self, code: int, msg: str):
        super().__init__(f"mx230 status {code}: {msg}")
        self.code = code


_CTYPE = {
    "int": C.c_int, "float": C.c_float, "size_t": C.c_size_t, "long long": C.c_longlong, "void": None, "uint32_t": C.c_uint32,
    "uint64_t": C.c_uint64,
}


def _parse_type(t: str):
    t = t.replace("const", "").strip()
    if t.endswith("**"):
        return C.POINTER(C.c_void_p)
    if t.endswith("*"):
        return C.c_void_p
    return _CTYPE[t]


def declared_functions(header: str = HEADER) -> dict[str, tuple[str, list[str]]]:
    """name -> (return type, [argument types]) for every prototype in the C header."""
    text = open(header).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    protos = {}
    for m in re.finditer(r"\n((?:const\s+)?[\w ]+?[\s\*]+)(mx230_\w+)\s*\(([^;{]*?)\)\s*;", text):
        ret, name, args = m.group(1).strip(), m.group(2), m.group(3)
        argt = []
        for a in args.split(","):
            a = " ".join(a.split())
            if a in ("void", ""):
                continue
            mm = re.match(r"(.*?)(\w+)$", a)
            argt.append(mm.group(1).strip())
        protos[name] = (ret, argt)
    return protos


_lib = None


def lib() -> C.CDLL:
    """Loads the shared library (building nothing): raises if it is missing."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m mx230_b200.build` "
                "(nvcc, sm_100a). There is no fallback path.")
        L = C.CDLL(LIB_PATH)
        for name, (ret, argt) in declared_functions().items():
            fn = getattr(L, name)
            fn.argtypes = [_parse_type(a) for a in argt]
            if ret.replace("const", "").strip().endswith("*"):
                fn.restype = C.c_char_p
            else:
                fn.restype = _CTYPE[ret]
        _lib = L
    return _lib


def check(code: int) -> None:
    if code != OK:
        raise Mx230Error(code, lib().mx230_last_error().decode())


def ptr(t) -> C.c_void_p | None:
    """Device (or host) address of a torch tensor / numpy array / int / None."""
    if t is None:
        return None
    if isinstance(t, int):
        return C.c_void_p(t)
    if hasattr(t, "data_ptr"):
        return C.c_void_p(t.data_ptr())
    return C.c_void_p(t.ctypes.data)
