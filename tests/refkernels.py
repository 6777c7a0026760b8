"""Launcher for the reference project's own CUDA kernels (test infrastructure).

`oracle/build.py` compiles the reference's unmodified attention-path `.cu` files into
cubins under `oracle/_ref/`.  This module loads such a cubin with the CUDA driver API
(plain ctypes on libcuda) into torch's primary context and launches kernels by their C
symbol name with the reference's own grid/block shapes, exactly as its Rust host does
through cudarc (02-flash-attention/src/main.rs:80-87).  Used only to pin the oracle
against the real reference on a GPU; skipped when `oracle/_ref` is absent.
"""
from __future__ import annotations

import ctypes as C
import os

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_DIR = os.path.join(ROOT, "oracle", "_ref")


def available(name: str) -> bool:
    return os.path.exists(os.path.join(REF_DIR, name + ".cubin"))


class RefModule:
    def __init__(self, name: str):
        import torch
        torch.cuda.init()
        torch.zeros(1, device="cuda")  # make the primary context current
        self.cu = C.CDLL("libcuda.so.1")
        data = open(os.path.join(REF_DIR, name + ".cubin"), "rb").read()
        self._image = C.create_string_buffer(data, len(data))
        self.mod = C.c_void_p()
        self._check(self.cu.cuModuleLoadData(C.byref(self.mod), self._image), "cuModuleLoadData")
        self._fn = {}

    def _check(self, rc, what):
        if rc != 0:
            raise RuntimeError(f"{what} failed with CUresult {rc}")

    def function(self, sym: str):
        if sym not in self._fn:
            f = C.c_void_p()
            self._check(self.cu.cuModuleGetFunction(C.byref(f), self.mod, sym.encode()),
                        f"cuModuleGetFunction({sym})")
            self._fn[sym] = f
        return self._fn[sym]

    def launch(self, sym: str, grid, block, args, stream=None, smem: int = 0):
        """args: torch CUDA tensors (passed as device pointers), Python ints (int32) or floats (f32)."""
        import torch
        store, ptrs = [], []
        for a in args:
            if hasattr(a, "data_ptr"):
                v = C.c_void_p(a.data_ptr())
            elif isinstance(a, float):
                v = C.c_float(a)
            else:
                v = C.c_int(int(a))
            store.append(v)
            ptrs.append(C.cast(C.pointer(v), C.c_void_p))
        arr = (C.c_void_p * len(ptrs))(*ptrs)
        g = tuple(grid) + (1,) * (3 - len(grid))
        b = tuple(block) + (1,) * (3 - len(block))
        s = stream if stream is not None else torch.cuda.current_stream()
        rc = self.cu.cuLaunchKernel(self.function(sym), *[C.c_uint(x) for x in g],
                                    *[C.c_uint(x) for x in b], C.c_uint(smem),
                                    C.c_void_p(s.cuda_stream), arr, None)
        self._check(rc, f"cuLaunchKernel({sym})")
