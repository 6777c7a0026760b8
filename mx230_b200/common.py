"""Runtime utilities mirroring the reference's `common` crate (common/src/lib.rs):
the library handle (in place of `load_ptx`), the CUDA-event median timer, the two
error metrics and the xorshift64* generator."""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib
from ._lib import check, lib, ptr


class Handle:
    """Per-device library state: replaces CudaContext + the loaded-module tables
    (common/src/lib.rs:11-18; 02-flash-attention/src/main.rs:392-415)."""

    def __init__(self, device: int = 0, workspace_bytes: int = 0):
        self._h = C.c_void_p()
        check(lib().mx230_create(C.byref(self._h), device, workspace_bytes))
        self.device = device

    def reserve(self, nbytes: int) -> None:
        check(lib().mx230_reserve(self._h, nbytes))

    def set_option(self, option: int, value: int) -> None:
        check(lib().mx230_set_option(self._h, option, value))

    def check_status(self, stream=None) -> None:
        check(lib().mx230_check_status(self._h, stream_ptr(stream)))

    # per-kernel device timing (the reference's opt-in prof_*_us attribution, gpu.rs:1922-1928)
    def profile_enable(self, on: bool = True) -> None:
        check(lib().mx230_profile_enable(self._h, int(on)))

    def profile_reset(self) -> None:
        check(lib().mx230_profile_reset(self._h))

    def profile_read(self) -> dict:
        """kernel name -> (launches, total device ms) since the last reset."""
        out = {}
        for k in range(_lib.K_COUNT):
            n, ms = C.c_longlong(), C.c_double()
            check(lib().mx230_profile_read(self._h, k, C.byref(n), C.byref(ms)))
            if n.value:
                out[lib().mx230_kernel_name(k).decode()] = (int(n.value), float(ms.value))
        return out

    @property
    def launches(self) -> int:
        return int(lib().mx230_launch_count(self._h))

    def close(self) -> None:
        if self._h:
            lib().mx230_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def stream_ptr(stream=None):
    """Raw CUstream of a torch stream (None = torch's current stream)."""
    if isinstance(stream, int):
        return C.c_void_p(stream)
    import torch
    s = stream if stream is not None else torch.cuda.current_stream()
    return C.c_void_p(s.cuda_stream)


def time_median_ms(stream, warmup: int, iters: int, f) -> float:
    """common/src/lib.rs:22-43: warm-up, then one CUDA-event pair per iteration on
    the launching stream, median in milliseconds."""
    import torch
    s = stream if stream is not None else torch.cuda.current_stream()
    for _ in range(warmup):
        f()
    s.synchronize()
    times = []
    for _ in range(iters):
        a = torch.cuda.Event(enable_timing=True)
        b = torch.cuda.Event(enable_timing=True)
        a.record(s)
        f()
        b.record(s)
        b.synchronize()
        times.append(a.elapsed_time(b))
    times.sort()
    return times[len(times) // 2]


def max_rel_err(got, want) -> float:
    """common/src/lib.rs:46-53"""
    g = np.asarray(got, np.float32).ravel()
    w = np.asarray(want, np.float32).ravel()
    return float(np.max(np.abs(g - w) / np.maximum(np.abs(w), np.float32(1e-6)))) if g.size else 0.0


def allclose_err(got, want, rtol: float, atol: float) -> float:
    """common/src/lib.rs:58-64: max |g - w| / (atol + rtol |w|); <= 1 passes allclose."""
    g = np.asarray(got, np.float32).ravel()
    w = np.asarray(want, np.float32).ravel()
    if g.size == 0:
        return 0.0
    return float(np.max(np.abs(g - w) / (np.float32(atol) + np.float32(rtol) * np.abs(w))))


def pseudo_rand(n: int, seed: int) -> np.ndarray:
    """common/src/lib.rs:67-78: xorshift64* uniform in [-1, 1) (host code of the library)."""
    out = np.empty(n, np.float32)
    check(lib().mx230_pseudo_rand(out.ctypes.data_as(C.c_void_p), n, seed))
    return out


def normal(shape, seed: int, tensor_index: int) -> np.ndarray:
    """Seeded N(0,1) inputs for benchmarks and tests: the xorshift64* stream of `pseudo_rand`, started at
    splitmix64(seed * 16 + tensor_index), through Box-Muller in double precision."""
    out = np.empty(int(np.prod(shape)), np.float32)
    check(lib().mx230_fill_normal(out.ctypes.data_as(C.c_void_p), out.size, seed, tensor_index))
    return out.reshape(shape)


__all__ = ["Handle", "stream_ptr", "time_median_ms", "max_rel_err", "allclose_err", "pseudo_rand", "normal",
           "_lib"]
