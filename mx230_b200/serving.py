"""Continuous batching over the batched decode attention step.

Mirror of `Engine::run_continuous` (03-llm-engine/src/gpu.rs:3800-3915) on the C ABI's
`mx230_sched_*` state machine.  The reference scheduler is welded to its model; here the model is
whatever the caller passes in: an object with

    prefill(request_index, prompt_tokens, table: np.ndarray[int32, n_log]) -> int   # first generated token
    decode_batched(cur: np.ndarray[uint32, n], pos: np.ndarray[int32, n],
                   tables: np.ndarray[int32, n x n_log]) -> sequence of n next tokens

whose attention runs through `llm_attention.prefill_step` / `batched_step` with those block tables.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np

from ._lib import check, lib
from .paging import KvPool


@dataclass
class Request:
    """Request, gpu.rs:356-359."""
    prompt: list
    max_new: int


@dataclass
class ServeStats:
    """ServeStats, gpu.rs:366-370."""
    decode_steps: int = 0
    seq_decodes: int = 0
    admitted: int = 0


class Scheduler:
    def __init__(self, pool: KvPool, n_ctx: int, max_batch: int, requests: list[Request]):
        self._s = C.c_void_p()
        self.pool, self.max_batch, self.n_req = pool, max_batch, len(requests)
        pl = np.ascontiguousarray([len(r.prompt) for r in requests], np.int32)
        mn = np.ascontiguousarray([r.max_new for r in requests], np.int32)
        check(lib().mx230_sched_create(C.byref(self._s), pool._p, n_ctx, max_batch,
                                       pl.ctypes.data_as(C.c_void_p), mn.ctypes.data_as(C.c_void_p), len(requests)))
        self.n_log = lib().mx230_sched_n_log(self._s)

    def close(self):
        if self._s:
            lib().mx230_sched_destroy(self._s)
            self._s = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def admit(self):
        """(request index, block table) of the next admission, or None."""
        r = C.c_int(-1)
        table = np.empty(self.n_log, np.int32)
        check(lib().mx230_sched_admit(self._s, C.byref(r), table.ctypes.data_as(C.c_void_p)))
        return None if r.value < 0 else (r.value, table)

    def admitted(self, request: int, first_token: int) -> None:
        check(lib().mx230_sched_admitted(self._s, request, int(first_token)))

    def batch(self):
        """(cur, pos, tables) of the active set; cur is empty when everything has been served."""
        n = C.c_int(0)
        cur = np.empty(self.max_batch, np.uint32)
        pos = np.empty(self.max_batch, np.int32)
        tables = np.empty((self.max_batch, self.n_log), np.int32)
        check(lib().mx230_sched_batch(self._s, C.byref(n), cur.ctypes.data_as(C.c_void_p),
                                      pos.ctypes.data_as(C.c_void_p), tables.ctypes.data_as(C.c_void_p)))
        return cur[:n.value], pos[:n.value], tables[:n.value]

    def step_done(self, next_tokens) -> None:
        nt = np.ascontiguousarray(next_tokens, np.uint32)
        check(lib().mx230_sched_step_done(self._s, nt.ctypes.data_as(C.c_void_p)))

    def result(self, request: int) -> list[int]:
        n = C.c_int(0)
        check(lib().mx230_sched_result(self._s, request, None, 0, C.byref(n)))
        out = np.empty(max(1, n.value), np.uint32)
        check(lib().mx230_sched_result(self._s, request, out.ctypes.data_as(C.c_void_p), out.size, C.byref(n)))
        return out[:n.value].tolist()

    def stats(self) -> ServeStats:
        f = lib().mx230_sched_stat
        return ServeStats(f(self._s, 0), f(self._s, 1), f(self._s, 2))


def run_continuous(model, pool: KvPool, n_ctx: int, requests: list[Request], max_batch: int, trace=None):
    """Serves `requests` keeping up to `max_batch` sequences decoding together; returns each
    request's generated tokens (request order) and the occupancy statistics.  `trace`, when given,
    receives one tuple per event (for tests)."""
    s = Scheduler(pool, n_ctx, max_batch, requests)
    try:
        while True:
            while (adm := s.admit()) is not None:
                r, table = adm
                first = model.prefill(r, requests[r].prompt, table)
                if trace is not None:
                    trace.append(("admit", r, table.tolist(), int(first)))
                s.admitted(r, first)
            cur, pos, tables = s.batch()
            if cur.size == 0:
                break
            nxt = model.decode_batched(cur.copy(), pos.copy(), tables.copy())
            if trace is not None:
                trace.append(("step", cur.tolist(), pos.tolist(), tables.tolist(), [int(x) for x in nxt]))
            s.step_done(nxt)
        return [s.result(r) for r in range(len(requests))], s.stats()
    finally:
        s.close()
