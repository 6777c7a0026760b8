"""Host side of paged attention: the KV block pool with its prefix tree, and the prefix-cached
prefill of the attention step.

Mirror of `Paging` / `RadixCache` (03-llm-engine/src/gpu.rs:211-343,372-539) and of
`Engine::prefill_cached` (gpu.rs:2273-2345) over the C ABI's `mx230_kv_pool_*` functions.  The
reference runs the whole model inside `prefill`; this package owns only the attention step, so the
caller supplies the qkv rows of the tokens that still have to be computed.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np

from ._lib import check, lib

KV_BLOCK = 16  # gpu.rs:209


@dataclass
class PrefixStats:
    """PrefixStats, gpu.rs:346-351."""
    total_tokens: int
    reused_tokens: int
    reused_blocks: int


def _tok(tokens):
    a = np.ascontiguousarray(tokens, dtype=np.uint32)
    return a, a.ctypes.data_as(C.c_void_p)


class KvPool:
    """`Paging::new` (prefix_cache=False) or `Paging::new_pool` (prefix_cache=True) over `n_slots`
    cache positions."""

    def __init__(self, n_slots: int, block_size: int = KV_BLOCK, prefix_cache: bool = True):
        self._p = C.c_void_p()
        check(lib().mx230_kv_pool_create(C.byref(self._p), n_slots, block_size, int(prefix_cache)))
        self.block_size, self.prefix_cache = block_size, prefix_cache
        self.n_blocks = lib().mx230_kv_pool_n_blocks(self._p)

    def close(self):
        if self._p:
            lib().mx230_kv_pool_destroy(self._p)
            self._p = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # ---- observers
    @property
    def free_blocks(self) -> int:
        return lib().mx230_kv_pool_free_blocks(self._p)

    @property
    def cached_blocks(self) -> int:
        return lib().mx230_kv_pool_cached_blocks(self._p)

    @property
    def evictions(self) -> int:
        return lib().mx230_kv_pool_evictions(self._p)

    def refcount(self, block: int) -> int:
        return lib().mx230_kv_pool_refcount(self._p, block)

    def table(self, n: int | None = None) -> np.ndarray:
        n = self.n_blocks if n is None else n
        out = np.empty(n, np.int32)
        check(lib().mx230_kv_pool_table(self._p, out.ctypes.data_as(C.c_void_p), n))
        return out

    def phys_row(self, t: int) -> int:
        return lib().mx230_kv_pool_phys_row(self._p, t)

    def audit(self) -> None:
        check(lib().mx230_kv_pool_audit(self._p))

    # ---- primitives
    def alloc(self) -> int:
        b = C.c_int(-1)
        check(lib().mx230_kv_pool_alloc(self._p, C.byref(b)))
        return b.value

    def incref(self, block: int) -> None:
        check(lib().mx230_kv_pool_incref(self._p, block))

    def decref(self, block: int) -> None:
        check(lib().mx230_kv_pool_decref(self._p, block))

    def evict(self) -> int:
        b = C.c_int(-1)
        check(lib().mx230_kv_pool_evict(self._p, C.byref(b)))
        return b.value

    def lookup(self, tokens) -> list[int]:
        a, pa = _tok(tokens)
        out = np.empty(max(1, a.size // self.block_size), np.int32)
        n = C.c_int(0)
        check(lib().mx230_kv_pool_lookup(self._p, pa, a.size, out.ctypes.data_as(C.c_void_p), out.size, C.byref(n)))
        return out[:n.value].tolist()

    def insert(self, tokens, blocks) -> list[int]:
        a, pa = _tok(tokens)
        b = np.ascontiguousarray(blocks, dtype=np.int32)
        out = np.empty(max(1, b.size), np.int32)
        n = C.c_int(0)
        check(lib().mx230_kv_pool_insert(self._p, pa, a.size, b.ctypes.data_as(C.c_void_p), b.size,
                                         out.ctypes.data_as(C.c_void_p), out.size, C.byref(n)))
        return out[:n.value].tolist()

    # ---- request protocol
    def begin_request(self, tokens) -> int:
        """Match + borrow + claim; returns the number of leading positions already resident."""
        a, pa = _tok(tokens)
        k = C.c_int(0)
        check(lib().mx230_kv_pool_begin_request(self._p, pa, a.size, C.byref(k)))
        return k.value

    def end_request(self, tokens) -> None:
        a, pa = _tok(tokens)
        check(lib().mx230_kv_pool_end_request(self._p, pa, a.size))

    def abort_request(self) -> None:
        """Drops the open request without letting the tree adopt its (unwritten) blocks."""
        check(lib().mx230_kv_pool_abort_request(self._p))


def prefill_cached(h, pool: KvPool, cache, tokens, qkv_rows, out, n_head, n_kv_head, theta,
                   table_dev, use_rope=True, stream=None) -> PrefixStats:
    """The attention step of `prefill_cached` (gpu.rs:2273-2345): the KV of the longest cached
    whole-chunk prefix of `tokens` is reused through the block table, only the suffix is written and
    attended.  `qkv_rows(k)` returns the device tensor [n - k][q_dim + 2 kv_dim] of the suffix rows
    (positions k .. n-1); the attention of those rows goes to `out[: n - k]`.  `table_dev` is an int32
    device tensor of at least ceil(n / block) entries that receives the block table."""
    import torch
    from . import llm_attention as la
    n = len(tokens)
    k = pool.begin_request(tokens)
    try:
        n_log = -(-n // pool.block_size)
        table_dev[:n_log].copy_(torch.from_numpy(pool.table(n_log)), non_blocking=False)
        pg = la.Paging(table_dev, pool.block_size)
        rows = qkv_rows(k)
        stride = rows.shape[-1]
        la.prefill_step(h, out, rows, cache, k, n - k, n_head, n_kv_head, 64, theta, stride, out.shape[-1],
                        pg, use_rope, stream)
    except BaseException:
        # the KV rows of the fresh blocks were not (all) enqueued: the tree must not adopt them
        pool.abort_request()
        raise
    # only now, with RoPE -> KV write -> attention enqueued, may the tree take over the new full chunks
    pool.end_request(tokens)
    return PrefixStats(n, k, k // pool.block_size)
