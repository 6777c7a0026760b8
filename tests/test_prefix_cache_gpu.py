"""Prefix-cached prefill of the attention step (KV block pool + paged prefill kernels): a prompt
whose leading chunks are resident attends through the reused blocks and computes only its suffix;
the suffix rows equal those of a cold prefill of the same prompt, and the oracle's attention."""
import numpy as np
import pytest
import torch

import oracle
from mx230_b200 import llm_attention as la
from mx230_b200.paging import KvPool, prefill_cached
from tests.conftest import assert_close

pytestmark = pytest.mark.gpu

NH, NKV, THETA, BS = 8, 2, 1e6, 16
QD, KVD = NH * 64, NKV * 64
STRIDE = QD + 2 * KVD


def rows_of(tokens):
    """qkv row of position t as a function of tokens[0..t] only, like a causal model's activations."""
    out = np.empty((len(tokens), STRIDE), np.float32)
    hsh = 1469598103
    for t, tok in enumerate(tokens):
        hsh = (hsh * 1000003 + int(tok) + 1) % (1 << 31)
        out[t] = oracle.normal((STRIDE,), hsh, 0)
    return out


def run(handle, pool, cache, table_dev, tokens):
    rows = rows_of(tokens)
    out = torch.zeros(len(tokens), QD, device="cuda")
    stats = prefill_cached(handle, pool, cache, tokens,
                           lambda k: torch.from_numpy(rows[k:].copy()).cuda(), out, NH, NKV, THETA, table_dev)
    handle.check_status()
    return out[: len(tokens) - stats.reused_tokens].cpu().numpy(), stats


@pytest.mark.parametrize("quant", [False, True])
def test_reused_prefix_gives_the_cold_result(handle, quant):
    n_slots = 16 * BS
    rng = np.random.default_rng(5)
    a = rng.integers(0, 1000, size=45).tolist()
    b = a[:37] + rng.integers(0, 1000, size=13).tolist()

    pool, cache = KvPool(n_slots, BS), la.KvCache(n_slots, NKV, 64, quant)
    table_dev = torch.zeros(pool.n_blocks, dtype=torch.int32, device="cuda")
    out_a, st_a = run(handle, pool, cache, table_dev, a)
    assert (st_a.total_tokens, st_a.reused_tokens, st_a.reused_blocks) == (45, 0, 0)
    out_b, st_b = run(handle, pool, cache, table_dev, b)
    assert (st_b.total_tokens, st_b.reused_tokens, st_b.reused_blocks) == (50, 32, 2)
    pool.audit()

    # cold prefill of b in a fresh pool and cache
    pool2, cache2 = KvPool(n_slots, BS), la.KvCache(n_slots, NKV, 64, quant)
    out_cold, st_c = run(handle, pool2, cache2, table_dev, b)
    assert st_c.reused_tokens == 0
    np.testing.assert_array_equal(out_b, out_cold[32:])   # the same kernels on the same bytes

    # and the oracle: attention of the suffix rows over an unpaged cache built position by position
    rows = rows_of(b)
    kc, vc = np.zeros((64, KVD), np.float32), np.zeros((64, KVD), np.float32)
    q8 = oracle.Q8Cache(64, NKV)
    for t in range(len(b)):
        oracle.rope_qkv_row(rows[t], t, NH, NKV, 64, THETA)
        oracle.copy_kv_row(kc, vc, rows[t], t, QD, KVD)
        oracle.quantize_kv_row(q8, rows[t], t, QD)
    # (over the int8 cache the default score mode is the reference kernel's int8 arithmetic: oracle mode 1)
    kw = dict(cache=q8, mode=1) if quant else dict(kcache=kc, vcache=vc)
    want = oracle.prefill(rows[32:], 32, len(b) - 32, NH, NKV, STRIDE, QD, **kw)
    assert_close(out_b, want, "prefix-cached prefill vs oracle")

    # sending a again: three of its... two full chunks are resident (45 tokens = 2 chunks + 13)
    out_a2, st_a2 = run(handle, pool, cache, table_dev, a)
    assert st_a2.reused_tokens == 32
    np.testing.assert_array_equal(out_a2, out_a[32:])
    pool.audit()


def test_eviction_under_pressure_keeps_results_right(handle):
    n_slots = 6 * BS   # room for 6 blocks only
    pool, cache = KvPool(n_slots, BS), la.KvCache(n_slots, NKV, 64, True)
    table_dev = torch.zeros(pool.n_blocks, dtype=torch.int32, device="cuda")
    rng = np.random.default_rng(9)
    first = rng.integers(0, 1000, size=40).tolist()
    ref, _ = run(handle, pool, cache, table_dev, first)
    for _ in range(5):   # unrelated prompts push the first one's chunks out
        run(handle, pool, cache, table_dev, rng.integers(0, 1000, size=int(rng.integers(20, 60))).tolist())
        pool.audit()
    assert pool.evictions > 0
    again, st = run(handle, pool, cache, table_dev, first)
    np.testing.assert_array_equal(again, ref[st.reused_tokens:])
    pool.audit()
