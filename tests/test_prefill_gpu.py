"""Prefill attention (n_tok new rows over the KV cache) through the C ABI vs the oracle.

Operands go through the tensor cores in bf16, so the gate is the floating-point parity bar:
max-abs 2e-2, norm-wise mean-rel 5e-3 against the oracle's fp32 result -- cpu.rs attention
over the fp32 cache; over the int8 cache both score modes, each against its own oracle on the same
(bit-exact) codes: the reference kernel's int8 scores (default, attn_prefill_q8's arithmetic) and
exact scores over the dequantised codes; and the reference's opt-in int8-score approximation over an
fp32 cache (attn_prefill_dp4a).
"""
import numpy as np
import pytest
import torch

import oracle
from mx230_b200 import _lib
from mx230_b200 import llm_attention as la
from mx230_b200._lib import check, lib, ptr
from mx230_b200.common import stream_ptr
from tests.conftest import assert_close

pytestmark = pytest.mark.gpu


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def i32(a):
    return torch.tensor(a, dtype=torch.int32, device="cuda")


CASES = [  # n_head, n_kv_head, pos0, n_tok
    (14, 2, 0, 300), (14, 2, 77, 130), (32, 4, 0, 257), (12, 12, 5, 64), (8, 2, 200, 1), (4, 4, 0, 512),
]


@pytest.mark.parametrize("quant", [False, True])
@pytest.mark.parametrize("paged", [False, True])
@pytest.mark.parametrize("nh,nkv,pos0,n_tok", CASES)
def test_prefill_matches_oracle(handle, nh, nkv, pos0, n_tok, quant, paged):
    qd, kvd, bs = nh * 64, nkv * 64, 16
    stride = qd + 2 * kvd + 64       # padded row stride, as a qkv buffer with extra columns
    out_stride = qd + 32
    n_keys = pos0 + n_tok
    rows = np.zeros((n_keys, stride), np.float32)
    rows[:, :qd + 2 * kvd] = oracle.normal((n_keys, qd + 2 * kvd), 300 + nh + pos0, 0)
    n_log = (n_keys + bs - 1) // bs
    table = (np.random.default_rng(1).permutation(n_log).astype(np.int32) + 1) if paged else None
    slots = (n_log + 1) * bs
    kc, vc = np.zeros((slots, kvd), np.float32), np.zeros((slots, kvd), np.float32)
    q8 = oracle.Q8Cache(slots, nkv)
    for t in range(n_keys):
        oracle.rope_qkv_row(rows[t], t, nh, nkv, 64, 1e6)
        oracle.copy_kv_row(kc, vc, rows[t], t, qd, kvd, table, bs)
        oracle.quantize_kv_row(q8, rows[t], t, qd, table, bs)
    c = la.KvCache(slots, nkv, 64, quant)
    new = np.ascontiguousarray(rows[pos0:])
    pg = la.Paging(i32(table), bs) if paged else None
    okw = dict(table=table, block_size=bs)
    if quant:
        c.k.copy_(dev(q8.kq)), c.v.copy_(dev(q8.vq)), c.ks.copy_(dev(q8.ks)), c.vs.copy_(dev(q8.vs))
        c.kb.copy_(dev(q8.kb)), c.vb.copy_(dev(q8.vb))
        modes = [(_lib.Q8_SCORE_REF, oracle.prefill(new, pos0, n_tok, nh, nkv, stride, out_stride, cache=q8, mode=1, **okw)),
                 (_lib.Q8_SCORE_EXACT, oracle.prefill(new, pos0, n_tok, nh, nkv, stride, out_stride, cache=q8, mode=0, **okw))]
    else:
        c.k.copy_(dev(kc)), c.v.copy_(dev(vc))
        modes = [(_lib.Q8_SCORE_REF, oracle.prefill(new, pos0, n_tok, nh, nkv, stride, out_stride, kcache=kc, vcache=vc, **okw))]
    try:
        for mode, want in modes:
            handle.set_option(_lib.OPT_Q8_SCORE_MODE, mode)
            out = torch.zeros(n_tok, out_stride, device="cuda")
            la.attn_prefill(handle, out, dev(new), c, pos0, n_tok, nh, nkv, stride, out_stride, pg)
            handle.check_status()
            got = out.cpu().numpy()
            assert_close(got[:, :qd], want[:, :qd], f"prefill, score mode {mode}")
            assert (got[:, qd:] == 0).all()  # the padding columns of the output rows are not touched
    finally:
        handle.set_option(_lib.OPT_Q8_SCORE_MODE, _lib.Q8_SCORE_REF)
    if not quant:
        # attn_prefill_dp4a[_paged]: int8 scores with K quantised on the fly, over the same fp32 cache
        want = oracle.prefill(new, pos0, n_tok, nh, nkv, stride, out_stride, kcache=kc, vcache=vc, mode=1, **okw)
        out = torch.zeros(n_tok, out_stride, device="cuda")
        args = [handle._h, stream_ptr(None), ptr(out), ptr(dev(new)), ptr(c.k), ptr(c.v), pos0, n_tok, nh, nkv, stride,
                out_stride]
        if paged:
            check(lib().mx230_attn_prefill_dp4a_paged(*args, ptr(pg.table_dev), bs))
        else:
            check(lib().mx230_attn_prefill_dp4a(*args))
        handle.check_status()
        assert_close(out.cpu().numpy()[:, :qd], want[:, :qd], "prefill dp4a")


def test_prefill_step_writes_cache_then_attends(handle):
    """RoPE -> KV write -> attention on the device for a chunk that follows 40 cached tokens."""
    nh, nkv, pos0, n_tok, theta = 14, 2, 40, 100, 1e6
    qd, kvd = nh * 64, nkv * 64
    stride = qd + 2 * kvd
    raw = oracle.normal((pos0 + n_tok, stride), 400, 0)
    c = la.KvCache(pos0 + n_tok, nkv, 64, True)
    d = dev(raw)
    out0 = torch.zeros(pos0, qd, device="cuda")
    la.prefill_step(handle, out0, d[:pos0], c, 0, pos0, nh, nkv, 64, theta, stride, qd)
    out = torch.zeros(n_tok, qd, device="cuda")
    la.prefill_step(handle, out, d[pos0:], c, pos0, n_tok, nh, nkv, 64, theta, stride, qd)
    handle.check_status()
    # oracle on the device's RoPE output so that the int8 codes agree bit for bit
    roped = d.cpu().numpy()
    w = oracle.Q8Cache(pos0 + n_tok, nkv)
    for t in range(pos0 + n_tok):
        oracle.quantize_kv_row(w, roped[t], t, qd)
    assert np.array_equal(c.k.cpu().numpy(), w.kq) and np.array_equal(c.v.cpu().numpy(), w.vq)
    want = oracle.prefill(roped[pos0:], pos0, n_tok, nh, nkv, stride, qd, cache=w, mode=1)
    assert_close(out.cpu().numpy(), want, "prefill step")
    # the last prefill row equals a decode step at the same position: both use the reference's int8 score arithmetic
    o1 = torch.zeros(qd, device="cuda")
    la.attn_decode(handle, o1, d[pos0 + n_tok - 1], c, pos0 + n_tok - 1, nh, nkv, 64)
    assert_close(out[-1].cpu().numpy(), o1.cpu().numpy(), "prefill row vs decode")


@pytest.mark.parametrize("scale", [1.0, 6.0])
def test_prefill_fp32_cache_small_and_large_scores(handle, scale):
    """The staging kernels leave the row norms of Q and K; bounded scores (scale 1) let the attention kernel run without
    a row max, large ones (scale 6: |q . k| / 8 * log2(e) far above 80) must take the running-max path.  Both against
    the oracle; the inputs are bf16-representable after staging so that at large scores the comparison is not about
    the rounding of q and k."""
    nh, nkv, pos0, n_tok = 8, 2, 40, 260
    qd, kvd = nh * 64, nkv * 64
    stride = qd + 2 * kvd
    n_keys = pos0 + n_tok
    bf = lambda x: torch.from_numpy(np.ascontiguousarray(x, np.float32)).to(torch.bfloat16).float().numpy()
    c = np.float32(0.125 * 1.4426950408889634)
    rows = oracle.normal((n_keys, stride), 555, 0)
    rows[:, :qd] = bf(scale * rows[:, :qd] * c) / c     # q is staged as q * scale * log2(e)
    rows[:, qd:] = bf(np.concatenate([scale * rows[:, qd:qd + kvd], rows[:, qd + kvd:]], axis=1))
    rows = rows.astype(np.float32)
    kc, vc = np.zeros((n_keys, kvd), np.float32), np.zeros((n_keys, kvd), np.float32)
    for t in range(n_keys):
        oracle.copy_kv_row(kc, vc, rows[t], t, qd, kvd)
    cch = la.KvCache(n_keys, nkv)
    cch.k.copy_(dev(kc)), cch.v.copy_(dev(vc))
    new = np.ascontiguousarray(rows[pos0:])
    want = oracle.prefill(new, pos0, n_tok, nh, nkv, stride, qd, kcache=kc, vcache=vc)
    out = torch.zeros(n_tok, qd, device="cuda")
    la.attn_prefill(handle, out, dev(new), cch, pos0, n_tok, nh, nkv, stride, qd)
    handle.check_status()
    assert_close(out.cpu().numpy(), want, f"prefill, score scale {scale}")
