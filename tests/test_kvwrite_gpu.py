"""RoPE, fp32 KV copy and int8 quantize-on-write through the C ABI vs the oracle.

int8 codes, scales and betas must be BIT-EXACT (03-llm-engine/kernels/llm.cu:1137-1149);
the copy is exact; RoPE is floating point: tolerance 1e-4 at small positions and 5e-3
absolute at position ~2047 (a 1-ulp difference in the f32 frequency moves the angle by
pos * 2^-24; the reference's own GPU kernel uses fast intrinsics and is looser still).
"""
import numpy as np
import pytest
import torch

import oracle
from mx230_b200 import llm_attention as la

pytestmark = pytest.mark.gpu


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def i32(a):
    return torch.tensor(a, dtype=torch.int32, device="cuda")


@pytest.mark.parametrize("nh,nkv,theta", [(14, 2, 1e6), (32, 4, 1e4), (12, 12, 1e4)])
def test_rope_variants(handle, nh, nkv, theta):
    stride = (nh + 2 * nkv) * 64
    rows = oracle.normal((6, stride), 21, 0)
    for pos, tol in ((0, 1e-6), (37, 1e-4), (2047, 5e-3)):
        want = oracle.rope_qkv_row(rows[0].copy(), pos, nh, nkv, 64, theta)
        d = dev(rows[0])
        la.rope(handle, d, pos, nh, nkv, 64, theta)
        assert np.abs(d.cpu().numpy() - want).max() <= tol, pos
        assert np.array_equal(d.cpu().numpy()[(nh + nkv) * 64:], rows[0][(nh + nkv) * 64:])  # V untouched
        d2 = dev(rows[0])
        la.rope_dyn(handle, d2, i32([pos]), nh, nkv, 64, theta)
        assert torch.equal(d, d2)
    # batch: rows at pos0 + t; seqpos: rows at pos[s]
    want = np.stack([oracle.rope_qkv_row(rows[t].copy(), 11 + t, nh, nkv, 64, theta) for t in range(6)])
    d = dev(rows)
    la.rope_batch(handle, d, 11, 6, nh, nkv, 64, stride, theta)
    assert np.abs(d.cpu().numpy() - want).max() <= 1e-4
    pos = [5, 0, 63, 17, 2, 40]
    want = np.stack([oracle.rope_qkv_row(rows[t].copy(), pos[t], nh, nkv, 64, theta) for t in range(6)])
    d = dev(rows)
    la.rope_seqpos(handle, d, i32(pos), 6, nh, nkv, 64, stride, theta)
    assert np.abs(d.cpu().numpy() - want).max() <= 1e-4
    handle.check_status()


def _rows(nh, nkv, n, seed):
    r = oracle.normal((n, (nh + 2 * nkv) * 64), seed, 0)
    r[1, nh * 64:nh * 64 + 64] = 0.25     # constant K head: hi == lo -> scale 1
    r[2, (nh + nkv) * 64:(nh + nkv) * 64 + 64] = 0.0  # zero V head
    r[3, nh * 64] = 1e4                   # outlier
    r[3, nh * 64 + 1] = -3e-5
    return r


def _q8_equal(c: la.KvCache, w: oracle.Q8Cache):
    assert np.array_equal(c.k.cpu().numpy(), w.kq), "K codes differ"
    assert np.array_equal(c.v.cpu().numpy(), w.vq), "V codes differ"
    assert np.array_equal(c.ks.cpu().numpy(), w.ks) and np.array_equal(c.vs.cpu().numpy(), w.vs), "scales differ"
    if w.affine:
        assert np.array_equal(c.kb.cpu().numpy(), w.kb) and np.array_equal(c.vb.cpu().numpy(), w.vb), "betas differ"


@pytest.mark.parametrize("affine", [True, False])
@pytest.mark.parametrize("nh,nkv", [(14, 2), (32, 4), (12, 12)])
def test_quantize_kv_bit_exact_all_variants(handle, nh, nkv, affine):
    n, bs = 40, 16
    qd = nh * 64
    rows = _rows(nh, nkv, n, 22)
    stride = rows.shape[1]
    drows = dev(rows)
    n_log = (n + bs - 1) // bs
    table = (np.arange(n_log, dtype=np.int32)[::-1] + 1).copy()  # non-identity block table
    slots = (n_log + 1) * bs
    # linear: single (host pos), dyn (device pos), batch
    w = oracle.Q8Cache(slots, nkv, 64, affine)
    for t in range(n):
        oracle.quantize_kv_row(w, rows[t], t, qd)
    c = la.KvCache(slots, nkv, 64, True, affine)
    for t in range(0, n, 2):
        la.quantize_kv(handle, c, drows[t], t, qd, nkv, 64)
        la.quantize_kv_dyn(handle, c, drows[t + 1], i32([t + 1]), qd, nkv, 64)
    _q8_equal(c, w)
    c2 = la.KvCache(slots, nkv, 64, True, affine)
    la.quantize_kv_batch(handle, c2, drows, 0, n, qd, nkv, 64, stride)
    _q8_equal(c2, w)
    # paged: batch_paged, paged_dyn, seqpos
    wp = oracle.Q8Cache(slots, nkv, 64, affine)
    for t in range(n):
        oracle.quantize_kv_row(wp, rows[t], t, qd, table, bs)
    pg = la.Paging(i32(table), bs)
    c3 = la.KvCache(slots, nkv, 64, True, affine)
    la.quantize_kv_batch(handle, c3, drows, 0, n, qd, nkv, 64, stride, pg)
    _q8_equal(c3, wp)
    c4 = la.KvCache(slots, nkv, 64, True, affine)
    for t in range(n):
        la.quantize_kv_paged_dyn(handle, c4, drows[t], i32([t]), qd, nkv, 64, pg)
    _q8_equal(c4, wp)
    # seqpos: 3 sequences, each with its own table row and position
    tables = np.stack([table, np.roll(table, 1), np.roll(table, 2)]).astype(np.int32)
    pos = [7, 33, 16]
    ws = oracle.Q8Cache(slots, nkv, 64, affine)
    for s in range(3):
        oracle.quantize_kv_row(ws, rows[s], pos[s], qd, tables[s], bs)
    c5 = la.KvCache(slots, nkv, 64, True, affine)
    la.quantize_kv_seqpos(handle, c5, drows, i32(pos), 3, qd, nkv, 64, stride, la.Paging(i32(tables), bs))
    _q8_equal(c5, ws)
    handle.check_status()


def test_copy_kv_all_variants(handle):
    nh, nkv, n, bs = 14, 2, 40, 16
    qd, kvd = nh * 64, nkv * 64
    rows = _rows(nh, nkv, n, 23)
    stride = rows.shape[1]
    drows = dev(rows)
    n_log = (n + bs - 1) // bs
    table = (np.arange(n_log, dtype=np.int32)[::-1] + 1).copy()
    slots = (n_log + 1) * bs
    wk, wv = np.zeros((slots, kvd), np.float32), np.zeros((slots, kvd), np.float32)
    for t in range(n):
        oracle.copy_kv_row(wk, wv, rows[t], t, qd, kvd)
    c = la.KvCache(slots, nkv)
    for t in range(0, n, 2):
        la.copy_kv(handle, c, drows[t], t, qd, kvd)
        la.copy_kv_dyn(handle, c, drows[t + 1], i32([t + 1]), qd, kvd)
    assert np.array_equal(c.k.cpu().numpy(), wk) and np.array_equal(c.v.cpu().numpy(), wv)
    c = la.KvCache(slots, nkv)
    la.copy_kv_batch(handle, c, drows, 0, n, qd, kvd, stride)
    assert np.array_equal(c.k.cpu().numpy(), wk) and np.array_equal(c.v.cpu().numpy(), wv)
    pk, pv = np.zeros_like(wk), np.zeros_like(wv)
    for t in range(n):
        oracle.copy_kv_row(pk, pv, rows[t], t, qd, kvd, table, bs)
    pg = la.Paging(i32(table), bs)
    c = la.KvCache(slots, nkv)
    la.copy_kv_batch(handle, c, drows, 0, n, qd, kvd, stride, pg)
    assert np.array_equal(c.k.cpu().numpy(), pk) and np.array_equal(c.v.cpu().numpy(), pv)
    c = la.KvCache(slots, nkv)
    for t in range(n):
        la.copy_kv_paged_dyn(handle, c, drows[t], i32([t]), qd, kvd, pg)
    assert np.array_equal(c.k.cpu().numpy(), pk) and np.array_equal(c.v.cpu().numpy(), pv)
    tables = np.stack([table, np.roll(table, 1)]).astype(np.int32)
    sk, sv = np.zeros_like(wk), np.zeros_like(wv)
    pos = [9, 38]
    for s in range(2):
        oracle.copy_kv_row(sk, sv, rows[s], pos[s], qd, kvd, tables[s], bs)
    c = la.KvCache(slots, nkv)
    la.copy_kv_seqpos(handle, c, drows, i32(pos), 2, qd, kvd, stride, la.Paging(i32(tables), bs))
    assert np.array_equal(c.k.cpu().numpy(), sk) and np.array_equal(c.v.cpu().numpy(), sv)
    handle.check_status()


def test_bad_arguments_are_rejected(handle):
    from mx230_b200 import _lib
    c = la.KvCache(16, 2, 64, True)
    row = torch.zeros(18 * 64, device="cuda")
    with pytest.raises(_lib.Mx230Error) as e:
        la.quantize_kv(handle, c, row, 0, 14 * 64, 2, 128)  # head_dim 128 unsupported
    assert e.value.code == _lib.ERR_UNSUPPORTED
    with pytest.raises(_lib.Mx230Error) as e:
        la.rope(handle, None, 0, 14, 2, 64, 1e6)
    assert e.value.code == _lib.ERR_INVALID_ARG
