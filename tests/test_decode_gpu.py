"""Decode attention (fp32 and int8 KV cache) through the C ABI vs the oracle.

Gates: fp32-cache output vs the cpu.rs attention (oracle.gqa_decode_f32); int8-cache
output in the reference score mode vs the kernel-faithful oracle (mode 1) and in the
exact score mode vs the dequant-exact oracle (mode 0), on bit-identical codes.  All
arithmetic is fp32, so the tolerance is max-abs 2e-5 / mean-rel 1e-4, far inside the
2e-2 / 5e-3 of the parity bar; the summation order differs from the oracle's.
"""
import numpy as np
import pytest
import torch

import oracle
from mx230_b200 import _lib
from mx230_b200 import llm_attention as la
from tests.conftest import assert_close

pytestmark = pytest.mark.gpu
TOL = dict(max_abs=2e-5, mean_rel=1e-4)


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def i32(a):
    return torch.tensor(a, dtype=torch.int32, device="cuda")


def build_caches(nh, nkv, ctx, seed, affine=True, theta=1e6):
    """Oracle-side caches filled position by position: RoPE -> write, like the engine."""
    qd, kvd = nh * 64, nkv * 64
    rows = oracle.normal((ctx, qd + 2 * kvd), seed, 0)
    kc = np.zeros((ctx, kvd), np.float32)
    vc = np.zeros_like(kc)
    q8 = oracle.Q8Cache(ctx, nkv, 64, affine)
    for t in range(ctx):
        oracle.rope_qkv_row(rows[t], t, nh, nkv, 64, theta)
        oracle.copy_kv_row(kc, vc, rows[t], t, qd, kvd)
        oracle.quantize_kv_row(q8, rows[t], t, qd)
    return rows, kc, vc, q8


def to_dev_f32(kc, vc, nkv):
    c = la.KvCache(kc.shape[0], nkv)
    c.k.copy_(dev(kc)), c.v.copy_(dev(vc))
    return c


def to_dev_q8(w: oracle.Q8Cache):
    c = la.KvCache(w.rows, w.n_kv_head, 64, True, w.affine)
    c.k.copy_(dev(w.kq)), c.v.copy_(dev(w.vq)), c.ks.copy_(dev(w.ks)), c.vs.copy_(dev(w.vs))
    if w.affine:
        c.kb.copy_(dev(w.kb)), c.vb.copy_(dev(w.vb))
    return c


SHAPES = [(14, 2, 300), (32, 4, 257), (12, 12, 130), (32, 2, 100), (4, 2, 1), (8, 1, 2500)]


@pytest.mark.parametrize("nh,nkv,ctx", SHAPES)
def test_decode_f32_matches_oracle(handle, nh, nkv, ctx):
    rows, kc, vc, _ = build_caches(nh, nkv, ctx, 31)
    c = to_dev_f32(kc, vc, nkv)
    for t_cur in sorted({0, ctx // 2, ctx - 1}):
        want = oracle.gqa_decode_f32(rows[t_cur], kc, vc, t_cur, nh, nkv)
        out = torch.full((nh * 64,), float("nan"), device="cuda")
        la.attn_decode(handle, out, dev(rows[t_cur]), c, t_cur, nh, nkv, 64)
        assert_close(out.cpu().numpy(), want, f"decode f32 t={t_cur}", **TOL)
        out2 = torch.full((nh * 64,), float("nan"), device="cuda")
        la.attn_decode_dyn(handle, out2, dev(rows[t_cur]), c, i32([t_cur]), nh, nkv, 64)
        assert_close(out2.cpu().numpy(), want, f"decode f32 dyn t={t_cur}", **TOL)
    handle.check_status()


@pytest.mark.parametrize("affine", [True, False])
@pytest.mark.parametrize("nh,nkv,ctx", SHAPES)
def test_decode_q8_matches_both_oracles(handle, nh, nkv, ctx, affine):
    rows, _, _, q8 = build_caches(nh, nkv, ctx, 32, affine)
    c = to_dev_q8(q8)
    t_cur = ctx - 1
    q = dev(rows[t_cur])
    try:
        for mode, omode in ((_lib.Q8_SCORE_REF, 1), (_lib.Q8_SCORE_EXACT, 0)):
            handle.set_option(_lib.OPT_Q8_SCORE_MODE, mode)
            want = oracle.gqa_decode_q8(rows[t_cur], q8, t_cur, nh, omode)
            out = torch.full((nh * 64,), float("nan"), device="cuda")
            la.attn_decode(handle, out, q, c, t_cur, nh, nkv, 64)
            assert_close(out.cpu().numpy(), want, f"decode q8 mode {mode}", **TOL)
            out2 = torch.full((nh * 64,), float("nan"), device="cuda")
            la.attn_decode_dyn(handle, out2, q, c, i32([t_cur]), nh, nkv, 64)
            assert_close(out2.cpu().numpy(), want, f"decode q8 dyn mode {mode}", **TOL)
    finally:
        handle.set_option(_lib.OPT_Q8_SCORE_MODE, _lib.Q8_SCORE_REF)
    handle.check_status()


@pytest.mark.parametrize("nh,nkv,ctx", [(14, 2, 300), (32, 4, 1000), (8, 8, 77)])
def test_decode_q8_ref_mode_on_cuda_cores_equals_tensor_path(handle, nh, nkv, ctx):
    """The reference score mode has two implementations (tensor-core tiles, default, and CUDA
    cores): both meet the oracle's kernel-faithful mode at the same tolerance."""
    rows, _, _, q8 = build_caches(nh, nkv, ctx, 33, True)
    c = to_dev_q8(q8)
    t_cur = ctx - 1
    want = oracle.gqa_decode_q8(rows[t_cur], q8, t_cur, nh, 1)
    try:
        for tensor in (1, 0):
            handle.set_option(_lib.OPT_DECODE_TENSOR, tensor)
            out = torch.full((nh * 64,), float("nan"), device="cuda")
            la.attn_decode(handle, out, dev(rows[t_cur]), c, t_cur, nh, nkv, 64)
            assert_close(out.cpu().numpy(), want, f"decode q8 ref, tensor={tensor}", **TOL)
    finally:
        handle.set_option(_lib.OPT_DECODE_TENSOR, 1)
    handle.check_status()


def test_decode_q8_large_value_scales(handle):
    """V rows a thousand times larger than usual: the weights p * vs of the tensor-core path stay
    inside the f16 range (no inf / nan) and the result scales with the values."""
    nh, nkv, ctx = 16, 2, 520
    qd, kvd = nh * 64, nkv * 64
    q = oracle.normal((qd,), 90, 0)
    kv = oracle.normal((ctx, 2 * kvd), 91, 0)
    kv[:, kvd:] *= 1000.0
    q8 = oracle.Q8Cache(ctx, nkv)
    for t in range(ctx):
        oracle.quantize_kv_row(q8, kv[t], t, 0)
    want = oracle.gqa_decode_q8(q, q8, ctx - 1, nh, 1)
    out = torch.full((qd,), float("nan"), device="cuda")
    la.attn_decode(handle, out, dev(q), to_dev_q8(q8), ctx - 1, nh, nkv, 64)
    got = out.cpu().numpy()
    assert np.isfinite(got).all()
    assert_close(got / 1000.0, want / 1000.0, "decode q8 large V", **TOL)
    handle.check_status()


@pytest.mark.parametrize("chunk", [0, 128, 256, 1024])
def test_decode_key_splits_agree(handle, chunk):
    """Any split of the key axis gives the same answer as the oracle (merge by log-sum-exp)."""
    nh, nkv, ctx = 14, 2, 2048
    rows, kc, vc, q8 = build_caches(nh, nkv, ctx, 33)
    cf, cq = to_dev_f32(kc, vc, nkv), to_dev_q8(q8)
    q = dev(rows[ctx - 1])
    handle.set_option(_lib.OPT_DECODE_CHUNK, chunk)
    try:
        out = torch.zeros(nh * 64, device="cuda")
        la.attn_decode(handle, out, q, cf, ctx - 1, nh, nkv, 64)
        assert_close(out.cpu().numpy(), oracle.gqa_decode_f32(rows[ctx - 1], kc, vc, ctx - 1, nh, nkv),
                     "split f32", **TOL)
        out = torch.zeros(nh * 64, device="cuda")
        la.attn_decode(handle, out, q, cq, ctx - 1, nh, nkv, 64)
        assert_close(out.cpu().numpy(), oracle.gqa_decode_q8(rows[ctx - 1], q8, ctx - 1, nh, 1),
                     "split q8", **TOL)
        # twice in a row: the self-resetting arrival counters are back at zero
        out2 = torch.zeros(nh * 64, device="cuda")
        la.attn_decode(handle, out2, q, cq, ctx - 1, nh, nkv, 64)
        assert torch.equal(out, out2)
    finally:
        handle.set_option(_lib.OPT_DECODE_CHUNK, 0)
    handle.check_status()


@pytest.mark.parametrize("quant", [False, True])
def test_decode_paged_and_batched(handle, quant):
    """Non-identity block tables (as the reference's --paged gate, gpu.rs:408-413), one table
    row and one position per sequence."""
    nh, nkv, bs, n_seq = 14, 2, 16, 5
    qd, kvd = nh * 64, nkv * 64
    pos = [70, 0, 33, 127, 15]
    n_log = 8
    rng = np.random.default_rng(0)
    perm = rng.permutation(n_seq * n_log).astype(np.int32)
    tables = perm.reshape(n_seq, n_log)
    slots = n_seq * n_log * bs
    stride = qd + 2 * kvd
    qkv = np.zeros((n_seq, stride), np.float32)
    kc = np.zeros((slots, kvd), np.float32)
    vc = np.zeros_like(kc)
    q8 = oracle.Q8Cache(slots, nkv)
    for s in range(n_seq):
        rows = oracle.normal((pos[s] + 1, stride), 40 + s, 0)
        for t in range(pos[s] + 1):
            oracle.rope_qkv_row(rows[t], t, nh, nkv, 64, 1e6)
            oracle.copy_kv_row(kc, vc, rows[t], t, qd, kvd, tables[s], bs)
            oracle.quantize_kv_row(q8, rows[t], t, qd, tables[s], bs)
        qkv[s] = rows[pos[s]]
    c = to_dev_q8(q8) if quant else to_dev_f32(kc, vc, nkv)
    if quant:
        want = oracle.gqa_decode_batched(qkv, pos, nh, nkv, cache=q8, tables=tables, block_size=bs, mode=1)
    else:
        want = oracle.gqa_decode_batched(qkv, pos, nh, nkv, kcache=kc, vcache=vc, tables=tables, block_size=bs)
    out = torch.full((n_seq, qd), float("nan"), device="cuda")
    la.attn_decode_batched(handle, out, dev(qkv), c, i32(pos), n_seq, nh, nkv, 64,
                           la.Paging(i32(tables), bs), stride, qd)
    assert_close(out.cpu().numpy(), want, "batched paged", **TOL)
    # single-sequence paged forms against the same pool
    for s in (0, 3):
        pg = la.Paging(i32(tables[s]), bs)
        o1 = torch.zeros(qd, device="cuda")
        la.attn_decode(handle, o1, dev(qkv[s]), c, pos[s], nh, nkv, 64, pg)
        assert_close(o1.cpu().numpy(), want[s], "paged", **TOL)
        o2 = torch.zeros(qd, device="cuda")
        la.attn_decode_dyn(handle, o2, dev(qkv[s]), c, i32([pos[s]]), nh, nkv, 64, pg)
        assert_close(o2.cpu().numpy(), want[s], "paged dyn", **TOL)
    handle.check_status()


@pytest.mark.parametrize("quant", [False, True])
def test_full_step_rope_write_attend(handle, quant):
    """RoPE -> KV write -> attention chained on the device, token by token (gpu.rs:2570-2672),
    against the oracle running the same three steps.  RoPE differs by libm rounding, so the
    int8 codes are compared only where the device RoPE output equals the oracle's."""
    nh, nkv, ctx, theta = 14, 2, 48, 1e6
    qd, kvd = nh * 64, nkv * 64
    raw = oracle.normal((ctx, qd + 2 * kvd), 50, 0)
    c = la.KvCache(ctx, nkv, 64, quant)
    w8 = oracle.Q8Cache(ctx, nkv)
    kc, vc = np.zeros((ctx, kvd), np.float32), np.zeros((ctx, kvd), np.float32)
    for t in range(ctx):
        row = dev(raw[t])
        out = torch.zeros(qd, device="cuda")
        la.decode_step(handle, out, row, c, t, nh, nkv, 64, theta)
        wrow = oracle.rope_qkv_row(raw[t].copy(), t, nh, nkv, 64, theta)
        oracle.copy_kv_row(kc, vc, wrow, t, qd, kvd)
        oracle.quantize_kv_row(w8, wrow, t, qd)
        want = oracle.gqa_decode_q8(wrow, w8, t, nh, 1) if quant else \
            oracle.gqa_decode_f32(wrow, kc, vc, t, nh, nkv)
        assert_close(out.cpu().numpy(), want, f"step t={t}", max_abs=2e-3, mean_rel=5e-3)
    handle.check_status()


def test_slab_batched_and_partial_merge(handle):
    """Contiguous per-sequence slabs; split-KV partial triples merged by log-sum-exp equal
    the unsplit result and the oracle's merge."""
    nh, nkv, ctx, n_seq = 32, 4, 700, 3
    qd, kvd = nh * 64, nkv * 64
    stride = qd
    qs = oracle.normal((n_seq, qd), 60, 0)
    kq = np.zeros((n_seq * ctx, kvd), np.int8)
    q8 = oracle.Q8Cache(n_seq * ctx, nkv)
    for s in range(n_seq):
        kv = oracle.normal((ctx, 2 * kvd), 61 + s, 0)
        for t in range(ctx):
            oracle.quantize_kv_row(q8, kv[t], s * ctx + t, 0)
    c = to_dev_q8(q8)
    pos = [ctx - 1, 100, 511]
    want = oracle.gqa_decode_batched(qs, pos, nh, nkv, cache=q8, seq_rows=ctx, mode=1)
    out = torch.zeros(n_seq, qd, device="cuda")
    la.attn_decode_slab(handle, out, dev(qs), c, i32(pos), n_seq, nh, nkv, 64, ctx, stride, qd)
    assert_close(out.cpu().numpy(), want, "slab", **TOL)
    # split the key axis in 3 "ranks", gather, merge
    handle.set_option(_lib.OPT_Q8_SCORE_MODE, _lib.Q8_SCORE_EXACT)
    try:
        cuts = [0, 256, 300, ctx]
        rows = n_seq * nh
        pm = torch.zeros(3, rows, device="cuda")
        pl = torch.zeros(3, rows, device="cuda")
        pa = torch.zeros(3, rows, 64, device="cuda")
        for r in range(3):
            la.attn_decode_partial(handle, pm[r], pl[r], pa[r], dev(qs), c, cuts[r], cuts[r + 1], n_seq,
                                   nh, nkv, 64, ctx, stride)
        merged = torch.zeros(rows, 64, device="cuda")
        la.merge_partials(handle, merged, pm, pl, pa, 3, rows)
        full = oracle.gqa_decode_batched(qs, [ctx - 1] * n_seq, nh, nkv, cache=q8, seq_rows=ctx, mode=0)
        assert_close(merged.cpu().numpy().reshape(n_seq, qd), full, "partial+merge", **TOL)
        om = oracle.merge_partials(pm.cpu().numpy(), pl.cpu().numpy(), pa.cpu().numpy())
        assert_close(merged.cpu().numpy(), om, "merge kernel vs oracle merge", **TOL)
        # the same merge straight from the ranks' packed [m | l | acc] buffers
        packed = torch.cat([pm, pl, pa.reshape(3, rows * 64)], dim=1).contiguous()
        merged2 = torch.full((rows, 64), 7.0, device="cuda")
        la.merge_partials_packed(handle, merged2, packed, 3, rows)
        assert torch.equal(merged2, merged)
        with pytest.raises(_lib.Mx230Error):   # odd row count: the parts would lose their alignment
            la.merge_partials_packed(handle, merged2, packed, 3, rows - 1)
        # one partial of the oracle for rank 1 of sequence 2
        m, l, acc = oracle.gqa_partial(qs[2], cuts[1], cuts[2], nh, nkv, 64, cache=_slab(q8, 2, ctx))
        got_acc = pa[1].cpu().numpy().reshape(n_seq, nh, 64)[2]
        got_m = pm[1].cpu().numpy().reshape(n_seq, nh)[2]
        got_l = pl[1].cpu().numpy().reshape(n_seq, nh)[2]
        w = np.exp(got_m - m)  # the device may hold a different (but consistent) running max
        assert_close(got_acc * w[:, None], acc, "partial acc", max_abs=1e-3, mean_rel=1e-4)
        assert_close(got_l * w, l, "partial l", max_abs=1e-3, mean_rel=1e-4)
    finally:
        handle.set_option(_lib.OPT_Q8_SCORE_MODE, _lib.Q8_SCORE_REF)
    handle.check_status()


def _slab(q8: oracle.Q8Cache, s, ctx):
    v = oracle.Q8Cache(ctx, q8.n_kv_head, 64, q8.affine)
    sl = slice(s * ctx, (s + 1) * ctx)
    v.kq, v.vq = np.ascontiguousarray(q8.kq[sl]), np.ascontiguousarray(q8.vq[sl])
    v.ks, v.vs = np.ascontiguousarray(q8.ks[sl]), np.ascontiguousarray(q8.vs[sl])
    v.kb, v.vb = np.ascontiguousarray(q8.kb[sl]), np.ascontiguousarray(q8.vb[sl])
    return v


def test_decode_rejects_bad_shapes(handle):
    c = la.KvCache(16, 3)
    out = torch.zeros(14 * 64, device="cuda")
    q = torch.zeros(20 * 64, device="cuda")
    with pytest.raises(_lib.Mx230Error) as e:
        la.attn_decode(handle, out, q, c, 3, 14, 3, 64)  # 14 % 3 != 0
    assert e.value.code == _lib.ERR_UNSUPPORTED
    with pytest.raises(_lib.Mx230Error) as e:
        la.attn_decode(handle, out, q, la.KvCache(16, 2), -1, 14, 2, 64)
    assert e.value.code == _lib.ERR_INVALID_ARG
