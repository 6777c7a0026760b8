"""Pins the CPU oracle against the reference project's own CUDA kernels run on the GPU.

The reference's kernels (compiled unmodified from the reference checkout into
oracle/_ref by oracle/build.py) are launched with the reference's grid shapes on the
reference's own test inputs (02-flash-attention/src/main.rs:419-499: N=512, uniform
seeds 1,2,3 / 11..14, allclose rtol 1e-3 atol 1e-4) and compared with the oracle.
This is the reference's own GPU==CPU test with our C restatement in the CPU seat.
"""
import numpy as np
import pytest
import torch

import oracle
from tests import refkernels

pytestmark = pytest.mark.gpu
RTOL, ATOL = 1e-3, 1e-4
N = 512


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.fixture(scope="module")
def flash_mod():
    if not refkernels.available("attention_flash"):
        pytest.skip("oracle/_ref not built (no reference checkout at build time)")
    return refkernels.RefModule("attention_flash")


@pytest.fixture(scope="module")
def bwd_mod():
    if not refkernels.available("attention_bwd"):
        pytest.skip("oracle/_ref not built")
    return refkernels.RefModule("attention_bwd")


@pytest.fixture(scope="module")
def llm_mod():
    if not refkernels.available("llm"):
        pytest.skip("oracle/_ref not built")
    return refkernels.RefModule("llm")


@pytest.mark.parametrize("causal", [0, 1])
def test_reference_flash_forward_equals_oracle(flash_mod, causal):
    q, k, v = (oracle.pseudo_rand(N * 64, s).reshape(N, 64) for s in (1, 2, 3))
    o = torch.zeros(N, 64, device="cuda")
    l = torch.zeros(N, device="cuda")
    flash_mod.launch("attn_flash_lse", ((N + 63) // 64,), (64,), [dev(q), dev(k), dev(v), o, l, N, causal])
    torch.cuda.synchronize()
    want_o, want_l = oracle.attn_fwd(q, k, v, bool(causal))
    assert oracle.allclose_err(o.cpu().numpy(), want_o, RTOL, ATOL) < 1.0
    assert np.abs(l.cpu().numpy() - want_l).max() < 1e-4


@pytest.mark.parametrize("causal", [0, 1])
def test_reference_flash_backward_equals_oracle(flash_mod, bwd_mod, causal):
    q, k, v, do = (oracle.pseudo_rand(N * 64, s).reshape(N, 64) for s in (11, 12, 13, 14))
    dq_, dk_, dv_, do_ = dev(q), dev(k), dev(v), dev(do)
    o = torch.zeros(N, 64, device="cuda")
    l = torch.zeros(N, device="cuda")
    delta = torch.zeros(N, device="cuda")
    g = ((N + 63) // 64,)
    flash_mod.launch("attn_flash_lse", g, (64,), [dq_, dk_, dv_, o, l, N, causal])
    bwd_mod.launch("attn_bwd_preprocess", ((N + 255) // 256,), (256,), [do_, o, delta, N])
    gq, gk, gv = (torch.zeros(N, 64, device="cuda") for _ in range(3))
    bwd_mod.launch("attn_bwd_dq", g, (64,), [dq_, dk_, dv_, do_, l, delta, gq, N, causal])
    bwd_mod.launch("attn_bwd_dkv", g, (64,), [dq_, dk_, dv_, do_, l, delta, gk, gv, N, causal])
    torch.cuda.synchronize()
    wq, wk, wv = oracle.attn_bwd(q, k, v, do, bool(causal))
    o_want, _ = oracle.attn_fwd(q, k, v, bool(causal))
    assert np.abs(delta.cpu().numpy() - oracle.bwd_preprocess(do, o_want)).max() < 1e-4
    for name, got, want in (("dQ", gq, wq), ("dK", gk, wk), ("dV", gv, wv)):
        assert oracle.allclose_err(got.cpu().numpy(), want, RTOL, ATOL) < 1.0, name


def test_reference_quantize_kv_equals_oracle_bit_exact(llm_mod):
    nh, nkv, ctx = 14, 2, 96
    qd, kvd = nh * 64, nkv * 64
    rows = oracle.normal((ctx, qd + 2 * kvd), 17, 0)
    rows[5, qd:qd + 64] = 0.5          # constant K row: hi == lo
    rows[6, qd + kvd:qd + kvd + 64] = 0.0
    want = oracle.Q8Cache(ctx, nkv)
    kq = torch.zeros(ctx, kvd, dtype=torch.int8, device="cuda")
    vq = torch.zeros_like(kq)
    ks, vs, kb, vb = (torch.zeros(ctx, nkv, device="cuda") for _ in range(4))
    drows = dev(rows)
    for t in range(ctx):
        oracle.quantize_kv_row(want, rows[t], t, qd)
        llm_mod.launch("quantize_kv", (nkv,), (64,), [kq, vq, ks, vs, kb, vb, drows[t], t, qd, nkv, 64])
    torch.cuda.synchronize()
    assert np.array_equal(kq.cpu().numpy(), want.kq) and np.array_equal(vq.cpu().numpy(), want.vq)
    for got, w in ((ks, want.ks), (vs, want.vs), (kb, want.kb), (vb, want.vb)):
        assert np.array_equal(got.cpu().numpy(), w)


def test_reference_decode_kernels_equal_oracle(llm_mod):
    nh, nkv, ctx = 14, 2, 300
    qd, kvd = nh * 64, nkv * 64
    rows = oracle.normal((ctx, qd + 2 * kvd), 18, 0)
    cache = oracle.Q8Cache(ctx, nkv)
    kc = np.zeros((ctx, kvd), np.float32)
    vc = np.zeros_like(kc)
    for t in range(ctx):
        oracle.rope_qkv_row(rows[t], t, nh, nkv, 64, 1e6)
        oracle.quantize_kv_row(cache, rows[t], t, qd)
        oracle.copy_kv_row(kc, vc, rows[t], t, qd, kvd)
    q = dev(rows[ctx - 1])
    out = torch.zeros(qd, device="cuda")
    llm_mod.launch("attn_decode", (nh,), (128,), [out, q, dev(kc), dev(vc), ctx - 1, nh, nkv, 64])
    torch.cuda.synchronize()
    want = oracle.gqa_decode_f32(rows[ctx - 1], kc, vc, ctx - 1, nh, nkv)
    assert oracle.allclose_err(out.cpu().numpy(), want, RTOL, ATOL) < 1.0
    out8 = torch.zeros(qd, device="cuda")
    llm_mod.launch("attn_decode_q8", (nh,), (128,),
                   [out8, q, dev(cache.kq), dev(cache.vq), dev(cache.ks), dev(cache.vs), dev(cache.kb),
                    dev(cache.vb), ctx - 1, nh, nkv, 64])
    torch.cuda.synchronize()
    want8 = oracle.gqa_decode_q8(rows[ctx - 1], cache, ctx - 1, nh, 1)  # kernel-faithful oracle
    assert oracle.allclose_err(out8.cpu().numpy(), want8, RTOL, ATOL) < 1.0


def test_reference_rope_kernel_close_to_oracle(llm_mod):
    """The reference GPU RoPE uses fast intrinsics; the oracle follows its CPU code."""
    nh, nkv = 14, 2
    row = oracle.normal(((nh + 2 * nkv) * 64,), 19, 0)
    d = dev(row)
    llm_mod.launch("rope", (((nh + nkv) * 32 + 255) // 256,), (256,), [d, 37, nh, nkv, 64, 1e6])
    torch.cuda.synchronize()
    want = oracle.rope_qkv_row(row.copy(), 37, nh, nkv, 64, 1e6)
    assert np.abs(d.cpu().numpy() - want).max() < 1e-3


# ---------------------------------------------------------------------------------------------
# The stage-3 variants: the reference's own batched / paged / prefill / projection kernels against the
# oracle functions that the product tests are gated with (grids and blocks as 03-llm-engine/src/gpu.rs
# launches them: prefill (n_head, ceil(n/64)) x 64, gpu.rs:3235-3239; batched decode (n_head, n_seq) x 128,
# gpu.rs:3543-3547; quantize_kv_batch (n_kv_head, n_tok) x 64, gpu.rs:3292-3296; gemv ceil(n_out/256) x 256
# with the activations in dynamic shared memory, gpu.rs:1184-1188).
# ---------------------------------------------------------------------------------------------
def _filled_caches(nh, nkv, ctx, seed, table=None, bs=16, slots=None):
    """RoPE'd qkv rows for positions 0..ctx-1 written to an fp32 and an int8 cache by the oracle (through `table`
    when given)."""
    qd, kvd = nh * 64, nkv * 64
    slots = slots or ctx
    rows = oracle.normal((ctx, qd + 2 * kvd), seed, 0)
    kc = np.zeros((slots, kvd), np.float32)
    vc = np.zeros_like(kc)
    q8 = oracle.Q8Cache(slots, nkv)
    for t in range(ctx):
        oracle.rope_qkv_row(rows[t], t, nh, nkv, 64, 1e6)
        oracle.copy_kv_row(kc, vc, rows[t], t, qd, kvd, table, bs)
        oracle.quantize_kv_row(q8, rows[t], t, qd, table, bs)
    return rows, kc, vc, q8


def _q8_dev(c):
    return [dev(c.kq), dev(c.vq), dev(c.ks), dev(c.vs), dev(c.kb), dev(c.vb)]


def test_reference_paged_and_dyn_decode_equal_oracle(llm_mod):
    nh, nkv, ctx, bs = 14, 2, 200, 16
    qd = nh * 64
    n_log = (ctx + bs - 1) // bs
    table = np.random.RandomState(3).permutation(n_log + 3)[:n_log].astype(np.int32)
    rows, kc, vc, q8 = _filled_caches(nh, nkv, ctx, 41, table, bs, (n_log + 3) * bs)
    q, bt = dev(rows[ctx - 1]), dev(table)
    pos = torch.tensor([ctx - 1], dtype=torch.int32, device="cuda")
    want = oracle.gqa_decode_f32(rows[ctx - 1], kc, vc, ctx - 1, nh, nkv, 64, table, bs)
    want8 = oracle.gqa_decode_q8(rows[ctx - 1], q8, ctx - 1, nh, 1, table, bs)
    for sym, args, w in (
            ("attn_decode_paged", [q, dev(kc), dev(vc), ctx - 1, nh, nkv, 64, bt, bs], want),
            ("attn_decode_paged_dyn", [q, dev(kc), dev(vc), pos, nh, nkv, 64, bt, bs], want),
            ("attn_decode_q8_paged", [q, *_q8_dev(q8), ctx - 1, nh, nkv, 64, bt, bs], want8),
            ("attn_decode_q8_paged_dyn", [q, *_q8_dev(q8), pos, nh, nkv, 64, bt, bs], want8)):
        out = torch.zeros(qd, device="cuda")
        llm_mod.launch(sym, (nh,), (128,), [out, *args])
        torch.cuda.synchronize()
        assert oracle.allclose_err(out.cpu().numpy(), w, RTOL, ATOL) < 1.0, sym
    # the linear _dyn forms on a linear cache
    rows, kc, vc, q8 = _filled_caches(nh, nkv, ctx, 42)
    q = dev(rows[ctx - 1])
    for sym, args, w in (
            ("attn_decode_dyn", [q, dev(kc), dev(vc), pos, nh, nkv, 64],
             oracle.gqa_decode_f32(rows[ctx - 1], kc, vc, ctx - 1, nh, nkv)),
            ("attn_decode_q8_dyn", [q, *_q8_dev(q8), pos, nh, nkv, 64],
             oracle.gqa_decode_q8(rows[ctx - 1], q8, ctx - 1, nh, 1))):
        out = torch.zeros(qd, device="cuda")
        llm_mod.launch(sym, (nh,), (128,), [out, *args])
        torch.cuda.synchronize()
        assert oracle.allclose_err(out.cpu().numpy(), w, RTOL, ATOL) < 1.0, sym


def test_reference_batched_decode_equals_oracle(llm_mod):
    nh, nkv, bs, n_seq = 14, 2, 16, 3
    qd, kvd = nh * 64, nkv * 64
    lens = [37, 150, 96]
    n_log = (max(lens) + bs - 1) // bs
    perm = np.random.RandomState(5).permutation(n_seq * n_log).astype(np.int32)
    tables = perm.reshape(n_seq, n_log)
    slots = n_seq * n_log * bs
    kc = np.zeros((slots, kvd), np.float32)
    vc = np.zeros_like(kc)
    q8 = oracle.Q8Cache(slots, nkv)
    qkv = np.zeros((n_seq, qd + 2 * kvd), np.float32)
    for s, n in enumerate(lens):
        rows = oracle.normal((n, qd + 2 * kvd), 50 + s, 0)
        for t in range(n):
            oracle.rope_qkv_row(rows[t], t, nh, nkv, 64, 1e6)
            oracle.copy_kv_row(kc, vc, rows[t], t, qd, kvd, tables[s], bs)
            oracle.quantize_kv_row(q8, rows[t], t, qd, tables[s], bs)
        qkv[s] = rows[n - 1]
    pos = np.array([n - 1 for n in lens], np.int32)
    stride = qkv.shape[1]
    want = oracle.gqa_decode_batched(qkv, pos, nh, nkv, kcache=kc, vcache=vc, tables=tables, block_size=bs)
    want8 = oracle.gqa_decode_batched(qkv, pos, nh, nkv, cache=q8, tables=tables, block_size=bs, mode=1)
    out = torch.zeros(n_seq, qd, device="cuda")
    llm_mod.launch("attn_decode_batched", (nh, n_seq), (128,),
                   [out, dev(qkv), dev(kc), dev(vc), dev(pos), nh, nkv, 64, dev(tables), bs, n_log, stride, qd])
    torch.cuda.synchronize()
    assert oracle.allclose_err(out.cpu().numpy(), want, RTOL, ATOL) < 1.0
    out8 = torch.zeros(n_seq, qd, device="cuda")
    llm_mod.launch("attn_decode_q8_batched", (nh, n_seq), (128,),
                   [out8, dev(qkv), *_q8_dev(q8), dev(pos), nh, nkv, 64, dev(tables), bs, n_log, stride, qd])
    torch.cuda.synchronize()
    assert oracle.allclose_err(out8.cpu().numpy(), want8, RTOL, ATOL) < 1.0


def test_reference_batch_and_seqpos_quantisers_equal_oracle_bit_exact(llm_mod):
    nh, nkv, bs = 14, 2, 16
    qd, kvd = nh * 64, nkv * 64
    stride = qd + 2 * kvd
    n_tok, pos0 = 40, 7
    rows = oracle.normal((n_tok, stride), 61, 0)
    n_log = (pos0 + n_tok + bs - 1) // bs
    table = np.random.RandomState(7).permutation(n_log + 2)[:n_log].astype(np.int32)
    slots = (n_log + 2) * bs
    for paged in (False, True):
        want = oracle.Q8Cache(slots, nkv)
        for t in range(n_tok):
            oracle.quantize_kv_row(want, rows[t], pos0 + t, qd, table if paged else None, bs)
        kq = torch.zeros(slots, kvd, dtype=torch.int8, device="cuda")
        vq = torch.zeros_like(kq)
        side = [torch.zeros(slots, nkv, device="cuda") for _ in range(4)]
        args = [kq, vq, *side, dev(rows), pos0, qd, nkv, 64, stride]
        llm_mod.launch("quantize_kv_batch_paged" if paged else "quantize_kv_batch", (nkv, n_tok), (64,),
                       args + ([dev(table), bs] if paged else []))
        torch.cuda.synchronize()
        assert np.array_equal(kq.cpu().numpy(), want.kq) and np.array_equal(vq.cpu().numpy(), want.vq)
        for got, w in zip(side, (want.ks, want.vs, want.kb, want.vb)):
            assert np.array_equal(got.cpu().numpy(), w)
    # per-sequence positions and tables (continuous batching)
    n_seq = 3
    pos = np.array([5, 33, 18], np.int32)
    tables = np.random.RandomState(8).permutation(n_seq * 3).astype(np.int32).reshape(n_seq, 3)
    slots = n_seq * 3 * bs
    want = oracle.Q8Cache(slots, nkv)
    for s in range(n_seq):
        oracle.quantize_kv_row(want, rows[s], int(pos[s]), qd, tables[s], bs)
    kq = torch.zeros(slots, kvd, dtype=torch.int8, device="cuda")
    vq = torch.zeros_like(kq)
    side = [torch.zeros(slots, nkv, device="cuda") for _ in range(4)]
    llm_mod.launch("quantize_kv_seqpos", (nkv, n_seq), (64,),
                   [kq, vq, *side, dev(rows[:n_seq]), dev(pos), qd, nkv, 64, stride, dev(tables), bs, 3])
    torch.cuda.synchronize()
    assert np.array_equal(kq.cpu().numpy(), want.kq) and np.array_equal(vq.cpu().numpy(), want.vq)
    for got, w in zip(side, (want.ks, want.vs, want.kb, want.vb)):
        assert np.array_equal(got.cpu().numpy(), w)


@pytest.mark.parametrize("paged", [False, True])
def test_reference_prefill_kernels_equal_oracle(llm_mod, paged):
    """attn_prefill / _paged (exact scores) against oracle.prefill mode 0; attn_prefill_q8 / _q8_paged (the
    reference's int8 score arithmetic) and attn_prefill_dp4a / _dp4a_paged against mode 1."""
    nh, nkv, bs = 14, 2, 16
    qd, kvd = nh * 64, nkv * 64
    pos0, n_tok = 70, 100
    ctx = pos0 + n_tok
    n_log = (ctx + bs - 1) // bs
    table = np.random.RandomState(11).permutation(n_log + 2)[:n_log].astype(np.int32) if paged else None
    rows, kc, vc, q8 = _filled_caches(nh, nkv, ctx, 71, table, bs, (n_log + 2) * bs)
    new = np.ascontiguousarray(rows[pos0:])
    stride = new.shape[1]
    grid, tail = (nh, (n_tok + 63) // 64), ([dev(table), bs] if paged else [])
    sfx = "_paged" if paged else ""
    cases = (
        ("attn_prefill" + sfx, [dev(kc), dev(vc)], dict(kcache=kc, vcache=vc, mode=0)),
        ("attn_prefill_dp4a" + sfx, [dev(kc), dev(vc)], dict(kcache=kc, vcache=vc, mode=1)),
        ("attn_prefill_q8" + sfx, _q8_dev(q8), dict(cache=q8, mode=1)),
    )
    for sym, cache_args, okw in cases:
        out = torch.zeros(n_tok, qd, device="cuda")
        llm_mod.launch(sym, grid, (64,), [out, dev(new), *cache_args, pos0, n_tok, nh, nkv, stride, qd, *tail])
        torch.cuda.synchronize()
        want = oracle.prefill(new, pos0, n_tok, nh, nkv, stride, qd, table=table, block_size=bs, **okw)
        assert oracle.allclose_err(out.cpu().numpy(), want, RTOL, ATOL) < 1.0, sym


def test_reference_gemv_kernels_equal_oracle(llm_mod):
    """gemv, gemv_half, gemv_int8 (llm.cu:144-177,226-316; activation group AG = 4, the module's default) against
    the oracle's gemv functions."""
    n_in, n_out = 896, 1152
    rs = np.random.RandomState(13)
    x = oracle.normal((n_in,), 81, 0)
    w = (oracle.normal((n_in, n_out), 82, 0) * 0.05).astype(np.float32)
    b = oracle.normal((n_out,), 83, 0)
    y0 = oracle.normal((n_out,), 84, 0)
    g = ((n_out + 255) // 256,)
    for accum in (0, 1):
        y = dev(y0.copy())
        llm_mod.launch("gemv", g, (256,), [y, dev(x), dev(w), dev(b), n_in, n_out, accum], smem=n_in * 4)
        torch.cuda.synchronize()
        want = oracle.gemv(x, w, b, y0 if accum else None, bool(accum))
        assert oracle.allclose_err(y.cpu().numpy(), want, RTOL, ATOL) < 1.0
    wh = w.astype(np.float16)
    y = torch.zeros(n_out, device="cuda")
    llm_mod.launch("gemv_half", g, (256,), [y, dev(x), dev(wh), dev(b), n_in, n_out, 0], smem=n_in * 4)
    torch.cuda.synchronize()
    assert oracle.allclose_err(y.cpu().numpy(), oracle.gemv(x, wh, b), RTOL, ATOL) < 1.0
    w8 = rs.randint(-127, 128, size=(n_in, n_out)).astype(np.int8)
    scales = (rs.rand(n_out).astype(np.float32) * 0.01 + 0.001)
    w32 = oracle.pack_int8_weights(w8)
    y = torch.zeros(n_out, device="cuda")
    llm_mod.launch("gemv_int8", g, (256,), [y, dev(x), dev(w32), dev(scales), dev(b), n_in, n_out, 0],
                   smem=n_in + (n_in // 4) * 4)
    torch.cuda.synchronize()
    assert oracle.allclose_err(y.cpu().numpy(), oracle.gemv_int8(x, w32, scales, b, ag=4), RTOL, ATOL) < 1.0


def test_reference_gemm_kernels_equal_oracle(llm_mod):
    """gemm_f32_wide / gemm_half_wide (the prefill tier, M > 64: grid (ceil(n/128), ceil(m/128)) x 256 threads,
    gpu.rs:1117-1123) and gemm_f32 (the 64-row tier, grid (ceil(n/64), ceil(m/64)) x (16, 16), gpu.rs:1109-1115)
    against the oracle's gemm, the function the library's mx230_gemm is tested with."""
    m, n, k = 200, 1152, 896
    a = oracle.normal((m, k), 91, 0)
    w = (oracle.normal((k, n), 92, 0) / np.sqrt(k)).astype(np.float32)
    b = oracle.normal((n,), 93, 0)
    want = oracle.gemm(a, w, b)
    c = torch.zeros(m, n, device="cuda")
    llm_mod.launch("gemm_f32_wide", ((n + 127) // 128, (m + 127) // 128), (256,), [c, dev(a), dev(w), dev(b), m, n, k])
    torch.cuda.synchronize()
    assert oracle.allclose_err(c.cpu().numpy(), want, RTOL, ATOL) < 1.0
    c.zero_()
    llm_mod.launch("gemm_f32", ((n + 63) // 64, (m + 63) // 64), (16, 16), [c, dev(a), dev(w), dev(b), m, n, k])
    torch.cuda.synchronize()
    assert oracle.allclose_err(c.cpu().numpy(), want, RTOL, ATOL) < 1.0
    wh = w.astype(np.float16)
    c.zero_()
    llm_mod.launch("gemm_half_wide", ((n + 127) // 128, (m + 127) // 128), (256,), [c, dev(a), dev(wh), dev(b), m, n, k])
    torch.cuda.synchronize()
    assert oracle.allclose_err(c.cpu().numpy(), oracle.gemm(a, wh, b), RTOL, ATOL) < 1.0


def test_library_int8_prefill_against_the_reference_int8_prefill(llm_mod, handle):
    """The reference's attn_prefill_q8 quantises q per (row, head) to int8 and scores with integer dots; the library's
    default score mode over an int8 cache reproduces that arithmetic (the codes cross the tensor cores exactly), its
    EXACT mode scores with fp32 q on dequantised K.  On benchmark-shaped data (14q/2kv, RoPE theta 1e6, N(0,1), 512
    tokens at position 1536) both read the same codes: the default mode is gated against the reference KERNEL'S own
    output at the parity bar, the exact mode against the exact-score oracle; the distance between the two arithmetics
    (q quantisation alone, about 5.7e-3) is printed."""
    from mx230_b200 import _lib
    from mx230_b200 import llm_attention as la
    nh, nkv = 14, 2
    qd = nh * 64
    pos0, n_tok = 1536, 512
    ctx = pos0 + n_tok
    rows, kc, vc, q8 = _filled_caches(nh, nkv, ctx, 91)
    new = np.ascontiguousarray(rows[pos0:])
    stride = new.shape[1]
    ref = torch.zeros(n_tok, qd, device="cuda")
    llm_mod.launch("attn_prefill_q8", (nh, (n_tok + 63) // 64), (64,),
                   [ref, dev(new), *_q8_dev(q8), pos0, n_tok, nh, nkv, stride, qd])
    c8 = la.KvCache(ctx, nkv, 64, True)
    for t, a in zip((c8.k, c8.v, c8.ks, c8.vs, c8.kb, c8.vb), (q8.kq, q8.vq, q8.ks, q8.vs, q8.kb, q8.vb)):
        t.copy_(dev(a))
    handle.reserve(la.prefill_workspace_bytes(n_tok, ctx, nh, nkv))
    got = {}
    try:
        for mode in (_lib.Q8_SCORE_REF, _lib.Q8_SCORE_EXACT):
            handle.set_option(_lib.OPT_Q8_SCORE_MODE, mode)
            o = torch.zeros(n_tok, qd, device="cuda")
            la.attn_prefill(handle, o, dev(new), c8, pos0, n_tok, nh, nkv, stride, qd)
            handle.check_status()
            got[mode] = o.cpu().numpy()
    finally:
        handle.set_option(_lib.OPT_Q8_SCORE_MODE, _lib.Q8_SCORE_REF)
    ref_n = ref.cpu().numpy()
    exact = oracle.prefill(new, pos0, n_tok, nh, nkv, stride, qd, cache=q8, mode=0)
    faithful = oracle.prefill(new, pos0, n_tok, nh, nkv, stride, qd, cache=q8, mode=1)
    print(f"\nprefill int8 cache, 512 tokens at pos0 1536 (mean-rel): default mode vs reference attn_prefill_q8 "
          f"{oracle.mean_rel_err(got[_lib.Q8_SCORE_REF], ref_n):.2e}; exact mode vs exact-score oracle "
          f"{oracle.mean_rel_err(got[_lib.Q8_SCORE_EXACT], exact):.2e}; exact mode vs reference kernel "
          f"{oracle.mean_rel_err(got[_lib.Q8_SCORE_EXACT], ref_n):.2e}; kernel-faithful vs exact oracle "
          f"{oracle.mean_rel_err(faithful, exact):.2e}")
    assert oracle.allclose_err(ref_n, faithful, RTOL, ATOL) < 1.0          # the reference kernel is what mode 1 restates
    for name, g, w in (("default mode vs the reference kernel", got[_lib.Q8_SCORE_REF], ref_n),
                       ("exact mode vs the exact-score oracle", got[_lib.Q8_SCORE_EXACT], exact)):
        assert oracle.max_abs_err(g, w) <= 2e-2 and oracle.mean_rel_err(g, w) <= 5e-3, name
