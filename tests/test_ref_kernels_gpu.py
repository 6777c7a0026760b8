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
