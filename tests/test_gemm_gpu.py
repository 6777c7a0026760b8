"""The prefill-side projections (mx230_gemm) through the C ABI against the oracle's sequential fp32 sums.

fp32 weights go through the tensor cores as two bf16 terms per operand (16 bits of mantissa, three products), so
the gate is close to fp32's own: max-abs 2e-4, mean-rel 2e-5 on outputs of order 1.  fp16 weights are used as they
lie and the activations are rounded to fp16 (11 bits): max-abs 5e-3, mean-rel 1e-3.
"""
import numpy as np
import pytest
import torch

import oracle
from mx230_b200 import llm_attention as la
from mx230_b200._lib import Mx230Error, check, lib, ptr
from tests.conftest import assert_close

pytestmark = pytest.mark.gpu


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


SHAPES = [  # m, n, k
    (512, 1152, 896),    # Qwen2-0.5B qkv projection of a 512-token chunk (gpu.rs:3187-3198)
    (512, 896, 896),     # its output projection (gpu.rs:3354-3365)
    (300, 2560, 2048),   # TinyLlama-like qkv, ragged m
    (130, 136, 80),      # ragged in every dimension: partial tiles in m and n, a partial k step
    (9, 64, 64), (1, 8, 16),
]


@pytest.mark.parametrize("fp16", [False, True])
@pytest.mark.parametrize("bias", [True, False])
@pytest.mark.parametrize("m,n,k", SHAPES)
def test_gemm_matches_oracle(handle, m, n, k, bias, fp16):
    a = oracle.normal((m, k), 700 + m, 0)
    w = (oracle.normal((k, n), 700 + n, 1) / np.sqrt(k)).astype(np.float32)
    b = oracle.normal((n,), 700 + k, 2) if bias else None
    if fp16:
        w = w.astype(np.float16)
    want = oracle.gemm(a, w, b)
    c = torch.full((m, n), float("nan"), device="cuda")
    la.gemm(handle, c, dev(a), dev(w), None if b is None else dev(b))
    handle.check_status()
    tol = dict(max_abs=5e-3, mean_rel=1e-3) if fp16 else dict(max_abs=2e-4, mean_rel=2e-5)
    assert_close(c.cpu().numpy(), want, f"gemm {m}x{n}x{k} fp16={fp16}", **tol)


def test_gemm_is_deterministic_and_rejects_bad_shapes(handle):
    m, n, k = 200, 256, 192
    a, w = dev(oracle.normal((m, k), 1, 0)), dev(oracle.normal((k, n), 1, 1))
    c1, c2 = torch.zeros(m, n, device="cuda"), torch.zeros(m, n, device="cuda")
    la.gemm(handle, c1, a, w)
    la.gemm(handle, c2, a, w)
    assert torch.equal(c1, c2)
    with pytest.raises(Mx230Error):   # k must be a multiple of 16
        check(lib().mx230_gemm(handle._h, None, ptr(c1), ptr(a), ptr(w), 0, None, m, n, 24))
    with pytest.raises(Mx230Error):   # n must be a multiple of 8
        check(lib().mx230_gemm(handle._h, None, ptr(c1), ptr(a), ptr(w), 0, None, m, 12, k))
    check(lib().mx230_gemm(handle._h, None, ptr(c1), ptr(a), ptr(w), 0, None, 0, n, k))   # no rows: nothing to do


@pytest.mark.parametrize("quant", [False, True])
def test_prefill_layer_attention_with_projections(handle, quant):
    """qkv projection -> RoPE -> KV write -> prefill attention -> output projection for a 200-token chunk that
    follows 56 cached tokens (Qwen-like 14q/2kv, e = 896), against the same chain in the oracle.  The oracle's
    attention runs on the device's own qkv rows after RoPE (so that int8 codes agree bit for bit, as in the
    prefill tests); the projections are checked on their own above."""
    nh, nkv, e, pos0, n_tok, theta = 14, 2, 896, 56, 200, 1e6
    qd, kvd = nh * 64, nkv * 64
    qkvd = qd + 2 * kvd
    x = oracle.normal((pos0 + n_tok, e), 801, 0)
    w_qkv = (oracle.normal((e, qkvd), 802, 0) / np.sqrt(e)).astype(np.float32)
    b_qkv = oracle.normal((qkvd,), 803, 0) * 0.1
    w_proj = (oracle.normal((qd, e), 804, 0) / np.sqrt(qd)).astype(np.float32)
    b_proj = oracle.normal((e,), 805, 0) * 0.1
    c = la.KvCache(pos0 + n_tok, nkv, 64, quant)
    dx, dwq, dbq, dwp, dbp = dev(x), dev(w_qkv), dev(b_qkv), dev(w_proj), dev(b_proj)
    qkv = torch.zeros(pos0 + n_tok, qkvd, device="cuda")
    attn = torch.zeros(pos0 + n_tok, qd, device="cuda")
    y = torch.full((pos0 + n_tok, e), float("nan"), device="cuda")
    la.prefill_layer_attention(handle, y[:pos0], dx[:pos0], dwq, dbq, dwp, dbp, qkv[:pos0], attn[:pos0], c, 0, pos0, nh, nkv,
                               64, theta)
    la.prefill_layer_attention(handle, y[pos0:], dx[pos0:], dwq, dbq, dwp, dbp, qkv[pos0:], attn[pos0:], c, pos0, n_tok, nh,
                               nkv, 64, theta)
    handle.check_status()
    roped = qkv.cpu().numpy()
    # the qkv rows before RoPE are the projection of x: undo nothing, compare the un-rotated V third, which RoPE leaves alone
    want_qkv = oracle.gemm(x, w_qkv, b_qkv)
    assert_close(roped[:, qd + kvd:], want_qkv[:, qd + kvd:], "v columns of the qkv projection", max_abs=2e-4, mean_rel=2e-5)
    if quant:
        w8 = oracle.Q8Cache(pos0 + n_tok, nkv)
        for t in range(pos0 + n_tok):
            oracle.quantize_kv_row(w8, roped[t], t, qd)
        want_attn = oracle.prefill(roped[pos0:], pos0, n_tok, nh, nkv, qkvd, qd, cache=w8, mode=1)
    else:
        kc, vc = np.zeros((pos0 + n_tok, kvd), np.float32), np.zeros((pos0 + n_tok, kvd), np.float32)
        for t in range(pos0 + n_tok):
            oracle.copy_kv_row(kc, vc, roped[t], t, qd, kvd)
        want_attn = oracle.prefill(roped[pos0:], pos0, n_tok, nh, nkv, qkvd, qd, kcache=kc, vcache=vc)
    assert_close(attn[pos0:].cpu().numpy(), want_attn, "attention rows")
    want_y = oracle.gemm(attn[pos0:].cpu().numpy(), w_proj, b_proj)
    assert_close(y[pos0:].cpu().numpy(), want_y, "output projection", max_abs=2e-4, mean_rel=2e-5)
