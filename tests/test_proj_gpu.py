"""The projections either side of the attention step: gemv (fp32 / fp16 weights, fused residual)
against the oracle's sequential sums, and the fused qkv step (gemv + RoPE + KV write) against the
separate oracle operations; the int8 codes are checked bit-exactly against the oracle quantiser
fed with the very k, v values the kernel produced."""
import numpy as np
import pytest
import torch

import oracle
from mx230_b200 import llm_attention as la
from tests.conftest import assert_close

pytestmark = pytest.mark.gpu

TOL = dict(max_abs=2e-4, mean_rel=2e-5)   # fp32 sums in a different order than the oracle's


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.parametrize("n_in,n_out", [(896, 1152), (896, 896), (64, 4), (2048, 2560), (100, 132), (4864, 896)])
@pytest.mark.parametrize("fp16", [False, True])
def test_gemv_matches_oracle(handle, n_in, n_out, fp16):
    x = oracle.normal((n_in,), 600, 0)
    w = (oracle.normal((n_in, n_out), 601, 0) * 0.05).astype(np.float16 if fp16 else np.float32)
    b = oracle.normal((n_out,), 602, 0)
    y0 = oracle.normal((n_out,), 603, 0)
    for accum, bias in ((False, True), (True, True), (False, False)):
        want = oracle.gemv(x, w, b if bias else None, y0, accum)
        y = dev(y0)
        la.gemv(handle, y, dev(x), dev(w), dev(b) if bias else None, accum)
        handle.check_status()
        assert_close(y.cpu().numpy(), want, f"gemv accum={accum} bias={bias}", **TOL)
    # deterministic: the slices are added in a fixed order
    y1, y2 = dev(y0), dev(y0)
    la.gemv(handle, y1, dev(x), dev(w), dev(b))
    la.gemv(handle, y2, dev(x), dev(w), dev(b))
    assert torch.equal(y1, y2)


@pytest.mark.parametrize("quant,affine", [(False, True), (True, True), (True, False)])
@pytest.mark.parametrize("paged,dyn", [(False, False), (True, True)])
def test_fused_qkv_step(handle, quant, affine, paged, dyn):
    nh, nkv, n_in, theta, bs, pos = 14, 2, 896, 1e6, 16, 37
    qd, kvd = nh * 64, nkv * 64
    n_out = qd + 2 * kvd
    x = oracle.normal((n_in,), 610, 0)
    w = (oracle.normal((n_in, n_out), 611, 0) * 0.05).astype(np.float16)
    b = oracle.normal((n_out,), 612, 0)
    table = np.random.default_rng(2).permutation(8).astype(np.int32) if paged else None
    slots = 8 * bs
    c = la.KvCache(slots, nkv, 64, quant, affine)
    qkv = torch.full((n_out,), float("nan"), device="cuda")
    pg = la.Paging(dev(table), bs) if paged else None
    p = torch.tensor([pos], dtype=torch.int32, device="cuda") if dyn else pos
    la.qkv_rope_kvwrite(handle, qkv, dev(x), dev(w), dev(b), p, c, nh, nkv, theta, pg)
    handle.check_status()
    got = qkv.cpu().numpy()
    want = oracle.rope_qkv_row(oracle.gemv(x, w, b), pos, nh, nkv, 64, theta)
    assert_close(got, want, "fused qkv row", **TOL)
    row = int(table[pos // bs]) * bs + pos % bs if paged else pos
    if not quant:
        assert np.array_equal(c.k[row].cpu().numpy(), got[qd:qd + kvd])
        assert np.array_equal(c.v[row].cpu().numpy(), got[qd + kvd:])
        assert float(c.k.abs().sum()) == float(c.k[row].abs().sum())   # no other row was touched
    else:
        # the oracle quantiser on the kernel's own k, v values: codes, scales and betas bit-exact
        q8 = oracle.Q8Cache(slots, nkv, 64, affine)
        oracle.quantize_kv_row(q8, got, pos, qd, table, bs)
        for name, dev_t, ref in (("kq", c.k, q8.kq), ("vq", c.v, q8.vq), ("ks", c.ks, q8.ks), ("vs", c.vs, q8.vs)):
            assert np.array_equal(dev_t[row].cpu().numpy(), ref[row]), name
        if affine:
            assert np.array_equal(c.kb[row].cpu().numpy(), q8.kb[row]) and np.array_equal(c.vb[row].cpu().numpy(), q8.vb[row])
    # the fused step feeds the decode attention like the separate launches do
    if pos == 37 and not paged:
        out = torch.zeros(qd, device="cuda")
        c2 = la.KvCache(slots, nkv, 64, quant, affine)
        for t in range(pos + 1):   # fill the earlier positions through the fused step as well
            xt = oracle.normal((n_in,), 620 + t, 0)
            la.qkv_rope_kvwrite(handle, qkv, dev(xt), dev(w), dev(b), t, c2, nh, nkv, theta)
        la.attn_decode(handle, out, qkv, c2, pos, nh, nkv, 64)
        handle.check_status()
        assert torch.isfinite(out).all()


@pytest.mark.parametrize("n_in,n_out", [(896, 1152), (2048, 2560), (64, 8), (4864, 896)])
@pytest.mark.parametrize("ag", [4, 8])
def test_gemv_int8_matches_oracle(handle, n_in, n_out, ag):
    rng = np.random.default_rng(n_in + ag)
    x = oracle.normal((n_in,), 630, 0)
    x[: 2 * ag] = 0.0                                   # an all-zero activation group (scale 1, codes 0)
    w32 = oracle.pack_int8_weights(rng.integers(-127, 128, size=(n_in, n_out), dtype=np.int8))
    scales = (np.abs(oracle.normal((n_out,), 631, 0)) * 0.01 + 0.001).astype(np.float32)
    b = oracle.normal((n_out,), 632, 0)
    y0 = oracle.normal((n_out,), 633, 0)
    for accum, bias in ((False, True), (True, False)):
        want = oracle.gemv_int8(x, w32, scales, b if bias else None, y0, accum, ag)
        y = dev(y0)
        la.gemv_int8(handle, y, dev(x), dev(w32), dev(scales), dev(b) if bias else None, accum, ag)
        handle.check_status()
        assert_close(y.cpu().numpy(), want, f"gemv_int8 ag={ag} accum={accum}", max_abs=2e-4 * max(1.0, float(np.abs(want).max())), mean_rel=2e-5)


def test_fused_qkv_step_with_int8_weights(handle):
    nh, nkv, n_in, theta, pos = 14, 2, 896, 1e6, 21
    qd, kvd = nh * 64, nkv * 64
    n_out = qd + 2 * kvd
    rng = np.random.default_rng(7)
    x = oracle.normal((n_in,), 640, 0)
    w32 = oracle.pack_int8_weights(rng.integers(-127, 128, size=(n_in, n_out), dtype=np.int8))
    scales = np.full(n_out, 0.002, np.float32)
    b = oracle.normal((n_out,), 641, 0)
    c = la.KvCache(64, nkv, 64, True)
    qkv = torch.full((n_out,), float("nan"), device="cuda")
    la.qkv_rope_kvwrite(handle, qkv, dev(x), dev(w32), dev(b), pos, c, nh, nkv, theta, w_scales=dev(scales), act_group=8)
    handle.check_status()
    got = qkv.cpu().numpy()
    want = oracle.rope_qkv_row(oracle.gemv_int8(x, w32, scales, b, ag=8), pos, nh, nkv, 64, theta)
    assert_close(got, want, "fused qkv row, int8 weights", max_abs=2e-4 * float(np.abs(want).max()), mean_rel=2e-5)
    q8 = oracle.Q8Cache(64, nkv)
    oracle.quantize_kv_row(q8, got, pos, qd)
    assert np.array_equal(c.k[pos].cpu().numpy(), q8.kq[pos]) and np.array_equal(c.v[pos].cpu().numpy(), q8.vq[pos])
    assert np.array_equal(c.ks[pos].cpu().numpy(), q8.ks[pos]) and np.array_equal(c.vb[pos].cpu().numpy(), q8.vb[pos])


def test_gemv_rejects_bad_arguments(handle):
    from mx230_b200._lib import Mx230Error
    with pytest.raises(Mx230Error):
        la.gemv(handle, torch.zeros(6, device="cuda"), torch.zeros(8, device="cuda"), torch.zeros(8, 6, device="cuda"))
