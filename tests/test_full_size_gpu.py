"""Size-independent properties at the full sizes of the two largest configurations, where the
oracle cannot be run on everything: the 32768-token non-causal forward (B=1 H=8 N=32768 d=64)
and the 131072-key int8 decode (32 query / 4 KV heads)."""
import numpy as np
import pytest
import torch

import oracle
from mx230_b200 import _lib, flash_attention as fa, llm_attention as la
from tests.conftest import assert_close

pytestmark = pytest.mark.gpu


def test_forward_32768_non_causal(handle):
    n, bh = 32768, 2
    q, k, v = (torch.from_numpy(oracle.normal((bh, n, 64), 21, i)).cuda() for i in range(3))
    handle.reserve(fa.workspace_bytes(bh, n, False))
    o = torch.empty_like(q)
    l = torch.empty(bh, n, device="cuda")
    fa.run_flash_lse(handle, q, k, torch.ones_like(v), o, l, n, False)
    handle.check_status()
    assert float((o - 1.0).abs().max()) < 2e-2           # softmax weights of every row sum to one
    fa.run_flash_lse(handle, q, k, v, o, l, n, False)
    o2 = torch.empty_like(o)
    fa.run_flash_lse(handle, q, k, 2.0 * v, o2, l, n, False)
    handle.check_status()
    assert torch.equal(o2, 2.0 * o)                       # linear in V (scaling by 2 is exact)
    # sampled rows and their log-sum-exp against the oracle's per-row arithmetic
    qn, kn, vn = (t.cpu().numpy() for t in (q, k, v))
    rows = oracle.attn_fwd_rows(qn, kn, vn, False, 7, 4099)
    assert_close(o.cpu().numpy()[:, 7::4099], rows, "sampled rows at N=32768")
    s = (qn[0, 7] @ kn[0].T) * 0.125
    lse = float(s.max() + np.log(np.exp(s - s.max()).sum()))
    assert abs(float(l[0, 7]) - lse) < 2e-2


def test_int8_decode_131072_keys(handle):
    nh, nkv, ctx, n_seq = 32, 4, 131072, 2
    qd, kvd = nh * 64, nkv * 64
    c = la.KvCache(n_seq * ctx, nkv, 64, True)
    g = torch.Generator(device="cuda").manual_seed(3)
    c.k.random_(-128, 128, generator=g), c.v.random_(-128, 128, generator=g)
    c.ks.uniform_(0.01, 0.03, generator=g), c.vs.uniform_(0.01, 0.03, generator=g)
    c.kb.normal_(generator=g), c.vb.normal_(generator=g)
    q = torch.randn(n_seq, qd, device="cuda", generator=g)
    pos = torch.full((n_seq,), ctx - 1, dtype=torch.int32, device="cuda")
    handle.reserve(max(1 << 20, int(_lib.lib().mx230_decode_workspace_bytes(n_seq, nh, 256))))
    out = torch.zeros(n_seq, qd, device="cuda")
    la.attn_decode_slab(handle, out, q, c, pos, n_seq, nh, nkv, 64, ctx, qd, qd)
    # the same context as four key ranges (as four ranks would hold them), merged by log-sum-exp
    rows = n_seq * nh
    cuts = [0, 32768, 65536, 100000, ctx]
    pm, pl = torch.zeros(4, rows, device="cuda"), torch.zeros(4, rows, device="cuda")
    pa = torch.zeros(4, rows, 64, device="cuda")
    for r in range(4):
        la.attn_decode_partial(handle, pm[r], pl[r], pa[r], q, c, cuts[r], cuts[r + 1], n_seq, nh, nkv, 64, ctx, qd)
    merged = torch.zeros(rows, 64, device="cuda")
    la.merge_partials(handle, merged, pm, pl, pa, 4, rows)
    handle.check_status()
    assert_close(merged.cpu().numpy().reshape(n_seq, qd), out.cpu().numpy(), "split-KV merge vs unsplit",
                 max_abs=2e-5, mean_rel=1e-4)
    # sequence 1 against the oracle (kernel-faithful mode) over all 131072 keys
    w = oracle.Q8Cache(ctx, nkv)
    sl = slice(ctx, 2 * ctx)
    w.kq, w.vq = c.k[sl].cpu().numpy(), c.v[sl].cpu().numpy()
    w.ks, w.vs, w.kb, w.vb = (t[sl].cpu().numpy() for t in (c.ks, c.vs, c.kb, c.vb))
    want = oracle.gqa_decode_q8(q[1].cpu().numpy(), w, ctx - 1, nh, 1)
    # (the oracle adds 131072 fp32 terms one after the other, the device in tiles and splits: the two
    # orders differ by ~1e-4 here, far inside the parity bar of 2e-2 / 5e-3)
    assert_close(out[1].cpu().numpy(), want, "decode over 131072 keys vs oracle", max_abs=1e-3, mean_rel=1e-3)
    # V codes all equal within a head: the output is that constant (weights sum to one)
    c.v.fill_(7), c.vs.fill_(0.5), c.vb.fill_(-1.0)
    la.attn_decode_slab(handle, out, q, c, pos, n_seq, nh, nkv, 64, ctx, qd, qd)
    handle.check_status()
    assert float((out - 2.5).abs().max()) < 1e-4
