"""The handle-free, allocation-free decode entry point against the ordinary one.

`mx230_attn_decode_q8_noalloc` exists for hosts that cannot call cudaMalloc at the moment they
need attention (every free byte of HBM already belongs to their KV pool, or they may only enqueue
work on a stream they were given), so it keeps its split-KV scratch in a fixed array inside the
library instead of a handle's workspace.  It must give what `mx230_attn_decode_q8` gives, on two
calls in a row (the array keeps the first call's contents), and refuse shapes beyond its array.
This file sorts last on purpose: a run that stops at the first failure has then run everything else.
"""
import numpy as np
import pytest
import torch

import oracle
from mx230_b200 import _lib
from mx230_b200 import llm_attention as la
from tests.conftest import assert_close

pytestmark = pytest.mark.gpu
TOL = dict(max_abs=2e-5, mean_rel=1e-4)  # the tolerance of the other decode tests


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _cache(nh, nkv, ctx, seed):
    qd = nh * 64
    rows = oracle.normal((ctx, qd + 2 * nkv * 64), seed, 0)
    w = oracle.Q8Cache(ctx, nkv)
    for t in range(ctx):
        oracle.rope_qkv_row(rows[t], t, nh, nkv, 64, 1e6)
        oracle.quantize_kv_row(w, rows[t], t, qd)
    c = la.KvCache(ctx, nkv, 64, True)
    c.k.copy_(dev(w.kq)), c.v.copy_(dev(w.vq)), c.ks.copy_(dev(w.ks)), c.vs.copy_(dev(w.vs))
    c.kb.copy_(dev(w.kb)), c.vb.copy_(dev(w.vb))
    return rows, w, c


@pytest.mark.parametrize("nh,nkv,ctx", [(14, 2, 2048), (32, 4, 700), (12, 12, 300)])
def test_noalloc_decode_matches_handle_path_twice(handle, nh, nkv, ctx):
    torch.cuda.set_device(0)
    rows, w, c = _cache(nh, nkv, ctx, 90 + nh)
    qd = nh * 64
    for t_cur in (ctx - 1, ctx // 3):      # two calls in a row share the built-in scratch array
        q = dev(rows[t_cur])
        ref = torch.full((qd,), float("nan"), device="cuda")
        la.attn_decode(handle, ref, q, c, t_cur, nh, nkv, 64)
        got = torch.full((qd,), float("nan"), device="cuda")
        la.attn_decode_q8_noalloc(got, q, c, t_cur, nh, nkv, 64)
        torch.cuda.synchronize()
        assert_close(got.cpu().numpy(), ref.cpu().numpy(), f"noalloc vs handle t={t_cur}", **TOL)
        assert_close(got.cpu().numpy(), oracle.gqa_decode_q8(rows[t_cur], w, t_cur, nh, 1),
                     f"noalloc vs oracle t={t_cur}", **TOL)
    handle.check_status()


def test_noalloc_rejects_what_does_not_fit(handle):
    nh, nkv = 4096, 512   # 4096 heads x 1 key split x 264 B = 1.03 MiB > the 1 MiB of built-in scratch
    c = la.KvCache(16, nkv, 64, True)
    out = torch.zeros(nh * 64, device="cuda")
    q = torch.zeros((nh + 2 * nkv) * 64, device="cuda")
    with pytest.raises(_lib.Mx230Error) as e:
        la.attn_decode_q8_noalloc(out, q, c, 15, nh, nkv, 64)
    assert e.value.code == _lib.ERR_WORKSPACE
    with pytest.raises(_lib.Mx230Error) as e:
        la.attn_decode_q8_noalloc(out, q, c, 5, 14, 2, 128)
    assert e.value.code == _lib.ERR_UNSUPPORTED
