"""The bounded-wait exit of the tensor kernels, run for real: a wait that is made to run out returns a status
instead of hanging, and the handle keeps working.

Every device-side barrier wait gives up after the limit of MX230_OPT_WAIT_LIMIT and records a status word; all
roles of the CTA then leave their loops, tensor memory is released and the kernel returns by itself.  The test
hook MX230_OPT_TEST_DROP_TILE makes the TMA producer of one CTA never request one K/V (or Q/dO) tile, so the MMA
issuer that waits for it runs into the limit (set to about a millisecond here: long enough for every load that WAS
issued to have landed before the CTA leaves).  Nothing faults and nothing spins without bound: the launch ends,
mx230_check_status reports MX230_ERR_DEVICE_STATUS, and the next ordinary call on the same handle meets the oracle.
"""
import numpy as np
import pytest
import torch

import oracle
from mx230_b200 import _lib
from mx230_b200 import flash_attention as fa
from mx230_b200.common import Handle
from tests.conftest import assert_close

pytestmark = pytest.mark.gpu


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _inputs(n=640, bh=2, seed=55):
    return tuple(oracle.normal((bh, n, 64), seed, i) for i in range(4))


def test_forward_wait_runs_out_and_handle_recovers():
    torch.cuda.set_device(0)
    h = Handle(0, 64 << 20)
    q, k, v, _ = _inputs()
    n = q.shape[1]
    Q, K, V = dev(q), dev(k), dev(v)
    o, l = torch.zeros_like(Q), torch.zeros(q.shape[0], n, device="cuda")
    try:
        h.set_option(_lib.OPT_WAIT_LIMIT, 2000)        # 2e6 SM cycles, about 1 ms
        h.set_option(_lib.OPT_TEST_DROP_TILE, 1)       # CTA 0 never gets its second K/V tile
        fa.run_flash_lse(h, Q, K, V, o, l, n, True)
        with pytest.raises(_lib.Mx230Error) as e:
            h.check_status()
        assert e.value.code == _lib.ERR_DEVICE_STATUS
    finally:
        h.set_option(_lib.OPT_TEST_DROP_TILE, -1)
        h.set_option(_lib.OPT_WAIT_LIMIT, 4000000)
    # the status was cleared by the read; the same handle computes a correct forward right after
    fa.run_flash_lse(h, Q, K, V, o, l, n, True)
    h.check_status()
    wo, wl = oracle.attn_fwd(q, k, v, True)
    assert_close(o.cpu().numpy(), wo, "O after the aborted launch")
    assert_close(l.cpu().numpy(), wl, "L after the aborted launch")
    h.close()


def test_fused_backward_wait_runs_out_and_handle_recovers():
    torch.cuda.set_device(0)
    h = Handle(0, 64 << 20)
    q, k, v, do = _inputs(seed=56)
    n = q.shape[1]
    Q, K, V, DO = dev(q), dev(k), dev(v), dev(do)
    o, l = torch.zeros_like(Q), torch.zeros(q.shape[0], n, device="cuda")
    delta = torch.zeros_like(l)
    gq, gk, gv = (torch.zeros_like(Q) for _ in range(3))
    fa.run_flash_lse(h, Q, K, V, o, l, n, True)
    fa.run_preprocess(h, DO, o, delta, n)
    h.check_status()
    try:
        h.set_option(_lib.OPT_WAIT_LIMIT, 2000)
        h.set_option(_lib.OPT_TEST_DROP_TILE, 1)       # CTA 0 never gets its second streamed Q/dO tile
        fa.run_bwd_flash(h, Q, K, V, DO, l, delta, gq, gk, gv, n, True)
        with pytest.raises(_lib.Mx230Error) as e:
            h.check_status()
        assert e.value.code == _lib.ERR_DEVICE_STATUS
    finally:
        h.set_option(_lib.OPT_TEST_DROP_TILE, -1)
        h.set_option(_lib.OPT_WAIT_LIMIT, 4000000)
    fa.run_bwd_flash(h, Q, K, V, DO, l, delta, gq, gk, gv, n, True)
    h.check_status()
    wq, wk, wv = oracle.attn_bwd(q, k, v, do, True)
    assert_close(gq.cpu().numpy(), wq, "dQ after the aborted launch")
    assert_close(gk.cpu().numpy(), wk, "dK after the aborted launch")
    assert_close(gv.cpu().numpy(), wv, "dV after the aborted launch")
    h.close()
