"""The fused split-KV exchange + merge kernel (mx230_splitkv_*) on ONE GPU.

Ranks of a real run sit on different GPUs and their kernels wait on one another, so two ranks'
kernels are never in flight together here.  What one GPU can show:

* world 1: push to the own region, wait on the own flags, merge -- equal to mx230_merge_partials_packed;
* world 2 emulated in one process (each communicator attached to the other's region by address): the
  rank launched FIRST pushes its triples and then waits for a step number that nothing publishes
  while it runs, so its bounded wait runs out: the kernel records the status and returns without
  writing its output.  The rank launched SECOND finds the first one's push complete and must produce
  exactly the merge of both triples.  The roles swap on the next step, which also covers the second
  half of the double-buffered region.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from mx230_b200 import _lib
from mx230_b200 import llm_attention as la
from mx230_b200._lib import Mx230Error, check, lib, ptr
from mx230_b200.common import Handle
from mx230_b200.multi_gpu import PeerExchange

pytestmark = pytest.mark.gpu


def _triples(rows, seed, empty=False):
    g = torch.Generator(device="cpu").manual_seed(seed)
    m = torch.randn(rows, generator=g) * 3
    l = torch.rand(rows, generator=g) + 0.5
    acc = torch.randn(rows, 64, generator=g)
    if empty:   # a rank whose key range is empty
        m[:] = float("-inf")
        l[:] = 0
        acc[:] = 0
    return torch.cat([m, l, acc.reshape(-1)]).cuda()


@pytest.mark.parametrize("rows", [2, 16, 250, 2048])
def test_world_one_equals_packed_merge(handle, rows):
    local = _triples(rows, rows)
    ex = PeerExchange(handle, 0, 1, rows)
    try:
        want = torch.zeros(rows, 64, device="cuda")
        la.merge_partials_packed(handle, want, local, 1, rows)
        for _ in range(3):   # both halves of the region and a reuse
            out = torch.full((rows, 64), float("nan"), device="cuda")
            ex.exchange_merge(out, local)
            handle.check_status()
            assert torch.equal(out, want)
    finally:
        ex.close()


def _comm(h, rank, world, rows):
    c = C.c_void_p()
    check(lib().mx230_splitkv_comm_create(h._h, rank, world, rows, 64, C.byref(c)))
    return c


@pytest.mark.parametrize("rows,empty", [(64, False), (30, True)])
def test_two_ranks_in_turn_first_times_out_second_merges(rows, empty):
    hs = [Handle(0, 1 << 20), Handle(0, 1 << 20)]
    comms = [_comm(hs[r], r, 2, rows) for r in range(2)]
    try:
        for r in range(2):
            base, nbytes = C.c_void_p(), C.c_size_t()
            check(lib().mx230_splitkv_comm_region(comms[1 - r], C.byref(base), C.byref(nbytes)))
            assert nbytes.value >= 2 * 2 * rows * 66 * 4
            check(lib().mx230_splitkv_comm_attach(comms[r], 1 - r, base))
        for h in hs:
            h.set_option(_lib.OPT_WAIT_LIMIT, 2000)   # 2e6 cycles, about a millisecond
        for step in range(4):
            local = [_triples(rows, 10 * step + r, empty and r == 1) for r in range(2)]
            want = torch.zeros(rows, 64, device="cuda")
            la.merge_partials_packed(hs[0], want, torch.stack(local), 2, rows)
            first = step & 1
            outs = [torch.full((rows, 64), float("nan"), device="cuda") for _ in range(2)]
            check(lib().mx230_splitkv_exchange_merge(comms[first], None, ptr(outs[first]), ptr(local[first])))
            with pytest.raises(Mx230Error) as e:
                hs[first].check_status()
            assert e.value.code == _lib.ERR_DEVICE_STATUS
            assert bool(torch.isnan(outs[first]).all())      # nothing written after the wait ran out
            check(lib().mx230_splitkv_exchange_merge(comms[1 - first], None, ptr(outs[1 - first]), ptr(local[1 - first])))
            hs[1 - first].check_status()
            assert torch.equal(outs[1 - first], want)
            hs[first].check_status()                          # the status was cleared by the read above
    finally:
        for c in comms:
            check(lib().mx230_splitkv_comm_disconnect(c))
        for c in comms:
            lib().mx230_splitkv_comm_destroy(c)
        for h in hs:
            h.close()


def test_argument_checks(handle):
    c = C.c_void_p()
    for rank, world, rows in ((0, 17, 8), (2, 2, 8), (0, 2, 7), (0, 2, 0)):
        with pytest.raises(Mx230Error):
            check(lib().mx230_splitkv_comm_create(handle._h, rank, world, rows, 64, C.byref(c)))
    c = _comm(handle, 0, 2, 8)
    try:
        out, local = torch.zeros(8, 64, device="cuda"), torch.zeros(8 * 66, device="cuda")
        with pytest.raises(Mx230Error):   # rank 1 was never connected
            check(lib().mx230_splitkv_exchange_merge(c, None, ptr(out), ptr(local)))
        with pytest.raises(Mx230Error):
            check(lib().mx230_splitkv_comm_attach(c, 0, ptr(local)))   # the own rank is not a peer
    finally:
        lib().mx230_splitkv_comm_destroy(c)


def _random_q8_cache(rows, nkv, seed):
    torch.manual_seed(seed)
    c = la.KvCache(rows, nkv, 64, True)
    c.k.random_(-128, 128), c.v.random_(-128, 128)
    c.ks.uniform_(0.01, 0.03), c.vs.uniform_(0.01, 0.03), c.kb.uniform_(-0.1, 0.1), c.vb.uniform_(-0.1, 0.1)
    return c


@pytest.mark.parametrize("one_kernel", [False, True])
@pytest.mark.parametrize("t1", [700, 0])
def test_partial_push_two_ranks_in_turn(t1, one_kernel):
    """The attention kernel stores its triples itself (mx230_attn_decode_partial_push) and a second kernel only
    waits and merges, or the attention kernel does that as well (mx230_attn_decode_splitkv).  Rank 0 holds keys [0, 1300), rank 1 keys [0, t1) of its own cache (t1 = 0: an empty
    range, the neutral triple).  Same turn-taking as above: the rank that goes first runs out of its wait."""
    n_seq, nh, nkv, span = 3, 8, 2, 1300
    rows = n_seq * nh
    hs = [Handle(0, 16 << 20), Handle(0, 16 << 20)]
    comms = [_comm(hs[r], r, 2, rows) for r in range(2)]
    try:
        for r in range(2):
            base = C.c_void_p()
            check(lib().mx230_splitkv_comm_region(comms[1 - r], C.byref(base), None))
            check(lib().mx230_splitkv_comm_attach(comms[r], 1 - r, base))
        for h in hs:
            h.set_option(_lib.OPT_WAIT_LIMIT, 2000)
        caches = [_random_q8_cache(n_seq * span, nkv, 5 + r) for r in range(2)]
        ranges = [span, t1]
        q = torch.randn(n_seq, nh * 64, device="cuda")
        # what the all-gather path would merge: each rank's packed triples, in rank order
        packed = torch.zeros(2, rows * 66, device="cuda")
        for r in range(2):
            m, l, acc = packed[r, :rows], packed[r, rows:2 * rows], packed[r, 2 * rows:]
            if ranges[r] > 0:
                la.attn_decode_partial(hs[r], m, l, acc, q, caches[r], 0, ranges[r], n_seq, nh, nkv, 64, span, nh * 64)
            else:
                m.fill_(float("-inf"))
        want = torch.zeros(rows, 64, device="cuda")
        la.merge_partials_packed(hs[0], want, packed, 2, rows)
        for step in range(3):
            first = step & 1
            outs = [torch.full((rows, 64), float("nan"), device="cuda") for _ in range(2)]
            for r in (first, 1 - first):
                if one_kernel:
                    la.attn_decode_splitkv(hs[r], comms[r], outs[r], q, caches[r], 0, ranges[r], n_seq, nh, nkv, 64, span,
                                           nh * 64)
                else:
                    la.attn_decode_partial_push(hs[r], comms[r], q, caches[r], 0, ranges[r], n_seq, nh, nkv, 64, span,
                                                nh * 64)
                    check(lib().mx230_splitkv_wait_merge(comms[r], None, ptr(outs[r])))
                if r == first:
                    with pytest.raises(Mx230Error):
                        hs[r].check_status()
                    assert bool(torch.isnan(outs[r]).all())
                else:
                    hs[r].check_status()
                    assert torch.equal(outs[r], want)
    finally:
        for c in comms:
            check(lib().mx230_splitkv_comm_disconnect(c))
        for c in comms:
            lib().mx230_splitkv_comm_destroy(c)
        for h in hs:
            h.close()


@pytest.mark.parametrize("n_seq,quant", [(3, True), (3, False), (80, True)])
def test_one_kernel_step_world_one(handle, n_seq, quant):
    """World 1: the one-kernel step equals partial attention + merge of the single triple, for the int8 and the
    fp32 cache; with 80 sequences x 2 KV heads there are more groups than SMs and the entry point puts the wait
    and the merge into a kernel of its own."""
    nh, nkv, span = 8, 2, 900
    rows = n_seq * nh
    c = _random_q8_cache(n_seq * span, nkv, 9) if quant else la.KvCache(n_seq * span, nkv)
    if not quant:
        c.k.normal_(), c.v.normal_()
    q = torch.randn(n_seq, nh * 64, device="cuda")
    packed = torch.zeros(rows * 66, device="cuda")
    la.attn_decode_partial(handle, packed[:rows], packed[rows:2 * rows], packed[2 * rows:], q, c, 0, span, n_seq, nh, nkv,
                           64, span, nh * 64)
    want = torch.zeros(rows, 64, device="cuda")
    la.merge_partials_packed(handle, want, packed, 1, rows)
    ex = PeerExchange(handle, 0, 1, rows)
    try:
        for _ in range(3):
            out = torch.full((rows, 64), float("nan"), device="cuda")
            la.attn_decode_splitkv(handle, ex._c, out, q, c, 0, span, n_seq, nh, nkv, 64, span, nh * 64)
            handle.check_status()
            assert torch.equal(out, want)
    finally:
        ex.close()
