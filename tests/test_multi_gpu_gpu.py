"""Two GPUs, one process each, NCCL: split-KV decode (partial attention on each rank's key
range, one all-gather, log-sum-exp merge) and (batch, head) sharding of the flash forward.
Skipped on a box with fewer than two GPUs.  NVLS is switched off for these short-lived
child processes.  The same decode step is then repeated with the all-gather and the merge fused into
one kernel over peer memory (plain peer stores and flags, no multimem): its output must equal the
NCCL path's bit for bit, since both merge the same triples in the same order."""
import os
import socket

import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu

TOL = dict(max_abs=2e-2, mean_rel=5e-3)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _problem(ctx, n_seq, nh, nkv):
    qs = oracle.normal((n_seq, nh * 64), 170, 0)
    q8 = oracle.Q8Cache(n_seq * ctx, nkv)
    for s in range(n_seq):
        kv = oracle.normal((ctx, 2 * nkv * 64), 171 + s, 0)
        for t in range(ctx):
            oracle.quantize_kv_row(q8, kv[t], s * ctx + t, 0)
    return qs, q8


def _worker(rank, world, port, ctx, n_seq, nh, nkv, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    from mx230_b200 import _lib, flash_attention as fa, llm_attention as la
    from mx230_b200.common import Handle
    from mx230_b200.multi_gpu import SplitKvDecoder, SplitKvPlan, shard_range
    import datetime
    torch.cuda.set_device(rank)
    # a short collective timeout: if the peer fails, this rank's next collective ends with an error
    # instead of spinning on the GPU
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank),
                            timeout=datetime.timedelta(seconds=60))
    try:
        h = Handle(rank, 64 << 20)
        dev = f"cuda:{rank}"
        # ---- split-KV decode: this rank holds keys [t0, t1) of every sequence ----
        qs, q8 = _problem(ctx, n_seq, nh, nkv)
        plan = SplitKvPlan(ctx=ctx, world=world, n_seq=n_seq, n_head=nh)
        t0, t1 = plan.key_range(rank)
        span = max(1, t1 - t0)
        c = la.KvCache(n_seq * span, nkv, 64, True, True, device=dev)
        for s in range(n_seq):
            sl, dl = slice(s * ctx + t0, s * ctx + t1), slice(s * span, s * span + (t1 - t0))
            c.k[dl] = torch.from_numpy(q8.kq[sl]).to(dev)
            c.v[dl] = torch.from_numpy(q8.vq[sl]).to(dev)
            c.ks[dl] = torch.from_numpy(q8.ks[sl]).to(dev)
            c.vs[dl] = torch.from_numpy(q8.vs[sl]).to(dev)
            c.kb[dl] = torch.from_numpy(q8.kb[sl]).to(dev)
            c.vb[dl] = torch.from_numpy(q8.vb[sl]).to(dev)
        h.set_option(_lib.OPT_Q8_SCORE_MODE, _lib.Q8_SCORE_EXACT)
        dec = SplitKvDecoder(h, plan, rank, device=dev)
        q_dev = torch.from_numpy(qs).to(dev)
        for _ in range(2):  # the second step reuses every buffer
            out = dec.step(q_dev, c, nkv, span, nh * 64)
        torch.cuda.synchronize()
        h.check_status()
        # the same step with exchange + merge in one kernel over peer memory; three steps walk both
        # halves of the double-buffered exchange region
        fused_equal = True
        for how in ("exchange", "push", "one"):   # stores by the merge kernel / by the attention kernel / all in one kernel
            fdec = SplitKvDecoder(h, plan, rank, device=dev, fused=how)
            try:
                for _ in range(3):
                    fout = fdec.step(q_dev, c, nkv, span, nh * 64)
                torch.cuda.synchronize()
                h.check_status()
                fused_equal = fused_equal and bool(torch.equal(fout, out))
            finally:
                fdec.close()
        want = oracle.gqa_decode_batched(qs, [ctx - 1] * n_seq, nh, nkv, cache=q8, seq_rows=ctx, mode=0)
        got = out.cpu().numpy().reshape(n_seq, nh * 64)
        err_dec = float(np.abs(got - want).max())
        rel_dec = float(np.abs(got - want).sum() / np.abs(want).sum())
        # ---- (batch, head) sharding of the forward: no collective on the data path ----
        bh, n = 6, 384
        Q, K, V = (oracle.normal((bh, n, 64), 180 + i, 0) for i in range(3))
        lo, hi = shard_range(bh, rank, world)
        o = torch.zeros(hi - lo, n, 64, device=dev)
        l = torch.zeros(hi - lo, n, device=dev)
        fa.run_flash_lse(h, *(torch.from_numpy(x[lo:hi]).to(dev) for x in (Q, K, V)), o, l, n, True)
        torch.cuda.synchronize()
        h.check_status()
        wo, _ = oracle.attn_fwd(Q[lo:hi], K[lo:hi], V[lo:hi], True)
        err_fwd = float(np.abs(o.cpu().numpy() - wo).max())
        # every rank ends with the same merged decode output
        chk = torch.tensor([float(out.double().sum())], device=dev)
        both = [torch.zeros_like(chk) for _ in range(world)]
        dist.all_gather(both, chk)
        ret[rank] = (err_dec, rel_dec, err_fwd, [float(b) for b in both], (lo, hi), fused_equal)
        dist.barrier()   # success path only: a rank that raised must not enter a collective its peer is not in
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("ctx", [640, 130])
def test_split_kv_decode_and_sharded_forward_two_gpus(ctx):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    world, n_seq, nh, nkv = 2, 2, 8, 2
    ctxm = mp.get_context("spawn")
    ret = ctxm.Manager().dict()
    port = _free_port()
    procs = [ctxm.Process(target=_worker, args=(r, world, port, ctx, n_seq, nh, nkv, ret), daemon=True)
             for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(300)
    codes = [p.exitcode for p in procs]
    for p in procs:   # never leave a rank behind on the GPUs
        if p.is_alive():
            p.terminate()
            p.join(10)
            if p.is_alive():
                p.kill()
    assert codes == [0] * world, f"rank exit codes {codes}"
    assert sorted(ret.keys()) == [0, 1]
    for r in range(world):
        err_dec, rel_dec, err_fwd, sums, _, fused_equal = ret[r]
        assert fused_equal, f"rank {r}: fused exchange+merge differs from all-gather + merge"
        assert err_dec < TOL["max_abs"] and rel_dec < TOL["mean_rel"], (r, err_dec, rel_dec)
        assert err_fwd < TOL["max_abs"], (r, err_fwd)
        assert abs(sums[0] - sums[1]) <= 1e-6 * max(1.0, abs(sums[0]))
    assert ret[0][4] == (0, 3) and ret[1][4] == (3, 6)


def test_two_handles_in_one_process():
    """One process driving two GPUs round-robin, a handle and a stream per device: the kernels'
    per-device function attributes and workspaces do not leak from one device to the other."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from mx230_b200 import flash_attention as fa, llm_attention as la
    from mx230_b200.common import Handle
    bh, n = 3, 300
    Q, K, V, dO = (oracle.normal((bh, n, 64), 190 + i, 0) for i in range(4))
    wo, wl = oracle.attn_fwd(Q, K, V, True)
    handles = [Handle(d, 32 << 20) for d in (1, 0)]   # device 1 first: nothing may assume device 0
    outs = []
    for h, d in zip(handles, (1, 0)):
        with torch.cuda.device(d):
            q, k, v, do = (torch.from_numpy(x).cuda(d) for x in (Q, K, V, dO))
            o, l = torch.zeros_like(q), torch.zeros(bh, n, device=f"cuda:{d}")
            delta = torch.zeros_like(l)
            dq, dk, dv = (torch.zeros_like(q) for _ in range(3))
            fa.run_flash_lse(h, q, k, v, o, l, n, True)
            fa.run_preprocess(h, do, o, delta, n)
            fa.run_bwd_flash(h, q, k, v, do, l, delta, dq, dk, dv, n, True)
            # int8 decode on this device too
            nh, nkv, ctx = 8, 2, 200
            c = la.KvCache(ctx, nkv, 64, True, device=f"cuda:{d}")
            c.k.random_(-128, 128), c.v.random_(-128, 128), c.ks.uniform_(0.01, 0.03), c.vs.uniform_(0.01, 0.03)
            qd = torch.randn(nh * 64, device=f"cuda:{d}")
            od = torch.zeros(nh * 64, device=f"cuda:{d}")
            la.attn_decode(h, od, qd, c, ctx - 1, nh, nkv, 64)
            h.check_status()
            outs.append((o.cpu().numpy(), dq.cpu().numpy(), dk.cpu().numpy(), dv.cpu().numpy(), od.cpu().numpy()))
    for o, dq, dk, dv, od in outs:
        assert np.abs(o - wo).max() < TOL["max_abs"] and np.isfinite(od).all()
    # both devices ran the same kernels on the same inputs: O, dK, dV are written once by their owner and
    # must agree bit for bit; dQ of the fused backward is a sum of fp32 reductions in no fixed order
    for i in (0, 2, 3):
        np.testing.assert_array_equal(outs[0][i], outs[1][i])
    assert np.abs(outs[0][1] - outs[1][1]).max() <= 1e-4


def _absent_peer_worker(rank, world, port, ret):
    """Failure detection without a GPU fault: after two good steps rank 1 stops taking part (a host-side decision,
    between steps, nothing of its own in flight).  Rank 0's next step stores its triples, waits for rank 1's with a
    short limit, and its kernel returns by itself with the status word set; the context stays usable and a fresh
    communicator works again."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import datetime
    import torch.distributed as dist
    from mx230_b200 import _lib, llm_attention as la
    from mx230_b200._lib import Mx230Error
    from mx230_b200.common import Handle
    from mx230_b200.multi_gpu import SplitKvDecoder, SplitKvPlan
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank),
                            timeout=datetime.timedelta(seconds=60))
    try:
        dev = f"cuda:{rank}"
        h = Handle(rank, 16 << 20)
        n_seq, nh, nkv, span = 2, 8, 2, 300
        plan = SplitKvPlan(ctx=span * world, world=world, n_seq=n_seq, n_head=nh, align=4)
        torch.manual_seed(7 + rank)
        c = la.KvCache(n_seq * span, nkv, 64, True, True, device=dev)
        c.k.random_(-128, 128), c.v.random_(-128, 128), c.ks.uniform_(0.01, 0.03), c.vs.uniform_(0.01, 0.03)
        q = torch.randn(n_seq, nh * 64, device=dev)
        dec = SplitKvDecoder(h, plan, rank, device=dev, fused=True)
        for _ in range(2):
            good = dec.step(q, c, nkv, span, nh * 64).clone()
        torch.cuda.synchronize()
        h.check_status()
        dist.barrier()
        status = None
        if rank == 0:   # rank 1 sits this step out
            h.set_option(_lib.OPT_WAIT_LIMIT, 4000)   # 4e6 cycles, about 2 ms
            dec.out.fill_(float("nan"))
            dec.step(q, c, nkv, span, nh * 64)
            try:
                h.check_status()
            except Mx230Error as e:
                status = e.code
            untouched = bool(torch.isnan(dec.out).all())
            h.set_option(_lib.OPT_WAIT_LIMIT, 4000000)
        dist.barrier()          # rank 1 learns on the host that the step is over
        dec.close()             # the step counts of the two ranks no longer agree: this communicator is done
        dec2 = SplitKvDecoder(h, plan, rank, device=dev, fused=True)
        again = dec2.step(q, c, nkv, span, nh * 64)
        torch.cuda.synchronize()
        h.check_status()
        same = bool(torch.equal(again, good))
        dec2.close()
        ret[rank] = (status, untouched if rank == 0 else None, same)
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_absent_peer_is_detected_by_the_bounded_wait_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    from mx230_b200 import _lib
    ctxm = mp.get_context("spawn")
    ret = ctxm.Manager().dict()
    port = _free_port()
    procs = [ctxm.Process(target=_absent_peer_worker, args=(r, 2, port, ret), daemon=True) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(240)
    codes = [p.exitcode for p in procs]
    for p in procs:
        if p.is_alive():
            p.terminate()
            p.join(10)
            if p.is_alive():
                p.kill()
    assert codes == [0, 0], f"rank exit codes {codes}"
    assert ret[0][0] == _lib.ERR_DEVICE_STATUS and ret[0][1] is True   # the wait ran out, nothing was written
    assert ret[0][2] and ret[1][2]                                      # a fresh communicator gives the same result as before
