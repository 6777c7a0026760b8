"""Host-side multi-GPU logic on CPU: sharding arithmetic, the split-KV plan, and the
all-gather layout over a world-size-2 gloo group (no GPU).  The compute of each rank is
played by the oracle, so the test exercises exactly the plumbing the GPU path uses."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from mx230_b200.multi_gpu import SplitKvPlan, gather_partials, shard_range


def test_shard_range_covers_all_units():
    for n in (0, 1, 6, 8, 48, 49, 64):
        for world in (1, 2, 4, 8):
            got = [shard_range(n, r, world) for r in range(world)]
            assert got[0][0] == 0 and got[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(got, got[1:]))
            sizes = [hi - lo for lo, hi in got]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_range(8, 2, 2)


def test_split_kv_plan_ranges():
    p = SplitKvPlan(ctx=131072, world=8, n_seq=8, n_head=32)
    r = [p.key_range(i) for i in range(8)]
    assert r[0] == (0, 16384) and r[-1] == (114688, 131072)
    assert p.bytes_per_rank() == 67584  # 256 rows x 66 floats
    p = SplitKvPlan(ctx=1000, world=4, n_seq=1, n_head=2)
    r = [p.key_range(i) for i in range(4)]
    assert r == [(0, 256), (256, 512), (512, 768), (768, 1000)]
    p = SplitKvPlan(ctx=130, world=4, n_seq=1, n_head=2)
    assert [p.key_range(i) for i in range(4)] == [(0, 128), (128, 130), (130, 130), (130, 130)]


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, ctx, results):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        nh, nkv, n_seq = 8, 2, 3
        plan = SplitKvPlan(ctx=ctx, world=world, n_seq=n_seq, n_head=nh)
        # every rank builds the same full problem from the seed and attends only its range
        qs = oracle.normal((n_seq, nh * 64), 70, 0)
        caches = []
        for s in range(n_seq):
            kv = oracle.normal((ctx, 2 * nkv * 64), 71 + s, 0)
            c = oracle.Q8Cache(ctx, nkv)
            for t in range(ctx):
                oracle.quantize_kv_row(c, kv[t], t, 0)
            caches.append(c)
        t0, t1 = plan.key_range(rank)
        local = torch.zeros(plan.floats_per_rank)
        m = local[:plan.rows].view(n_seq, nh)
        l = local[plan.rows:2 * plan.rows].view(n_seq, nh)
        acc = local[2 * plan.rows:].view(n_seq, nh, 64)
        for s in range(n_seq):
            if t1 > t0:
                pm, pl, pa = oracle.gqa_partial(qs[s], t0, t1, nh, nkv, 64, cache=caches[s])
            else:
                pm, pl, pa = np.full(nh, -np.inf, np.float32), np.zeros(nh, np.float32), np.zeros((nh, 64), np.float32)
            m[s], l[s], acc[s] = torch.from_numpy(pm), torch.from_numpy(pl), torch.from_numpy(pa)
        gathered = torch.zeros(world, plan.floats_per_rank)
        gather_partials(plan, local, gathered)
        gm, gl, ga = plan.unpack(gathered)
        merged = oracle.merge_partials(gm.numpy(), gl.numpy(), ga.numpy())
        want = np.stack([oracle.gqa_decode_q8(qs[s], caches[s], ctx - 1, nh, 0) for s in range(n_seq)])
        err = float(np.abs(merged.reshape(n_seq, -1) - want).max())
        results[rank] = err
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("ctx", [300, 130])
def test_split_kv_over_gloo_world2(ctx):
    world = 2
    with mp.Manager() as mgr:
        results = mgr.dict()
        mp.spawn(_worker, args=(world, _free_port(), ctx, results), nprocs=world, join=True)
        assert len(results) == world
        for r in range(world):
            assert results[r] < 5e-6, dict(results)


def test_split_kv_decoder_rejects_bad_fused_arguments_before_touching_the_device():
    """An odd row count or an unknown mode is refused by the constructor itself, before any library call."""
    from mx230_b200.multi_gpu import SplitKvDecoder, SplitKvPlan
    with pytest.raises(ValueError):
        SplitKvDecoder(None, SplitKvPlan(ctx=256, world=2, n_seq=1, n_head=7), 0, device="cpu", fused=True)
    with pytest.raises(ValueError):
        SplitKvDecoder(None, SplitKvPlan(ctx=256, world=2, n_seq=1, n_head=8), 0, device="cpu", fused="both")
