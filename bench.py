#!/usr/bin/env python
"""Benchmark of the attention hot path: causal flash-attention forward + backward.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (one "step"): the causal forward + backward of B=4, H=12, N=4096, d=64 through
the fp32-in / fp32-out C-ABI entry points -- attn_flash_lse, attn_bwd_preprocess,
attn_bwd_flash -- on seeded synthetic N(0,1) tensors (the library's own generator).  Operands are
rounded to bf16 by the library's staging kernel inside the timed region; accumulation is fp32.
Algorithmic work per step: forward 2*B*H*N^2*d = 103.08 GFLOP, backward 2.5x = 257.70 GFLOP
(the two recomputed matmuls of the atomic-free split are not counted).

`value`   whole-job TFLOP/s with the inputs resident in HBM, CUDA-event timed, max over ranks.
`e2e`     the same metric with the inputs in pinned HOST memory: every step copies Q, K, V, dO
          host->device and O, L, dQ, dK, dV device->host inside the timed region.
`roofline` per-launch achieved TFLOP/s of the dominant kernel, from event pairs the library
          records around each launch during the timed steps, against the measured dense
          bf16 peak of this pool (read from the driver-written peaks file when present).
`cpu_baseline` the CPU restatement of the reference's attention (oracle/) on a bounded sample.
`decode`  HBM GB/s of the int8-KV GQA decode step (14q/2kv, ctx 2048, batch 64; 32q/4kv, ctx 131072,
          batch 8) and of the fp32-KV control, launches replayed from a CUDA graph over rotated caches.
`prefill` TFLOP/s of the per-layer prefill attention (staging + kernel), 512 new tokens.

With N > 1 GPUs (torchrun) every rank runs the same per-GPU workload on its own (batch, head)
units -- no data-path collective -- and the job value is N * units / max-over-ranks time
(weak scaling); `multi_gpu` then adds the partitioned configurations: the long-context decode with
its key axis split over the ranks (partial attention, one all-gather, log-sum-exp merge), the
32768-token forward with its heads over the ranks and the batch-64 decode with its sequences over
the ranks (strong scaling).  `--impl reference` times the CPU oracle with all host threads instead.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

B, H, N, D = 4, 12, 4096, 64
BH = B * H
FWD_FLOP = 2.0 * BH * N * N * D          # causal forward
BWD_FLOP = 2.5 * FWD_FLOP                # five matmuls of the same size
STEP_FLOP = FWD_FLOP + BWD_FLOP
# share of the backward's algorithmic work attributed to each pass: dQ owns 1 matmul, dK/dV own
# 2, and the two shared ones (S, dP) are split evenly
DQ_FLOP = BWD_FLOP * 2.0 / 5.0
DKV_FLOP = BWD_FLOP * 3.0 / 5.0
WORKLOAD = "causal flash-attention fwd+bwd, B=4 H=12 N=4096 d=64, fp32 in/out, bf16 operands"
# dram__bytes_read.sum + dram__bytes_write.sum per launch of the tensor kernels on this exact workload, from one
# ncu capture each (the operands, 4 x 25 MB bf16 + fp32 outputs, mostly stay in the 126 MB L2)
NCU_DRAM_BYTES_PER_LAUNCH = {"flash_fwd_kernel": 86331904 + 18123776, "bwd_fused_kernel": 328961536 + 207100928,
                             "bwd_dq_kernel": 106472960 + 25134592, "bwd_dkv_kernel": 108812800 + 60150016}
NOMINAL_BF16_TFLOPS = 2250.0
NOMINAL_HBM_GBS = 8000.0


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return {"bf16_tflops": p.get("bf16_tflops"), "bf16_tflops_sustained": p.get("bf16_tflops_sustained"),
                "hbm_gbs": p.get("hbm_gbs"), "source": "measured"}
    return {"bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "hbm_gbs": 6650.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while a region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        # `index` is the CUDA device ordinal of this process; nvidia-smi numbers the physical GPUs, which
        # differs under CUDA_VISIBLE_DEVICES, so the GPU is named by its UUID when torch can give it
        self.index, self.rows, self.proc = str(index), [], None
        try:
            import torch
            name = "GPU-" + str(torch.cuda.get_device_properties(index).uuid)
            if subprocess.run(["nvidia-smi", f"--id={name}", "--query-gpu=index", "--format=csv,noheader"],
                              capture_output=True, timeout=20).returncode == 0:
                self.index = name
        except Exception:
            pass

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.thread.join(timeout=2)
        mhz, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                mhz.append(float(r[0]))
                mx = float(r[1])
                for nm, v in zip(names, r[3:7]):
                    if v.lower().startswith("active"):
                        reasons.add(nm)
            except Exception:
                pass
        mhz.sort()
        # clocks under load: the upper half of the samples (idle samples pull the median down)
        load = mhz[len(mhz) // 2:] if mhz else []
        return {"sm_mhz": (load[len(load) // 2] if load else None), "sm_max_mhz": mx,
                "reasons": sorted(reasons), "samples": len(mhz)}


def host_threads() -> int:
    """Cores this process may run on.  Not omp_get_max_threads: torchrun exports OMP_NUM_THREADS=1 to its workers, which
    would turn the all-cores CPU arm into a single-threaded one; the oracle takes its thread count as an argument."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


# ----------------------------------------------------------------------------- CPU arm
def cpu_sample(heads: int, threads: int):
    """Forward + backward of `heads` heads of the workload on the CPU oracle; returns seconds."""
    import oracle
    q, k, v, do = (oracle.normal((heads, N, D), 1234, i) for i in range(4))
    t0 = time.perf_counter()
    oracle.attn_fwd(q, k, v, True, threads=threads)
    oracle.attn_bwd(q, k, v, do, True, threads=threads)
    return time.perf_counter() - t0


def run_reference(args):
    """The reference's CPU attention path (C restatement: the Rust sources cannot be built here) with all
    host threads.  A step is the whole workload -- all B*H heads, forward + backward -- as in the GPU arm."""
    rank, world, _ = dist_env()
    if rank != 0:
        return
    import oracle
    threads = host_threads()
    q, k, v, do = (oracle.normal((BH, N, D), 1234, i) for i in range(4))

    def step():
        t0 = time.perf_counter()
        oracle.attn_fwd(q, k, v, True, threads=threads)
        oracle.attn_bwd(q, k, v, do, True, threads=threads)
        return time.perf_counter() - t0

    if args.warmup > 0:
        cpu_sample(min(threads, 4), threads)   # one short untimed pass: page in the library, spin up the thread pool
    # every step is the full workload; on a box whose cores would need more than about four minutes for the
    # requested steps the run is cut to as many whole steps as fit (at least one) and `steps` reports that number
    times, budget = [], 240.0
    for _ in range(max(1, args.steps)):
        times.append(step())
        if sum(times) + times[-1] > budget:
            break
    sec = sum(times) / len(times)
    tflops = STEP_FLOP / sec / 1e12
    line = {
        "impl": "reference", "metric": "attn_fwd_bwd_tflops", "value": tflops, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": len(times), "warmup": args.warmup, "ms_per_step": sec * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": {"workload": WORKLOAD, "per_gpu_units": f"{BH} (batch, head) units"},
        "cpu_baseline": {"value": tflops, "unit": "TFLOP/s", "cores": threads, "kind": "port",
                         "sample": f"all {BH} heads, N={N}, forward+backward, {threads} OpenMP threads, {len(times)} steps"},
        "e2e": {"value": tflops, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------- GPU arm
def decode_bench(h, torch, la, n_seq=64, nh=14, nkv=2, ctx=2048, quants=(True, False), replays=5):
    """int8-KV GQA decode (and fp32 control): GB/s of algorithmic bytes.  A launch of a few microseconds cannot be
    timed by an event pair around it (that measures the host's submission gap), so a sequence of launches over
    rotated caches -- consecutive launches never touch L2-resident data -- is captured in a CUDA graph once and
    replayed; the figure is the graph's device time per launch."""
    out = {}
    qd, kvd = nh * 64, nkv * 64
    for quant in quants:
        per_seq = ctx * kvd * 2 * (1 if quant else 4) + (ctx * nkv * 16 if quant else 0) + qd * 8
        nbytes = n_seq * per_seq
        copies = max(2, int(4 * 126e6 / nbytes) + 1)
        caches = []
        for _ in range(copies):
            c = la.KvCache(n_seq * ctx, nkv, 64, quant)
            if quant:
                c.k.random_(-128, 128), c.v.random_(-128, 128)
                c.ks.uniform_(0.01, 0.03), c.vs.uniform_(0.01, 0.03), c.kb.normal_(), c.vb.normal_()
            else:
                c.k.normal_(), c.v.normal_()
            caches.append(c)
        q = torch.randn(n_seq, qd, device="cuda")
        o = torch.empty(n_seq, qd, device="cuda")
        pos = torch.full((n_seq,), ctx - 1, dtype=torch.int32, device="cuda")
        launches = [(lambda cc=cc: la.attn_decode_slab(h, o, q, cc, pos, n_seq, nh, nkv, 64, ctx, qd, qd))
                    for cc in (caches * 12)[:max(copies, 12)]]
        g_us = graph_time_us(torch, launches, replays)
        out["int8_kv" if quant else "fp32_kv"] = {
            "gbs": nbytes / g_us / 1e3, "us_per_launch": g_us, "bytes_per_launch": nbytes,
            "timing": f"CUDA graph of {len(launches)} launches over {copies} rotated caches, {replays} replays",
            "batch": n_seq, "ctx": ctx, "heads": f"{nh}q/{nkv}kv", "cache_copies_rotated": copies}
        del caches
    return out


def prefill_bench(h, torch, la, n_tok=512, nh=14, nkv=2, reps=10):
    """Per-layer prefill attention (Qwen2.5-0.5B layout): `n_tok` new rows at positions pos0.. over the cache,
    staging kernels + attention kernel, fp32 and int8 cache, at pos0 = 0 and 1536.  Algorithmic FLOPs: 4 * 64 per
    (query, visible key) pair and head."""
    out = {}
    qd, kvd = nh * 64, nkv * 64
    stride = qd + 2 * kvd
    for quant in (False, True):
        for pos0 in (0, 1536):
            n_keys = pos0 + n_tok
            h.reserve(la.prefill_workspace_bytes(n_tok, n_keys, nh, nkv))
            c = la.KvCache(n_keys, nkv, 64, quant)
            if quant:
                c.k.random_(-128, 128), c.v.random_(-128, 128)
                c.ks.uniform_(0.01, 0.03), c.vs.uniform_(0.01, 0.03), c.kb.normal_(), c.vb.normal_()
            else:
                c.k.normal_(), c.v.normal_()
            qkv = torch.randn(n_tok, stride, device="cuda")
            o = torch.empty(n_tok, qd, device="cuda")
            f = lambda: la.attn_prefill(h, o, qkv, c, pos0, n_tok, nh, nkv, stride, qd)
            us = graph_time_us(torch, [f] * 8)   # three launches of a few microseconds each: timed from a CUDA graph
            pairs = n_tok * pos0 + n_tok * (n_tok + 1) // 2
            out[f"{'int8' if quant else 'fp32'}_kv_pos0_{pos0}"] = {
                "us": us, "tflops": 4.0 * 64 * pairs * nh / us / 1e6, "n_tok": n_tok, "n_keys": n_keys,
                "heads": f"{nh}q/{nkv}kv", "launches_per_call": 3, "timing": "CUDA graph of 8 calls, 5 replays"}
    # the projections either side (gpu.rs:3187-3198, 3354-3365): qkv = x W + b and y = attn W + b for the same chunk
    e = 896
    x = torch.randn(n_tok, e, device="cuda")
    for name, dt in (("fp32_w", torch.float32), ("fp16_w", torch.float16)):
        w1 = (torch.randn(e, stride, device="cuda") / 30).to(dt)
        w2 = (torch.randn(qd, e, device="cuda") / 30).to(dt)
        b1, b2 = torch.randn(stride, device="cuda"), torch.randn(e, device="cuda")
        qkv = torch.empty(n_tok, stride, device="cuda")
        att = torch.randn(n_tok, qd, device="cuda")
        y = torch.empty(n_tok, e, device="cuda")
        la.gemm(h, qkv, x, w1, b1), la.gemm(h, y, att, w2, b2)   # workspace grown outside the capture
        u1 = graph_time_us(torch, [lambda: la.gemm(h, qkv, x, w1, b1)] * 8)
        u2 = graph_time_us(torch, [lambda: la.gemm(h, y, att, w2, b2)] * 8)
        out[f"proj_{name}"] = {"qkv_us": u1, "out_us": u2, "qkv_tflops": 2.0 * n_tok * e * stride / u1 / 1e6,
                               "out_tflops": 2.0 * n_tok * qd * e / u2 / 1e6, "shape": f"{n_tok} x {e} -> {stride} / {qd} -> {e}",
                               "launches_per_call": 2, "timing": "CUDA graph of 8 calls, 5 replays"}
    return out


def multi_gpu_bench(h, torch, dist, la, fa, rank, world, local, steps):
    """The partitioned configurations at N > 1 (strong scaling: the total problem is fixed), each timed on the
    device between a barrier and all-ranks-done, max over ranks:
      splitkv   32q/4kv, ctx 131072, 8 sequences, int8 cache: keys split over the ranks, one all-gather of the
                (m, l, acc) triples, log-sum-exp merge on every rank;
      fwd_32768 non-causal forward, 8 heads of 32768 tokens, heads over the ranks (no collective);
      decode_b64 14q/2kv, ctx 2048, batch 64, int8 cache: sequences over the ranks (no collective)."""
    from mx230_b200.multi_gpu import SplitKvDecoder, SplitKvPlan, shard_range
    out = {}

    def timed(fn, n, warm=3):
        for _ in range(warm):
            fn()
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(n):
            fn(i)
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / n], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t[0])

    # ---- split-KV decode
    nh, nkv, ctx, n_seq = 32, 4, 131072, 8
    plan = SplitKvPlan(ctx=ctx, world=world, n_seq=n_seq, n_head=nh)
    t0, t1 = plan.key_range(rank)
    span = max(1, t1 - t0)
    caches = []
    for _ in range(2):   # two copies of this rank's share: together larger than L2
        c = la.KvCache(n_seq * span, nkv, 64, True)
        c.k.random_(-128, 128), c.v.random_(-128, 128), c.ks.uniform_(0.01, 0.03), c.vs.uniform_(0.01, 0.03)
        caches.append(c)
    q = torch.randn(n_seq, nh * 64, device="cuda")
    dec = SplitKvDecoder(h, plan, rank, device=f"cuda:{local}")
    ms = timed(lambda i=0: dec.step(q, caches[i % 2], nkv, span, nh * 64), max(steps, 10))
    total = n_seq * ctx * nkv * (128 + 16)
    out["splitkv"] = {"ms_per_step": ms, "aggregate_gbs": total / ms / 1e6, "kv_bytes_total": total,
                      "exchange_bytes_per_rank": plan.bytes_per_rank(), "scaling": "strong",
                      "workload": "int8-KV GQA decode 32q/4kv ctx 131072 x 8 sequences, keys split over ranks, "
                                  "ncclAllGather of the partial triples, merge on every rank"}
    # the same step with the exchange and the merge in one kernel over peer memory (no collective call per step),
    # host-launched like the line above and replayed from a CUDA graph of 16 steps (the reference captures its
    # decode step in a graph, 03-llm-engine/src/gpu.rs:4024-4054; the exchange's step numbers live in device memory)
    fdec = SplitKvDecoder(h, plan, rank, device=f"cuda:{local}", fused=True)
    try:
        ms_f = timed(lambda i=0: fdec.step(q, caches[i % 2], nkv, span, nh * 64), max(steps, 10))
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            for i in range(16):
                fdec.step(q, caches[i % 2], nkv, span, nh * 64)
        ms_g = timed(lambda i=0: g.replay(), 8) / 16
        h.check_status()
    finally:
        fdec.close()
    out["splitkv_fused"] = {"ms_per_step": ms_f, "aggregate_gbs": total / ms_f / 1e6, "scaling": "strong",
                            "ms_per_step_graph": ms_g, "aggregate_gbs_graph": total / ms_g / 1e6,
                            "workload": "the same step as ONE kernel per rank: the CTA that finishes a (sequence, KV head) "
                                        "group stores its triples into every other rank's exchange region over NVLink "
                                        "({value, step} words, plain peer stores), waits (bounded) for theirs and merges; "
                                        "no collective call per step"}
    del caches, dec, fdec
    # ---- 32768-token forward, heads over ranks
    n, heads = 32768, 8
    lo, hi = shard_range(heads, rank, world)
    mine = max(1, hi - lo)
    h.reserve(fa.workspace_bytes(mine, n, False))
    qq, kk, vv = (torch.randn(mine, n, 64, device="cuda") for _ in range(3))
    oo, ll = torch.empty_like(qq), torch.empty(mine, n, device="cuda")
    ms = timed(lambda i=0: fa.run_flash_lse(h, qq, kk, vv, oo, ll, n, False), 3, warm=2)
    out["fwd_32768"] = {"ms_per_step": ms, "aggregate_tflops": 4.0 * heads * n * n * 64 / ms / 1e9,
                        "heads_per_rank": hi - lo, "scaling": "strong",
                        "workload": "non-causal forward B=1 H=8 N=32768 d=64 (cast + kernel), heads over ranks"}
    del qq, kk, vv, oo
    # ---- batch-64 decode, sequences over ranks
    nh, nkv, ctx, batch = 14, 2, 2048, 64
    lo, hi = shard_range(batch, rank, world)
    mine = max(1, hi - lo)
    d = decode_bench(h, torch, la, n_seq=mine, nh=nh, nkv=nkv, ctx=ctx, quants=(True,))["int8_kv"]
    t = torch.tensor([d["us_per_launch"]], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    tot = batch * (ctx * nkv * 64 * 2 + ctx * nkv * 16 + nh * 64 * 8)
    out["decode_b64"] = {"us_per_step": float(t[0]), "aggregate_gbs": tot / float(t[0]) / 1e3, "seqs_per_rank": hi - lo,
                         "scaling": "strong", "workload": "int8-KV GQA decode 14q/2kv ctx 2048 batch 64, sequences over ranks"}
    return out


def run_ours(args):
    import torch
    import torch.distributed as dist
    from mx230_b200 import flash_attention as fa
    from mx230_b200 import llm_attention as la
    from mx230_b200.common import Handle

    rank, world, local = dist_env()
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the CUDA library is the only implementation")
    torch.cuda.set_device(local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    from mx230_b200 import _lib
    from mx230_b200.common import normal
    h = Handle(local, fa.workspace_bytes(BH, N, True))
    # the training step keeps Q, K, V unchanged between its forward and backward: the backward then reuses the bf16
    # copies the forward staged (an option of the library, documented in its header) and stages only dO
    h.set_option(_lib.OPT_BWD_REUSE_STAGED, 1)
    # seeded N(0,1) inputs from the library's generator (seed 1000 + rank, tensor index 0..3), uploaded once
    q, k, v, do = (torch.from_numpy(normal((B, H, N, D), 1000 + rank, i)).cuda() for i in range(4))
    o = torch.empty_like(q)
    lse = torch.empty(B, H, N, device="cuda")
    delta = torch.empty_like(lse)
    dq, dk, dv = torch.empty_like(q), torch.empty_like(q), torch.empty_like(q)
    stream = torch.cuda.current_stream()

    def step():
        fa.run_flash_lse(h, q, k, v, o, lse, N, True)
        fa.run_preprocess(h, do, o, delta, N)
        fa.run_bwd_flash(h, q, k, v, do, lse, delta, dq, dk, dv, N, True)

    for _ in range(max(args.warmup, 3)):
        step()
    h.check_status()
    barrier()

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    l0 = h.launches
    h.profile_reset()
    h.profile_enable(True)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(args.steps):
        step()
    e1.record(stream)
    barrier()
    ms = e0.elapsed_time(e1)
    h.profile_enable(False)
    launches = h.launches - l0
    prof = h.profile_read()
    h.check_status()

    # the reference's atomic-free split (a dQ pass and a dK/dV pass, bit-reproducible) on the same step
    h.set_option(_lib.OPT_BWD_TWO_PASS, 1)
    for _ in range(2):
        step()
    torch.cuda.synchronize()
    h.profile_reset()
    h.profile_enable(True)
    for _ in range(5):
        step()
    h.profile_enable(False)
    prof2 = h.profile_read()
    h.set_option(_lib.OPT_BWD_TWO_PASS, 0)
    h.check_status()

    # ---- end to end: pinned host tensors in, results out, every step ----
    hq, hk, hv, hdo = (t.cpu().pin_memory() for t in (q, k, v, do))
    ho, hl, hdq, hdk, hdv = (torch.empty(t.shape, dtype=t.dtype).pin_memory() for t in (o, lse, dq, dk, dv))

    # Software pipeline over three streams and two sets of device buffers: the host->device copy of
    # step i+1 and the device->host copy of step i-1 run under the kernels of step i (PCIe is full
    # duplex).  Every step still moves all of its inputs in and all of its results out inside the
    # timed region.
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    dev_in = [(q, k, v, do), tuple(torch.empty_like(t) for t in (q, k, v, do))]
    dev_out = [(o, lse, dq, dk, dv), tuple(torch.empty_like(t) for t in (o, lse, dq, dk, dv))]
    delta2 = [delta, torch.empty_like(delta)]
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_c = [torch.cuda.Event() for _ in range(2)]
    ev_out = [torch.cuda.Event() for _ in range(2)]

    def e2e_run(n_steps):
        for i in range(n_steps):
            b = i & 1
            qi, ki, vi, doi = dev_in[b]
            oi, li, dqi, dki, dvi = dev_out[b]
            with torch.cuda.stream(s_in):
                if i >= 2:
                    s_in.wait_event(ev_c[b])      # the kernels of step i-2 have read these inputs
                for dst, src in ((qi, hq), (ki, hk), (vi, hv), (doi, hdo)):
                    dst.copy_(src, non_blocking=True)
                ev_in[b].record(s_in)
            stream.wait_event(ev_in[b])
            if i >= 2:
                stream.wait_event(ev_out[b])      # the results of step i-2 have left these outputs
            fa.run_flash_lse(h, qi, ki, vi, oi, li, N, True)
            fa.run_preprocess(h, doi, oi, delta2[b], N)
            fa.run_bwd_flash(h, qi, ki, vi, doi, li, delta2[b], dqi, dki, dvi, N, True)
            ev_c[b].record(stream)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_c[b])
                for dst, src in ((ho, oi), (hl, li), (hdq, dqi), (hdk, dki), (hdv, dvi)):
                    dst.copy_(src, non_blocking=True)
                ev_out[b].record(s_out)
        stream.wait_event(ev_out[0])
        stream.wait_event(ev_out[1])

    e2e_steps = max(4, min(args.steps, 10))
    e2e_run(2)
    barrier()
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record(stream)
    s_in.wait_event(f0)
    e2e_run(e2e_steps)
    f1.record(stream)
    barrier()
    e2e_ms = f0.elapsed_time(f1)
    h.check_status()
    clocks = sampler.stop() if rank == 0 else None
    h2d = sum(t.numel() * 4 for t in (hq, hk, hv, hdo))
    d2h = sum(t.numel() * 4 for t in (ho, hl, hdq, hdk, hdv))

    if world > 1:
        t = torch.tensor([ms, e2e_ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_ms = float(t[0]), float(t[1])

    multi = multi_gpu_bench(h, torch, dist, la, fa, rank, world, local, args.steps) if world > 1 else None
    dec = decode_bench(h, torch, la) if rank == 0 else None
    pre = prefill_bench(h, torch, la) if rank == 0 else None
    if dec is not None:  # the long-context configuration: 32q/4kv, ctx 131072, 8 sequences, int8 cache (604 MB per launch)
        dec["int8_kv_long"] = decode_bench(h, torch, la, n_seq=8, nh=32, nkv=4, ctx=131072, quants=(True,))["int8_kv"]
    if rank == 0:
        peaks = measured_peaks()
        ms_step = ms / args.steps
        value = world * STEP_FLOP / (ms_step * 1e-3) / 1e12
        e2e_val = world * STEP_FLOP / (e2e_ms / e2e_steps * 1e-3) / 1e12
        kern = {}
        for name, flop in (("flash_fwd_kernel", FWD_FLOP), ("bwd_fused_kernel", BWD_FLOP), ("bwd_dq_kernel", DQ_FLOP),
                           ("bwd_dkv_kernel", DKV_FLOP)):
            if name in prof:
                cnt, tot = prof[name]
                kern[name] = {"launches": cnt, "ms_per_launch": tot / cnt,
                              "achieved_tflops": flop / (tot / cnt * 1e-3) / 1e12, "flop_per_launch": flop}
        for name in ("cast_bf16_kernel", "bwd_preprocess_kernel"):
            if name in prof:
                cnt, tot = prof[name]
                kern[name] = {"launches": cnt, "ms_per_launch": tot / cnt}
        # dominant kernel = the one with the largest share of device time
        dom = max((n for n in kern if "achieved_tflops" in kern[n]), key=lambda n: kern[n]["ms_per_launch"] * kern[n]["launches"])
        peak = peaks["bf16_tflops"]
        roofline = {"bound": "tensor", "kernel": dom, "achieved": kern[dom]["achieved_tflops"], "peak": peak,
                    "unit": "TFLOP/s", "frac": kern[dom]["achieved_tflops"] / peak,
                    "traffic": NCU_DRAM_BYTES_PER_LAUNCH.get(dom), "traffic_unit": "bytes per launch (dram read + write)",
                    "traffic_source": "one ncu --set full capture of this kernel on this workload (not re-measured by this run)",
                    "peak_source": f"{peaks['source']} dense bf16 burst",
                    "frac_of_nominal": kern[dom]["achieved_tflops"] / NOMINAL_BF16_TFLOPS,
                    "per_kernel": kern}
        import oracle
        cores = host_threads()
        heads = max(1, min(cores, BH))   # one head per thread: every core busy
        sec = cpu_sample(heads, cores)
        sec1 = cpu_sample(1, 1)   # what the reference itself does: one head on one thread
        cpu = {"value": STEP_FLOP * heads / BH / sec / 1e12, "unit": "TFLOP/s", "cores": cores, "kind": "port",
               "sample": f"{heads} of {BH} heads, N={N}, forward+backward, {cores} OpenMP threads, {sec:.1f} s",
               "single_thread": {"value": STEP_FLOP / BH / sec1 / 1e12, "unit": "TFLOP/s", "cores": 1,
                                 "sample": f"1 of {BH} heads, N={N}, forward+backward, {sec1:.1f} s"}}
        if dec:
            for kk in dec:
                dec[kk]["frac_of_measured_hbm"] = dec[kk]["gbs"] / peaks["hbm_gbs"]
        line = {
            "metric": "attn_fwd_bwd_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": WORKLOAD, "per_gpu_units": f"{BH} (batch, head) units",
                       "l2": "inputs larger than L2 (4 x 50 MB fp32 operands per step)",
                       "entry_points": "mx230_attn_flash_lse + mx230_attn_bwd_preprocess + mx230_attn_bwd_flash",
                       "options": "MX230_OPT_BWD_REUSE_STAGED = 1 (the backward reuses the forward's staged Q, K, V and the dO copy the Delta pre-pass leaves)",
                       "inputs": "N(0,1), library generator, seed 1000 + rank"},
            "fwd_tflops": world * FWD_FLOP / (kern["flash_fwd_kernel"]["ms_per_launch"] * 1e-3) / 1e12,
            "bwd_tflops": world * BWD_FLOP / (sum(kern[k]["ms_per_launch"] for k in kern if k.startswith("bwd_") and
                                                  "achieved_tflops" in kern[k]) * 1e-3) / 1e12,
            "bwd_two_pass_tflops": world * BWD_FLOP / (sum(prof2[k][1] / prof2[k][0] for k in ("bwd_dq_kernel", "bwd_dkv_kernel")
                                                            if k in prof2) * 1e-3) / 1e12 if "bwd_dq_kernel" in prof2 else None,
            "roofline": roofline, "cpu_baseline": cpu,
            "e2e": {"value": e2e_val, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": e2e_ms / e2e_steps, "steps": e2e_steps,
                    "pipeline": "3 streams, 2 buffer sets: the copies of steps i+1 / i-1 overlap the kernels of step i"},
            "gpu_launches": launches, "clocks": clocks, "decode": dec, "prefill": pre, "multi_gpu": multi,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    h.close()


def run_case(args):
    """One kernel family on a fixed shape, a few launches and nothing else: the command that the
    ncu captures wrap (`--case fwd|bwd|bwd_two_pass|decode_c4|decode_long`)."""
    import torch
    from mx230_b200 import flash_attention as fa
    from mx230_b200 import llm_attention as la
    from mx230_b200.common import Handle
    torch.cuda.set_device(0)
    h = Handle(0, 1 << 30)
    reps = max(1, args.steps)
    if args.case in ("fwd", "bwd", "bwd_two_pass"):
        from mx230_b200 import _lib
        h.set_option(_lib.OPT_BWD_TWO_PASS, 1 if args.case == "bwd_two_pass" else 0)
        q, k, v, do = (torch.randn(BH, N, D, device="cuda") for _ in range(4))
        o = torch.empty_like(q)
        l = torch.empty(BH, N, device="cuda")
        delta = torch.empty_like(l)
        dq, dk, dv = (torch.empty_like(q) for _ in range(3))
        for _ in range(reps):
            fa.run_flash_lse(h, q, k, v, o, l, N, True)
            if args.case != "fwd":
                fa.run_preprocess(h, do, o, delta, N)
                fa.run_bwd_flash(h, q, k, v, do, l, delta, dq, dk, dv, N, True)
    else:
        nh, nkv, ctx, n_seq = (14, 2, 2048, 64) if args.case == "decode_c4" else (32, 4, 32768, 8)
        caches = []
        for _ in range(3):
            c = la.KvCache(n_seq * ctx, nkv, 64, True)
            c.k.random_(-128, 128), c.v.random_(-128, 128), c.ks.uniform_(0.01, 0.03), c.vs.uniform_(0.01, 0.03)
            caches.append(c)
        qd = nh * 64
        q = torch.randn(n_seq, qd, device="cuda")
        out = torch.empty(n_seq, qd, device="cuda")
        pos = torch.full((n_seq,), ctx - 1, dtype=torch.int32, device="cuda")
        for i in range(reps):
            la.attn_decode_slab(h, out, q, caches[i % 3], pos, n_seq, nh, nkv, 64, ctx, qd, qd)
    h.check_status()
    print(json.dumps({"case": args.case, "launches": h.launches}))
    h.close()


def run_splitkv(args):
    """Long-context int8-KV decode (32q/4kv, ctx 131072, 8 sequences) with the key axis split over the ranks
    (strong scaling: the total context is fixed), in every form the library has, each host-launched back to
    back and replayed from a CUDA graph of 16 steps, device time, max over ranks:
      nccl      partial attention, all-gather of the (m, l, acc) triples, merge kernel
      exchange  partial attention, then one kernel that stores the triples to every rank, waits and merges
      push      the attention kernel stores the triples itself; a second kernel waits and merges
      one       the whole step in one kernel
    and the pieces of the first two on their own (partial kernel, all-gather, merge, exchange kernel).
    Run under torchrun for N > 1; prints one JSON line on rank 0."""
    import torch
    import torch.distributed as dist
    from mx230_b200 import llm_attention as la
    from mx230_b200.common import Handle
    from mx230_b200.multi_gpu import SplitKvDecoder, SplitKvPlan, gather_partials
    rank, world, local = dist_env()
    torch.cuda.set_device(local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29533")
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", local))
    nh, nkv, ctx, n_seq = 32, 4, 131072, 8
    h = Handle(local, 64 << 20)
    plan = SplitKvPlan(ctx=ctx, world=world, n_seq=n_seq, n_head=nh)
    t0, t1 = plan.key_range(rank)
    span = t1 - t0
    caches = []
    for _ in range(2):  # two copies of this rank's share (604 MB / world each): larger than L2 together
        c = la.KvCache(n_seq * span, nkv, 64, True)
        c.k.random_(-128, 128), c.v.random_(-128, 128), c.ks.uniform_(0.01, 0.03), c.vs.uniform_(0.01, 0.03)
        caches.append(c)
    q = torch.randn(n_seq, nh * 64, device="cuda")
    decs = {"nccl": SplitKvDecoder(h, plan, rank)}
    for how in ("exchange", "push", "one"):
        decs[how] = SplitKvDecoder(h, plan, rank, fused=how)
    d0 = decs["nccl"]
    fns = {k: (lambda i, d=d: d.step(q, caches[i % 2], nkv, span, nh * 64)) for k, d in decs.items()}
    fns["piece_partial"] = lambda i: la.attn_decode_partial(h, d0.m, d0.l, d0.acc, q, caches[i % 2], 0, span, n_seq, nh,
                                                            nkv, 64, span, nh * 64)
    fns["piece_all_gather"] = lambda i: gather_partials(plan, d0.local, d0.gathered, None)
    fns["piece_merge"] = lambda i: la.merge_partials_packed(h, d0.out, d0.gathered, world, plan.rows, 64)
    fns["piece_exchange_merge"] = lambda i: decs["exchange"].peer.exchange_merge(decs["exchange"].out, d0.local)
    reps = max(10, args.steps)

    def max_over_ranks(us):
        t = torch.tensor([us], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return round(float(t[0]), 2)

    def timed(run, n):
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(n):
            run(i)
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1e3

    host, graph = {}, {}
    for name, fn in fns.items():
        for i in range(max(3, args.warmup)):
            fn(i)
        host[name] = max_over_ranks(timed(fn, reps) / reps)
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            for i in range(16):
                fn(i)
        for _ in range(3):
            g.replay()
        graph[name] = max_over_ranks(timed(lambda i: g.replay(), 10) / 160)
    h.check_status()
    total_bytes = n_seq * ctx * nkv * (128 + 16)
    if rank == 0:
        print(json.dumps({"case": "splitkv", "n_gpus": world, "us_per_step_host_launched": host, "us_per_step_graph": graph,
                          "kv_bytes_total": total_bytes, "aggregate_gbs_one_kernel_graph": total_bytes / graph["one"] / 1e3,
                          "aggregate_gbs_nccl_graph": total_bytes / graph["nccl"] / 1e3, "scaling": "strong",
                          "exchange_bytes_per_rank": plan.bytes_per_rank(),
                          "config": {"workload": "int8-KV GQA decode 32q/4kv ctx 131072 x 8 sequences, keys split over ranks"}}))
    for d in decs.values():
        d.close()
    dist.barrier()
    dist.destroy_process_group()
    h.close()


def graph_time_us(torch, launches, replays=5):
    """Device time per launch of a list of enqueue-only callables, replayed from a CUDA graph: for
    kernels of a few microseconds the host cannot submit launches fast enough for an event pair around
    each one to measure anything but the submission gap."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())   # the caller's tensors (positions, caches) were filled on its stream
    with torch.cuda.stream(side):
        for f in launches:
            f()
    side.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=side):
        for f in launches:
            f()
    g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(replays):
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / (replays * len(launches))


def run_configs(args):
    """Every benchmark configuration on one GPU, kernel time from the library's own event pairs
    (median-free mean over `--steps` launches after warm-up): C1 and C3 forward through the fp32 entry
    point (cast + kernel), C4 decode at batch 1 / 16 / 64 (int8 affine cache and fp32 control), C5 decode.
    One JSON line per configuration."""
    import torch
    from mx230_b200 import flash_attention as fa
    from mx230_b200 import llm_attention as la
    from mx230_b200.common import Handle
    torch.cuda.set_device(0)
    h = Handle(0, 1 << 30)
    peaks = measured_peaks()
    reps = max(5, args.steps)

    def fwd_config(name, bh, n, causal):
        q, k, v = (torch.randn(bh, n, D, device="cuda") for _ in range(3))
        o = torch.empty_like(q)
        l = torch.empty(bh, n, device="cuda")
        for _ in range(3):
            fa.run_flash_lse(h, q, k, v, o, l, n, causal)
        torch.cuda.synchronize()
        h.profile_reset()
        h.profile_enable(True)
        for _ in range(reps):
            fa.run_flash_lse(h, q, k, v, o, l, n, causal)
        h.profile_enable(False)
        prof = h.profile_read()
        flop = (2 if causal else 4) * bh * n * n * D
        kms = prof["flash_fwd_kernel"][1] / prof["flash_fwd_kernel"][0]
        cms = prof["cast_bf16_kernel"][1] / prof["cast_bf16_kernel"][0]
        print(json.dumps({"config": name, "shape": f"BH={bh} N={n} d=64 causal={causal}", "flop": flop,
                          "kernel_ms": kms, "kernel_tflops": flop / kms / 1e9, "with_cast_tflops": flop / (kms + cms) / 1e9,
                          "frac_of_measured_bf16": flop / kms / 1e9 / peaks["bf16_tflops"]}), flush=True)
        del q, k, v, o

    fwd_config("C1", 12, 1024, True)
    fwd_config("C2-forward", 48, 4096, True)
    fwd_config("C3", 8, 32768, False)
    for b in (1, 16, 64):
        d = decode_bench(h, torch, la, n_seq=b)
        for kname, v in d.items():
            v["frac_of_measured_hbm"] = v["gbs"] / peaks["hbm_gbs"]
            print(json.dumps({"config": f"C4 batch {b} {kname}", **v}), flush=True)
    d = decode_bench(h, torch, la, n_seq=8, nh=32, nkv=4, ctx=131072, quants=(True,))["int8_kv"]
    d["frac_of_measured_hbm"] = d["gbs"] / peaks["hbm_gbs"]
    print(json.dumps({"config": "C5 one GPU int8_kv", **d}), flush=True)
    h.check_status()
    h.close()


def run_proj(args):
    """The projections either side of attention for one decode token (Qwen2-0.5B-like 896 -> 1152 and
    TinyLlama-like 2048 -> 2560, fp16 and fp32 weights): GB/s of weight bytes per launch, and the decode
    step with the fused qkv launch against the reference's sequence of gemv + rope + KV write."""
    import torch
    from mx230_b200 import llm_attention as la
    from mx230_b200.common import Handle
    torch.cuda.set_device(0)
    h = Handle(0, 64 << 20)
    peaks = measured_peaks()
    reps = max(20, args.steps)

    def timed(fn, name):
        for _ in range(5):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1e3 / reps   # us per call, launches back to back

    for model, n_in, nh, nkv in (("qwen2-0.5b-like", 896, 14, 2), ("tinyllama-like", 2048, 32, 4)):
        n_out = (nh + 2 * nkv) * 64
        for dt in (torch.float16, torch.float32):
            # a ring of weight copies larger than L2, as successive layers of a model would be
            copies = max(2, int(2 * 126e6 / (n_in * n_out * dt.itemsize)) + 1)
            ws = [(torch.randn(n_in, n_out, device="cuda") * 0.05).to(dt) for _ in range(copies)]
            b = torch.randn(n_out, device="cuda")
            x = torch.randn(n_in, device="cuda")
            qkv = torch.empty(n_out, device="cuda")
            c = la.KvCache(256, nkv, 64, True)
            st = {"i": 0}

            def w():
                st["i"] += 1
                return ws[st["i"] % copies]
            t_gemv = timed(lambda: la.gemv(h, qkv, x, w(), b), "gemv")
            t_fused = timed(lambda: la.qkv_rope_kvwrite(h, qkv, x, w(), b, 100, c, nh, nkv, 1e6), "fused")
            # the kernels alone: the library's event pair around each launch
            h.profile_reset()
            h.profile_enable(True)
            for _ in range(reps):
                la.gemv(h, qkv, x, w(), b)
            h.profile_enable(False)
            cnt, ms = h.profile_read()["gemv_heads_kernel"]
            k_gemv = 1e3 * ms / cnt
            h.profile_reset()
            h.profile_enable(True)
            for _ in range(reps):
                la.qkv_rope_kvwrite(h, qkv, x, w(), b, 100, c, nh, nkv, 1e6)
            h.profile_enable(False)
            cnt, ms = h.profile_read()["gemv_heads_kernel"]
            k_fused = 1e3 * ms / cnt

            def separate():
                la.gemv(h, qkv, x, w(), b)
                la.rope(h, qkv, 100, nh, nkv, 64, 1e6)
                la.quantize_kv(h, c, qkv, 100, nh * 64, nkv, 64)
            t_sep = timed(separate, "separate")
            g_gemv = graph_time_us(torch, [(lambda ww=ww: la.gemv(h, qkv, x, ww, b)) for ww in (ws * 12)[:max(copies, 12)]])
            g_fused = graph_time_us(torch, [(lambda ww=ww: la.qkv_rope_kvwrite(h, qkv, x, ww, b, 100, c, nh, nkv, 1e6))
                                            for ww in (ws * 12)[:max(copies, 12)]])

            def sep3(ww):
                la.gemv(h, qkv, x, ww, b)
                la.rope(h, qkv, 100, nh, nkv, 64, 1e6)
                la.quantize_kv(h, c, qkv, 100, nh * 64, nkv, 64)
            g_sep = graph_time_us(torch, [(lambda ww=ww: sep3(ww)) for ww in (ws * 12)[:max(copies, 12)]])
            wbytes = n_in * n_out * dt.itemsize
            print(json.dumps({"case": "proj", "model": model, "weights": str(dt).split(".")[-1], "n_in": n_in, "n_out": n_out,
                              "weight_bytes": wbytes, "graph_us": {"gemv": g_gemv, "fused_qkv_rope_kvwrite": g_fused,
                                                                       "gemv+rope+quantize_kv (3 launches)": g_sep},
                              "gemv_gbs": wbytes / g_gemv / 1e3, "gemv_frac_of_measured_hbm": wbytes / g_gemv / 1e3 / peaks["hbm_gbs"],
                              "fused_gbs": wbytes / g_fused / 1e3,
                              "event_pair_us": {"gemv": k_gemv, "fused_qkv_rope_kvwrite": k_fused},
                              "host_call_us": {"gemv": t_gemv, "fused_qkv_rope_kvwrite": t_fused,
                                               "gemv+rope+quantize_kv (3 launches)": t_sep},
                              "weight_copies_rotated": copies}), flush=True)
            del ws
    h.check_status()
    h.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--case", default=None, choices=["fwd", "bwd", "bwd_two_pass", "decode_c4", "decode_long", "splitkv", "configs", "proj"],
                    help="fwd|bwd|decode_*: profiling aid, runs one kernel family a few times and exits; "
                         "splitkv: long-context decode with keys split over the ranks (torchrun for N > 1); "
                         "configs: every benchmark configuration on one GPU; "
                         "proj: the projections either side of attention for one decode token")
    args = ap.parse_args()
    if args.case == "splitkv":
        run_splitkv(args)
    elif args.case == "configs":
        run_configs(args)
    elif args.case == "proj":
        run_proj(args)
    elif args.case:
        run_case(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
