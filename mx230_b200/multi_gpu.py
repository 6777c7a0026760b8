"""Multi-GPU plumbing for the attention path: one process per GPU, torch.distributed
(NCCL over NVLink/NVSwitch on GPUs, gloo in the CPU tests) for the only exchange step.

The reference is single-device (`CudaContext::new(0)`, 02-flash-attention/src/main.rs:514;
03-llm-engine/src/main.rs:401), so everything here is new:

* (batch, head) sharding for flash-attention forward/backward and (sequence) sharding for
  batched decode: the units are independent, every rank works on its own slice and no
  data-path collective exists (`shard_range`);
* split-KV decode for very long contexts: rank r attends keys [t0_r, t1_r) of every sequence
  and produces the unnormalised triple (m, l, acc) per (sequence, query head); one all-gather
  of the triples (66 floats per row and rank) and a log-sum-exp merge on every rank give the
  full-context output (`SplitKvPlan`, `gather_partials`, `SplitKvDecoder`).  With `fused=True`
  the all-gather and the merge are ONE kernel over peer memory (`PeerExchange`): every rank stores
  its triples into every rank's exchange region over NVLink, publishes a step number, waits for
  the others' and merges; the collective library is used only once, to pass the 64-byte IPC
  handles of the regions at set-up.
"""
from __future__ import annotations

from dataclasses import dataclass


def shard_range(n_units: int, rank: int, world: int) -> tuple[int, int]:
    """Contiguous slice [lo, hi) of `n_units` independent units owned by `rank`; the first
    n_units % world ranks get one extra unit."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError(f"bad rank/world {rank}/{world}")
    base, extra = divmod(n_units, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


@dataclass
class SplitKvPlan:
    """Key ranges and buffer layout of a split-KV decode step."""
    ctx: int          # keys per sequence (positions 0 .. ctx-1 are attended)
    world: int
    n_seq: int
    n_head: int
    head_dim: int = 64
    align: int = 128  # range boundaries are multiples of this many keys

    def key_range(self, rank: int) -> tuple[int, int]:
        """[t0, t1) of `rank`: contiguous chunks of ceil(ctx / world) keys rounded up to `align`;
        trailing ranks may get a shorter or empty range."""
        per = -(-self.ctx // self.world)
        per = -(-per // self.align) * self.align
        t0 = min(self.ctx, rank * per)
        return t0, min(self.ctx, t0 + per)

    @property
    def rows(self) -> int:
        return self.n_seq * self.n_head

    @property
    def floats_per_rank(self) -> int:
        return self.rows * (self.head_dim + 2)

    def bytes_per_rank(self) -> int:
        return 4 * self.floats_per_rank

    def unpack(self, gathered):
        """gathered: [world, floats_per_rank] -> (m [world, rows], l [world, rows],
        acc [world, rows, head_dim]) views of one rank-major buffer."""
        r, d = self.rows, self.head_dim
        m = gathered[:, :r]
        l = gathered[:, r:2 * r]
        acc = gathered[:, 2 * r:].reshape(self.world, r, d)
        return m, l, acc


def gather_partials(plan: SplitKvPlan, local, gathered, group=None):
    """All-gathers each rank's packed partial buffer ([m | l | acc], `floats_per_rank` floats)
    into `gathered` [world, floats_per_rank].  One collective per decode step."""
    import torch.distributed as dist
    if plan.world == 1:
        if local.data_ptr() != gathered.data_ptr():
            gathered[0].copy_(local)
        return gathered
    dist.all_gather_into_tensor(gathered.view(-1), local.view(-1), group=group)
    return gathered


class PeerExchange:
    """Exchange regions of the fused split-KV step (mx230_splitkv_*): one region per rank, allocated
    by the library, mapped into every other rank's process through CUDA IPC.  The handles travel
    once through `torch.distributed` (any backend); the steps themselves use no collective."""

    def __init__(self, handle, rank: int, world: int, rows: int, head_dim: int = 64, group=None):
        import ctypes as C
        from ._lib import check, lib
        self.h, self.rank, self.world, self.group = handle, rank, world, group
        c = C.c_void_p()
        check(lib().mx230_splitkv_comm_create(handle._h, rank, world, rows, head_dim, C.byref(c)))
        self._c = c
        if world > 1:
            import torch.distributed as dist
            mine = C.create_string_buffer(64)
            check(lib().mx230_splitkv_comm_export(c, mine))
            handles = [None] * world
            dist.all_gather_object(handles, bytes(mine.raw), group=group)
            for peer, hb in enumerate(handles):
                if peer != rank:
                    check(lib().mx230_splitkv_comm_import(c, peer, C.create_string_buffer(hb, 64)))
            dist.barrier(group=group)   # every rank has opened every region before the first push

    def exchange_merge(self, out, local, stream=None):
        """One kernel: push `local` ([m | l | acc]) to every rank, wait for the others, merge into `out`."""
        from ._lib import check, lib, ptr
        from .common import stream_ptr
        check(lib().mx230_splitkv_exchange_merge(self._c, stream_ptr(stream), ptr(out), ptr(local)))

    def wait_merge(self, out, stream=None):
        """Second half of a step whose push was done by `llm_attention.attn_decode_partial_push`."""
        from ._lib import check, lib, ptr
        from .common import stream_ptr
        check(lib().mx230_splitkv_wait_merge(self._c, stream_ptr(stream), ptr(out)))

    def close(self):
        """Two-phase teardown: all ranks close their imports, then each frees its own region."""
        from ._lib import check, lib
        if self._c is None:
            return
        check(lib().mx230_splitkv_comm_disconnect(self._c))
        if self.world > 1:
            import torch.distributed as dist
            dist.barrier(group=self.group)
        lib().mx230_splitkv_comm_destroy(self._c)
        self._c = None


class SplitKvDecoder:
    """Pre-allocated buffers and the per-step call sequence of split-KV decode on one rank:
    local partial attention -> all-gather -> merge (`fused=False`).  With `fused=True` ("one") the whole
    step is one kernel: the CTA that finishes a (sequence, KV head) group stores the group's triples
    into every other rank's exchange region, waits for theirs and merges.  `fused="push"` leaves the
    wait and the merge to a second kernel, `fused="exchange"` also the stores.  All forms give the same
    bits.  Nothing is allocated per step."""

    def __init__(self, handle, plan: SplitKvPlan, rank: int, device="cuda", group=None, fused=False):
        import torch
        self.h, self.plan, self.rank, self.group = handle, plan, rank, group
        if fused and plan.rows % 2:
            raise ValueError("the fused exchange needs an even number of (sequence, head) rows")
        self.mode = "one" if fused is True else fused
        if fused and self.mode not in ("one", "push", "exchange"):
            raise ValueError(f"unknown fused mode {fused!r}")
        self.peer = PeerExchange(handle, rank, plan.world, plan.rows, plan.head_dim, group) if fused else None
        self.gathered = torch.zeros(plan.world, plan.floats_per_rank, dtype=torch.float32, device=device)
        # alone, the rank writes its partial straight into the gathered buffer
        self.local = self.gathered[0] if plan.world == 1 and not fused else torch.zeros(
            plan.floats_per_rank, dtype=torch.float32, device=device)
        self.out = torch.zeros(plan.rows, plan.head_dim, dtype=torch.float32, device=device)
        # packed views: [m | l | acc] of this rank, and contiguous gathered m / l / acc
        r = plan.rows
        self.m, self.l, self.acc = self.local[:r], self.local[r:2 * r], self.local[2 * r:]
        self.gm = torch.zeros(plan.world, r, dtype=torch.float32, device=device)
        self.gl = torch.zeros(plan.world, r, dtype=torch.float32, device=device)
        self.ga = torch.zeros(plan.world, r, plan.head_dim, dtype=torch.float32, device=device)

    def step(self, qkv, cache, n_kv_head: int, seq_rows: int, qkv_stride: int):
        """`cache` holds only this rank's key range: local row i of sequence s is key t0 + i."""
        from . import llm_attention as la
        p = self.plan
        t0, t1 = p.key_range(self.rank)
        if self.peer is not None and self.mode == "one":
            la.attn_decode_splitkv(self.h, self.peer._c, self.out, qkv, cache, 0, t1 - t0, p.n_seq, p.n_head, n_kv_head,
                                   p.head_dim, seq_rows, qkv_stride)
            return self.out
        if self.peer is not None and self.mode == "push":
            la.attn_decode_partial_push(self.h, self.peer._c, qkv, cache, 0, t1 - t0, p.n_seq, p.n_head, n_kv_head,
                                        p.head_dim, seq_rows, qkv_stride)
            self.peer.wait_merge(self.out)
            return self.out
        if t1 > t0:
            la.attn_decode_partial(self.h, self.m, self.l, self.acc, qkv, cache, 0, t1 - t0, p.n_seq,
                                   p.n_head, n_kv_head, p.head_dim, seq_rows, qkv_stride)
        else:  # an empty range contributes nothing: m = -inf, l = 0, acc = 0
            self.m.fill_(float("-inf"))
            self.l.zero_()
            self.acc.zero_()
        if self.peer is not None:
            self.peer.exchange_merge(self.out, self.local)
            return self.out
        gather_partials(p, self.local, self.gathered, self.group)
        if p.rows % 2 == 0:   # merge straight from the gathered buffer
            la.merge_partials_packed(self.h, self.out, self.gathered, p.world, p.rows, p.head_dim)
        else:
            m, l, acc = p.unpack(self.gathered)
            self.gm.copy_(m), self.gl.copy_(l), self.ga.copy_(acc)
            la.merge_partials(self.h, self.out, self.gm, self.gl, self.ga, p.world, p.rows, p.head_dim)
        return self.out

    def close(self):
        if self.peer is not None:
            self.peer.close()
            self.peer = None
