"""Host mirror of the reference engine's per-layer attention step
(03-llm-engine/src/gpu.rs:2570-2672 decode, :2808-2918 graph decode, :3204-3347 prefill
write path, :3530-3628 batched decode): RoPE -> KV write -> attention, with the kernel
chosen by (cache format, paging).  One Python function per reference kernel symbol,
same argument order; `KvCache` and `Paging` mirror gpu.rs:188-205 and :381-539.
Tensors are torch CUDA tensors; nothing here synchronises or allocates on the step path.
"""
from __future__ import annotations

import torch

from ._lib import check, lib, ptr
from .common import Handle, stream_ptr

KV_BLOCK = 16  # 03-llm-engine/src/gpu.rs:209


class KvCache:
    """One layer's KV cache: fp32 `[slots][n_kv_head*64]`, or int8 codes of that shape
    plus per-(slot, kv head) fp32 scale (and beta when `affine`), gpu.rs:188-205."""

    def __init__(self, slots: int, n_kv_head: int, head_dim: int = 64, quant: bool = False,
                 affine: bool = True, device="cuda"):
        self.slots, self.n_kv_head, self.head_dim = slots, n_kv_head, head_dim
        self.quant, self.affine = quant, affine
        kvd = n_kv_head * head_dim
        if quant:
            self.k = torch.zeros(slots, kvd, dtype=torch.int8, device=device)
            self.v = torch.zeros(slots, kvd, dtype=torch.int8, device=device)
            self.ks = torch.zeros(slots, n_kv_head, dtype=torch.float32, device=device)
            self.vs = torch.zeros(slots, n_kv_head, dtype=torch.float32, device=device)
            self.kb = torch.zeros(slots, n_kv_head, dtype=torch.float32, device=device) if affine else None
            self.vb = torch.zeros(slots, n_kv_head, dtype=torch.float32, device=device) if affine else None
        else:
            self.k = torch.zeros(slots, kvd, dtype=torch.float32, device=device)
            self.v = torch.zeros(slots, kvd, dtype=torch.float32, device=device)

    def q8_args(self):
        return (ptr(self.k), ptr(self.v), ptr(self.ks), ptr(self.vs), ptr(self.kb), ptr(self.vb))

    def nbytes(self) -> int:
        n = self.k.numel() * self.k.element_size() * 2
        if self.quant:
            n += self.ks.numel() * 4 * (4 if self.affine else 2)
        return n


class Paging:
    """Logical position -> physical row through a block table (gpu.rs:381-539):
    row = table[t // block_size] * block_size + t % block_size."""

    def __init__(self, table, block_size: int = KV_BLOCK):
        self.table_dev = table  # int32 CUDA tensor [n_log] or [n_seq][n_log]
        self.block_size = block_size
        self.n_log = table.shape[-1]

    def phys_row(self, host_table, pos: int) -> int:
        return int(host_table[pos // self.block_size]) * self.block_size + pos % self.block_size


# ---------------------------------------------------------------- rope
def rope(h: Handle, qkv, pos: int, n_head, n_kv_head, head_dim, theta, stream=None):
    check(lib().mx230_rope(h._h, stream_ptr(stream), ptr(qkv), pos, n_head, n_kv_head, head_dim, theta))


def rope_dyn(h: Handle, qkv, pos_ptr, n_head, n_kv_head, head_dim, theta, stream=None):
    check(lib().mx230_rope_dyn(h._h, stream_ptr(stream), ptr(qkv), ptr(pos_ptr), n_head, n_kv_head,
                               head_dim, theta))


def rope_batch(h: Handle, qkv, pos0, n_tok, n_head, n_kv_head, head_dim, stride, theta, stream=None):
    check(lib().mx230_rope_batch(h._h, stream_ptr(stream), ptr(qkv), pos0, n_tok, n_head, n_kv_head,
                                 head_dim, stride, theta))


def rope_seqpos(h: Handle, qkv, pos, n_seq, n_head, n_kv_head, head_dim, stride, theta, stream=None):
    check(lib().mx230_rope_seqpos(h._h, stream_ptr(stream), ptr(qkv), ptr(pos), n_seq, n_head,
                                  n_kv_head, head_dim, stride, theta))


# ---------------------------------------------------------------- fp32 KV write
def copy_kv(h: Handle, c: KvCache, qkv, pos: int, q_dim, kv_dim, stream=None):
    check(lib().mx230_copy_kv(h._h, stream_ptr(stream), ptr(c.k), ptr(c.v), ptr(qkv), pos, q_dim, kv_dim))


def copy_kv_dyn(h: Handle, c: KvCache, qkv, pos_ptr, q_dim, kv_dim, stream=None):
    check(lib().mx230_copy_kv_dyn(h._h, stream_ptr(stream), ptr(c.k), ptr(c.v), ptr(qkv),
                                  ptr(pos_ptr), q_dim, kv_dim))


def copy_kv_paged_dyn(h: Handle, c: KvCache, qkv, pos_ptr, q_dim, kv_dim, pg: Paging, stream=None):
    check(lib().mx230_copy_kv_paged_dyn(h._h, stream_ptr(stream), ptr(c.k), ptr(c.v), ptr(qkv),
                                        ptr(pos_ptr), q_dim, kv_dim, ptr(pg.table_dev), pg.block_size))


def copy_kv_batch(h: Handle, c: KvCache, qkv, pos0, n_tok, q_dim, kv_dim, stride, pg: Paging | None = None,
                  stream=None):
    if pg is None:
        check(lib().mx230_copy_kv_batch(h._h, stream_ptr(stream), ptr(c.k), ptr(c.v), ptr(qkv), pos0,
                                        n_tok, q_dim, kv_dim, stride))
    else:
        check(lib().mx230_copy_kv_batch_paged(h._h, stream_ptr(stream), ptr(c.k), ptr(c.v), ptr(qkv),
                                              pos0, n_tok, q_dim, kv_dim, stride, ptr(pg.table_dev),
                                              pg.block_size))


def copy_kv_seqpos(h: Handle, c: KvCache, qkv, pos, n_seq, q_dim, kv_dim, qkv_stride, pg: Paging,
                   stream=None):
    check(lib().mx230_copy_kv_seqpos(h._h, stream_ptr(stream), ptr(c.k), ptr(c.v), ptr(qkv), ptr(pos),
                                     n_seq, q_dim, kv_dim, qkv_stride, ptr(pg.table_dev),
                                     pg.block_size, pg.n_log))


# ---------------------------------------------------------------- int8 quantize-on-write
def quantize_kv(h: Handle, c: KvCache, qkv, pos: int, q_dim, n_kv_head, head_dim, stream=None):
    check(lib().mx230_quantize_kv(h._h, stream_ptr(stream), *c.q8_args(), ptr(qkv), pos, q_dim,
                                  n_kv_head, head_dim))


def quantize_kv_dyn(h: Handle, c: KvCache, qkv, pos_ptr, q_dim, n_kv_head, head_dim, stream=None):
    check(lib().mx230_quantize_kv_dyn(h._h, stream_ptr(stream), *c.q8_args(), ptr(qkv), ptr(pos_ptr),
                                      q_dim, n_kv_head, head_dim))


def quantize_kv_paged_dyn(h: Handle, c: KvCache, qkv, pos_ptr, q_dim, n_kv_head, head_dim, pg: Paging,
                          stream=None):
    check(lib().mx230_quantize_kv_paged_dyn(h._h, stream_ptr(stream), *c.q8_args(), ptr(qkv),
                                            ptr(pos_ptr), q_dim, n_kv_head, head_dim,
                                            ptr(pg.table_dev), pg.block_size))


def quantize_kv_batch(h: Handle, c: KvCache, qkv, pos0, n_tok, q_dim, n_kv_head, head_dim, stride,
                      pg: Paging | None = None, stream=None):
    if pg is None:
        check(lib().mx230_quantize_kv_batch(h._h, stream_ptr(stream), *c.q8_args(), ptr(qkv), pos0,
                                            n_tok, q_dim, n_kv_head, head_dim, stride))
    else:
        check(lib().mx230_quantize_kv_batch_paged(h._h, stream_ptr(stream), *c.q8_args(), ptr(qkv),
                                                  pos0, n_tok, q_dim, n_kv_head, head_dim, stride,
                                                  ptr(pg.table_dev), pg.block_size))


def quantize_kv_seqpos(h: Handle, c: KvCache, qkv, pos, n_seq, q_dim, n_kv_head, head_dim, qkv_stride,
                       pg: Paging, stream=None):
    check(lib().mx230_quantize_kv_seqpos(h._h, stream_ptr(stream), *c.q8_args(), ptr(qkv), ptr(pos),
                                         n_seq, q_dim, n_kv_head, head_dim, qkv_stride,
                                         ptr(pg.table_dev), pg.block_size, pg.n_log))


# ---------------------------------------------------------------- decode attention
def attn_decode(h: Handle, out, qkv, c: KvCache, t_cur: int, n_head, n_kv_head, head_dim,
                pg: Paging | None = None, stream=None):
    """attn_decode / attn_decode_paged / attn_decode_q8 / attn_decode_q8_paged, chosen by
    (cache format, paging) as gpu.rs:2607-2670."""
    s = stream_ptr(stream)
    L = lib()
    if c.quant:
        if pg is None:
            check(L.mx230_attn_decode_q8(h._h, s, ptr(out), ptr(qkv), *c.q8_args(), t_cur, n_head,
                                         n_kv_head, head_dim))
        else:
            check(L.mx230_attn_decode_q8_paged(h._h, s, ptr(out), ptr(qkv), *c.q8_args(), t_cur, n_head,
                                               n_kv_head, head_dim, ptr(pg.table_dev), pg.block_size))
    else:
        if pg is None:
            check(L.mx230_attn_decode(h._h, s, ptr(out), ptr(qkv), ptr(c.k), ptr(c.v), t_cur, n_head,
                                      n_kv_head, head_dim))
        else:
            check(L.mx230_attn_decode_paged(h._h, s, ptr(out), ptr(qkv), ptr(c.k), ptr(c.v), t_cur,
                                            n_head, n_kv_head, head_dim, ptr(pg.table_dev),
                                            pg.block_size))


def attn_decode_dyn(h: Handle, out, qkv, c: KvCache, pos_ptr, n_head, n_kv_head, head_dim,
                    pg: Paging | None = None, stream=None):
    """The `_dyn` forms of gpu.rs:2808-2918: position read from device memory."""
    s = stream_ptr(stream)
    L = lib()
    if c.quant:
        if pg is None:
            check(L.mx230_attn_decode_q8_dyn(h._h, s, ptr(out), ptr(qkv), *c.q8_args(), ptr(pos_ptr),
                                             n_head, n_kv_head, head_dim))
        else:
            check(L.mx230_attn_decode_q8_paged_dyn(h._h, s, ptr(out), ptr(qkv), *c.q8_args(),
                                                   ptr(pos_ptr), n_head, n_kv_head, head_dim,
                                                   ptr(pg.table_dev), pg.block_size))
    else:
        if pg is None:
            check(L.mx230_attn_decode_dyn(h._h, s, ptr(out), ptr(qkv), ptr(c.k), ptr(c.v), ptr(pos_ptr),
                                          n_head, n_kv_head, head_dim))
        else:
            check(L.mx230_attn_decode_paged_dyn(h._h, s, ptr(out), ptr(qkv), ptr(c.k), ptr(c.v),
                                                ptr(pos_ptr), n_head, n_kv_head, head_dim,
                                                ptr(pg.table_dev), pg.block_size))


def attn_decode_batched(h: Handle, out, qkv, c: KvCache, pos, n_seq, n_head, n_kv_head, head_dim,
                        pg: Paging, qkv_stride, out_stride, stream=None):
    """attn_decode_batched / attn_decode_q8_batched, gpu.rs:3530-3628."""
    s = stream_ptr(stream)
    if c.quant:
        check(lib().mx230_attn_decode_q8_batched(h._h, s, ptr(out), ptr(qkv), *c.q8_args(), ptr(pos),
                                                 n_seq, n_head, n_kv_head, head_dim, ptr(pg.table_dev),
                                                 pg.block_size, pg.n_log, qkv_stride, out_stride))
    else:
        check(lib().mx230_attn_decode_batched(h._h, s, ptr(out), ptr(qkv), ptr(c.k), ptr(c.v), ptr(pos),
                                              n_seq, n_head, n_kv_head, head_dim, ptr(pg.table_dev),
                                              pg.block_size, pg.n_log, qkv_stride, out_stride))


def _cache_args(c: KvCache):
    if c.quant:
        return (None, None) + c.q8_args()
    return (ptr(c.k), ptr(c.v), None, None, None, None, None, None)


def attn_decode_slab(h: Handle, out, qkv, c: KvCache, pos, n_seq, n_head, n_kv_head, head_dim,
                     seq_rows, qkv_stride, out_stride, stream=None):
    """Batched decode over contiguous per-sequence cache slabs of `seq_rows` rows."""
    check(lib().mx230_attn_decode_slab(h._h, stream_ptr(stream), ptr(out), ptr(qkv), *_cache_args(c),
                                       ptr(pos), n_seq, n_head, n_kv_head, head_dim, seq_rows,
                                       qkv_stride, out_stride))


def attn_decode_partial(h: Handle, part_m, part_l, part_acc, qkv, c: KvCache, t0, t1, n_seq, n_head,
                        n_kv_head, head_dim, seq_rows, qkv_stride, stream=None):
    """Unnormalised (m, l, acc) of keys [t0, t1) per (sequence, query head)."""
    check(lib().mx230_attn_decode_partial(h._h, stream_ptr(stream), ptr(part_m), ptr(part_l),
                                          ptr(part_acc), ptr(qkv), *_cache_args(c), t0, t1, n_seq,
                                          n_head, n_kv_head, head_dim, seq_rows, qkv_stride))


def attn_decode_partial_push(h: Handle, comm, qkv, c: KvCache, t0, t1, n_seq, n_head, n_kv_head, head_dim, seq_rows,
                             qkv_stride, stream=None):
    """attn_decode_partial whose finishing CTAs store the triples into every rank's split-KV exchange region
    (`comm`: the mx230_splitkv_comm of `multi_gpu.PeerExchange`)."""
    check(lib().mx230_attn_decode_partial_push(h._h, stream_ptr(stream), comm, ptr(qkv), *_cache_args(c), t0, t1,
                                               n_seq, n_head, n_kv_head, head_dim, seq_rows, qkv_stride))


def attn_decode_splitkv(h: Handle, comm, out, qkv, c: KvCache, t0, t1, n_seq, n_head, n_kv_head, head_dim, seq_rows,
                        qkv_stride, stream=None):
    """A whole split-KV step in one kernel: partial attention over keys [t0, t1), stores to every other rank's
    exchange region, wait for their triples, merged rows to out[n_seq * n_head][64]."""
    check(lib().mx230_attn_decode_splitkv(h._h, stream_ptr(stream), comm, ptr(out), ptr(qkv), *_cache_args(c), t0, t1,
                                          n_seq, n_head, n_kv_head, head_dim, seq_rows, qkv_stride))


def merge_partials(h: Handle, out, m, l, acc, parts, rows, head_dim=64, stream=None):
    check(lib().mx230_merge_partials(h._h, stream_ptr(stream), ptr(out), ptr(m), ptr(l), ptr(acc),
                                     parts, rows, head_dim))


def merge_partials_packed(h: Handle, out, gathered, parts, rows, head_dim=64, stream=None):
    """Merge straight from the all-gathered buffer [parts][m | l | acc] (rows even)."""
    check(lib().mx230_merge_partials_packed(h._h, stream_ptr(stream), ptr(out), ptr(gathered), parts, rows, head_dim))


# ---------------------------------------------------------------- the step
def decode_step(h: Handle, out, qkv, c: KvCache, pos: int, n_head, n_kv_head, head_dim, theta,
                pg: Paging | None = None, host_table=None, use_rope=True, stream=None):
    """One token of one sequence, as forward_layers does per layer (gpu.rs:2570-2672):
    RoPE, KV write at the host-resolved physical row, then attention over 0..=pos."""
    q_dim, kv_dim = n_head * head_dim, n_kv_head * head_dim
    if use_rope:
        rope(h, qkv, pos, n_head, n_kv_head, head_dim, theta, stream)
    phys = pos if pg is None else pg.phys_row(host_table, pos)
    if c.quant:
        quantize_kv(h, c, qkv, phys, q_dim, n_kv_head, head_dim, stream)
    else:
        copy_kv(h, c, qkv, phys, q_dim, kv_dim, stream)
    attn_decode(h, out, qkv, c, pos, n_head, n_kv_head, head_dim, pg, stream)


def decode_step_dyn(h: Handle, out, qkv, c: KvCache, pos_ptr, n_head, n_kv_head, head_dim, theta,
                    pg: Paging | None = None, use_rope=True, stream=None):
    """The graph-capturable step of forward_body_dyn (gpu.rs:2808-2918)."""
    q_dim, kv_dim = n_head * head_dim, n_kv_head * head_dim
    if use_rope:
        rope_dyn(h, qkv, pos_ptr, n_head, n_kv_head, head_dim, theta, stream)
    if c.quant:
        if pg is None:
            quantize_kv_dyn(h, c, qkv, pos_ptr, q_dim, n_kv_head, head_dim, stream)
        else:
            quantize_kv_paged_dyn(h, c, qkv, pos_ptr, q_dim, n_kv_head, head_dim, pg, stream)
    else:
        if pg is None:
            copy_kv_dyn(h, c, qkv, pos_ptr, q_dim, kv_dim, stream)
        else:
            copy_kv_paged_dyn(h, c, qkv, pos_ptr, q_dim, kv_dim, pg, stream)
    attn_decode_dyn(h, out, qkv, c, pos_ptr, n_head, n_kv_head, head_dim, pg, stream)


def batched_step(h: Handle, out, qkv, c: KvCache, pos, n_seq, n_head, n_kv_head, head_dim, theta,
                 pg: Paging, qkv_stride, out_stride, use_rope=True, stream=None):
    """One token for each of n_seq sequences, as forward_batched (gpu.rs:3530-3628)."""
    q_dim, kv_dim = n_head * head_dim, n_kv_head * head_dim
    if use_rope:
        rope_seqpos(h, qkv, pos, n_seq, n_head, n_kv_head, head_dim, qkv_stride, theta, stream)
    if c.quant:
        quantize_kv_seqpos(h, c, qkv, pos, n_seq, q_dim, n_kv_head, head_dim, qkv_stride, pg, stream)
    else:
        copy_kv_seqpos(h, c, qkv, pos, n_seq, q_dim, kv_dim, qkv_stride, pg, stream)
    attn_decode_batched(h, out, qkv, c, pos, n_seq, n_head, n_kv_head, head_dim, pg, qkv_stride,
                        out_stride, stream)


# ---------------------------------------------------------------- prefill attention
def prefill_workspace_bytes(n_tok, n_keys, n_head, n_kv_head) -> int:
    return int(lib().mx230_prefill_workspace_bytes(n_tok, n_keys, n_head, n_kv_head))


def attn_prefill(h: Handle, out, qkv, c: KvCache, pos0, n_tok, n_head, n_kv_head, qkv_stride, out_stride,
                 pg: Paging | None = None, stream=None):
    """attn_prefill / _paged / _q8 / _q8_paged chosen by (cache format, paging) as
    batch_body_from does (gpu.rs:3269-3345).  The cache must already hold the new rows."""
    s = stream_ptr(stream)
    L = lib()
    if c.quant:
        if pg is None:
            check(L.mx230_attn_prefill_q8(h._h, s, ptr(out), ptr(qkv), *c.q8_args(), pos0, n_tok, n_head,
                                          n_kv_head, qkv_stride, out_stride))
        else:
            check(L.mx230_attn_prefill_q8_paged(h._h, s, ptr(out), ptr(qkv), *c.q8_args(), pos0, n_tok, n_head,
                                                n_kv_head, qkv_stride, out_stride, ptr(pg.table_dev),
                                                pg.block_size))
    else:
        if pg is None:
            check(L.mx230_attn_prefill(h._h, s, ptr(out), ptr(qkv), ptr(c.k), ptr(c.v), pos0, n_tok, n_head,
                                       n_kv_head, qkv_stride, out_stride))
        else:
            check(L.mx230_attn_prefill_paged(h._h, s, ptr(out), ptr(qkv), ptr(c.k), ptr(c.v), pos0, n_tok,
                                             n_head, n_kv_head, qkv_stride, out_stride, ptr(pg.table_dev),
                                             pg.block_size))


def prefill_step(h: Handle, out, qkv, c: KvCache, pos0, n_tok, n_head, n_kv_head, head_dim, theta,
                 qkv_stride, out_stride, pg: Paging | None = None, use_rope=True, stream=None):
    """The prefill attention step of batch_body_from (gpu.rs:3204-3347): RoPE on the n_tok rows,
    KV write of all of them, then causal attention over the cache."""
    q_dim, kv_dim = n_head * head_dim, n_kv_head * head_dim
    if use_rope:
        rope_batch(h, qkv, pos0, n_tok, n_head, n_kv_head, head_dim, qkv_stride, theta, stream)
    if c.quant:
        quantize_kv_batch(h, c, qkv, pos0, n_tok, q_dim, n_kv_head, head_dim, qkv_stride, pg, stream)
    else:
        copy_kv_batch(h, c, qkv, pos0, n_tok, q_dim, kv_dim, qkv_stride, pg, stream)
    attn_prefill(h, out, qkv, c, pos0, n_tok, n_head, n_kv_head, qkv_stride, out_stride, pg, stream)


def attn_decode_q8_noalloc(out, qkv, c: KvCache, t_cur: int, n_head, n_kv_head, head_dim, stream=None):
    """Handle-free int8-cache decode of one sequence whose split-KV scratch is a fixed array inside
    the library: for hosts that may not call cudaMalloc (all HBM already owned by their KV pool, or
    only allowed to enqueue on a given stream).  Current device; see include/mx230_attn.h."""
    check(lib().mx230_attn_decode_q8_noalloc(stream_ptr(stream), ptr(out), ptr(qkv), *c.q8_args(), t_cur,
                                             n_head, n_kv_head, head_dim))


# ---------------------------------------------------------------- projections either side of attention
def gemv(h: Handle, y, x, w, b=None, accum=False, stream=None):
    """gemv / gemv_half (llm.cu:144-177; gpu.rs:1158-1198): y (+)= x W + b, W [n_in][n_out] fp32 or fp16."""
    n_in, n_out = w.shape
    check(lib().mx230_gemv(h._h, stream_ptr(stream), ptr(y), ptr(x), ptr(w), int(w.dtype == torch.float16),
                           ptr(b), n_in, n_out, int(accum)))


def gemm(h: Handle, c, a, w, b=None, stream=None):
    """gemm (gpu.rs:1291-1420) for the prefill-side projections: c [m][n] = a [m][k] . w [k][n] + b, `w` fp32 or
    fp16.  Grows the handle's workspace when it is too small for the staged operands."""
    m, k = a.shape
    n = w.shape[1]
    fp16 = 1 if w.dtype == torch.float16 else 0
    h.reserve(lib().mx230_gemm_workspace_bytes(m, n, k, fp16))
    check(lib().mx230_gemm(h._h, stream_ptr(stream), ptr(c), ptr(a), ptr(w), fp16, ptr(b), m, n, k))


def prefill_layer_attention(h: Handle, y, x, w_qkv, b_qkv, w_proj, b_proj, qkv, attn, c: KvCache, pos0, n_tok, n_head,
                            n_kv_head, head_dim, theta, pg: Paging | None = None, use_rope=True, stream=None):
    """The attention half of one layer for a prefill chunk, as batch_body_from runs it (gpu.rs:3187-3365):
    qkv = x W_qkv + b (gemm), RoPE, KV write, causal attention over the cache, y = attn W_proj + b (gemm).
    `qkv` [n_tok][q_dim + 2 kv_dim] and `attn` [n_tok][q_dim] are the caller's scratch rows (the reference's batch_qkv
    and batch_attn); the residual add that follows stays with the caller, as in the reference."""
    q_dim = n_head * head_dim
    gemm(h, qkv, x, w_qkv, b_qkv, stream)
    prefill_step(h, attn, qkv, c, pos0, n_tok, n_head, n_kv_head, head_dim, theta, qkv.shape[1], q_dim, pg, use_rope, stream)
    gemm(h, y, attn, w_proj, b_proj, stream)


def gemv_int8(h: Handle, y, x, w_packed, scales, b=None, accum=False, act_group=8, stream=None):
    """gemv_int8 (llm.cu:226-316): `w_packed` int32 [n_in / 4][n_out], four consecutive input rows per word."""
    n_in, n_out = w_packed.shape[0] * 4, w_packed.shape[1]
    check(lib().mx230_gemv_int8(h._h, stream_ptr(stream), ptr(y), ptr(x), ptr(w_packed), ptr(scales), ptr(b),
                                n_in, n_out, int(accum), act_group))


def qkv_rope_kvwrite(h: Handle, qkv, x, w, b, pos, c: KvCache, n_head, n_kv_head, theta, pg: Paging | None = None,
                     stream=None, w_scales=None, act_group=8):
    """The qkv step of one decode token in one launch (gemv + rope + KV write of gpu.rs:2558-2646):
    `pos` is a host int or an int32 device tensor (the graph-captured form)."""
    int8 = w.dtype == torch.int32   # packed int8 weights
    n_in = w.shape[0] * (4 if int8 else 1)
    kind = 2 if int8 else int(w.dtype == torch.float16)
    dyn = not isinstance(pos, int)
    caches = (None, None, *c.q8_args()) if c.quant else (ptr(c.k), ptr(c.v), None, None, None, None, None, None)
    check(lib().mx230_qkv_rope_kvwrite(h._h, stream_ptr(stream), ptr(qkv), ptr(x), ptr(w),
                                       kind, ptr(w_scales), act_group, ptr(b), n_in, 0 if dyn else pos,
                                       ptr(pos) if dyn else None, n_head, n_kv_head, 64, theta, *caches,
                                       ptr(pg.table_dev) if pg else None, pg.block_size if pg else 0))
