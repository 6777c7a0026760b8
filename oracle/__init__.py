"""CPU oracle for the attention path -- TEST INFRASTRUCTURE ONLY.

numpy-facing bindings of ``oracle/attn_oracle.c``.  Only ``tests/``, the smoke
check and the CPU-baseline / reference legs of ``bench.py`` may import this
package; the product (``mx230_b200``) never does.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

from . import build as _build

_f32p = C.POINTER(C.c_float)
_i8p = C.POINTER(C.c_int8)
_i32p = C.POINTER(C.c_int)

_lib = None


def lib():
    global _lib
    if _lib is None:
        path = _build.ORACLE_SO
        if not os.path.exists(path) or os.path.getmtime(path) < os.path.getmtime(
                os.path.join(_build.HERE, "attn_oracle.c")):
            path = _build.build_oracle()
        L = C.CDLL(path)
        L.orc_attn_loss.restype = C.c_double
        L.orc_max_rel_err.restype = C.c_float
        L.orc_allclose_err.restype = C.c_float
        L.orc_max_threads.restype = C.c_int
        L.orc_attn_fwd_rows.restype = C.c_int
        _lib = L
    return _lib


def _f(a):
    if a is None:
        return None
    assert a.dtype == np.float32 and a.flags.c_contiguous
    return a.ctypes.data_as(_f32p)


def _b(a):
    if a is None:
        return None
    assert a.dtype == np.int8 and a.flags.c_contiguous
    return a.ctypes.data_as(_i8p)


def _i(a):
    if a is None:
        return None
    assert a.dtype == np.int32 and a.flags.c_contiguous
    return a.ctypes.data_as(_i32p)


def max_threads() -> int:
    return int(lib().orc_max_threads())


# ---- common/src/lib.rs ------------------------------------------------------
def pseudo_rand(n: int, seed: int) -> np.ndarray:
    out = np.empty(n, np.float32)
    lib().orc_pseudo_rand(_f(out), C.c_size_t(n), C.c_uint64(seed))
    return out


def normal(shape, seed: int, tensor_index: int) -> np.ndarray:
    out = np.empty(int(np.prod(shape)), np.float32)
    lib().orc_normal(_f(out), C.c_size_t(out.size), C.c_uint64(seed), C.c_uint64(tensor_index))
    return out.reshape(shape)


def max_rel_err(got, want) -> float:
    g = np.ascontiguousarray(got, np.float32).ravel()
    w = np.ascontiguousarray(want, np.float32).ravel()
    return float(lib().orc_max_rel_err(_f(g), _f(w), C.c_size_t(g.size)))


def allclose_err(got, want, rtol: float, atol: float) -> float:
    g = np.ascontiguousarray(got, np.float32).ravel()
    w = np.ascontiguousarray(want, np.float32).ravel()
    return float(lib().orc_allclose_err(_f(g), _f(w), C.c_size_t(g.size), C.c_float(rtol),
                                        C.c_float(atol)))


# ---- the build's own parity metrics (tolerances of the north star) -----------
def max_abs_err(got, want) -> float:
    return float(np.max(np.abs(np.asarray(got, np.float64) - np.asarray(want, np.float64)))) \
        if np.size(want) else 0.0


def mean_rel_err(got, want) -> float:
    """Norm-wise mean relative error: sum|got-want| / sum|want|."""
    g = np.asarray(got, np.float64)
    w = np.asarray(want, np.float64)
    den = np.sum(np.abs(w))
    return float(np.sum(np.abs(g - w)) / den) if den > 0 else float(np.sum(np.abs(g - w)))


# ---- 02-flash-attention -------------------------------------------------------
def attn_fwd(q, k, v, causal: bool, threads: int = 0):
    """q,k,v: [..., n, 64] float32 -> (o [..., n, 64], lse [..., n])."""
    q = np.ascontiguousarray(q, np.float32)
    k = np.ascontiguousarray(k, np.float32)
    v = np.ascontiguousarray(v, np.float32)
    n = q.shape[-2]
    heads = int(np.prod(q.shape[:-2])) if q.ndim > 2 else 1
    o = np.empty_like(q)
    lse = np.empty(q.shape[:-1], np.float32)
    lib().orc_attn_fwd(_f(q), _f(k), _f(v), _f(o), _f(lse), heads, n, int(causal), threads)
    return o, lse


def attn_bwd(q, k, v, dout, causal: bool, threads: int = 0):
    q = np.ascontiguousarray(q, np.float32)
    k = np.ascontiguousarray(k, np.float32)
    v = np.ascontiguousarray(v, np.float32)
    dout = np.ascontiguousarray(dout, np.float32)
    n = q.shape[-2]
    heads = int(np.prod(q.shape[:-2])) if q.ndim > 2 else 1
    dq, dk, dv = np.empty_like(q), np.empty_like(q), np.empty_like(q)
    lib().orc_attn_bwd(_f(q), _f(k), _f(v), _f(dout), _f(dq), _f(dk), _f(dv), heads, n,
                       int(causal), threads)
    return dq, dk, dv


def attn_fwd_rows(q, k, v, causal: bool, row0: int, stride: int, threads: int = 0):
    q = np.ascontiguousarray(q, np.float32)
    n = q.shape[-2]
    heads = int(np.prod(q.shape[:-2])) if q.ndim > 2 else 1
    rows = len(range(row0, n, stride))
    o = np.empty((heads, rows, 64), np.float32)
    lib().orc_attn_fwd_rows(_f(q), _f(np.ascontiguousarray(k, np.float32)),
                            _f(np.ascontiguousarray(v, np.float32)), _f(o), heads, n, int(causal),
                            row0, stride, threads)
    return o


def bwd_preprocess(dout, o):
    dout = np.ascontiguousarray(dout, np.float32)
    o = np.ascontiguousarray(o, np.float32)
    delta = np.empty(o.shape[:-1], np.float32)
    lib().orc_bwd_preprocess(_f(dout), _f(o), _f(delta), C.c_size_t(delta.size))
    return delta


def attn_loss(q, k, v, dout, causal: bool) -> float:
    n = q.shape[0]
    return float(lib().orc_attn_loss(_f(np.ascontiguousarray(q, np.float32)),
                                     _f(np.ascontiguousarray(k, np.float32)),
                                     _f(np.ascontiguousarray(v, np.float32)),
                                     _f(np.ascontiguousarray(dout, np.float32)), n, int(causal)))


# ---- 03-llm-engine attention step --------------------------------------------
def rope(x, n_heads: int, head_dim: int, pos: int, theta: float):
    """In place on a contiguous float32 vector of n_heads*head_dim values."""
    assert x.dtype == np.float32 and x.flags.c_contiguous
    lib().orc_rope(_f(x), n_heads, head_dim, pos, C.c_float(theta))
    return x


def rope_qkv_row(row, pos, n_head, n_kv_head, head_dim, theta):
    """RoPE on the Q heads then the K heads of one qkv row (K follows Q)."""
    qd = n_head * head_dim
    kd = n_kv_head * head_dim
    rope(row[:qd], n_head, head_dim, pos, theta)
    rope(row[qd:qd + kd], n_kv_head, head_dim, pos, theta)
    return row


def quant_affine(src):
    src = np.ascontiguousarray(src, np.float32)
    dst = np.empty(src.shape, np.int8)
    s, b = C.c_float(), C.c_float()
    lib().orc_quant_affine(_f(src), _b(dst), C.byref(s), C.byref(b), src.size)
    return dst, np.float32(s.value), np.float32(b.value)


def quant_absmax(src):
    src = np.ascontiguousarray(src, np.float32)
    dst = np.empty(src.shape, np.int8)
    s = C.c_float()
    lib().orc_quant_absmax(_f(src), _b(dst), C.byref(s), src.size)
    return dst, np.float32(s.value)


class Q8Cache:
    """int8 KV cache in the reference layout (03-llm-engine/src/gpu.rs:197-204):
    codes [rows][n_kv_head*head_dim], side arrays [rows][n_kv_head]."""

    def __init__(self, rows, n_kv_head, head_dim=64, affine=True):
        self.rows, self.n_kv_head, self.head_dim, self.affine = rows, n_kv_head, head_dim, affine
        kvd = n_kv_head * head_dim
        self.kq = np.zeros((rows, kvd), np.int8)
        self.vq = np.zeros((rows, kvd), np.int8)
        self.ks = np.zeros((rows, n_kv_head), np.float32)
        self.vs = np.zeros((rows, n_kv_head), np.float32)
        self.kb = np.zeros((rows, n_kv_head), np.float32) if affine else None
        self.vb = np.zeros((rows, n_kv_head), np.float32) if affine else None


def quantize_kv_row(cache: Q8Cache, qkv_row, pos, q_dim, table=None, block_size=16):
    qkv_row = np.ascontiguousarray(qkv_row, np.float32)
    lib().orc_quantize_kv_row(_b(cache.kq), _b(cache.vq), _f(cache.ks), _f(cache.vs), _f(cache.kb),
                              _f(cache.vb), _f(qkv_row), pos, q_dim, cache.n_kv_head,
                              cache.head_dim, _i(table), block_size, 0 if cache.affine else 1)


def copy_kv_row(kcache, vcache, qkv_row, pos, q_dim, kv_dim, table=None, block_size=16):
    lib().orc_copy_kv_row(_f(kcache), _f(vcache), _f(np.ascontiguousarray(qkv_row, np.float32)),
                          pos, q_dim, kv_dim, _i(table), block_size)


def gqa_decode_f32(q, kcache, vcache, t_cur, n_head, n_kv_head, head_dim=64, table=None,
                   block_size=16):
    out = np.empty(n_head * head_dim, np.float32)
    lib().orc_gqa_decode_f32(_f(out), _f(np.ascontiguousarray(q, np.float32)), _f(kcache),
                             _f(vcache), t_cur, n_head, n_kv_head, head_dim, _i(table), block_size)
    return out


def gqa_decode_q8(q, cache: Q8Cache, t_cur, n_head, mode, table=None, block_size=16):
    """mode 0: dequant-exact oracle; mode 1: kernel-faithful (q also int8)."""
    out = np.empty(n_head * cache.head_dim, np.float32)
    lib().orc_gqa_decode_q8(_f(out), _f(np.ascontiguousarray(q, np.float32)), _b(cache.kq),
                            _b(cache.vq), _f(cache.ks), _f(cache.vs), _f(cache.kb), _f(cache.vb),
                            t_cur, n_head, cache.n_kv_head, cache.head_dim, _i(table), block_size,
                            mode)
    return out


def gqa_partial(q, t0, t1, n_head, n_kv_head, head_dim=64, kcache=None, vcache=None, cache=None):
    m = np.empty(n_head, np.float32)
    l = np.empty(n_head, np.float32)
    acc = np.empty((n_head, head_dim), np.float32)
    c = cache
    lib().orc_gqa_partial(_f(m), _f(l), _f(acc), _f(np.ascontiguousarray(q, np.float32)),
                          _f(kcache), _f(vcache), _b(c.kq) if c else None,
                          _b(c.vq) if c else None, _f(c.ks) if c else None,
                          _f(c.vs) if c else None, _f(c.kb) if c else None,
                          _f(c.vb) if c else None, t0, t1, n_head, n_kv_head, head_dim)
    return m, l, acc


def merge_partials(m, l, acc):
    """m,l [parts][rows]; acc [parts][rows][hd] -> out [rows][hd]."""
    m = np.ascontiguousarray(m, np.float32)
    l = np.ascontiguousarray(l, np.float32)
    acc = np.ascontiguousarray(acc, np.float32)
    parts, rows, hd = acc.shape
    out = np.empty((rows, hd), np.float32)
    lib().orc_merge_partials(_f(out), _f(m), _f(l), _f(acc), parts, rows, hd)
    return out


def gqa_decode_batched(qkv, pos, n_head, n_kv_head, head_dim=64, kcache=None, vcache=None,
                       cache=None, tables=None, block_size=16, seq_rows=0, qkv_stride=None,
                       out_stride=None, mode=0, threads=0):
    qkv = np.ascontiguousarray(qkv, np.float32)
    pos = np.ascontiguousarray(pos, np.int32)
    n_seq = pos.size
    qkv_stride = qkv_stride or qkv.shape[-1]
    out_stride = out_stride or n_head * head_dim
    out = np.zeros((n_seq, out_stride), np.float32)
    c = cache
    n_log = tables.shape[1] if tables is not None else 0
    lib().orc_gqa_decode_batched(
        _f(out), _f(qkv), _f(kcache), _f(vcache), _b(c.kq) if c else None, _b(c.vq) if c else None,
        _f(c.ks) if c else None, _f(c.vs) if c else None, _f(c.kb) if c else None,
        _f(c.vb) if c else None, _i(pos), n_seq, n_head, n_kv_head, head_dim, _i(tables),
        block_size, n_log, C.c_size_t(seq_rows), qkv_stride, out_stride, mode, threads)
    return out


def prefill(qkv, pos0, n_tok, n_head, n_kv_head, qkv_stride, out_stride, kcache=None, vcache=None,
            cache=None, table=None, block_size=16, threads=0, mode=0):
    """mode 0: exact scores (fp32 cache, or int8 cache dequantised).  mode 1: the reference kernels' int8 score
    arithmetic -- over an int8 cache its attn_prefill_q8, over an fp32 cache its opt-in attn_prefill_dp4a."""
    qkv = np.ascontiguousarray(qkv, np.float32)
    out = np.zeros((n_tok, out_stride), np.float32)
    c = cache
    lib().orc_prefill(_f(out), _f(qkv), _f(kcache), _f(vcache), _b(c.kq) if c else None,
                      _b(c.vq) if c else None, _f(c.ks) if c else None, _f(c.vs) if c else None,
                      _f(c.kb) if c else None, _f(c.vb) if c else None, pos0, n_tok, n_head,
                      n_kv_head, qkv_stride, out_stride, _i(table), block_size,
                      (2 if mode else 1) if c is not None else (3 if mode else 0), threads)
    return out


def gemv(x, w, b=None, y=None, accum=False):
    """The reference gemv (llm.cu:144-177): y[o] (+)= sum_i x[i] w[i, o] + b[o]; fp16 weights are
    widened to fp32 first, as gemv_half does."""
    x = np.ascontiguousarray(x, np.float32)
    w = np.ascontiguousarray(np.asarray(w).astype(np.float32))
    n_in, n_out = w.shape
    out = np.zeros(n_out, np.float32) if y is None else np.ascontiguousarray(y, np.float32).copy()
    lib().orc_gemv(_f(out), _f(x), _f(w), _f(None if b is None else np.ascontiguousarray(b, np.float32)),
                   n_in, n_out, 1 if accum else 0)
    return out


def gemm(a, w, b=None):
    """The reference gemm (gpu.rs:1291-1420; kernels gemm_f32* / gemm_half*, llm.cu:1632-1733): c[r][o] =
    sum_i a[r][i] w[i][o] + b[o], every row the sequential fp32 sum of `gemv`."""
    a = np.ascontiguousarray(a, np.float32)
    return np.stack([gemv(a[r], w, b) for r in range(a.shape[0])]) if a.shape[0] else np.zeros((0, np.asarray(w).shape[1]), np.float32)


def pack_int8_weights(w8):
    """int8 [n_in][n_out] -> int32 words of four consecutive input rows, w32[(i/4)][o], byte j = row 4(i/4)+j
    (the reference's load-time repacking, llm.cu:183-188)."""
    w8 = np.ascontiguousarray(w8, np.int8)
    n_in, n_out = w8.shape
    u = w8.astype(np.uint8).astype(np.uint32).reshape(n_in // 4, 4, n_out)
    return np.ascontiguousarray((u[:, 0] | (u[:, 1] << 8) | (u[:, 2] << 16) | (u[:, 3] << 24)).astype(np.uint32).view(np.int32))


def gemv_int8(x, w32, scales, b=None, y=None, accum=False, ag=8):
    """The reference gemv_int8 (llm.cu:226-316) on packed weights."""
    x = np.ascontiguousarray(x, np.float32)
    w32 = np.ascontiguousarray(w32, np.int32)
    n_in, n_out = w32.shape[0] * 4, w32.shape[1]
    out = np.zeros(n_out, np.float32) if y is None else np.ascontiguousarray(y, np.float32).copy()
    lib().orc_gemv_int8(_f(out), _f(x), _i(w32), _f(np.ascontiguousarray(scales, np.float32)),
                        _f(None if b is None else np.ascontiguousarray(b, np.float32)), n_in, n_out,
                        1 if accum else 0, ag)
    return out
