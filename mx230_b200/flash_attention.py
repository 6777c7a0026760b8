"""Host mirror of the reference's stage-2 launch wrappers
(02-flash-attention/src/main.rs:68-210): same names, argument order and meaning, with
the library handle in place of the `CudaFunction` tables and torch CUDA tensors in
place of `CudaSlice<f32>`.  Tensors are `[n, 64]` (the reference call) or
`[..., n, 64]` contiguous fp32; leading dimensions are independent (batch, head) units.
Everything is enqueued on torch's current stream (or `stream`) and nothing synchronises.
"""
from __future__ import annotations

from ._lib import check, lib, ptr
from .common import Handle, stream_ptr

D = 64  # 02-flash-attention/src/main.rs:12


def _bh(q, n: int) -> int:
    assert q.is_cuda and q.is_contiguous() and q.shape[-1] == D and q.shape[-2] == n, \
        "expected a contiguous CUDA tensor [..., n, 64]"
    bh = 1
    for s in q.shape[:-2]:
        bh *= s
    return bh


def workspace_bytes(batch_heads: int, n: int, with_backward: bool) -> int:
    return int(lib().mx230_flash_workspace_bytes(batch_heads, n, int(with_backward)))


def run_flash(h: Handle, q, k, v, o, n: int, causal: bool, stream=None) -> None:
    """run_flash, 02-flash-attention/src/main.rs:68-88."""
    check(lib().mx230_attn_flash(h._h, stream_ptr(stream), ptr(q), ptr(k), ptr(v), ptr(o),
                                 _bh(q, n), n, int(causal)))


def run_flash_lse(h: Handle, q, k, v, o, l, n: int, causal: bool, stream=None) -> None:
    """run_flash_lse, 02-flash-attention/src/main.rs:102-123."""
    check(lib().mx230_attn_flash_lse(h._h, stream_ptr(stream), ptr(q), ptr(k), ptr(v), ptr(o),
                                     ptr(l), _bh(q, n), n, int(causal)))


def run_preprocess(h: Handle, do_, o, delta, n: int, stream=None) -> None:
    """run_preprocess, 02-flash-attention/src/main.rs:126-143."""
    check(lib().mx230_attn_bwd_preprocess(h._h, stream_ptr(stream), ptr(do_), ptr(o), ptr(delta),
                                          _bh(o, n), n))


def run_bwd_flash(h: Handle, q, k, v, do_, l, delta, dq, dk, dv, n: int, causal: bool,
                  stream=None) -> None:
    """run_bwd_flash, 02-flash-attention/src/main.rs:179-210: dQ pass then dK/dV pass;
    outputs are fully overwritten (no zeroing needed)."""
    check(lib().mx230_attn_bwd_flash(h._h, stream_ptr(stream), ptr(q), ptr(k), ptr(v), ptr(do_),
                                     ptr(l), ptr(delta), ptr(dq), ptr(dk), ptr(dv), _bh(q, n), n,
                                     int(causal)))


def run_bwd_dq(h: Handle, q, k, v, do_, l, delta, dq, n: int, causal: bool, stream=None) -> None:
    check(lib().mx230_attn_bwd_dq(h._h, stream_ptr(stream), ptr(q), ptr(k), ptr(v), ptr(do_),
                                  ptr(l), ptr(delta), ptr(dq), _bh(q, n), n, int(causal)))


def run_bwd_dkv(h: Handle, q, k, v, do_, l, delta, dk, dv, n: int, causal: bool,
                stream=None) -> None:
    check(lib().mx230_attn_bwd_dkv(h._h, stream_ptr(stream), ptr(q), ptr(k), ptr(v), ptr(do_),
                                   ptr(l), ptr(delta), ptr(dk), ptr(dv), _bh(q, n), n, int(causal)))


# ---- bf16-resident forms (operands staged once, as a training loop would keep them) ----
def cast_bf16(h: Handle, src, dst, stream=None) -> None:
    check(lib().mx230_cast_bf16(h._h, stream_ptr(stream), ptr(src), ptr(dst), src.numel()))


def run_flash_bf16(h: Handle, qb, kb, vb, o, l, n: int, causal: bool, stream=None) -> None:
    check(lib().mx230_attn_flash_bf16(h._h, stream_ptr(stream), ptr(qb), ptr(kb), ptr(vb), ptr(o),
                                      ptr(l), _bh(o, n), n, int(causal)))


def run_bwd_flash_bf16(h: Handle, qb, kb, vb, dob, l, delta, dq, dk, dv, n: int, causal: bool,
                       stream=None) -> None:
    check(lib().mx230_attn_bwd_flash_bf16(h._h, stream_ptr(stream), ptr(qb), ptr(kb), ptr(vb),
                                          ptr(dob), ptr(l), ptr(delta), ptr(dq), ptr(dk), ptr(dv),
                                          _bh(dq, n), n, int(causal)))
