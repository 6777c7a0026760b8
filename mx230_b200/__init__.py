"""mx230_b200: B200-native (sm_100a) attention path of glaucomaa/mx230.

Hand-written CUDA behind a C ABI (include/mx230_attn.h, built in-tree into
libmx230_attn.so) plus thin host mirrors of the reference's call sites:

* flash_attention -- 02-flash-attention's launch wrappers (forward, backward);
* llm_attention   -- 03-llm-engine's per-layer attention step (RoPE, KV write, decode);
* common          -- handle, CUDA-event timer, metrics, xorshift generator.

The CUDA library is mandatory; nothing here falls back to PyTorch or the CPU.
"""
from . import _lib, common  # noqa: F401
from .common import Handle  # noqa: F401

__all__ = ["Handle", "common", "_lib"]
