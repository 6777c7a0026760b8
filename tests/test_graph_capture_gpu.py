"""The `_dyn` decode step (RoPE -> KV write -> attention, position read from device memory) is
captured once into a CUDA graph and replayed for successive tokens, as the reference engine does
(capture_decode_graph, 03-llm-engine/src/gpu.rs:4024-4054): nothing on the launch path allocates,
synchronises or depends on a host-side position."""
import numpy as np
import pytest
import torch

import oracle
from mx230_b200 import llm_attention as la
from tests.conftest import assert_close

pytestmark = pytest.mark.gpu

TOL = dict(max_abs=2e-3, mean_rel=5e-3)  # device RoPE (precise powf/sincosf) vs libm may flip an int8 code


@pytest.mark.parametrize("quant", [True, False])
def test_decode_step_dyn_replays_from_a_cuda_graph(handle, quant):
    nh, nkv, ctx, theta = 14, 2, 48, 1e6
    qd, kvd = nh * 64, nkv * 64
    stride = qd + 2 * kvd
    rows = oracle.normal((ctx, stride), 300, 0)
    c = la.KvCache(ctx, nkv, 64, quant)
    qkv = torch.zeros(stride, device="cuda")
    out = torch.zeros(qd, device="cuda")
    pos = torch.zeros(1, dtype=torch.int32, device="cuda")
    # oracle-side caches, filled position by position exactly like the device step
    kc = np.zeros((ctx, kvd), np.float32)
    vc = np.zeros_like(kc)
    q8 = oracle.Q8Cache(ctx, nkv)

    side = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    # warm-up outside capture (first-launch function attributes), on the capture stream
    with torch.cuda.stream(side):
        qkv.copy_(torch.from_numpy(rows[0]))
        la.decode_step_dyn(handle, out, qkv, c, pos, nh, nkv, 64, theta)
    side.synchronize()
    with torch.cuda.graph(graph, stream=side):
        la.decode_step_dyn(handle, out, qkv, c, pos, nh, nkv, 64, theta)
    for t in range(ctx):
        row = rows[t].copy()
        qkv.copy_(torch.from_numpy(row))
        pos.fill_(t)
        torch.cuda.synchronize()
        graph.replay()
        torch.cuda.synchronize()
        row = oracle.rope_qkv_row(row, t, nh, nkv, 64, theta)
        if quant:
            oracle.quantize_kv_row(q8, row, t, qd)
            want = oracle.gqa_decode_q8(row, q8, t, nh, 1)
        else:
            oracle.copy_kv_row(kc, vc, row, t, qd, kvd)
            want = oracle.gqa_decode_f32(row, kc, vc, t, nh, nkv)
        if t in (0, 1, 17, ctx - 1):
            assert_close(out.cpu().numpy(), want, f"graph replay t={t}", **TOL)
    handle.check_status()
