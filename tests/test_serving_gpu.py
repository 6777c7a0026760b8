"""Continuous batching over the real batched decode attention: a stand-in model whose only real
layer is the attention step (token embedding -> RoPE -> KV write -> attention -> fixed projection
-> argmax).  Serving a queue with up to four sequences decoding together gives, token for token,
what serving the requests one at a time gives (the reference's gate for its scheduler,
03-llm-engine/src/gpu.rs:3811-3813), and the batch stays occupied."""
import numpy as np
import pytest
import torch

import oracle
from mx230_b200 import _lib, llm_attention as la
from mx230_b200.paging import KvPool
from mx230_b200.serving import Request, run_continuous

pytestmark = pytest.mark.gpu

NH, NKV, THETA, BS, VOCAB, N_CTX = 8, 2, 1e6, 16, 61, 160
QD, KVD = NH * 64, NKV * 64
STRIDE = QD + 2 * KVD


class AttentionOnlyModel:
    def __init__(self, handle, n_slots, quant):
        self.h = handle
        self.cache = la.KvCache(n_slots, NKV, 64, quant)
        self.emb = torch.from_numpy(oracle.normal((VOCAB, STRIDE), 500, 0)).cuda()
        self.proj = oracle.normal((QD, VOCAB), 501, 0).astype(np.float64)
        self.n_log = -(-N_CTX // BS)

    def _next(self, out_rows):
        # projection and argmax on the host in float64: independent of the batch composition
        return np.argmax(out_rows.double().cpu().numpy() @ self.proj, axis=1)

    def prefill(self, r, prompt, table):
        n = len(prompt)
        rows = self.emb[torch.tensor(prompt, device="cuda", dtype=torch.long)].contiguous()
        out = torch.zeros(n, QD, device="cuda")
        pg = la.Paging(torch.from_numpy(np.ascontiguousarray(table)).cuda(), BS)
        la.prefill_step(self.h, out, rows, self.cache, 0, n, NH, NKV, 64, THETA, STRIDE, QD, pg)
        return int(self._next(out[-1:])[0])

    def decode_batched(self, cur, pos, tables):
        n = len(cur)
        rows = self.emb[torch.from_numpy(cur.astype(np.int64)).cuda()].contiguous()
        out = torch.zeros(n, QD, device="cuda")
        pg = la.Paging(torch.from_numpy(np.ascontiguousarray(tables)).cuda(), BS)
        la.batched_step(self.h, out, rows, self.cache, torch.from_numpy(pos).cuda(), n, NH, NKV, 64, THETA,
                        pg, STRIDE, QD)
        return self._next(out)


@pytest.mark.parametrize("quant", [False, True])
def test_continuous_batching_equals_serving_one_by_one(handle, quant):
    rng = np.random.default_rng(11)
    reqs = [Request(rng.integers(0, VOCAB, size=int(rng.integers(3, 60))).tolist(), int(rng.integers(1, 40)))
            for _ in range(9)]
    n_slots = 40 * BS
    # a fixed number of keys per decode CTA makes the key split, and with it the summation order,
    # independent of how many sequences share the launch
    handle.set_option(_lib.OPT_DECODE_CHUNK, 256)
    try:
        together, st = run_continuous(AttentionOnlyModel(handle, n_slots, quant), KvPool(n_slots, BS), N_CTX, reqs, 4)
        alone, st1 = run_continuous(AttentionOnlyModel(handle, n_slots, quant), KvPool(n_slots, BS), N_CTX, reqs, 1)
    finally:
        handle.set_option(_lib.OPT_DECODE_CHUNK, 0)
    handle.check_status()
    assert together == alone
    assert [len(t) for t in together] == [r.max_new for r in reqs]
    assert st.admitted == st1.admitted == len(reqs)
    assert st.seq_decodes == st1.seq_decodes and st.decode_steps < st1.decode_steps
    assert st.seq_decodes / st.decode_steps > 2.0
