"""The continuous-batching state machine of the library against the Python restatement of the
reference loop, event by event, with a pure-function stand-in for the model (no GPU)."""
import numpy as np
import pytest

from mx230_b200._lib import Mx230Error
from mx230_b200.paging import KvPool
from mx230_b200.serving import Request, Scheduler, run_continuous
from oracle import sched_oracle
from oracle.kvpool_oracle import PoolOracle

VOCAB = 1000


class FakeModel:
    def prefill(self, r, prompt, table):
        return (sum(int(t) for t in prompt) * 31 + 7 * r + int(sum(x for x in table if x >= 0))) % VOCAB

    def decode_batched(self, cur, pos, tables):
        return [(int(c) * 131 + int(p) * 17 + int(t[0]) + 3) % VOCAB for c, p, t in zip(cur, pos, tables)]


def make_requests(seed, n, max_prompt, max_new):
    rng = np.random.default_rng(seed)
    return [Request(rng.integers(0, VOCAB, size=int(rng.integers(1, max_prompt + 1))).tolist(),
                    int(rng.integers(1, max_new + 1))) for _ in range(n)]


@pytest.mark.parametrize("seed,n_blocks,max_batch", [(0, 64, 4), (1, 12, 8), (2, 9, 3), (3, 40, 1)])
def test_schedule_matches_the_restatement(seed, n_blocks, max_batch):
    bs, n_ctx = 16, 128
    reqs = make_requests(seed, 23, 70, 40)
    t_lib, t_ref = [], []
    got, st = run_continuous(FakeModel(), KvPool(n_blocks * bs, bs), n_ctx, reqs, max_batch, t_lib)
    want, sw = sched_oracle.run_continuous(FakeModel(), PoolOracle(n_blocks * bs, bs), n_ctx, reqs, max_batch, t_ref)
    assert t_lib == t_ref
    assert got == want
    assert (st.decode_steps, st.seq_decodes, st.admitted) == (sw["decode_steps"], sw["seq_decodes"], sw["admitted"])
    assert all(len(g) == r.max_new for g, r in zip(got, reqs)) and st.admitted == len(reqs)
    if max_batch > 1 and n_blocks >= 40:
        assert st.seq_decodes / st.decode_steps > 1.5   # the batch actually stays occupied


def test_all_blocks_return_to_the_pool_and_misuse_is_rejected():
    bs, n_ctx = 16, 64
    pool = KvPool(8 * bs, bs)
    reqs = [Request([1, 2, 3], 5), Request([4] * 20, 1), Request([5] * 10, 30)]
    out, st = run_continuous(FakeModel(), pool, n_ctx, reqs, 2)
    assert [len(o) for o in out] == [5, 1, 30] and pool.free_blocks == 8
    pool.audit()
    with pytest.raises(Mx230Error):
        Scheduler(pool, n_ctx, 2, [Request([1] * 60, 10)])   # prompt + max_new > n_ctx
    s = Scheduler(pool, n_ctx, 2, reqs)
    r, table = s.admit()
    assert r == 0 and (table[:1] >= 0).all() and (table[1:] == -1).all()
    with pytest.raises(Mx230Error):
        s.admit()                    # the first admission has not been confirmed
    with pytest.raises(Mx230Error):
        s.step_done([1])             # no decode step is open
    s.admitted(0, 42)
    cur, pos, tables = s.batch()
    assert cur.tolist() == [42] and pos.tolist() == [3]
    s.close()
