"""The KV block pool and prefix tree (host code of the library, no GPU): hand-worked sequences
pin both the library and the Python restatement; random request streams then compare the two
operation by operation (tables, reference counts, free and cached block counts, evictions)."""
import numpy as np
import pytest

from mx230_b200._lib import ERR_INVALID_ARG, ERR_WORKSPACE, Mx230Error
from mx230_b200.paging import KvPool
from oracle.kvpool_oracle import PoolOracle


def test_single_sequence_table_is_reversed():
    p = KvPool(8 * 16, 16, prefix_cache=False)
    assert p.table().tolist() == [7, 6, 5, 4, 3, 2, 1, 0]
    assert p.free_blocks == 0 and all(p.refcount(b) == 1 for b in range(8))
    assert p.phys_row(0) == 7 * 16 and p.phys_row(17) == 6 * 16 + 1 and p.phys_row(127) == 15
    o = PoolOracle(8 * 16, 16, prefix_cache=False)
    assert o.table == p.table().tolist() and o.phys_row(37) == p.phys_row(37)
    with pytest.raises(Mx230Error):
        p.lookup([1] * 16)          # no prefix tree in this mode
    p.audit()


def test_hand_worked_prefix_reuse_and_eviction():
    bs = 4
    p = KvPool(6 * bs, bs)          # 6 blocks
    a = [1, 2, 3, 4, 5, 6, 7, 8, 9, 10]          # 2 full chunks + 2 tokens
    assert p.begin_request(a) == 0
    assert p.table(3).tolist() == [5, 4, 3]      # LIFO free list
    p.end_request(a)
    # the tree keeps the two full chunks, the partial block went back to the pool
    assert p.cached_blocks == 2 and p.free_blocks == 4
    assert [p.refcount(b) for b in (5, 4, 3)] == [1, 1, 0]
    assert p.lookup(a) == [5, 4]
    # same prefix, different tail: both chunks reused, one fresh block
    b = [1, 2, 3, 4, 5, 6, 7, 8, 11, 12, 13]
    assert p.begin_request(b) == 8
    assert p.table(3).tolist() == [5, 4, 3]
    assert p.refcount(5) == 2 and p.refcount(4) == 2
    p.end_request(b)
    assert p.refcount(5) == 1 and p.cached_blocks == 2
    # a prompt that is exactly the cached prefix: the last token must still be computed,
    # so only the first chunk is reused
    c = [1, 2, 3, 4, 5, 6, 7, 8]
    assert p.begin_request(c) == 4
    t = p.table(2).tolist()
    assert t[0] == 5 and t[1] != 4
    p.end_request(c)
    assert p.cached_blocks == 2 and p.free_blocks == 4  # chunk 1 was already held: the duplicate block is released
    # fill the pool with unrelated prompts until the least recently used leaf is evicted
    for k in range(3):
        d = [100 + 10 * k + i for i in range(8)]
        p.begin_request(d)
        p.end_request(d)
    assert p.evictions >= 1 and p.cached_blocks + p.free_blocks == 6
    p.audit()


def test_pool_exhaustion_is_an_error_and_leaves_the_pool_intact():
    p = KvPool(2 * 4, 4)
    with pytest.raises(Mx230Error) as e:
        p.begin_request(list(range(9)))   # 3 blocks needed, 2 exist
    assert e.value.code == ERR_WORKSPACE
    assert p.free_blocks == 2
    p.audit()
    p.begin_request([1, 2, 3, 4, 5])
    with pytest.raises(Mx230Error) as e:
        p.begin_request([9])              # a request is already open
    assert e.value.code == ERR_INVALID_ARG
    p.end_request([1, 2, 3, 4, 5])
    p.audit()


@pytest.mark.parametrize("seed,n_blocks,bs", [(0, 12, 4), (1, 7, 4), (2, 40, 16), (3, 5, 2)])
def test_random_request_streams_match_the_restatement(seed, n_blocks, bs):
    rng = np.random.default_rng(seed)
    p, o = KvPool(n_blocks * bs, bs), PoolOracle(n_blocks * bs, bs)
    stems = [rng.integers(0, 50, size=rng.integers(bs, 4 * bs)).tolist() for _ in range(4)]
    for step in range(300):
        stem = stems[rng.integers(0, len(stems))]
        cut = rng.integers(1, len(stem) + 1)
        tail = rng.integers(0, 50, size=rng.integers(0, 2 * bs)).tolist()
        toks = (stem[:cut] + tail)[: (n_blocks - 1) * bs]
        if not toks:
            continue
        try:
            ko = o.begin_request(toks)
        except MemoryError:
            with pytest.raises(Mx230Error):
                p.begin_request(toks)
            break
        kp = p.begin_request(toks)
        n_log = -(-len(toks) // bs)
        assert kp == ko
        assert p.table(n_log).tolist() == o.table[:n_log], f"step {step}"
        assert [p.refcount(b) for b in range(n_blocks)] == o.refcount
        p.end_request(toks)
        o.end_request(toks)
        assert [p.refcount(b) for b in range(n_blocks)] == o.refcount
        assert (p.free_blocks, p.cached_blocks, p.evictions) == (len(o.free), o.cached_blocks(), o.evictions)
        if step % 25 == 0:
            p.audit()
            o.audit()
    p.audit()
    o.audit()


def test_primitives_alloc_insert_lookup_evict():
    bs = 2
    p, o = KvPool(4 * bs, bs), PoolOracle(4 * bs, bs)
    blocks = [p.alloc() for _ in range(3)]
    assert blocks == [o.alloc() for _ in range(3)] == [3, 2, 1]
    toks = [7, 7, 8, 8, 9, 9]
    assert p.insert(toks, blocks) == o.insert(toks, blocks) == [0, 1, 2]
    assert p.insert(toks[:4], [0, 0]) == o.insert(toks[:4], [0, 0]) == []   # already cached: nothing taken
    assert p.lookup(toks + [1]) == o.lookup(toks + [1]) == [3, 2, 1]
    assert p.lookup([7, 7, 0, 0]) == o.lookup([7, 7, 0, 0]) == [3]
    # leaves only: the deepest chunk goes first, then its parent becomes a leaf
    assert p.evict() == o.evict() == 1
    assert p.evict() == o.evict() == 2
    p.incref(3)                         # borrowed by a live request: not reclaimable
    o.incref(3)
    assert p.evict() == o.evict() == -1
    p.decref(3)
    o.decref(3)
    assert p.evict() == o.evict() == 3
    assert p.free_blocks == 4 and p.cached_blocks == 0 and p.evictions == 3
    p.audit()


def test_aborted_request_leaves_no_trace_in_the_tree():
    """A request whose attention step fails after begin_request is aborted: the fresh blocks were never
    written, so the tree must not adopt them and a later request with the same prefix must compute it."""
    bs = 4
    p = KvPool(6 * bs, bs)
    o = PoolOracle(6 * bs, bs)
    a = [1, 2, 3, 4, 5, 6, 7, 8, 9]
    assert p.begin_request(a) == 0 and o.begin_request(a) == 0
    p.abort_request()
    o.abort_request(a)
    p.audit()
    o.audit()
    assert p.cached_blocks == 0 and p.free_blocks == 6 and p.lookup(a) == [] and o.lookup(a) == []
    assert all(p.refcount(b) == 0 for b in range(6))
    with pytest.raises(Mx230Error):
        p.abort_request()                      # nothing open any more
    # the same prompt again: nothing is reused; after a successful end the prefix is there
    assert p.begin_request(a) == 0
    p.end_request(a)
    assert p.lookup(a) == p.table(2).tolist() and p.cached_blocks == 2
    # an abort on top of a borrowed prefix releases the borrow but keeps the tree's own reference
    b = [1, 2, 3, 4, 5, 6, 7, 8, 50, 51]
    assert p.begin_request(b) == 8
    held = p.table(2).tolist()
    assert [p.refcount(x) for x in held] == [2, 2]
    p.abort_request()
    assert [p.refcount(x) for x in held] == [1, 1] and p.cached_blocks == 2 and p.free_blocks == 4
    p.audit()


def test_prefill_cached_aborts_when_the_attention_step_raises():
    """paging.prefill_cached: a failure between begin_request and the enqueue of the attention step must not
    let the tree adopt the request's blocks (host logic only: the step is made to fail before any launch)."""
    from mx230_b200 import paging

    bs = 4
    p = KvPool(6 * bs, bs)
    tokens = list(range(1, 10))

    class Boom(RuntimeError):
        pass

    def qkv_rows(k):
        raise Boom("suffix rows unavailable")

    class FakeTable:
        shape = (8,)

        def __getitem__(self, sl):
            return self

        def copy_(self, src, non_blocking=False):
            return self

    with pytest.raises(Boom):
        paging.prefill_cached(None, p, None, tokens, qkv_rows, None, 2, 1, 1e4, FakeTable())
    p.audit()
    assert p.cached_blocks == 0 and p.free_blocks == 6 and p.lookup(tokens) == []
    assert p.begin_request(tokens) == 0        # the pool accepts a new request: nothing was left open
    p.end_request(tokens)
