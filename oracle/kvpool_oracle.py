"""TEST INFRASTRUCTURE ONLY: a plain-Python restatement of the reference's KV block pool and
prefix tree, used by tests/ to check the library's pool operation by operation.

Follows `RadixCache` (03-llm-engine/src/gpu.rs:219-343: lookup :254-271, insert :277-299,
alloc_node :302-316, evict_leaf :324-342), `Paging` (:387-539: new :409-431, new_pool :436-449,
alloc :455-462, evict :467-481, audit :488-525, incref/decref :530-533, phys_row :536-538) and the
request protocol of `prefill_cached` (gpu.rs:2273-2345).  The reference ships no unit test or
fixture for these structures (its gates run the whole model), so this restatement is checked
against hand-worked sequences in tests/test_kvpool_cpu.py: parity unpinned by reference fixtures.
"""
from __future__ import annotations


class _Node:
    def __init__(self, parent, key, block, t):
        self.children = {}      # tuple(chunk tokens) -> node index
        self.parent, self.key, self.block, self.last_used = parent, key, block, t


class PoolOracle:
    def __init__(self, n_slots, block_size=16, prefix_cache=True):
        self.bs = block_size
        self.n_blocks = n_slots // block_size
        self.prefix_cache = prefix_cache
        self.free = list(range(self.n_blocks))
        if prefix_cache:
            self.table = [-1] * self.n_blocks
            self.refcount = [0] * self.n_blocks
        else:
            self.table = [self.free.pop() for _ in range(self.n_blocks)]
            self.refcount = [1] * self.n_blocks
        self.nodes = [_Node(0, (), -1, 0)]
        self.free_nodes = []
        self.tick = 0
        self.evictions = 0

    # ---- tree
    def _chunks(self, tokens):
        for c in range(len(tokens) // self.bs):
            yield c, tuple(int(x) for x in tokens[c * self.bs:(c + 1) * self.bs])

    def lookup(self, tokens):
        self.tick += 1
        node, blocks = 0, []
        for _, chunk in self._chunks(tokens):
            child = self.nodes[node].children.get(chunk)
            if child is None:
                break
            node = child
            self.nodes[child].last_used = self.tick
            blocks.append(self.nodes[child].block)
        return blocks

    def insert(self, tokens, blocks):
        self.tick += 1
        node, created = 0, []
        for i, chunk in self._chunks(tokens):
            if i >= len(blocks):
                break
            child = self.nodes[node].children.get(chunk)
            if child is not None:
                node = child
                self.nodes[child].last_used = self.tick
            else:
                nn = _Node(node, chunk, blocks[i], self.tick)
                if self.free_nodes:
                    idx = self.free_nodes.pop()
                    self.nodes[idx] = nn
                else:
                    self.nodes.append(nn)
                    idx = len(self.nodes) - 1
                self.nodes[node].children[chunk] = idx
                node = idx
                created.append(i)
        return created

    def _evict_leaf(self):
        victim = None
        for i, nd in enumerate(self.nodes):
            if i == 0 or nd.block < 0 or nd.children or self.refcount[nd.block] != 1:
                continue
            if victim is None or nd.last_used < self.nodes[victim].last_used:
                victim = i
        if victim is None:
            return None
        nd = self.nodes[victim]
        blk = nd.block
        del self.nodes[nd.parent].children[nd.key]
        nd.key, nd.block = (), -1
        self.free_nodes.append(victim)
        return blk

    # ---- pool
    def incref(self, b):
        self.refcount[b] += 1

    def decref(self, b):
        self.refcount[b] -= 1
        if self.refcount[b] == 0:
            self.free.append(b)

    def evict(self):
        if not self.prefix_cache:
            return -1
        blk = self._evict_leaf()
        if blk is None:
            return -1
        self.decref(blk)
        self.evictions += 1
        return blk

    def alloc(self):
        if not self.free:
            self.evict()
        if not self.free:
            return None
        b = self.free.pop()
        self.refcount[b] = 1
        return b

    def phys_row(self, t):
        return self.table[t // self.bs] * self.bs + t % self.bs

    def cached_blocks(self):
        return sum(1 for i, nd in enumerate(self.nodes) if i and nd.block >= 0)

    # ---- prefill_cached, steps 1-2 and 4
    def begin_request(self, tokens):
        n, b = len(tokens), self.bs
        n_log = -(-n // b)
        matched = self.lookup(tokens)
        m = min(len(matched), (n - 1) // b)
        for j in range(m):
            self.table[j] = matched[j]
            self.incref(matched[j])
        for j in range(m, n_log):
            blk = self.alloc()
            if blk is None:
                raise MemoryError("pool exhausted")
            self.table[j] = blk
        return m * b

    def end_request(self, tokens):
        n, b = len(tokens), self.bs
        n_log, n_full = -(-n // b), n // b
        full = [self.table[j] for j in range(n_full)]
        for j in self.insert(tokens[:n_full * b], full):
            self.incref(full[j])
        for j in range(n_log):
            self.decref(self.table[j])

    def abort_request(self, tokens):
        """A request that failed after begin_request: its borrow is released, the tree adopts nothing."""
        n_log = -(-len(tokens) // self.bs)
        for j in range(n_log):
            self.decref(self.table[j])
            self.table[j] = -1

    def audit(self):
        owner = {}
        for i, nd in enumerate(self.nodes):
            if i == 0 or nd.block < 0:
                continue
            assert nd.block not in owner, "block owned twice"
            owner[nd.block] = i
            assert self.refcount[nd.block] >= 1, "tree block unreferenced"
        assert len(set(self.free)) == len(self.free), "duplicate in free list"
        for b in self.free:
            assert self.refcount[b] == 0 and b not in owner
