// Host side of paged attention: a pool of fixed-size KV blocks with reference counts and a
// block-granular prefix tree, so that a request whose token prefix is already resident reuses
// those cache blocks instead of recomputing them.  Pure host code (no CUDA calls): the block
// table it maintains is what the paged attention entry points take as `bt`.
//
// Reference semantics: RadixCache (lookup / insert / evict_leaf) and Paging (new, new_pool,
// alloc, evict, audit, incref / decref, phys_row), 03-llm-engine/src/gpu.rs:211-343,372-539,
// and the request protocol of prefill_cached, gpu.rs:2273-2345.  Observable behaviour is kept
// exactly -- which physical block a logical block gets (LIFO free list), what is evicted (the
// least recently used leaf held by the tree alone), which chunks an insert takes over -- so a
// block table produced here is the one the reference engine would upload.
#include <stdint.h>
#include <stdio.h>

#include <map>
#include <string>
#include <vector>

#include "common.cuh"

namespace {

struct TreeNode {
    std::map<std::vector<uint32_t>, int> children;  // chunk tokens (verbatim, never a hash) -> node
    int parent = 0;
    std::vector<uint32_t> key;   // this node's chunk under `parent`
    int block = -1;              // physical block; -1 for the root and for recycled slots
    unsigned long long last_used = 0;
};

}  // namespace

struct mx230_kv_pool {
    int block_size = 0;
    int n_blocks = 0;
    bool prefix_cache = false;
    std::vector<int> table;          // logical block -> physical block (-1 = unmapped)
    std::vector<int> free_list;      // LIFO: claimed from the back
    std::vector<unsigned> refcount;  // per physical block; 0 = free
    std::vector<TreeNode> nodes;     // nodes[0] is the root
    std::vector<int> free_nodes;     // recycled node slots
    unsigned long long tick = 0;     // logical clock of the LRU order
    long long evictions = 0;
    // the request between begin_request and end_request
    int req_log_blocks = 0;
};

namespace {

int pool_fail(int code, const char *fmt, long long a = 0, long long b = 0) {
    return mx230_fail(code, fmt, a, b);
}

void decref(mx230_kv_pool *p, int b) {
    if (--p->refcount[b] == 0) p->free_list.push_back(b);
}

// Longest cached whole-chunk prefix of tokens[0..n): its physical blocks, every matched node touched.
void tree_lookup(mx230_kv_pool *p, const uint32_t *tokens, int n, std::vector<int> &blocks) {
    const unsigned long long t = ++p->tick;
    int node = 0;
    const int bs = p->block_size;
    for (int c = 0; (c + 1) * bs <= n; ++c) {
        std::vector<uint32_t> chunk(tokens + c * bs, tokens + (c + 1) * bs);
        auto it = p->nodes[node].children.find(chunk);
        if (it == p->nodes[node].children.end()) break;
        node = it->second;
        p->nodes[node].last_used = t;
        blocks.push_back(p->nodes[node].block);
    }
}

int tree_new_node(mx230_kv_pool *p, int parent, const std::vector<uint32_t> &chunk, int block,
                  unsigned long long t) {
    TreeNode nn;
    nn.parent = parent;
    nn.key = chunk;
    nn.block = block;
    nn.last_used = t;
    if (!p->free_nodes.empty()) {
        int id = p->free_nodes.back();
        p->free_nodes.pop_back();
        p->nodes[id] = nn;
        return id;
    }
    p->nodes.push_back(nn);
    return (int)p->nodes.size() - 1;
}

// Caches blocks[i] under chunk i (full chunks only); `created` gets the chunk indices the tree took over.
void tree_insert(mx230_kv_pool *p, const uint32_t *tokens, int n, const int *blocks, int n_blk,
                 std::vector<int> &created) {
    const unsigned long long t = ++p->tick;
    int node = 0;
    const int bs = p->block_size;
    for (int c = 0; (c + 1) * bs <= n && c < n_blk; ++c) {
        std::vector<uint32_t> chunk(tokens + c * bs, tokens + (c + 1) * bs);
        auto it = p->nodes[node].children.find(chunk);
        if (it != p->nodes[node].children.end()) {
            node = it->second;
            p->nodes[node].last_used = t;
        } else {
            int id = tree_new_node(p, node, chunk, blocks[c], t);
            p->nodes[node].children[chunk] = id;
            node = id;
            created.push_back(c);
        }
    }
}

// The least recently used leaf whose block only the tree holds; -1 when nothing is reclaimable.
int tree_evict_leaf(mx230_kv_pool *p) {
    int victim = -1;
    for (int i = 1; i < (int)p->nodes.size(); ++i) {
        const TreeNode &nd = p->nodes[i];
        if (nd.block < 0 || !nd.children.empty() || p->refcount[nd.block] != 1) continue;
        if (victim < 0 || nd.last_used < p->nodes[victim].last_used) victim = i;
    }
    if (victim < 0) return -1;
    TreeNode &v = p->nodes[victim];
    const int blk = v.block;
    p->nodes[v.parent].children.erase(v.key);
    v.key.clear();
    v.block = -1;
    p->free_nodes.push_back(victim);
    return blk;
}

bool pool_evict(mx230_kv_pool *p, int *freed) {
    if (freed) *freed = -1;
    if (!p->prefix_cache) return false;
    int blk = tree_evict_leaf(p);
    if (blk < 0) return false;
    decref(p, blk);  // the tree's reference was the last one
    ++p->evictions;
    if (freed) *freed = blk;
    return true;
}

int pool_alloc(mx230_kv_pool *p) {
    if (p->free_list.empty()) pool_evict(p, nullptr);
    if (p->free_list.empty()) return -1;
    int b = p->free_list.back();
    p->free_list.pop_back();
    p->refcount[b] = 1;
    return b;
}

}  // namespace

extern "C" int mx230_kv_pool_create(mx230_kv_pool **out, int n_slots, int block_size, int prefix_cache) {
    MX_REQUIRE(out != nullptr, MX230_ERR_INVALID_ARG, "kv_pool_create: null output");
    MX_REQUIRE(block_size > 0 && n_slots > 0 && n_slots % block_size == 0, MX230_ERR_INVALID_ARG,
               "kv_pool_create: n_slots %d must be a positive multiple of block_size %d", n_slots, block_size);
    mx230_kv_pool *p = new mx230_kv_pool();
    p->block_size = block_size;
    p->n_blocks = n_slots / block_size;
    p->prefix_cache = prefix_cache != 0;
    p->nodes.emplace_back();  // root
    p->free_list.resize(p->n_blocks);
    for (int i = 0; i < p->n_blocks; ++i) p->free_list[i] = i;
    if (p->prefix_cache) {
        p->table.assign(p->n_blocks, -1);
        p->refcount.assign(p->n_blocks, 0);
    } else {
        // one sequence owns every block; claimed from the back, so the map is not the identity
        // and a wrong gather shows at once
        p->table.resize(p->n_blocks);
        for (int i = 0; i < p->n_blocks; ++i) {
            p->table[i] = p->free_list.back();
            p->free_list.pop_back();
        }
        p->refcount.assign(p->n_blocks, 1);
    }
    *out = p;
    return MX230_OK;
}

extern "C" void mx230_kv_pool_destroy(mx230_kv_pool *p) { delete p; }

extern "C" int mx230_kv_pool_n_blocks(const mx230_kv_pool *p) { return p ? p->n_blocks : -1; }
extern "C" int mx230_kv_pool_block_size(const mx230_kv_pool *p) { return p ? p->block_size : -1; }
extern "C" int mx230_kv_pool_free_blocks(const mx230_kv_pool *p) { return p ? (int)p->free_list.size() : -1; }
extern "C" long long mx230_kv_pool_evictions(const mx230_kv_pool *p) { return p ? p->evictions : -1; }
extern "C" int mx230_kv_pool_cached_blocks(const mx230_kv_pool *p) {
    if (!p) return -1;
    int n = 0;
    for (size_t i = 1; i < p->nodes.size(); ++i) n += p->nodes[i].block >= 0;
    return n;
}
extern "C" int mx230_kv_pool_refcount(const mx230_kv_pool *p, int block) {
    if (!p || block < 0 || block >= p->n_blocks) return -1;
    return (int)p->refcount[block];
}

extern "C" int mx230_kv_pool_table(const mx230_kv_pool *p, int *table_out, int n) {
    MX_REQUIRE(p && table_out && n >= 0 && n <= p->n_blocks, MX230_ERR_INVALID_ARG,
               "kv_pool_table: bad argument (n = %d)", n);
    for (int i = 0; i < n; ++i) table_out[i] = p->table[i];
    return MX230_OK;
}

extern "C" int mx230_kv_pool_phys_row(const mx230_kv_pool *p, int t) {
    if (!p || t < 0 || t / p->block_size >= p->n_blocks) return -1;
    int b = p->table[t / p->block_size];
    return b < 0 ? -1 : b * p->block_size + t % p->block_size;
}

extern "C" int mx230_kv_pool_alloc(mx230_kv_pool *p, int *block_out) {
    MX_REQUIRE(p && block_out, MX230_ERR_INVALID_ARG, "kv_pool_alloc: null argument");
    int b = pool_alloc(p);
    *block_out = b;
    if (b < 0) return pool_fail(MX230_ERR_WORKSPACE, "kv_pool_alloc: pool exhausted (every block is pinned by a live request)");
    return MX230_OK;
}

extern "C" int mx230_kv_pool_incref(mx230_kv_pool *p, int block) {
    MX_REQUIRE(p && block >= 0 && block < p->n_blocks && p->refcount[block] > 0, MX230_ERR_INVALID_ARG,
               "kv_pool_incref: block %d is not live", block);
    ++p->refcount[block];
    return MX230_OK;
}

extern "C" int mx230_kv_pool_decref(mx230_kv_pool *p, int block) {
    MX_REQUIRE(p && block >= 0 && block < p->n_blocks && p->refcount[block] > 0, MX230_ERR_INVALID_ARG,
               "kv_pool_decref: block %d is not live", block);
    decref(p, block);
    return MX230_OK;
}

extern "C" int mx230_kv_pool_evict(mx230_kv_pool *p, int *freed_block) {
    MX_REQUIRE(p != nullptr, MX230_ERR_INVALID_ARG, "kv_pool_evict: null pool");
    pool_evict(p, freed_block);
    return MX230_OK;
}

extern "C" int mx230_kv_pool_lookup(mx230_kv_pool *p, const uint32_t *tokens, int n, int *blocks_out,
                                    int cap, int *n_matched) {
    MX_REQUIRE(p && p->prefix_cache && (tokens || n == 0) && n >= 0 && n_matched, MX230_ERR_INVALID_ARG,
               "kv_pool_lookup: bad argument or pool without a prefix tree");
    std::vector<int> blocks;
    tree_lookup(p, tokens, n, blocks);
    *n_matched = (int)blocks.size();
    for (int i = 0; i < (int)blocks.size() && i < cap && blocks_out; ++i) blocks_out[i] = blocks[i];
    return MX230_OK;
}

extern "C" int mx230_kv_pool_insert(mx230_kv_pool *p, const uint32_t *tokens, int n, const int *blocks,
                                    int n_blk, int *created_out, int cap, int *n_created) {
    MX_REQUIRE(p && p->prefix_cache && (tokens || n == 0) && n >= 0 && (blocks || n_blk == 0) && n_created,
               MX230_ERR_INVALID_ARG, "kv_pool_insert: bad argument or pool without a prefix tree");
    std::vector<int> created;
    tree_insert(p, tokens, n, blocks, n_blk, created);
    *n_created = (int)created.size();
    for (int i = 0; i < (int)created.size() && i < cap && created_out; ++i) created_out[i] = created[i];
    return MX230_OK;
}

// Steps 1-2 of a prefix-cached prefill of tokens[0..n): borrow the blocks of the longest cached
// whole-chunk prefix (capped so that the last token is always computed), claim fresh blocks from
// the first divergence on; the table then maps logical blocks 0 .. ceil(n / bs) - 1.
extern "C" int mx230_kv_pool_begin_request(mx230_kv_pool *p, const uint32_t *tokens, int n,
                                           int *reused_tokens) {
    MX_REQUIRE(p && p->prefix_cache && tokens && n >= 1 && reused_tokens, MX230_ERR_INVALID_ARG,
               "kv_pool_begin_request: bad argument or pool without a prefix tree");
    MX_REQUIRE(p->req_log_blocks == 0, MX230_ERR_INVALID_ARG, "kv_pool_begin_request: a request is already open");
    const int bs = p->block_size;
    const int n_log = (n + bs - 1) / bs;
    MX_REQUIRE(n_log <= p->n_blocks, MX230_ERR_WORKSPACE, "kv_pool_begin_request: %d tokens exceed the pool", n);
    std::vector<int> matched;
    tree_lookup(p, tokens, n, matched);
    int m = (int)matched.size();
    if (m > (n - 1) / bs) m = (n - 1) / bs;
    // borrow before allocating: a fresh claim may evict, and the extra reference keeps the prefix
    // this request reads off the victim list
    for (int j = 0; j < m; ++j) {
        p->table[j] = matched[j];
        ++p->refcount[matched[j]];
    }
    for (int j = m; j < n_log; ++j) {
        int b = pool_alloc(p);
        if (b < 0) {  // undo, leave the pool as it was found
            for (int i = 0; i < j; ++i) {
                decref(p, p->table[i]);
                p->table[i] = -1;
            }
            return pool_fail(MX230_ERR_WORKSPACE, "kv_pool_begin_request: pool exhausted, working set exceeds the pool");
        }
        p->table[j] = b;
    }
    p->req_log_blocks = n_log;
    *reused_tokens = m * bs;
    return MX230_OK;
}

// Step 4: the tree takes over the freshly computed full chunks, then the request's borrow of every
// table block is released (a block the tree did not take returns to the pool).
extern "C" int mx230_kv_pool_end_request(mx230_kv_pool *p, const uint32_t *tokens, int n) {
    MX_REQUIRE(p && p->prefix_cache && tokens && n >= 1, MX230_ERR_INVALID_ARG,
               "kv_pool_end_request: bad argument or pool without a prefix tree");
    const int bs = p->block_size;
    const int n_log = (n + bs - 1) / bs, n_full = n / bs;
    MX_REQUIRE(p->req_log_blocks == n_log, MX230_ERR_INVALID_ARG,
               "kv_pool_end_request: no matching begin_request (open blocks %d, this request %d)",
               p->req_log_blocks, n_log);
    std::vector<int> full(p->table.begin(), p->table.begin() + n_full), created;
    tree_insert(p, tokens, n_full * bs, full.data(), n_full, created);
    for (int j : created) ++p->refcount[full[j]];
    for (int j = 0; j < n_log; ++j) decref(p, p->table[j]);
    p->req_log_blocks = 0;
    return MX230_OK;
}

// The open request is given up (its attention step could not be enqueued): every table block loses the
// request's reference and NOTHING is handed to the tree -- the fresh blocks were never written, and a later
// request with the same prefix must not find them.  The reference has no such path: it panics
// (03-llm-engine/src/gpu.rs:2273-2345).
extern "C" int mx230_kv_pool_abort_request(mx230_kv_pool *p) {
    MX_REQUIRE(p && p->prefix_cache, MX230_ERR_INVALID_ARG, "kv_pool_abort_request: bad argument or pool without a prefix tree");
    MX_REQUIRE(p->req_log_blocks > 0, MX230_ERR_INVALID_ARG, "kv_pool_abort_request: no open request");
    for (int j = 0; j < p->req_log_blocks; ++j) {
        decref(p, p->table[j]);
        p->table[j] = -1;
    }
    p->req_log_blocks = 0;
    return MX230_OK;
}

// No block owned by two tree nodes, every tree block referenced, the free list a duplicate-free
// set of unreferenced blocks disjoint from the tree.
extern "C" int mx230_kv_pool_audit(const mx230_kv_pool *p) {
    MX_REQUIRE(p != nullptr, MX230_ERR_INVALID_ARG, "kv_pool_audit: null pool");
    std::vector<int> owner(p->n_blocks, -1);
    for (int i = 1; i < (int)p->nodes.size(); ++i) {
        int b = p->nodes[i].block;
        if (b < 0) continue;
        if (owner[b] >= 0) return pool_fail(MX230_ERR_INVALID_ARG, "kv_pool_audit: block %lld owned by two tree nodes (second: %lld)", b, i);
        owner[b] = i;
        if (p->refcount[b] == 0) return pool_fail(MX230_ERR_INVALID_ARG, "kv_pool_audit: tree block %lld (node %lld) has refcount 0", b, i);
    }
    std::vector<char> seen(p->n_blocks, 0);
    for (int b : p->free_list) {
        if (seen[b]) return pool_fail(MX230_ERR_INVALID_ARG, "kv_pool_audit: block %lld appears twice in the free list", b);
        seen[b] = 1;
        if (p->refcount[b] != 0) return pool_fail(MX230_ERR_INVALID_ARG, "kv_pool_audit: free block %lld has refcount %lld", b, p->refcount[b]);
        if (owner[b] >= 0) return pool_fail(MX230_ERR_INVALID_ARG, "kv_pool_audit: block %lld is both free and tree-owned (node %lld)", b, owner[b]);
    }
    return MX230_OK;
}
