// Continuous-batching scheduler over batched decode attention: the state machine of
// Engine::run_continuous (03-llm-engine/src/gpu.rs:3800-3915) without the model.  It decides
// which request is admitted when (block reservation for the request's whole life, prompt +
// max_new, so a running sequence can never fail to allocate), builds each step's active batch
// (current tokens, positions, packed block tables -- the arguments of the *_batched attention
// entry points), and retires sequences as they reach their length, returning their blocks to
// the pool.  The caller owns the model: it prefills an admitted prompt through the given block
// table and reports the first generated token, runs one batched decode step per batch and
// reports the next tokens.  Pure host code.
#include <stdint.h>

#include <vector>

#include "common.cuh"

struct mx230_sched {
    mx230_kv_pool *pool = nullptr;
    int block = 0, n_ctx = 0, n_log = 0, max_batch = 0;
    std::vector<int> prompt_len, max_new;
    struct Slot {
        int req;
        std::vector<int> table;  // logical -> physical, padded to n_log with -1
        int need;                // blocks reserved for the whole lifetime
        int pos;                 // position of `cur` (its KV is written by the next step)
        uint32_t cur;
        int target;
    };
    std::vector<Slot> active;
    std::vector<std::vector<uint32_t>> results;
    int next_req = 0;
    // an admission handed out by mx230_sched_admit and not yet confirmed
    int pending_req = -1;
    std::vector<int> pending_table;
    int pending_need = 0;
    long long decode_steps = 0, seq_decodes = 0, admitted = 0;
    bool batch_open = false;
};

namespace {
void release(mx230_sched *s, const std::vector<int> &table, int need) {
    for (int i = 0; i < need; ++i) mx230_kv_pool_decref(s->pool, table[i]);
}
}  // namespace

extern "C" int mx230_sched_create(mx230_sched **out, mx230_kv_pool *pool, int n_ctx, int max_batch,
                                  const int *prompt_len, const int *max_new, int n_requests) {
    MX_REQUIRE(out && pool && n_ctx > 0 && max_batch >= 1 && n_requests >= 0 && (n_requests == 0 || (prompt_len && max_new)),
               MX230_ERR_INVALID_ARG, "sched_create: bad argument");
    int n_blocks = mx230_kv_pool_n_blocks(pool);
    MX_REQUIRE(n_blocks > 0, MX230_ERR_INVALID_ARG, "sched_create: empty pool");   // (before anything is allocated)
    mx230_sched *s = new mx230_sched();
    s->pool = pool;
    s->n_ctx = n_ctx;
    s->max_batch = max_batch;
    s->block = mx230_kv_pool_block_size(pool);
    s->n_log = (n_ctx + s->block - 1) / s->block;
    for (int r = 0; r < n_requests; ++r) {
        if (prompt_len[r] < 1 || max_new[r] < 1 || prompt_len[r] + max_new[r] > n_ctx) {
            delete s;
            return mx230_fail(MX230_ERR_INVALID_ARG, "sched_create: request %d (prompt %d + max_new %d) is empty or exceeds n_ctx %d",
                              r, prompt_len[r], max_new[r], n_ctx);
        }
        s->prompt_len.push_back(prompt_len[r]);
        s->max_new.push_back(max_new[r]);
    }
    s->results.resize(n_requests);
    *out = s;
    return MX230_OK;
}

extern "C" void mx230_sched_destroy(mx230_sched *s) { delete s; }

extern "C" int mx230_sched_n_log(const mx230_sched *s) { return s ? s->n_log : -1; }

// The next request to admit, with the block table its prompt must be prefilled through (n_log
// entries, -1 beyond the reservation); *request = -1 when no slot is free, no request is waiting,
// or the pool cannot hold the next request's whole life yet.
extern "C" int mx230_sched_admit(mx230_sched *s, int *request, int *table_out) {
    MX_REQUIRE(s && request && table_out, MX230_ERR_INVALID_ARG, "sched_admit: null argument");
    MX_REQUIRE(s->pending_req < 0, MX230_ERR_INVALID_ARG, "sched_admit: request %d awaits its first token", s->pending_req);
    MX_REQUIRE(!s->batch_open, MX230_ERR_INVALID_ARG, "sched_admit: a decode step is open");
    *request = -1;
    if ((int)s->active.size() >= s->max_batch || s->next_req >= (int)s->prompt_len.size()) return MX230_OK;
    const int r = s->next_req;
    const int need = (s->prompt_len[r] + s->max_new[r] + s->block - 1) / s->block;
    if (mx230_kv_pool_free_blocks(s->pool) < need) return MX230_OK;  // wait for a retire
    s->pending_table.assign(s->n_log, -1);
    for (int i = 0; i < need; ++i) {
        int rc = mx230_kv_pool_alloc(s->pool, &s->pending_table[i]);
        if (rc != MX230_OK) {
            for (int k = 0; k < i; ++k) mx230_kv_pool_decref(s->pool, s->pending_table[k]);
            return rc;
        }
    }
    s->pending_req = r;
    s->pending_need = need;
    for (int i = 0; i < s->n_log; ++i) table_out[i] = s->pending_table[i];
    *request = r;
    return MX230_OK;
}

// The prompt has been prefilled; `first_token` is its first generated token.
extern "C" int mx230_sched_admitted(mx230_sched *s, int request, uint32_t first_token) {
    MX_REQUIRE(s && request >= 0 && request == s->pending_req, MX230_ERR_INVALID_ARG,
               "sched_admitted: request %d was not handed out", request);
    s->results[request].push_back(first_token);
    ++s->admitted;
    ++s->next_req;
    if (s->max_new[request] == 1) {
        release(s, s->pending_table, s->pending_need);  // done at the prefill token
    } else {
        mx230_sched::Slot sl;
        sl.req = request;
        sl.table = s->pending_table;
        sl.need = s->pending_need;
        sl.pos = s->prompt_len[request];
        sl.cur = first_token;
        sl.target = s->max_new[request];
        s->active.push_back(sl);
    }
    s->pending_req = -1;
    return MX230_OK;
}

// One batched decode step over the active set: current tokens, their positions and the packed
// block tables [n_active][n_log].  *n_active = 0 means every request has been served.
extern "C" int mx230_sched_batch(mx230_sched *s, int *n_active, uint32_t *cur, int *pos, int *tables) {
    MX_REQUIRE(s && n_active && cur && pos && tables, MX230_ERR_INVALID_ARG, "sched_batch: null argument");
    MX_REQUIRE(s->pending_req < 0 && !s->batch_open, MX230_ERR_INVALID_ARG, "sched_batch: called out of order");
    *n_active = (int)s->active.size();
    for (int i = 0; i < *n_active; ++i) {
        cur[i] = s->active[i].cur;
        pos[i] = s->active[i].pos;
        for (int j = 0; j < s->n_log; ++j) tables[(size_t)i * s->n_log + j] = s->active[i].table[j];
    }
    s->batch_open = *n_active > 0;
    return MX230_OK;
}

// The step's next tokens, in batch order: appended to the results; finished sequences retire.
extern "C" int mx230_sched_step_done(mx230_sched *s, const uint32_t *next_tokens) {
    MX_REQUIRE(s && next_tokens && s->batch_open, MX230_ERR_INVALID_ARG, "sched_step_done: no open decode step");
    ++s->decode_steps;
    s->seq_decodes += (long long)s->active.size();
    std::vector<mx230_sched::Slot> keep;
    for (size_t i = 0; i < s->active.size(); ++i) {
        mx230_sched::Slot &sl = s->active[i];
        sl.cur = next_tokens[i];
        sl.pos += 1;
        s->results[sl.req].push_back(next_tokens[i]);
        if ((int)s->results[sl.req].size() >= sl.target) release(s, sl.table, sl.need);
        else keep.push_back(sl);
    }
    s->active.swap(keep);
    s->batch_open = false;
    return MX230_OK;
}

extern "C" int mx230_sched_result(const mx230_sched *s, int request, uint32_t *out, int cap, int *n) {
    MX_REQUIRE(s && n && request >= 0 && request < (int)s->results.size(), MX230_ERR_INVALID_ARG,
               "sched_result: bad request index %d", request);
    *n = (int)s->results[request].size();
    for (int i = 0; i < *n && i < cap && out; ++i) out[i] = s->results[request][i];
    return MX230_OK;
}

// ServeStats, gpu.rs:366-370: which = 0 decode_steps, 1 seq_decodes, 2 admitted
extern "C" long long mx230_sched_stat(const mx230_sched *s, int which) {
    if (!s) return -1;
    return which == 0 ? s->decode_steps : which == 1 ? s->seq_decodes : which == 2 ? s->admitted : -1;
}
