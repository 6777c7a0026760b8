"""TEST INFRASTRUCTURE ONLY: plain-Python restatement of the reference's continuous-batching
loop, `Engine::run_continuous` (03-llm-engine/src/gpu.rs:3821-3915), over the pool restatement
of oracle/kvpool_oracle.py and a caller-supplied model (same protocol as mx230_b200.serving).
The reference has no fixture for the schedule itself (its gate compares generated tokens of the
whole model): parity unpinned by reference fixtures; tests compare event traces."""
from __future__ import annotations


def run_continuous(model, pool, n_ctx, requests, max_batch, trace=None):
    b = pool.bs
    n_log = -(-n_ctx // b)
    results = [[] for _ in requests]
    stats = dict(decode_steps=0, seq_decodes=0, admitted=0)
    next_req, active = 0, []
    while True:
        while len(active) < max_batch and next_req < len(requests):
            r = next_req
            plen, target = len(requests[r].prompt), requests[r].max_new
            assert plen >= 1 and target >= 1 and plen + target <= n_ctx
            need = -(-(plen + target) // b)
            if len(pool.free) < need:
                break
            table = [-1] * n_log
            for i in range(need):
                table[i] = pool.alloc()
            first = int(model.prefill(r, requests[r].prompt, list(table)))
            if trace is not None:
                trace.append(("admit", r, list(table), first))
            results[r].append(first)
            stats["admitted"] += 1
            next_req += 1
            if target == 1:
                for blk in table[:need]:
                    pool.decref(blk)
            else:
                active.append(dict(req=r, table=table, need=need, pos=plen, cur=first, target=target))
        if not active:
            break
        cur = [s["cur"] for s in active]
        pos = [s["pos"] for s in active]
        tables = [list(s["table"]) for s in active]
        nxt = [int(x) for x in model.decode_batched(cur, pos, tables)]
        if trace is not None:
            trace.append(("step", cur, pos, tables, nxt))
        stats["decode_steps"] += 1
        stats["seq_decodes"] += len(active)
        keep = []
        for i, s in enumerate(active):
            s["cur"] = nxt[i]
            s["pos"] += 1
            results[s["req"]].append(nxt[i])
            if len(results[s["req"]]) >= s["target"]:
                for blk in s["table"][:s["need"]]:
                    pool.decref(blk)
            else:
                keep.append(s)
        active = keep
    return results, stats
