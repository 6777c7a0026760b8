// Split-KV decode, exchange + merge over peer memory in one kernel.
//
// Every rank holds the unnormalised (m, l, acc) triples of its own key range, packed as
// [m (rows) | l (rows) | acc (rows x 64)].  The full-context output needs every rank's triples on
// every rank.  Instead of a collective library call followed by a merge kernel, one kernel per rank
//   1. stores its triples into slot `rank` of every rank's exchange region (plain stores to peer
//      memory over NVLink; the own region is written the same way).  Every float travels in an
//      8-byte word {value, step number}; 8-byte stores are single-copy atomic, so a reader that sees
//      the step number of the current step in a word also sees that word's value: no fence and no
//      separate flag, hence one NVLink traversal between "computed" and "usable";
//   2. polls, bounded, the words of its rows in its own region until every source rank's words carry
//      the current step number, and
//   3. merges the `world` triples of its rows (log-sum-exp) into the output.
// A CTA owns a slice of 16 rows from the push to the merge, so CTAs never wait on one another; ranks
// wait on one another only across GPUs (one process and one GPU per rank).
//
// The exchange region is allocated by the library with cudaMalloc so that it can be exported as a
// CUDA IPC handle; the host passes the 64 handle bytes between the processes with whatever transport
// it has.  The region is double-buffered by step parity: a rank can be at most one step ahead of
// another (its step k+1 cannot complete before every rank has pushed step k+1, which every rank does
// only after it has finished merging step k), so slot parity k&1 is never overwritten while a slower
// rank still reads it; the words it holds from step k-2 carry a different step number.  The step
// number lives in device memory (one word per row in the own region, read by the threads that work on
// the row and advanced by the kernel that merges it), not in a kernel argument, so a captured launch
// can be replayed from a CUDA graph.
//
// The push (1.) can also be done by the partial-attention kernel itself (mx230_attn_decode_partial_push,
// decode.cu): the CTA that finishes a (sequence, KV head) group stores the group's triples straight
// into every region, so the transfer starts while other groups are still being computed, and the
// kernel here then only waits and merges (mx230_splitkv_wait_merge); or that CTA also waits for the other
// ranks' triples of its group and merges them, which makes the whole step one kernel
// (mx230_attn_decode_splitkv).
//
// The reference is single-device (03-llm-engine/src/main.rs:401); this has no counterpart there.
#include "common.cuh"

#include <math_constants.h>

#include <cstring>
#include <new>

namespace {

constexpr int MAX_WORLD = MX230_SPLITKV_MAX_WORLD;
constexpr int SLICE_ROWS = 16;
constexpr int THREADS = SLICE_ROWS * 16;   // one float4 of one row per thread

struct ExchangeParams {
    uint2 *region[MAX_WORLD];       // base of every rank's region, as mapped in this process
    const float *local;             // this rank's packed triples (null: nothing to push)
    float *out;                     // [rows][64] (null: push only)
    int *status;
    int rank, world, rows, slices;
    int neutral;                    // push (m, l, acc) = (-inf, 0, 0): a rank whose key range is empty
    size_t part_words;              // rows * 66 words {value, step} per (parity, source rank)
    size_t step_offset_words;       // the own step numbers [rows] start this many words into a region
};

// Bounded polling: `aborted` is CTA-shared, so that once one thread gave up the others leave too.
struct Poller {
    long long t0, limit;
    unsigned polls;
    volatile int *aborted;
    int *status;
    __device__ bool give_up() {
        if ((++polls & 31u) != 0u) return false;
        if (*aborted) return true;
        if (clock64() - t0 > limit) {
            *aborted = 1;
            atomicExch(status, mx::STATUS_WAIT_TIMEOUT);
            return true;
        }
        return false;
    }
};

__global__ void __launch_bounds__(THREADS) splitkv_exchange_merge_kernel(ExchangeParams P) {
    __shared__ int aborted;
    const int slice = blockIdx.x, tid = threadIdx.x;
    const int r0 = slice * SLICE_ROWS;
    const int nr = min(SLICE_ROWS, P.rows - r0);
    const int row = r0 + (tid >> 4), d4 = (tid & 15) * 4;
    const bool has_row = (tid >> 4) < nr;
    // threads 0..nr-1 carry m, threads 16..16+nr-1 carry l
    const int mr = tid & 15;
    const bool has_ml = tid < 32 && mr < nr;
    // one step number per row, advanced once per step by whichever kernel finishes the row's step; all of a
    // launch's rows carry the same number.  Every thread reads its row's before the row's first thread advances it.
    unsigned *steps = (unsigned *)(P.region[P.rank] + P.step_offset_words);
    const unsigned step = *(volatile unsigned *)(steps + (has_row ? row : r0 + (has_ml ? mr : 0))) + 1u;
    const size_t parity_off = (size_t)(step & 1u) * P.world * P.part_words;
    if (tid == 0) aborted = 0;
    const size_t acc_word = 2 * (size_t)P.rows + (size_t)row * 64 + d4;

    // 1. push this rank's rows of the slice into slot `rank` of every region
    if (P.local || P.neutral) {
        const size_t slot = parity_off + (size_t)P.rank * P.part_words;
        const size_t ml_word = (size_t)(tid >> 4) * P.rows + r0 + mr;
        float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
        float ml = tid < 16 ? -CUDART_INF_F : 0.f;
        if (!P.neutral) {
            if (has_row) a = *(const float4 *)(P.local + acc_word);
            if (has_ml) ml = P.local[ml_word];
        }
        for (int i = 0; i < P.world; ++i) {
            const int p = (P.rank + 1 + i) % P.world;   // the own region last; every rank starts at a different peer
            uint2 *dst = P.region[p] + slot;
            if (has_row) {
                mx::st_words2(dst + acc_word, a.x, a.y, step);
                mx::st_words2(dst + acc_word + 2, a.z, a.w, step);
            }
            if (has_ml) mx::st_word(dst + ml_word, ml, step);
        }
    }
    __syncthreads();   // `aborted` is initialised
    if (!P.out) return;   // push only: the step ends with the launch that merges

    // 2. wait for the words of this row from every source rank, 3. merge them
    Poller poll{clock64(), *(const volatile long long *)(P.status + mx::STATUS_LIMIT_WORD), 0u, &aborted, P.status};
    const uint2 *g = P.region[P.rank] + parity_off;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    float ll = 0.f;
    bool ok = true;
    auto wait_word = [&](const uint2 *p) {
        uint2 w = mx::ld_word(p);
        while (w.y != step) {
            if (poll.give_up()) {
                ok = false;
                break;
            }
            w = mx::ld_word(p);
        }
        return w;
    };
    auto wait_words2 = [&](const uint2 *p) {
        uint4 v = mx::ld_words2(p);
        while (v.y != step || v.w != step) {
            if (poll.give_up()) {
                ok = false;
                break;
            }
            v = mx::ld_words2(p);
        }
        return v;
    };
    if (has_row) {
        float mp[MAX_WORLD];
        float mm = -CUDART_INF_F;
#pragma unroll
        for (int p = 0; p < MAX_WORLD; ++p) {
            mp[p] = -CUDART_INF_F;
            if (p < P.world && ok) {
                mp[p] = __uint_as_float(wait_word(g + (size_t)p * P.part_words + row).x);
                mm = fmaxf(mm, mp[p]);
            }
        }
#pragma unroll
        for (int p = 0; p < MAX_WORLD; ++p) {
            if (p < P.world && ok) {
                const uint2 *gp = g + (size_t)p * P.part_words;
                const uint2 wl = wait_word(gp + P.rows + row);
                const uint4 v0 = wait_words2(gp + acc_word);
                const uint4 v1 = wait_words2(gp + acc_word + 2);
                const float w = (mp[p] == -CUDART_INF_F) ? 0.0f : __expf(mp[p] - mm);
                ll += __uint_as_float(wl.x) * w;
                acc.x += __uint_as_float(v0.x) * w, acc.y += __uint_as_float(v0.z) * w;
                acc.z += __uint_as_float(v1.x) * w, acc.w += __uint_as_float(v1.z) * w;
            }
        }
    }
    __syncthreads();
    if (has_row && d4 == 0) steps[row] = step;   // also after a wait that ran out: the ranks stay on the same step count
    if (aborted || !has_row) return;   // after a wait that ran out nothing is written
    const float inv = 1.0f / ll;
    *(float4 *)(P.out + (size_t)row * 64 + d4) = make_float4(acc.x * inv, acc.y * inv, acc.z * inv, acc.w * inv);
}

int upload_table(mx230_splitkv_comm *c) {
    MX_CHECK_CUDA(cudaMemcpy(c->region_dev, c->region, sizeof(c->region), cudaMemcpyHostToDevice));
    return MX230_OK;
}

int launch(mx230_splitkv_comm *c, void *stream, float *out, const float *local, int neutral) {
    for (int p = 0; p < c->world; ++p)
        MX_REQUIRE(c->region[p], MX230_ERR_INVALID_ARG, "splitkv: rank %d is not connected", p);
    mx230_handle *h = c->h;
    mx230_device_guard guard(h->device);
    cudaStream_t st = (cudaStream_t)stream;
    ExchangeParams P;
    for (int p = 0; p < MAX_WORLD; ++p) P.region[p] = c->region[p];
    P.local = local, P.out = out, P.status = h->status_dev;
    P.rank = c->rank, P.world = c->world, P.rows = c->rows, P.slices = c->slices;
    P.neutral = neutral;
    P.part_words = c->part_words, P.step_offset_words = c->step_offset_words;
    MX_LAUNCH(h, st, MX230_K_MERGE, (splitkv_exchange_merge_kernel<<<c->slices, THREADS, 0, st>>>(P)));
    MX_CHECK_CUDA(cudaGetLastError());
    return MX230_OK;
}

}  // namespace

extern "C" int mx230_splitkv_comm_create(mx230_handle *h, int rank, int world, int rows, int head_dim,
                                         mx230_splitkv_comm **out) {
    MX_REQUIRE(h && out, MX230_ERR_INVALID_ARG, "splitkv_comm_create: null argument");
    *out = nullptr;
    MX_REQUIRE(head_dim == 64, MX230_ERR_UNSUPPORTED, "splitkv_comm_create: head_dim must be 64");
    MX_REQUIRE(world >= 1 && world <= MAX_WORLD, MX230_ERR_INVALID_ARG, "splitkv_comm_create: world must be 1..%d",
               MAX_WORLD);
    MX_REQUIRE(rank >= 0 && rank < world, MX230_ERR_INVALID_ARG, "splitkv_comm_create: bad rank %d of %d", rank, world);
    MX_REQUIRE(rows > 0 && rows % 2 == 0 && rows <= (1 << 20), MX230_ERR_INVALID_ARG,
               "splitkv_comm_create: rows must be even and in 2..2^20");
    mx230_splitkv_comm *c = new (std::nothrow) mx230_splitkv_comm();
    MX_REQUIRE(c, MX230_ERR_CUDA, "splitkv_comm_create: out of host memory");
    c->h = h, c->rank = rank, c->world = world, c->rows = rows;
    c->slices = (rows + SLICE_ROWS - 1) / SLICE_ROWS;
    c->part_words = (size_t)rows * 66;
    c->step_offset_words = 2 * (size_t)world * c->part_words;
    c->region_bytes = 8 * c->step_offset_words + 4 * (size_t)rows;
    for (int p = 0; p < MAX_WORLD; ++p) c->region[p] = nullptr, c->imported[p] = false;
    c->region_dev = nullptr, c->local = nullptr;
    mx230_device_guard guard(h->device);
    void *base = nullptr;
    cudaError_t e = cudaMalloc(&base, c->region_bytes);
    if (e == cudaSuccess) e = cudaMemset(base, 0, c->region_bytes);
    if (e == cudaSuccess) e = cudaMalloc((void **)&c->region_dev, sizeof(c->region));
    if (e == cudaSuccess) e = cudaMalloc((void **)&c->local, c->part_words * sizeof(float));
    if (e == cudaSuccess) {
        c->region[rank] = (uint2 *)base;
        e = cudaMemcpy(c->region_dev, c->region, sizeof(c->region), cudaMemcpyHostToDevice);
    }
    if (e != cudaSuccess) {
        if (base) cudaFree(base);
        if (c->region_dev) cudaFree(c->region_dev);
        if (c->local) cudaFree(c->local);
        delete c;
        return mx230_fail(MX230_ERR_CUDA, "splitkv_comm_create: %s", cudaGetErrorString(e));
    }
    *out = c;
    return MX230_OK;
}

extern "C" int mx230_splitkv_comm_export(mx230_splitkv_comm *c, unsigned char *handle) {
    MX_REQUIRE(c && handle, MX230_ERR_INVALID_ARG, "splitkv_comm_export: null argument");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    mx230_device_guard guard(c->h->device);
    cudaIpcMemHandle_t ipc;
    MX_CHECK_CUDA(cudaIpcGetMemHandle(&ipc, c->region[c->rank]));
    memcpy(handle, &ipc, 64);
    return MX230_OK;
}

extern "C" int mx230_splitkv_comm_import(mx230_splitkv_comm *c, int peer, const unsigned char *handle) {
    MX_REQUIRE(c && handle, MX230_ERR_INVALID_ARG, "splitkv_comm_import: null argument");
    MX_REQUIRE(peer >= 0 && peer < c->world && peer != c->rank, MX230_ERR_INVALID_ARG,
               "splitkv_comm_import: peer %d is not another rank of %d", peer, c->world);
    MX_REQUIRE(!c->region[peer], MX230_ERR_INVALID_ARG, "splitkv_comm_import: peer %d is already connected", peer);
    mx230_device_guard guard(c->h->device);
    cudaIpcMemHandle_t ipc;
    memcpy(&ipc, handle, 64);
    void *base = nullptr;
    MX_CHECK_CUDA(cudaIpcOpenMemHandle(&base, ipc, cudaIpcMemLazyEnablePeerAccess));
    c->region[peer] = (uint2 *)base;
    c->imported[peer] = true;
    return upload_table(c);
}

extern "C" int mx230_splitkv_comm_region(mx230_splitkv_comm *c, void **base, size_t *bytes) {
    MX_REQUIRE(c && base, MX230_ERR_INVALID_ARG, "splitkv_comm_region: null argument");
    *base = c->region[c->rank];
    if (bytes) *bytes = c->region_bytes;
    return MX230_OK;
}

extern "C" int mx230_splitkv_comm_attach(mx230_splitkv_comm *c, int peer, void *region) {
    MX_REQUIRE(c && region, MX230_ERR_INVALID_ARG, "splitkv_comm_attach: null argument");
    MX_REQUIRE(peer >= 0 && peer < c->world && peer != c->rank, MX230_ERR_INVALID_ARG,
               "splitkv_comm_attach: peer %d is not another rank of %d", peer, c->world);
    MX_REQUIRE(!c->region[peer], MX230_ERR_INVALID_ARG, "splitkv_comm_attach: peer %d is already connected", peer);
    MX_REQUIRE((((uintptr_t)region) & 15) == 0, MX230_ERR_INVALID_ARG, "splitkv_comm_attach: region must be 16-byte aligned");
    mx230_device_guard guard(c->h->device);
    c->region[peer] = (uint2 *)region;
    return upload_table(c);
}

extern "C" int mx230_splitkv_exchange_merge(mx230_splitkv_comm *c, void *stream, float *out, const float *local) {
    MX_REQUIRE(c && out && local, MX230_ERR_INVALID_ARG, "splitkv_exchange_merge: null argument");
    MX_REQUIRE(((((uintptr_t)out) | ((uintptr_t)local)) & 15) == 0, MX230_ERR_INVALID_ARG,
               "splitkv_exchange_merge: buffers must be 16-byte aligned");
    return launch(c, stream, out, local, 0);
}

extern "C" int mx230_splitkv_wait_merge(mx230_splitkv_comm *c, void *stream, float *out) {
    MX_REQUIRE(c && out, MX230_ERR_INVALID_ARG, "splitkv_wait_merge: null argument");
    MX_REQUIRE((((uintptr_t)out) & 15) == 0, MX230_ERR_INVALID_ARG, "splitkv_wait_merge: out must be 16-byte aligned");
    return launch(c, stream, out, nullptr, 0);
}

// A rank whose key range is empty: the neutral triple is pushed; with `out` the step is also finished here
// (used by mx230_attn_decode_partial_push and mx230_attn_decode_splitkv).
int mx230_splitkv_push_neutral(mx230_splitkv_comm *c, void *stream, float *out) {
    return launch(c, stream, out, nullptr, 1);
}

extern "C" int mx230_splitkv_comm_disconnect(mx230_splitkv_comm *c) {
    MX_REQUIRE(c, MX230_ERR_INVALID_ARG, "splitkv_comm_disconnect: null argument");
    mx230_device_guard guard(c->h->device);
    MX_CHECK_CUDA(cudaDeviceSynchronize());
    for (int p = 0; p < c->world; ++p) {
        if (p == c->rank) continue;
        if (c->imported[p] && c->region[p]) cudaIpcCloseMemHandle(c->region[p]);
        c->region[p] = nullptr, c->imported[p] = false;
    }
    return MX230_OK;
}

extern "C" void mx230_splitkv_comm_destroy(mx230_splitkv_comm *c) {
    if (!c) return;
    mx230_splitkv_comm_disconnect(c);
    mx230_device_guard guard(c->h->device);
    if (c->region[c->rank]) cudaFree(c->region[c->rank]);
    if (c->region_dev) cudaFree(c->region_dev);
    if (c->local) cudaFree(c->local);
    delete c;
}
