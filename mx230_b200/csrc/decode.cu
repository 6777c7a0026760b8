// Per-layer attention step, part 2: decode attention (one query row per sequence)
// over the fp32 or int8 KV cache, grouped-query aware, split over the key axis.
//
// Reference semantics: attn_decode_impl / attn_decode_q8_impl and their wrappers,
// 03-llm-engine/kernels/llm.cu:1246-1487 -- one block per QUERY head, three phases
// (scores+max, exp+sum, PV), whole score row in shared s[2048].
//
// This design: one CTA per (key split, kv head, sequence) serves ALL query heads of
// the kv head's group, so every cache byte leaves HBM once.  Inside the CTA every warp
// streams its own key sub-range through a private cp.async shared-memory ring (memory
// parallelism independent of register pressure, no block barrier in the loop) and keeps
// a private online-softmax state, so the context length is unbounded; the warps are merged
// by log-sum-exp at the end.  Split CTAs leave (m, l, acc) partials in the workspace; the
// last CTA to arrive for a (sequence, kv head) merges them.  Three kernels share this
// skeleton: fp32 cache on CUDA cores; int8 cache on CUDA cores (exact score mode); int8
// cache with the GQA group on warp-level tensor-core tiles (reference score mode).
#include <math_constants.h>

#include <mutex>

#include "common.cuh"

namespace {

constexpr int DEC_THREADS = 128;

struct DecodeParams {
    float *out;               // [n_seq][out_stride]; head h at h*64 (null in partial mode)
    int out_stride;
    float *fin_m, *fin_l, *fin_acc;  // partial mode outputs [n_seq][n_head](x64), else null
    float *ws_m, *ws_l, *ws_acc;     // split partials [n_seq][n_head][n_splits](x64)
    unsigned *counters;
    const float *qkv;
    int qkv_stride;
    const float *kcache, *vcache;    // fp32 cache
    const int8_t *kq, *vq;           // int8 cache
    const float *ks, *vs, *kb, *vb;
    // key range of sequence s: [t0, t1) when range_mode, else [0, pos(s)+1)
    int range_mode, t0, t1;
    int pos_kind;  // 0 host scalar `pos`, 1 *pos_dev, 2 pos_dev[s]
    int pos;
    const int *pos_dev;
    const int *tables;  // block tables; kind 2: row s of n_log entries; null = linear
    int bs, n_log;
    long long seq_rows;  // linear batched slabs: sequence s starts at row s*seq_rows
    int max_keys;        // capacity of one sequence (slab rows, or table entries x block) when positions come from the device; 0 = unknown
    int n_head, n_kv_head, group, head_groups;
    int score_mode;
    // partial mode with a push: the finished triples also go, as {value, step} words, into slot `push_rank` of every
    // rank's split-KV exchange region (table of `push_world` region bases in device memory)
    uint2 *const *push_regions;
    unsigned *push_steps;        // [rows] the number of the last finished exchange step of every row (own region)
    float *push_out;             // [rows][64]: the finishing CTA also waits for the other ranks' triples and merges; else null
    int *push_status;            // where a wait that ran out is recorded
    size_t push_part_words;      // rows * 66
    int push_rank, push_world, push_rows;
};

__device__ __forceinline__ float warp_max_f(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
    return v;
}
__device__ __forceinline__ float warp_sum_f(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
    return v;
}

__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src, int src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src),
                 "r"(src_bytes)
                 : "memory");
}
__device__ __forceinline__ void cp_async4(uint32_t dst, const void *src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

__device__ __forceinline__ size_t cache_row(const DecodeParams &P, const int *table, long long base,
                                            int t) {
    if (table) return (size_t)(table[t / P.bs] * P.bs + t % P.bs);
    return (size_t)(base + t);
}

__device__ __forceinline__ void key_range(const DecodeParams &P, int s, int &kbeg, int &kend) {
    if (P.range_mode) {
        kbeg = P.t0;
        kend = P.t1;
    } else {
        int p = P.pos_kind == 0 ? P.pos : (P.pos_kind == 1 ? *P.pos_dev : P.pos_dev[s]);
        // a position read from device memory cannot be validated by the host: where the capacity of a sequence is
        // known, a wild value (a caller's ordering bug) is kept inside it rather than turned into wild addresses
        if (P.pos_kind == 2 && P.max_keys > 0) p = min(max(p, 0), P.max_keys - 1);
        kbeg = 0;
        kend = p + 1;
    }
}

// Split c of n covers a 32-aligned slice of [kbeg, kend).
__device__ __forceinline__ void split_range(int kbeg, int kend, int c, int n, int &a, int &b) {
    int len = kend - kbeg;
    int per = (len + n - 1) / n;
    per = (per + 31) & ~31;
    a = kbeg + c * per;
    b = min(kend, a + per);
    if (a > kend) a = kend;
    if (b < a) b = a;
}

// Final or partial write of one (sequence, kv head) group from merged values held
// by the first threads of the CTA.
template <int G>
__device__ void merge_and_store(const DecodeParams &P, int s, int head0, int gc, int n_splits,
                                int n_threads = DEC_THREADS) {
    // thread t handles (g = t / 16, 4 consecutive dims at (t % 16) * 4) and loops g
    for (int g = threadIdx.x / 16; g < gc; g += n_threads / 16) {
        int d4 = (threadIdx.x % 16) * 4;
        int h = head0 + g;
        size_t pbase = ((size_t)s * P.n_head + h) * n_splits;
        float mm = -CUDART_INF_F;
        for (int c = 0; c < n_splits; ++c) mm = fmaxf(mm, P.ws_m[pbase + c]);
        float ll = 0.0f;
        float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int c = 0; c < n_splits; ++c) {
            float mc = P.ws_m[pbase + c];
            float w = (mc == -CUDART_INF_F) ? 0.0f : __expf(mc - mm);
            ll += P.ws_l[pbase + c] * w;
            float4 v = *(const float4 *)(P.ws_acc + (pbase + c) * 64 + d4);
            a.x += v.x * w, a.y += v.y * w, a.z += v.z * w, a.w += v.w * w;
        }
        if (P.fin_acc) {
            size_t o = (size_t)s * P.n_head + h;
            *(float4 *)(P.fin_acc + o * 64 + d4) = a;
            if (d4 == 0) {
                P.fin_m[o] = mm;
                P.fin_l[o] = ll;
            }
            if (P.push_regions) {
                // the row's step number: read by the row's 16 threads here, advanced (by the kernel that merges the row)
                // only after a CTA-wide barrier
                const unsigned step = *(const volatile unsigned *)(P.push_steps + o) + 1u;
                const size_t parity = (size_t)(step & 1u) * P.push_world * P.push_part_words;
                const size_t acc_word = 2 * (size_t)P.push_rows + o * 64 + d4;
                // every other rank first, starting at a different peer on every rank; the own region last, and not
                // at all when this CTA merges the row itself (it has the own triple in registers)
                for (int i = 0; i < P.push_world - (P.push_out ? 1 : 0); ++i) {
                    uint2 *dst = P.push_regions[(P.push_rank + 1 + i) % P.push_world] + parity + P.push_rank * P.push_part_words;
                    mx::st_words2(dst + acc_word, a.x, a.y, step);
                    mx::st_words2(dst + acc_word + 2, a.z, a.w, step);
                    if (d4 == 0) mx::st_word(dst + o, mm, step);
                    if (d4 == 4) mx::st_word(dst + P.push_rows + o, ll, step);
                }
                if (P.push_out) {
                    // wait (bounded) for the other ranks' triples of this row and merge all of them in rank order
                    const uint2 *gsrc = P.push_regions[P.push_rank] + parity;
                    const long long t_start = clock64();
                    const long long limit = *(const volatile long long *)(P.push_status + mx::STATUS_LIMIT_WORD);
                    unsigned polls = 0;
                    bool ok = true;
                    auto give_up = [&]() {
                        if ((++polls & 31u) != 0u) return false;
                        if (clock64() - t_start > limit) {
                            atomicExch(P.push_status, mx::STATUS_WAIT_TIMEOUT);
                            return true;
                        }
                        return false;
                    };
                    auto wait_word = [&](const uint2 *p) {
                        uint2 w = mx::ld_word(p);
                        while (w.y != step) {
                            if (give_up()) {
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
                            if (give_up()) {
                                ok = false;
                                break;
                            }
                            v = mx::ld_words2(p);
                        }
                        return v;
                    };
                    float mp[MX230_SPLITKV_MAX_WORLD];
                    float gm = -CUDART_INF_F;
#pragma unroll
                    for (int p = 0; p < MX230_SPLITKV_MAX_WORLD; ++p) {
                        mp[p] = -CUDART_INF_F;
                        if (p < P.push_world && ok) {
                            mp[p] = p == P.push_rank ? mm : __uint_as_float(wait_word(gsrc + (size_t)p * P.push_part_words + o).x);
                            gm = fmaxf(gm, mp[p]);
                        }
                    }
                    float gl = 0.0f;
                    float4 ga = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                    for (int p = 0; p < MX230_SPLITKV_MAX_WORLD; ++p) {
                        if (p < P.push_world && ok) {
                            float lp = ll;
                            float4 v = a;
                            if (p != P.push_rank) {
                                const uint2 *gp = gsrc + (size_t)p * P.push_part_words;
                                lp = __uint_as_float(wait_word(gp + P.push_rows + o).x);
                                const uint4 v0 = wait_words2(gp + acc_word);
                                const uint4 v1 = wait_words2(gp + acc_word + 2);
                                v = make_float4(__uint_as_float(v0.x), __uint_as_float(v0.z), __uint_as_float(v1.x),
                                                __uint_as_float(v1.z));
                            }
                            const float w = (mp[p] == -CUDART_INF_F) ? 0.0f : __expf(mp[p] - gm);
                            gl += lp * w;
                            ga.x += v.x * w, ga.y += v.y * w, ga.z += v.z * w, ga.w += v.w * w;
                        }
                    }
                    if (ok) {   // after a wait that ran out the row is not written
                        const float inv = 1.0f / gl;
                        *(float4 *)(P.push_out + o * 64 + d4) = make_float4(ga.x * inv, ga.y * inv, ga.z * inv, ga.w * inv);
                    }
                }
            }
        } else {
            float inv = 1.0f / ll;
            *(float4 *)(P.out + (size_t)s * P.out_stride + h * 64 + d4) =
                make_float4(a.x * inv, a.y * inv, a.z * inv, a.w * inv);
        }
    }
    if (P.push_out) {
        // this CTA finished the step of its rows: their step numbers move on (also after a wait that ran out, so
        // that the ranks stay on the same step count)
        __syncthreads();
        if (threadIdx.x < gc) P.push_steps[(size_t)s * P.n_head + head0 + threadIdx.x] += 1u;
    }
}

// ---------------------------------------------------------------------------
// int8 cache: warp-autonomous streaming
//
// A CTA of Q8_WARPS warps owns one (key split, kv head, sequence); its key range is cut
// into one contiguous sub-range per warp.  Each warp streams its sub-range in tiles of 32
// keys through its own two-stage cp.async ring (K codes, V codes and the four side-array
// slices of the tile) and keeps a private online-softmax state, so the main loop contains
// no block-wide barrier: 16 independent warps per SM hide each other's latencies.
//   scores:  lane = key; the 64-byte K row against the G query heads (dp4a, or fp32 FMA in
//            the exact score mode); running max per head raised lazily (only when a score
//            exceeds it by more than RAISE, found with one vote per head and tile);
//   weights: w = exp(s - m) * vs through a per-warp shared buffer;
//   values:  lane = (key lane, 8-byte slice); int8 -> fp32 with byte permutes, packed FMAs.
// At the end the warps' (m, l, acc) are merged by log-sum-exp in shared memory.
// ---------------------------------------------------------------------------
constexpr int Q8_WARPS = 8;
constexpr int Q8_THREADS = Q8_WARPS * 32;
constexpr int WT_KEYS = 32;                         // keys per warp tile
constexpr int WT_STAGE = 2 * WT_KEYS * 64 + 4 * WT_KEYS * 4;  // K + V codes + ks,kb,vs,vb = 4608 B
constexpr int WT_STAGES = 2;
constexpr float RAISE = 8.0f;                       // natural-log units

template <int G>
struct Q8Smem {
    static constexpr int GP = (G + 3) & ~3;         // heads padded to a multiple of 4 floats
    static constexpr int Q_BYTES = G * 64 * 4 + G * 16 * 4 + 2 * G * 4 + 64;
    static constexpr int WBUF = WT_KEYS * GP * 4;   // per-warp weight exchange
    static constexpr int PER_WARP = WT_STAGES * WT_STAGE + WBUF;
    static constexpr int MERGE = Q8_WARPS * G * 68 * 4;  // per-warp (m, l, beta-sum, pad, acc[64])
    static constexpr int TOTAL = ((Q_BYTES + 127) & ~127) + (Q8_WARPS * PER_WARP > MERGE ? Q8_WARPS * PER_WARP : MERGE);
};

// four signed bytes of `w` -> four fp32 values on the integer/FMA pipes (int->float converts
// share the narrow special-function pipe): flip the sign bit to get u = b + 128, plant u into
// the mantissa of 2^23, subtract 2^23 + 128 (exact).  Scalar fp32 throughout: measured on B200,
// the packed f32x2 instructions issue slower than two scalar ones.
__device__ __forceinline__ void s8x4_to_f32(int w, float (&f)[4]) {
    const unsigned x = (unsigned)w ^ 0x80808080u;
    const unsigned magic = 0x4B000000u;
    f[0] = __uint_as_float(__byte_perm(x, magic, 0x7650)) - 8388736.0f;
    f[1] = __uint_as_float(__byte_perm(x, magic, 0x7651)) - 8388736.0f;
    f[2] = __uint_as_float(__byte_perm(x, magic, 0x7652)) - 8388736.0f;
    f[3] = __uint_as_float(__byte_perm(x, magic, 0x7653)) - 8388736.0f;
}

template <int G, bool PAGED>
__global__ void __launch_bounds__(Q8_THREADS, 2)
decode_q8_kernel(const DecodeParams P) {
    using SM = Q8Smem<G>;
    constexpr int GP = SM::GP;
    constexpr float LOG2E = 1.4426950408889634f;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    float *qf = (float *)smem_raw;                        // [G][64]
    int *qq = (int *)(qf + G * 64);                       // [G][16]
    float *hq = (float *)(qq + G * 16);                   // [2][G]: score scale (log2 domain), sum of q
    unsigned char *warp_base = smem_raw + ((SM::Q_BYTES + 127) & ~127);
    __shared__ int is_last;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int s = blockIdx.z;
    const int kvh = blockIdx.y / P.head_groups;
    const int hg = blockIdx.y - kvh * P.head_groups;
    const int head0 = kvh * P.group + hg * 8;
    const int gc = min(G, P.group - hg * 8);
    const int n_splits = gridDim.x;
    const int nkv = P.n_kv_head, kvd = nkv * 64;

    int kbeg, kend, ka, kb_;
    key_range(P, s, kbeg, kend);
    split_range(kbeg, kend, blockIdx.x, n_splits, ka, kb_);
    const int *table = PAGED ? P.tables + (P.pos_kind == 2 ? (size_t)s * P.n_log : 0) : nullptr;
    const long long base = PAGED ? 0 : (long long)s * P.seq_rows;
    const bool affine = P.kb != nullptr;
    const bool ref_mode = P.score_mode == MX230_Q8_SCORE_REF;
    const float scale = 0.125f * LOG2E;  // scores are kept in the log2 domain

    // ---- q: fp32 copy, and (reference score mode) per-head int8 codes ----
    const float *qrow = P.qkv + (size_t)s * P.qkv_stride + head0 * 64;
    for (int i = tid; i < G * 64; i += Q8_THREADS) qf[i] = (i / 64 < gc) ? qrow[i] : 0.0f;
    __syncthreads();
    for (int g = warp; g < G; g += Q8_WARPS) {
        float a = qf[g * 64 + lane], b = qf[g * 64 + 32 + lane];
        if (ref_mode) {
            float qmax = warp_max_f(fmaxf(fabsf(a), fabsf(b)));
            float qid = qmax > 0.0f ? __fdiv_rn(127.0f, qmax) : 0.0f;
            int ca = max(-127, min(127, __float2int_rn(a * qid)));
            int cb = max(-127, min(127, __float2int_rn(b * qid)));
            int8_t *qb = (int8_t *)(qq + g * 16);
            qb[lane] = (int8_t)ca;
            qb[32 + lane] = (int8_t)cb;
            float qsum = warp_sum_f((float)(ca + cb));  // exact: small integers
            if (lane == 0) {
                hq[g] = (qmax > 0.0f ? __fdiv_rn(qmax, 127.0f) : 0.0f) * scale;
                hq[G + g] = qsum;
            }
        } else {
            float qsum = warp_sum_f(a + b);
            if (lane == 0) {
                hq[g] = scale;
                hq[G + g] = qsum;
            }
        }
    }
    __syncthreads();

    // ---- this warp's key sub-range ----
    const int n_keys = kb_ - ka;
    int per_w = (n_keys + Q8_WARPS - 1) / Q8_WARPS;
    per_w = (per_w + WT_KEYS - 1) & ~(WT_KEYS - 1);
    const int wa = min(kb_, ka + warp * per_w), wb = min(kb_, wa + per_w);
    const int n_tiles = (wb - wa + WT_KEYS - 1) / WT_KEYS;
    unsigned char *ring = warp_base + warp * SM::PER_WARP;
    float *wbuf = (float *)(ring + WT_STAGES * WT_STAGE);
    const uint32_t ring_u32 = mx::smem_u32(ring);

    // Stage layout: K codes [32][64 B] with 16-byte pieces XOR-swizzled (lane = key reads),
    // V codes [32][64 B] plain, then ks, kb, vs, vb slices of 32 floats.
    // Lane l moves pieces l, l+32, l+64, l+96 of K and V: key = it*8 + l/4, piece = l%4.
    const int pk = lane >> 2, pp = lane & 3;
    const uint32_t dk0 = (uint32_t)(pk * 64 + ((pp ^ ((pk >> 1) & 3)) << 4));
    const uint32_t dv0 = (uint32_t)(WT_KEYS * 64 + pk * 64 + pp * 16);
    const uint32_t ds0 = (uint32_t)(2 * WT_KEYS * 64 + lane * 4);
    // linear caches: per-lane source cursors, advanced by one tile per issue
    const int8_t *ksrc = nullptr, *vsrc = nullptr;
    const float *s_ks = nullptr, *s_kb = nullptr, *s_vs = nullptr, *s_vb = nullptr;
    if (!PAGED) {
        size_t r0 = (size_t)(base + wa);
        ksrc = P.kq + (r0 + pk) * kvd + kvh * 64 + pp * 16;
        vsrc = P.vq + (r0 + pk) * kvd + kvh * 64 + pp * 16;
        size_t sd = (r0 + lane) * nkv + kvh;
        s_ks = P.ks + sd, s_vs = P.vs + sd;
        s_kb = affine ? P.kb + sd : P.ks + sd;
        s_vb = affine ? P.vb + sd : P.vs + sd;
    }
    const size_t it_stride = (size_t)8 * kvd, tile_stride = (size_t)WT_KEYS * kvd;

    auto issue = [&](int tile) {
        const uint32_t dst = ring_u32 + (tile % WT_STAGES) * WT_STAGE;
        const int key0 = wa + tile * WT_KEYS;
        if (!PAGED && key0 + WT_KEYS <= wb) {  // full tile of a linear cache: no predicates, no lookups
#pragma unroll
            for (int it = 0; it < 4; ++it) {
                cp_async16(dst + dk0 + it * 512, ksrc + it * it_stride, 16);
                cp_async16(dst + dv0 + it * 512, vsrc + it * it_stride, 16);
            }
            cp_async4(dst + ds0, s_ks);
            cp_async4(dst + ds0 + 128, s_kb);
            cp_async4(dst + ds0 + 256, s_vs);
            cp_async4(dst + ds0 + 384, s_vb);
        } else {
#pragma unroll
            for (int it = 0; it < 4; ++it) {
                int t = key0 + it * 8 + pk;
                bool ok = t < wb;
                size_t row = cache_row(P, table, base, ok ? t : wa);
                cp_async16(dst + dk0 + it * 512, P.kq + row * kvd + kvh * 64 + pp * 16, ok ? 16 : 0);
                cp_async16(dst + dv0 + it * 512, P.vq + row * kvd + kvh * 64 + pp * 16, ok ? 16 : 0);
            }
            int t = key0 + lane;
            size_t sd = cache_row(P, table, base, t < wb ? t : wa) * nkv + kvh;
            cp_async4(dst + ds0, P.ks + sd);
            cp_async4(dst + ds0 + 128, affine ? P.kb + sd : P.ks + sd);
            cp_async4(dst + ds0 + 256, P.vs + sd);
            cp_async4(dst + ds0 + 384, affine ? P.vb + sd : P.vs + sd);
        }
        if (!PAGED) {
            ksrc += tile_stride, vsrc += tile_stride;
            s_ks += WT_KEYS * nkv, s_kb += WT_KEYS * nkv, s_vs += WT_KEYS * nkv, s_vb += WT_KEYS * nkv;
        }
    };

    float m_run[G], l_thr[G], b_thr[G];
    float acc[G][8];
#pragma unroll
    for (int g = 0; g < G; ++g) {
        m_run[g] = -CUDART_INF_F;
        l_thr[g] = 0.0f;
        b_thr[g] = 0.0f;
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[g][j] = 0.0f;
    }

    if (n_tiles > 0) issue(0);
    cp_async_commit();
    const int kl = lane >> 3, dsl = lane & 7;
    const int koff = lane * 64, kswz = (lane >> 1) & 3;           // K row of this lane's key
    const int voff = WT_KEYS * 64 + kl * 64 + dsl * 8;            // V slice of (key lane, dims)
    for (int tile = 0; tile < n_tiles; ++tile) {
        if (tile + 1 < n_tiles) issue(tile + 1);
        cp_async_commit();
        cp_async_wait<1>();
        __syncwarp();
        const unsigned char *st = ring + (tile % WT_STAGES) * WT_STAGE;
        const float *side = (const float *)(st + 2 * WT_KEYS * 64);
        const bool ok = wa + tile * WT_KEYS + lane < wb;
        const float ksc = side[lane], kbe = affine ? side[32 + lane] : 0.0f;
        const float vsc = side[64 + lane], vbe = affine ? side[96 + lane] : 0.0f;

        // ---- scores (log2 domain) of this lane's key against the G heads ----
        float sco[G];
        if (ref_mode) {
            int dot[G];
#pragma unroll
            for (int g = 0; g < G; ++g) dot[g] = 0;
#pragma unroll
            for (int p = 0; p < 4; ++p) {
                int4 kw = *(const int4 *)(st + koff + ((p ^ kswz) << 4));
#pragma unroll
                for (int g = 0; g < G; ++g) {
                    int4 qw = *(const int4 *)(qq + g * 16 + p * 4);
                    dot[g] = __dp4a(kw.x, qw.x, dot[g]);
                    dot[g] = __dp4a(kw.y, qw.y, dot[g]);
                    dot[g] = __dp4a(kw.z, qw.z, dot[g]);
                    dot[g] = __dp4a(kw.w, qw.w, dot[g]);
                }
            }
#pragma unroll
            for (int g = 0; g < G; ++g) sco[g] = hq[g] * fmaf(ksc, (float)dot[g], kbe * hq[G + g]);
        } else {
            float dotf[G][2];
#pragma unroll
            for (int g = 0; g < G; ++g) dotf[g][0] = dotf[g][1] = 0.0f;
#pragma unroll
            for (int p = 0; p < 4; ++p) {
                int4 kw = *(const int4 *)(st + koff + ((p ^ kswz) << 4));
                const int w4[4] = {kw.x, kw.y, kw.z, kw.w};
#pragma unroll
                for (int w = 0; w < 4; ++w) {
                    float cf[4];
                    s8x4_to_f32(w4[w], cf);
#pragma unroll
                    for (int g = 0; g < G; ++g) {
                        const float4 qv = *(const float4 *)(qf + g * 64 + p * 16 + w * 4);
                        dotf[g][0] = fmaf(qv.x, cf[0], fmaf(qv.z, cf[2], dotf[g][0]));
                        dotf[g][1] = fmaf(qv.y, cf[1], fmaf(qv.w, cf[3], dotf[g][1]));
                    }
                }
            }
#pragma unroll
            for (int g = 0; g < G; ++g)
                sco[g] = hq[g] * fmaf(ksc, dotf[g][0] + dotf[g][1], kbe * hq[G + g]);
        }

        // ---- lazy running max, probabilities, weights ----
        float wv[GP];
#pragma unroll
        for (int g = 0; g < GP; ++g) wv[g] = 0.0f;
#pragma unroll
        for (int g = 0; g < G; ++g) {
            const float sg = ok ? sco[g] : -CUDART_INF_F;
            // raise the running max only when a score exceeds it by RAISE (warp-uniform, rare)
            if (__any_sync(0xFFFFFFFFu, sg > m_run[g] + RAISE * LOG2E)) {
                const float m_new = warp_max_f(fmaxf(sg, m_run[g]));
                const float alpha = (m_run[g] == -CUDART_INF_F) ? 0.0f : mx::ex2(m_run[g] - m_new);
                l_thr[g] *= alpha;
                b_thr[g] *= alpha;
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[g][j] *= alpha;
                m_run[g] = m_new;
            }
            const float p = mx::ex2(sg - m_run[g]);
            l_thr[g] += p;
            b_thr[g] = fmaf(p, vbe, b_thr[g]);
            wv[g] = p * vsc;
        }
#pragma unroll
        for (int g4 = 0; g4 < GP / 4; ++g4)
            *(float4 *)(wbuf + lane * GP + g4 * 4) = make_float4(wv[g4 * 4], wv[g4 * 4 + 1], wv[g4 * 4 + 2], wv[g4 * 4 + 3]);
        __syncwarp();

        // ---- values: lane = (key lane kl, 8-byte slice dsl), 8 steps of 4 keys ----
#pragma unroll 2
        for (int step = 0; step < WT_KEYS / 4; ++step) {
            const int2 vw = *(const int2 *)(st + voff + step * 256);
            float vlo[4], vhi[4];
            s8x4_to_f32(vw.x, vlo);
            s8x4_to_f32(vw.y, vhi);
            float wk[GP];
#pragma unroll
            for (int g4 = 0; g4 < GP / 4; ++g4) {
                const float4 w4 = *(const float4 *)(wbuf + (step * 4 + kl) * GP + g4 * 4);
                wk[g4 * 4] = w4.x, wk[g4 * 4 + 1] = w4.y, wk[g4 * 4 + 2] = w4.z, wk[g4 * 4 + 3] = w4.w;
            }
#pragma unroll
            for (int g = 0; g < G; ++g) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    acc[g][j] = fmaf(wk[g], vlo[j], acc[g][j]);
                    acc[g][4 + j] = fmaf(wk[g], vhi[j], acc[g][4 + j]);
                }
            }
        }
        __syncwarp();  // the ring slot and the weight buffer are rewritten by the next iterations
    }
    cp_async_wait<0>();

    // ---- warp totals, then the CTA-level log-sum-exp merge of the Q8_WARPS warps ----
#pragma unroll
    for (int g = 0; g < G; ++g) {
        l_thr[g] = warp_sum_f(l_thr[g]);
        b_thr[g] = warp_sum_f(b_thr[g]);
#pragma unroll
        for (int j = 0; j < 8; ++j) {  // key lanes differ in lane bits 3,4
            float v = acc[g][j];
            v += __shfl_xor_sync(0xFFFFFFFFu, v, 8);
            v += __shfl_xor_sync(0xFFFFFFFFu, v, 16);
            acc[g][j] = v;
        }
    }
    __syncthreads();  // every warp is done with its ring: reuse the memory for the merge
    float *mg = (float *)warp_base;  // [warp][g][68]: m (log2 domain), l, beta sum, pad, acc[64]
#pragma unroll
    for (int g = 0; g < G; ++g) {
        float *dst = mg + (warp * G + g) * 68;
        if (lane == 0) {
            dst[0] = m_run[g];
            dst[1] = l_thr[g];
            dst[2] = b_thr[g];
        }
        if (lane < 8) {
            *(float4 *)(dst + 4 + lane * 8) = make_float4(acc[g][0], acc[g][1], acc[g][2], acc[g][3]);
            *(float4 *)(dst + 8 + lane * 8) = make_float4(acc[g][4], acc[g][5], acc[g][6], acc[g][7]);
        }
    }
    __syncthreads();

    const bool direct = (n_splits == 1) && (P.fin_acc == nullptr);
    for (int i = tid; i < gc * 64; i += Q8_THREADS) {
        const int g = i >> 6, d = i & 63;
        float mm = -CUDART_INF_F;
#pragma unroll
        for (int w = 0; w < Q8_WARPS; ++w) mm = fmaxf(mm, mg[(w * G + g) * 68]);
        float lt = 0.0f, a = 0.0f;
#pragma unroll
        for (int w = 0; w < Q8_WARPS; ++w) {
            const float *src = mg + (w * G + g) * 68;
            const float wgt = (src[0] == -CUDART_INF_F) ? 0.0f : mx::ex2(src[0] - mm);
            lt += src[1] * wgt;
            a += (src[4 + d] + src[2]) * wgt;  // V's affine offset sum_j p_j vb_j folds into every dim
        }
        const int h = head0 + g;
        if (direct) {
            P.out[(size_t)s * P.out_stride + h * 64 + d] = a / lt;
        } else {
            // partial triples carry the max in natural-log units, as the split-KV interface states
            size_t pi = ((size_t)s * P.n_head + h) * n_splits + blockIdx.x;
            P.ws_acc[pi * 64 + d] = a;
            if (d == 0) {
                P.ws_m[pi] = mm * 0.6931471805599453f;
                P.ws_l[pi] = lt;
            }
        }
    }
    if (direct) return;

    // ---- last CTA of this (sequence, kv head group) merges the splits ----
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        unsigned prev = atomicInc(&P.counters[(size_t)s * gridDim.y + blockIdx.y], n_splits - 1);
        is_last = (prev == (unsigned)(n_splits - 1));
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    merge_and_store<G>(P, s, head0, gc, n_splits, Q8_THREADS);
}

// ---------------------------------------------------------------------------
// int8 cache, reference score mode: the same warp-autonomous streaming, with the two
// contractions of the GQA group on the warp-level tensor-core path
//
// With G query heads per K/V head a key costs 2*G*64 multiply-adds against 144 bytes: on the
// CUDA cores that is more issue slots than the HBM stream leaves (8 heads: ~22 warp instructions
// per key at best, ~6 available), so the group is treated as the M dimension of mma.sync tiles:
//   scores:  S[16 x 8 keys] = Qc[16 x 64] Kc^T, int8 x int8 -> int32 (m16n8k32, two per 8 keys);
//            rows >= G are zero padding.  The 64 dims are assigned to the MMA's k slots so that a
//            thread's B fragments are 16 contiguous bytes of a key (one shared-memory load);
//   weights: p = exp2(s - m) in the accumulator layout, which is the A-fragment layout of the
//            next MMA (thread (g, j) holds head g, keys 2j, 2j+1 of each 8-key group);
//   values:  O[16 x 64] += (p vs)[16 x 16 keys] Vc[16 x 64], f16 x f16 -> f32 (m16n8k16).  The int8
//            codes become f16 exactly (byte permutes onto the mantissa of 1024, minus 1152); p vs
//            goes in as a high and a low f16 part, so the product carries ~22 bits.
// ---------------------------------------------------------------------------
constexpr int MG = 8;                               // heads per CTA (rows 8..15 of the tiles are padding)
// Probabilities are taken against a running max that may lag by up to RAISE_MMA (natural-log units);
// kept small here because p * vs has to stay inside the f16 range (65504): p <= e^2, so any V scale
// below ~8000 is safe.
constexpr float RAISE_MMA = 2.0f;
#ifndef MX_MMA_STAGES
#define MX_MMA_STAGES 2
#endif
constexpr int MMA_STAGES = MX_MMA_STAGES;             // ring depth per warp: MMA_STAGES - 1 tiles of 4.6 KB in flight

__device__ __forceinline__ void mma_s8(int (&c)[4], int a0, int a2, int b0, int b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                 : "r"(a0), "r"(0), "r"(a2), "r"(0), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_f16(float &c0, float &c1, float &z0, float &z1, uint32_t a0, uint32_t a2,
                                        uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c0), "+f"(c1), "+f"(z0), "+f"(z1)
                 : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_f16(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}
__device__ __forceinline__ float2 unpack_f16(uint32_t v) {
    float2 r;
    asm("{.reg .f16 l, h; mov.b32 {l, h}, %2; cvt.f32.f16 %0, l; cvt.f32.f16 %1, h;}" : "=f"(r.x), "=f"(r.y) : "r"(v));
    return r;
}
__device__ __forceinline__ uint32_t hsub2(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("sub.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}

struct Q8MmaSmem {
    static constexpr int Q_BYTES = MG * 64 * 4 + MG * 16 * 4 + 2 * MG * 4 + 64;
    static constexpr int PER_WARP = MMA_STAGES * WT_STAGE;
    static constexpr int MERGE = Q8_WARPS * MG * 68 * 4;
    static constexpr int TOTAL = ((Q_BYTES + 127) & ~127) + (Q8_WARPS * PER_WARP > MERGE ? Q8_WARPS * PER_WARP : MERGE);
};

template <bool PAGED>
__global__ void __launch_bounds__(Q8_THREADS, 2)
decode_q8_mma_kernel(const DecodeParams P) {
    using SM = Q8MmaSmem;
    constexpr float LOG2E = 1.4426950408889634f;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    float *qf = (float *)smem_raw;                        // [8][64]
    int *qq = (int *)(qf + MG * 64);                      // [8][16] int8 codes
    float *hq = (float *)(qq + MG * 16);                  // [2][8]: score scale (log2 domain), sum of q codes
    unsigned char *warp_base = smem_raw + ((SM::Q_BYTES + 127) & ~127);
    __shared__ int is_last;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int s = blockIdx.z;
    const int kvh = blockIdx.y / P.head_groups;
    const int hg = blockIdx.y - kvh * P.head_groups;
    const int head0 = kvh * P.group + hg * 8;
    const int gc = min(MG, P.group - hg * 8);
    const int n_splits = gridDim.x;
    const int nkv = P.n_kv_head, kvd = nkv * 64;

    int kbeg, kend, ka, kb_;
    key_range(P, s, kbeg, kend);
    split_range(kbeg, kend, blockIdx.x, n_splits, ka, kb_);
    const int *table = PAGED ? P.tables + (P.pos_kind == 2 ? (size_t)s * P.n_log : 0) : nullptr;
    const long long base = PAGED ? 0 : (long long)s * P.seq_rows;
    const bool affine = P.kb != nullptr;
    const float scale = 0.125f * LOG2E;  // scores are kept in the log2 domain

    // ---- this warp's key sub-range ----
    const int n_keys = kb_ - ka;
    int per_w = (n_keys + Q8_WARPS - 1) / Q8_WARPS;
    per_w = (per_w + WT_KEYS - 1) & ~(WT_KEYS - 1);
    const int wa = min(kb_, ka + warp * per_w), wb = min(kb_, wa + per_w);
    const int n_tiles = (wb - wa + WT_KEYS - 1) / WT_KEYS;
    unsigned char *ring = warp_base + warp * SM::PER_WARP;
    const uint32_t ring_u32 = mx::smem_u32(ring);

    // Stage layout: K codes [32 keys][64 B] plain; V codes as 16 lines of 128 B (two keys each) whose
    // 16-byte pieces are XOR-swizzled with the line index, so that the 8-byte reads of four lines at
    // once are bank-conflict free; then ks, kb, vs, vb slices of 32 floats.
    // Lane l moves pieces l, l+32, l+64, l+96 of K and V: key = it*8 + l/4, piece = l%4.
    const int pk = lane >> 2, pp = lane & 3;
    const uint32_t dk0 = (uint32_t)(pk * 64 + pp * 16);
    auto v_dst = [&](int key) {  // key: tile-local
        return (uint32_t)(WT_KEYS * 64 + (key >> 1) * 128 + ((((key & 1) << 2) + pp) ^ (((key >> 1) & 3) << 1)) * 16);
    };
    const uint32_t ds0 = (uint32_t)(2 * WT_KEYS * 64 + lane * 4);
    const int8_t *ksrc = nullptr, *vsrc = nullptr;
    const float *s_ks = nullptr, *s_kb = nullptr, *s_vs = nullptr, *s_vb = nullptr;
    if (!PAGED) {
        size_t r0 = (size_t)(base + wa);
        ksrc = P.kq + (r0 + pk) * kvd + kvh * 64 + pp * 16;
        vsrc = P.vq + (r0 + pk) * kvd + kvh * 64 + pp * 16;
        size_t sd = (r0 + lane) * nkv + kvh;
        s_ks = P.ks + sd, s_vs = P.vs + sd;
        s_kb = affine ? P.kb + sd : P.ks + sd;
        s_vb = affine ? P.vb + sd : P.vs + sd;
    }
    const size_t it_stride = (size_t)8 * kvd, tile_stride = (size_t)WT_KEYS * kvd;

    auto issue = [&](int tile) {
        const uint32_t dst = ring_u32 + (tile % MMA_STAGES) * WT_STAGE;
        const int key0 = wa + tile * WT_KEYS;
        if (!PAGED && key0 + WT_KEYS <= wb) {  // full tile of a linear cache: no predicates, no lookups
#pragma unroll
            for (int it = 0; it < 4; ++it) {
                cp_async16(dst + dk0 + it * 512, ksrc + it * it_stride, 16);
                cp_async16(dst + v_dst(it * 8 + pk), vsrc + it * it_stride, 16);
            }
            cp_async4(dst + ds0, s_ks);
            cp_async4(dst + ds0 + 128, s_kb);
            cp_async4(dst + ds0 + 256, s_vs);
            cp_async4(dst + ds0 + 384, s_vb);
        } else {
#pragma unroll
            for (int it = 0; it < 4; ++it) {
                int t = key0 + it * 8 + pk;
                bool ok = t < wb;
                size_t row = cache_row(P, table, base, ok ? t : wa);
                cp_async16(dst + dk0 + it * 512, P.kq + row * kvd + kvh * 64 + pp * 16, ok ? 16 : 0);
                cp_async16(dst + v_dst(it * 8 + pk), P.vq + row * kvd + kvh * 64 + pp * 16, ok ? 16 : 0);
            }
            int t = key0 + lane;
            size_t sd = cache_row(P, table, base, t < wb ? t : wa) * nkv + kvh;
            cp_async4(dst + ds0, P.ks + sd);
            cp_async4(dst + ds0 + 128, affine ? P.kb + sd : P.ks + sd);
            cp_async4(dst + ds0 + 256, P.vs + sd);
            cp_async4(dst + ds0 + 384, affine ? P.vb + sd : P.vs + sd);
        }
        if (!PAGED) {
            ksrc += tile_stride, vsrc += tile_stride;
            s_ks += WT_KEYS * nkv, s_kb += WT_KEYS * nkv, s_vs += WT_KEYS * nkv, s_vb += WT_KEYS * nkv;
        }
    };

    // the first tiles are requested before anything else: their HBM latency then covers the q prologue below
#pragma unroll
    for (int t = 0; t < MMA_STAGES - 1; ++t) {
        if (t < n_tiles) issue(t);
        cp_async_commit();
    }

    // ---- q: per-head int8 codes as the reference kernel forms them (padding heads: zeros) ----
    const float *qrow = P.qkv + (size_t)s * P.qkv_stride + head0 * 64;
    for (int i = tid; i < MG * 64; i += Q8_THREADS) qf[i] = (i / 64 < gc) ? qrow[i] : 0.0f;
    __syncthreads();
    {
        const int g = warp;  // Q8_WARPS == MG
        float a = qf[g * 64 + lane], b = qf[g * 64 + 32 + lane];
        float qmax = warp_max_f(fmaxf(fabsf(a), fabsf(b)));
        float qid = qmax > 0.0f ? __fdiv_rn(127.0f, qmax) : 0.0f;
        int ca = max(-127, min(127, __float2int_rn(a * qid)));
        int cb = max(-127, min(127, __float2int_rn(b * qid)));
        int8_t *qb = (int8_t *)(qq + g * 16);
        qb[lane] = (int8_t)ca;
        qb[32 + lane] = (int8_t)cb;
        float qsum = warp_sum_f((float)(ca + cb));  // exact: small integers
        if (lane == 0) {
            hq[g] = (qmax > 0.0f ? __fdiv_rn(qmax, 127.0f) : 0.0f) * scale;
            hq[MG + g] = qsum;
        }
    }
    __syncthreads();
    static_assert(Q8_WARPS == MG, "one warp quantises one head");

    // fragment coordinates: g = head row (and key / value-dim column of the B fragments), j = k group
    const int g = lane >> 2, j = lane & 3;
    const int4 qa = *(const int4 *)(qq + g * 16 + 4 * j);   // bytes 16j .. 16j+15 of head g
    const float hq_g = hq[g], qsum_g = hq[MG + g];

    float m_run = -CUDART_INF_F, l_thr = 0.0f, b_thr = 0.0f;
    float oacc[8][2];
    float z0 = 0.0f, z1 = 0.0f;   // rows 8..15 of the output tiles: stay zero
#pragma unroll
    for (int t = 0; t < 8; ++t) oacc[t][0] = oacc[t][1] = 0.0f;

    const uint32_t MAGIC = 0x64646464u, BIAS = 0x64806480u;  // f16 1024 | byte, minus 1152
    for (int tile = 0; tile < n_tiles; ++tile) {
        if (tile + MMA_STAGES - 1 < n_tiles) issue(tile + MMA_STAGES - 1);
        cp_async_commit();
        cp_async_wait<MMA_STAGES - 1>();
        __syncwarp();
        const unsigned char *st = ring + (tile % MMA_STAGES) * WT_STAGE;
        const float *side = (const float *)(st + 2 * WT_KEYS * 64);
        const int key_lim = wb - (wa + tile * WT_KEYS);  // valid keys in this tile
#pragma unroll
        for (int blk = 0; blk < 2; ++blk) {
            // ---- scores (log2 domain): two 8-key groups ----
            float sc[2][2], vsw[2][2], vbw[2][2];
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                const int key8 = blk * 16 + r * 8;
                const int4 kw = *(const int4 *)(st + (key8 + g) * 64 + 16 * j);
                int c[4] = {0, 0, 0, 0};
                mma_s8(c, qa.x, qa.y, kw.x, kw.y);
                mma_s8(c, qa.z, qa.w, kw.z, kw.w);
                const float2 ks2 = *(const float2 *)(side + key8 + 2 * j);
                float2 kb2 = make_float2(0.0f, 0.0f), vb2 = make_float2(0.0f, 0.0f);
                if (affine) {
                    kb2 = *(const float2 *)(side + 32 + key8 + 2 * j);
                    vb2 = *(const float2 *)(side + 96 + key8 + 2 * j);
                }
                const float2 vs2 = *(const float2 *)(side + 64 + key8 + 2 * j);
                const float s0 = hq_g * fmaf(ks2.x, (float)c[0], kb2.x * qsum_g);
                const float s1 = hq_g * fmaf(ks2.y, (float)c[1], kb2.y * qsum_g);
                sc[r][0] = key8 + 2 * j < key_lim ? s0 : -CUDART_INF_F;
                sc[r][1] = key8 + 2 * j + 1 < key_lim ? s1 : -CUDART_INF_F;
                vsw[r][0] = vs2.x, vsw[r][1] = vs2.y, vbw[r][0] = vb2.x, vbw[r][1] = vb2.y;
            }
            // ---- lazy running max: raised only when a score exceeds it by RAISE (warp-uniform, rare) ----
            const float smax = fmaxf(fmaxf(sc[0][0], sc[0][1]), fmaxf(sc[1][0], sc[1][1]));
            if (__any_sync(0xFFFFFFFFu, smax > m_run + RAISE_MMA * LOG2E)) {
                float hm = fmaxf(smax, __shfl_xor_sync(0xFFFFFFFFu, smax, 1));
                hm = fmaxf(hm, __shfl_xor_sync(0xFFFFFFFFu, hm, 2));
                const float m_new = fmaxf(hm, m_run);
                const float alpha = (m_run == -CUDART_INF_F) ? 0.0f : mx::ex2(m_run - m_new);
                l_thr *= alpha;
                b_thr *= alpha;
#pragma unroll
                for (int t = 0; t < 8; ++t) oacc[t][0] *= alpha, oacc[t][1] *= alpha;
                m_run = m_new;
            }
            // ---- probabilities, weights (high + low f16 parts) ----
            uint32_t ah[2], al[2];
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                const float p0 = mx::ex2(sc[r][0] - m_run), p1 = mx::ex2(sc[r][1] - m_run);
                l_thr += p0 + p1;
                b_thr = fmaf(p0, vbw[r][0], fmaf(p1, vbw[r][1], b_thr));
                const float w0 = p0 * vsw[r][0], w1 = p1 * vsw[r][1];
                ah[r] = pack_f16(w0, w1);
                const float2 hf = unpack_f16(ah[r]);
                al[r] = pack_f16(w0 - hf.x, w1 - hf.y);
            }
            // ---- values: keys 2j, 2j+1 (+8) of the block, dims 8g .. 8g+7 -> eight 16x8 tiles ----
            uint32_t b[2][8];
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                const int line = blk * 8 + j + 4 * r;
                const unsigned char *lp = st + WT_KEYS * 64 + line * 128;
                const int2 v0 = *(const int2 *)(lp + ((g) ^ (4 * j)) * 8);          // key 2j   (+8r)
                const int2 v1 = *(const int2 *)(lp + ((8 + g) ^ (4 * j)) * 8);      // key 2j+1 (+8r)
                const uint32_t x0 = (uint32_t)v0.x ^ 0x80808080u, x1 = (uint32_t)v1.x ^ 0x80808080u;
                const uint32_t y0 = (uint32_t)v0.y ^ 0x80808080u, y1 = (uint32_t)v1.y ^ 0x80808080u;
                const uint32_t zx01 = __byte_perm(x0, x1, 0x5140), zx23 = __byte_perm(x0, x1, 0x7362);
                const uint32_t zy01 = __byte_perm(y0, y1, 0x5140), zy23 = __byte_perm(y0, y1, 0x7362);
                b[r][0] = hsub2(__byte_perm(zx01, MAGIC, 0x4140), BIAS);
                b[r][1] = hsub2(__byte_perm(zx01, MAGIC, 0x4342), BIAS);
                b[r][2] = hsub2(__byte_perm(zx23, MAGIC, 0x4140), BIAS);
                b[r][3] = hsub2(__byte_perm(zx23, MAGIC, 0x4342), BIAS);
                b[r][4] = hsub2(__byte_perm(zy01, MAGIC, 0x4140), BIAS);
                b[r][5] = hsub2(__byte_perm(zy01, MAGIC, 0x4342), BIAS);
                b[r][6] = hsub2(__byte_perm(zy23, MAGIC, 0x4140), BIAS);
                b[r][7] = hsub2(__byte_perm(zy23, MAGIC, 0x4342), BIAS);
            }
#pragma unroll
            for (int t = 0; t < 8; ++t) {
                mma_f16(oacc[t][0], oacc[t][1], z0, z1, ah[0], ah[1], b[0][t], b[1][t]);
                mma_f16(oacc[t][0], oacc[t][1], z0, z1, al[0], al[1], b[0][t], b[1][t]);
            }
        }
        __syncwarp();  // the ring slot is rewritten by the next iterations
    }
    cp_async_wait<0>();

    // ---- head totals over the four threads of a row, then the CTA-level merge of the warps ----
    l_thr += __shfl_xor_sync(0xFFFFFFFFu, l_thr, 1);
    l_thr += __shfl_xor_sync(0xFFFFFFFFu, l_thr, 2);
    b_thr += __shfl_xor_sync(0xFFFFFFFFu, b_thr, 1);
    b_thr += __shfl_xor_sync(0xFFFFFFFFu, b_thr, 2);
    __syncthreads();  // every warp is done with its ring: reuse the memory for the merge
    float *mg = (float *)warp_base;  // [warp][g][68]: m (log2 domain), l, beta sum, pad, acc[64]
    {
        float *dst = mg + (warp * MG + g) * 68;
        if (j == 0) {
            dst[0] = m_run;
            dst[1] = l_thr;
            dst[2] = b_thr;
        }
        // tile t, columns 2j, 2j+1 <-> dims 16j + t, 16j + 8 + t
#pragma unroll
        for (int t = 0; t < 8; ++t) {
            dst[4 + 16 * j + t] = oacc[t][0];
            dst[4 + 16 * j + 8 + t] = oacc[t][1];
        }
    }
    __syncthreads();

    const bool direct = (n_splits == 1) && (P.fin_acc == nullptr);
    for (int i = tid; i < gc * 64; i += Q8_THREADS) {
        const int gg = i >> 6, d = i & 63;
        float mm = -CUDART_INF_F;
#pragma unroll
        for (int w = 0; w < Q8_WARPS; ++w) mm = fmaxf(mm, mg[(w * MG + gg) * 68]);
        float lt = 0.0f, a = 0.0f;
#pragma unroll
        for (int w = 0; w < Q8_WARPS; ++w) {
            const float *src = mg + (w * MG + gg) * 68;
            const float wgt = (src[0] == -CUDART_INF_F) ? 0.0f : mx::ex2(src[0] - mm);
            lt += src[1] * wgt;
            a += (src[4 + d] + src[2]) * wgt;  // V's affine offset sum_j p_j vb_j folds into every dim
        }
        const int h = head0 + gg;
        if (direct) {
            P.out[(size_t)s * P.out_stride + h * 64 + d] = a / lt;
        } else {
            // partial triples carry the max in natural-log units, as the split-KV interface states
            size_t pi = ((size_t)s * P.n_head + h) * n_splits + blockIdx.x;
            P.ws_acc[pi * 64 + d] = a;
            if (d == 0) {
                P.ws_m[pi] = mm * 0.6931471805599453f;
                P.ws_l[pi] = lt;
            }
        }
    }
    if (direct) return;

    // ---- last CTA of this (sequence, kv head group) merges the splits ----
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        unsigned prev = atomicInc(&P.counters[(size_t)s * gridDim.y + blockIdx.y], n_splits - 1);
        is_last = (prev == (unsigned)(n_splits - 1));
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    merge_and_store<MG>(P, s, head0, gc, n_splits, Q8_THREADS);
}

// ---------------------------------------------------------------------------
// fp32 cache: warp-autonomous streaming on CUDA cores (a key is 512 B per kv head here, so the
// 2*G*64 multiply-adds per key fit the FMA pipes under the HBM stream)
//
// A CTA of F32_WARPS warps owns one (key split, kv head, sequence); each warp streams its own key
// sub-range in tiles of 16 keys (K and V rows, 8 KB) through a private two-stage cp.async ring.
//   scores:  lane = (key, half of the 64 dims); the halves are added with one shuffle per head;
//            running max per head raised lazily, as in the int8 kernel;
//   values:  lane = (key lane of 4, 8-dim slice), weights through a per-warp shared buffer.
// K rows are XOR-swizzled by key, V rows fold their upper half, so both read patterns are
// bank-conflict free.  Three CTAs are resident per SM.
// ---------------------------------------------------------------------------
constexpr int F32_WARPS = 4;
constexpr int F32_THREADS = F32_WARPS * 32;
constexpr int FT_KEYS = 16;                          // keys per warp tile
constexpr int FT_STAGE = 2 * FT_KEYS * 256;          // K + V rows = 8192 B
constexpr int FT_STAGES = 2;

template <int G>
struct F32Smem {
    static constexpr int GP = (G + 3) & ~3;
    static constexpr int Q_BYTES = G * 64 * 4;
    static constexpr int WBUF = FT_KEYS * GP * 4;
    static constexpr int PER_WARP = FT_STAGES * FT_STAGE + WBUF;
    static constexpr int MERGE = F32_WARPS * G * 68 * 4;
    static constexpr int TOTAL = ((Q_BYTES + 127) & ~127) + (F32_WARPS * PER_WARP > MERGE ? F32_WARPS * PER_WARP : MERGE);
};

template <int G, bool PAGED>
__global__ void __launch_bounds__(F32_THREADS, 3)
decode_f32_ring_kernel(const DecodeParams P) {
    using SM = F32Smem<G>;
    constexpr int GP = SM::GP;
    constexpr float LOG2E = 1.4426950408889634f;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    float *qf = (float *)smem_raw;                        // [G][64]
    unsigned char *warp_base = smem_raw + ((SM::Q_BYTES + 127) & ~127);
    __shared__ int is_last;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int s = blockIdx.z;
    const int kvh = blockIdx.y / P.head_groups;
    const int hg = blockIdx.y - kvh * P.head_groups;
    const int head0 = kvh * P.group + hg * 8;
    const int gc = min(G, P.group - hg * 8);
    const int n_splits = gridDim.x;
    const int nkv = P.n_kv_head, kvd = nkv * 64;

    int kbeg, kend, ka, kb_;
    key_range(P, s, kbeg, kend);
    split_range(kbeg, kend, blockIdx.x, n_splits, ka, kb_);
    const int *table = PAGED ? P.tables + (P.pos_kind == 2 ? (size_t)s * P.n_log : 0) : nullptr;
    const long long base = PAGED ? 0 : (long long)s * P.seq_rows;
    const float scale = 0.125f * LOG2E;  // scores are kept in the log2 domain

    const float *qrow = P.qkv + (size_t)s * P.qkv_stride + head0 * 64;
    for (int i = tid; i < G * 64; i += F32_THREADS) qf[i] = (i / 64 < gc) ? qrow[i] : 0.0f;
    __syncthreads();

    // ---- this warp's key sub-range ----
    const int n_keys = kb_ - ka;
    int per_w = (n_keys + F32_WARPS - 1) / F32_WARPS;
    per_w = (per_w + FT_KEYS - 1) & ~(FT_KEYS - 1);
    const int wa = min(kb_, ka + warp * per_w), wb = min(kb_, wa + per_w);
    const int n_tiles = (wb - wa + FT_KEYS - 1) / FT_KEYS;
    unsigned char *ring = warp_base + warp * SM::PER_WARP;
    float *wbuf = (float *)(ring + FT_STAGES * FT_STAGE);
    const uint32_t ring_u32 = mx::smem_u32(ring);

    // Lane l moves 16-byte pieces l, l+32, ... of the tile's K rows and V rows: piece p of a matrix is
    // (key = p / 16, chunk = p % 16) = (it*2 + l/16, l%16).
    const int pk = lane >> 4, pc = lane & 15;
    auto k_off = [&](int key) { return (uint32_t)(key * 256 + (((pc & 8) | ((pc ^ key) & 7)) << 4)); };
    const uint32_t v_chunk = (uint32_t)((pc ^ (pc >> 3)) << 4);
    const float *ksrc = nullptr, *vsrc = nullptr;
    if (!PAGED) {
        size_t r0 = (size_t)(base + wa);
        ksrc = P.kcache + (r0 + pk) * kvd + kvh * 64 + pc * 4;
        vsrc = P.vcache + (r0 + pk) * kvd + kvh * 64 + pc * 4;
    }
    const size_t it_stride = (size_t)2 * kvd, tile_stride = (size_t)FT_KEYS * kvd;

    auto issue = [&](int tile) {
        const uint32_t dst = ring_u32 + (tile % FT_STAGES) * FT_STAGE;
        const int key0 = wa + tile * FT_KEYS;
        if (!PAGED && key0 + FT_KEYS <= wb) {  // full tile of a linear cache: no predicates, no lookups
#pragma unroll
            for (int it = 0; it < 8; ++it) {
                const int key = it * 2 + pk;
                cp_async16(dst + k_off(key), ksrc + it * it_stride, 16);
                cp_async16(dst + FT_KEYS * 256 + key * 256 + v_chunk, vsrc + it * it_stride, 16);
            }
        } else {
#pragma unroll
            for (int it = 0; it < 8; ++it) {
                const int key = it * 2 + pk;
                const int t = key0 + key;
                const bool ok = t < wb;
                const size_t row = cache_row(P, table, base, ok ? t : wa);
                cp_async16(dst + k_off(key), P.kcache + row * kvd + kvh * 64 + pc * 4, ok ? 16 : 0);
                cp_async16(dst + FT_KEYS * 256 + key * 256 + v_chunk, P.vcache + row * kvd + kvh * 64 + pc * 4,
                           ok ? 16 : 0);
            }
        }
        if (!PAGED) ksrc += tile_stride, vsrc += tile_stride;
    };

    float m_run[G], l_thr[G];
    float acc[G][8];
#pragma unroll
    for (int g = 0; g < G; ++g) {
        m_run[g] = -CUDART_INF_F;
        l_thr[g] = 0.0f;
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[g][j] = 0.0f;
    }

    if (n_tiles > 0) issue(0);
    cp_async_commit();
    const int sk = lane & 15, sh = lane >> 4;          // scores: key, dim half
    const int kl = lane >> 3, dsl = lane & 7;          // values: key lane, 8-dim slice
    const uint32_t vo0 = (uint32_t)(((2 * dsl) ^ ((2 * dsl) >> 3)) << 4);
    const uint32_t vo1 = (uint32_t)(((2 * dsl + 1) ^ ((2 * dsl + 1) >> 3)) << 4);
    for (int tile = 0; tile < n_tiles; ++tile) {
        if (tile + 1 < n_tiles) issue(tile + 1);
        cp_async_commit();
        cp_async_wait<1>();
        __syncwarp();
        const unsigned char *st = ring + (tile % FT_STAGES) * FT_STAGE;
        const bool ok = wa + tile * FT_KEYS + sk < wb;

        // ---- scores (log2 domain): this lane's half of its key's row against the G heads ----
        float d0[G], d1[G];
#pragma unroll
        for (int g = 0; g < G; ++g) d0[g] = d1[g] = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float4 kv = *(const float4 *)(st + sk * 256 + (((sh << 3) | ((i ^ sk) & 7)) << 4));
#pragma unroll
            for (int g = 0; g < G; ++g) {
                const float4 qv = *(const float4 *)(qf + g * 64 + sh * 32 + i * 4);
                d0[g] = fmaf(qv.x, kv.x, fmaf(qv.z, kv.z, d0[g]));
                d1[g] = fmaf(qv.y, kv.y, fmaf(qv.w, kv.w, d1[g]));
            }
        }
        float wv[GP];
#pragma unroll
        for (int g = 0; g < GP; ++g) wv[g] = 0.0f;
#pragma unroll
        for (int g = 0; g < G; ++g) {
            float dot = d0[g] + d1[g];
            dot += __shfl_xor_sync(0xFFFFFFFFu, dot, 16);
            const float sg = ok ? dot * scale : -CUDART_INF_F;
            // raise the running max only when a score exceeds it by RAISE (warp-uniform, rare)
            if (__any_sync(0xFFFFFFFFu, sg > m_run[g] + RAISE * LOG2E)) {
                const float m_new = warp_max_f(fmaxf(sg, m_run[g]));
                const float alpha = (m_run[g] == -CUDART_INF_F) ? 0.0f : mx::ex2(m_run[g] - m_new);
                l_thr[g] *= alpha;
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[g][j] *= alpha;
                m_run[g] = m_new;
            }
            const float p = mx::ex2(sg - m_run[g]);
            if (sh == 0) l_thr[g] += p;   // the two halves of a key hold the same score
            wv[g] = p;
        }
        if (sh == 0) {
#pragma unroll
            for (int g4 = 0; g4 < GP / 4; ++g4)
                *(float4 *)(wbuf + sk * GP + g4 * 4) = make_float4(wv[g4 * 4], wv[g4 * 4 + 1], wv[g4 * 4 + 2], wv[g4 * 4 + 3]);
        }
        __syncwarp();

        // ---- values: lane = (key lane kl, 8-dim slice dsl), 4 steps of 4 keys ----
#pragma unroll
        for (int step = 0; step < FT_KEYS / 4; ++step) {
            const unsigned char *vr = st + FT_KEYS * 256 + (step * 4 + kl) * 256;
            const float4 va = *(const float4 *)(vr + vo0), vb4 = *(const float4 *)(vr + vo1);
            float wk[GP];
#pragma unroll
            for (int g4 = 0; g4 < GP / 4; ++g4) {
                const float4 w4 = *(const float4 *)(wbuf + (step * 4 + kl) * GP + g4 * 4);
                wk[g4 * 4] = w4.x, wk[g4 * 4 + 1] = w4.y, wk[g4 * 4 + 2] = w4.z, wk[g4 * 4 + 3] = w4.w;
            }
#pragma unroll
            for (int g = 0; g < G; ++g) {
                acc[g][0] = fmaf(wk[g], va.x, acc[g][0]);
                acc[g][1] = fmaf(wk[g], va.y, acc[g][1]);
                acc[g][2] = fmaf(wk[g], va.z, acc[g][2]);
                acc[g][3] = fmaf(wk[g], va.w, acc[g][3]);
                acc[g][4] = fmaf(wk[g], vb4.x, acc[g][4]);
                acc[g][5] = fmaf(wk[g], vb4.y, acc[g][5]);
                acc[g][6] = fmaf(wk[g], vb4.z, acc[g][6]);
                acc[g][7] = fmaf(wk[g], vb4.w, acc[g][7]);
            }
        }
        __syncwarp();  // the ring slot and the weight buffer are rewritten by the next iterations
    }
    cp_async_wait<0>();

    // ---- warp totals, then the CTA-level log-sum-exp merge of the warps ----
#pragma unroll
    for (int g = 0; g < G; ++g) {
        l_thr[g] = warp_sum_f(l_thr[g]);
#pragma unroll
        for (int j = 0; j < 8; ++j) {  // key lanes differ in lane bits 3,4
            float v = acc[g][j];
            v += __shfl_xor_sync(0xFFFFFFFFu, v, 8);
            v += __shfl_xor_sync(0xFFFFFFFFu, v, 16);
            acc[g][j] = v;
        }
    }
    __syncthreads();  // every warp is done with its ring: reuse the memory for the merge
    float *mg = (float *)warp_base;  // [warp][g][68]: m (log2 domain), l, pad, pad, acc[64]
#pragma unroll
    for (int g = 0; g < G; ++g) {
        float *dst = mg + (warp * G + g) * 68;
        if (lane == 0) {
            dst[0] = m_run[g];
            dst[1] = l_thr[g];
        }
        if (lane < 8) {
            *(float4 *)(dst + 4 + lane * 8) = make_float4(acc[g][0], acc[g][1], acc[g][2], acc[g][3]);
            *(float4 *)(dst + 8 + lane * 8) = make_float4(acc[g][4], acc[g][5], acc[g][6], acc[g][7]);
        }
    }
    __syncthreads();

    const bool direct = (n_splits == 1) && (P.fin_acc == nullptr);
    for (int i = tid; i < gc * 64; i += F32_THREADS) {
        const int g = i >> 6, d = i & 63;
        float mm = -CUDART_INF_F;
#pragma unroll
        for (int w = 0; w < F32_WARPS; ++w) mm = fmaxf(mm, mg[(w * G + g) * 68]);
        float lt = 0.0f, a = 0.0f;
#pragma unroll
        for (int w = 0; w < F32_WARPS; ++w) {
            const float *src = mg + (w * G + g) * 68;
            const float wgt = (src[0] == -CUDART_INF_F) ? 0.0f : mx::ex2(src[0] - mm);
            lt += src[1] * wgt;
            a += src[4 + d] * wgt;
        }
        const int h = head0 + g;
        if (direct) {
            P.out[(size_t)s * P.out_stride + h * 64 + d] = a / lt;
        } else {
            // partial triples carry the max in natural-log units, as the split-KV interface states
            size_t pi = ((size_t)s * P.n_head + h) * n_splits + blockIdx.x;
            P.ws_acc[pi * 64 + d] = a;
            if (d == 0) {
                P.ws_m[pi] = mm * 0.6931471805599453f;
                P.ws_l[pi] = lt;
            }
        }
    }
    if (direct) return;

    // ---- last CTA of this (sequence, kv head group) merges the splits ----
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        unsigned prev = atomicInc(&P.counters[(size_t)s * gridDim.y + blockIdx.y], n_splits - 1);
        is_last = (prev == (unsigned)(n_splits - 1));
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    merge_and_store<G>(P, s, head0, gc, n_splits, F32_THREADS);
}

// Log-sum-exp merge of gathered partial triples: one thread per (row, 4 dims).
// Part p keeps its maxima and sums at m + p*ml_stride, l + p*ml_stride and its accumulators at
// acc + p*acc_stride (floats): rows / rows*64 for separate arrays, rows*66 for both when the parts
// are the ranks' packed [m | l | acc] buffers as the all-gather leaves them.
__global__ void merge_partials_kernel(float *out, const float *m, const float *l, const float *acc,
                                      int parts, int rows, size_t ml_stride, size_t acc_stride) {
    int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= rows * 16) return;
    int r = idx >> 4, d4 = (idx & 15) * 4;
    float mm = -CUDART_INF_F;
    for (int p = 0; p < parts; ++p) mm = fmaxf(mm, m[(size_t)p * ml_stride + r]);
    float ll = 0.0f;
    float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int p = 0; p < parts; ++p) {
        float mp = m[(size_t)p * ml_stride + r];
        float w = (mp == -CUDART_INF_F) ? 0.0f : __expf(mp - mm);
        ll += l[(size_t)p * ml_stride + r] * w;
        float4 v = *(const float4 *)(acc + (size_t)p * acc_stride + (size_t)r * 64 + d4);
        a.x += v.x * w, a.y += v.y * w, a.z += v.z * w, a.w += v.w * w;
    }
    float inv = 1.0f / ll;
    *(float4 *)(out + (size_t)r * 64 + d4) = make_float4(a.x * inv, a.y * inv, a.z * inv, a.w * inv);
}

template <int G>
size_t q8_smem_bytes() {
    return (size_t)Q8Smem<G>::TOTAL;
}

template <int G>
int launch_g(mx230_handle *h, cudaStream_t st, const DecodeParams &P, dim3 grid, bool q8) {
    if (q8 && P.score_mode == MX230_Q8_SCORE_REF && h->decode_tensor) {
        // reference score mode: the tensor-core kernel serves any group size up to 8 per CTA
        size_t sm = (size_t)Q8MmaSmem::TOTAL;
        if (P.tables) {
            MX_SMEM_ATTR_ONCE(h->device, (decode_q8_mma_kernel<true>), sm);
            MX_LAUNCH(h, st, MX230_K_DECODE_Q8, (decode_q8_mma_kernel<true><<<grid, Q8_THREADS, sm, st>>>(P)));
        } else {
            MX_SMEM_ATTR_ONCE(h->device, (decode_q8_mma_kernel<false>), sm);
            MX_LAUNCH(h, st, MX230_K_DECODE_Q8, (decode_q8_mma_kernel<false><<<grid, Q8_THREADS, sm, st>>>(P)));
        }
    } else if (q8) {
        size_t sm = q8_smem_bytes<G>();
        if (P.tables) {
            MX_SMEM_ATTR_ONCE(h->device, (decode_q8_kernel<G, true>), sm);
            MX_LAUNCH(h, st, MX230_K_DECODE_Q8, (decode_q8_kernel<G, true><<<grid, Q8_THREADS, sm, st>>>(P)));
        } else {
            MX_SMEM_ATTR_ONCE(h->device, (decode_q8_kernel<G, false>), sm);
            MX_LAUNCH(h, st, MX230_K_DECODE_Q8, (decode_q8_kernel<G, false><<<grid, Q8_THREADS, sm, st>>>(P)));
        }
    } else {
        size_t sm = (size_t)F32Smem<G>::TOTAL;
        if (P.tables) {
            MX_SMEM_ATTR_ONCE(h->device, (decode_f32_ring_kernel<G, true>), sm);
            MX_LAUNCH(h, st, MX230_K_DECODE_F32, (decode_f32_ring_kernel<G, true><<<grid, F32_THREADS, sm, st>>>(P)));
        } else {
            MX_SMEM_ATTR_ONCE(h->device, (decode_f32_ring_kernel<G, false>), sm);
            MX_LAUNCH(h, st, MX230_K_DECODE_F32, (decode_f32_ring_kernel<G, false><<<grid, F32_THREADS, sm, st>>>(P)));
        }
    }
    return MX230_OK;
}

// `known_keys`: host-known upper bound of keys per sequence (<= 0 when the position
// lives on the device); only steers how many key splits are launched.
int launch_decode(mx230_handle *h, void *stream, DecodeParams P, int n_seq, int head_dim,
                  long long known_keys, mx230_splitkv_comm *comm = nullptr) {
    MX_REQUIRE(h && P.qkv, MX230_ERR_INVALID_ARG, "attn_decode: null argument");
    MX_REQUIRE(head_dim == 64, MX230_ERR_UNSUPPORTED, "attn_decode: head_dim %d unsupported (must be 64)",
               head_dim);
    MX_REQUIRE(P.n_head > 0 && P.n_kv_head > 0 && P.n_head % P.n_kv_head == 0, MX230_ERR_UNSUPPORTED,
               "attn_decode: n_head %d must be a positive multiple of n_kv_head %d", P.n_head,
               P.n_kv_head);
    const bool q8 = P.kq != nullptr;
    if (q8)
        MX_REQUIRE(P.vq && P.ks && P.vs && ((P.kb == nullptr) == (P.vb == nullptr)),
                   MX230_ERR_INVALID_ARG, "attn_decode_q8: missing cache array");
    else
        MX_REQUIRE(P.kcache && P.vcache, MX230_ERR_INVALID_ARG, "attn_decode: null cache");
    MX_REQUIRE(P.fin_acc || P.out, MX230_ERR_INVALID_ARG, "attn_decode: null output");
    MX_REQUIRE(P.tables == nullptr || P.bs > 0, MX230_ERR_INVALID_ARG, "attn_decode: block size %d",
               P.bs);
    MX_REQUIRE((((uintptr_t)P.qkv | (uintptr_t)P.out | (uintptr_t)P.kcache | (uintptr_t)P.vcache |
                 (uintptr_t)P.kq | (uintptr_t)P.vq) & 15) == 0 && P.qkv_stride % 4 == 0 &&
                   P.out_stride % 4 == 0,
               MX230_ERR_INVALID_ARG, "attn_decode: buffers must be 16-byte aligned");
    if (P.range_mode) MX_REQUIRE(P.t0 >= 0 && P.t1 > P.t0, MX230_ERR_INVALID_ARG,
                                 "attn_decode_partial: empty key range [%d, %d)", P.t0, P.t1);
    if (!P.range_mode && P.pos_kind == 0)
        MX_REQUIRE(P.pos >= 0, MX230_ERR_INVALID_ARG, "attn_decode: negative position %d", P.pos);
    if (n_seq <= 0) return n_seq == 0 ? MX230_OK
                                      : mx230_fail(MX230_ERR_INVALID_ARG, "attn_decode: negative n_seq");

    P.group = P.n_head / P.n_kv_head;
    P.head_groups = (P.group + 7) / 8;
    P.score_mode = h->q8_score_mode;
    P.max_keys = (P.pos_kind == 2 && known_keys > 0 && known_keys < 0x7FFFFFFF) ? (int)known_keys : 0;
    int gy = P.n_kv_head * P.head_groups;
    MX_REQUIRE((size_t)n_seq * gy <= h->n_counters, MX230_ERR_UNSUPPORTED,
               "attn_decode: n_seq*n_kv_head %lld exceeds %zu", (long long)n_seq * gy, h->n_counters);

    // how many key splits: fill the machine (2 resident CTAs per SM for the int8 kernel, 3 for
    // the fp32 one) but keep >= 256 keys each
    // (rounded down so that the whole grid is resident at once: a partial second wave would
    // nearly double the time)
    long long base_ctas = (long long)n_seq * gy;
    // One-kernel split-KV step: the CTA that finishes a group waits there for the other ranks.  At most one CTA per
    // group ever waits, so with fewer groups than SMs a slot always stays free for the CTAs that still have keys to
    // stream, on every rank, and no rank's waiting CTAs can keep another rank's pushes from happening.  With more
    // groups the wait moves into a kernel of its own behind this one.
    float *merge_after = nullptr;
    if (P.push_out && base_ctas >= h->sm_count) merge_after = P.push_out, P.push_out = nullptr;
    int want = (int)(((q8 ? 2LL : 3LL) * h->sm_count) / base_ctas);
    int n_splits;
    if (h->decode_chunk > 0 && known_keys > 0) {
        n_splits = (int)((known_keys + h->decode_chunk - 1) / h->decode_chunk);
    } else {
        long long keys = known_keys > 0 ? known_keys : 4096;
        int max_by_len = (int)((keys + 255) / 256);
        n_splits = want < 1 ? 1 : want;
        if (n_splits > max_by_len) n_splits = max_by_len;
        // a second split is not worth its merge pass when one CTA per (sequence, kv head) already
        // covers most of the SMs and the contexts are short (measured: batch 64 x 2048 keys, 19.7 vs 22.3 us)
        if (n_splits == 2 && base_ctas * 5 >= (long long)h->sm_count * 4 && keys <= 4096) n_splits = 1;
    }
    if (n_splits < 1) n_splits = 1;
    if (n_splits > 256) n_splits = 256;
    if (n_splits > 1 || P.fin_acc) {
        size_t need = (size_t)n_seq * P.n_head * n_splits * 66 * sizeof(float);
        MX_REQUIRE(h->ws && need <= h->ws_bytes, MX230_ERR_WORKSPACE,
                   "attn_decode: workspace %zu B < %zu B needed for %d key splits", h->ws_bytes, need,
                   n_splits);
        size_t rows = (size_t)n_seq * P.n_head * n_splits;
        h->staged.valid = 0;   // the workspace is about to hold something else
        P.ws_acc = (float *)h->ws;
        P.ws_m = P.ws_acc + rows * 64;
        P.ws_l = P.ws_m + rows;
    }
    P.counters = h->counters;

    mx230_device_guard guard(h->device);
    dim3 grid(n_splits, gy, n_seq);
    cudaStream_t st = (cudaStream_t)stream;
    int g = P.group > 8 ? 8 : P.group;
    int rc;
    if (g == 1) rc = launch_g<1>(h, st, P, grid, q8);
    else if (g == 2) rc = launch_g<2>(h, st, P, grid, q8);
    else if (g <= 4) rc = launch_g<4>(h, st, P, grid, q8);
    else if (g <= 7) rc = launch_g<7>(h, st, P, grid, q8);
    else rc = launch_g<8>(h, st, P, grid, q8);
    if (rc == MX230_OK && merge_after) rc = mx230_splitkv_wait_merge(comm, stream, merge_after);
    return rc;
}

DecodeParams base_params(float *out, int out_stride, const float *qkv, int qkv_stride, int n_head,
                         int n_kv_head) {
    DecodeParams P;
    memset(&P, 0, sizeof(P));
    P.out = out;
    P.out_stride = out_stride;
    P.qkv = qkv;
    P.qkv_stride = qkv_stride;
    P.n_head = n_head;
    P.n_kv_head = n_kv_head;
    return P;
}

}  // namespace

// ---- fp32 cache ----
extern "C" int mx230_attn_decode(mx230_handle *h, void *stream, float *out, const float *qkv,
                                 const float *kcache, const float *vcache, int t_cur, int n_head,
                                 int n_kv_head, int head_dim) {
    DecodeParams P = base_params(out, n_head * 64, qkv, 0, n_head, n_kv_head);
    P.kcache = kcache, P.vcache = vcache, P.pos_kind = 0, P.pos = t_cur;
    return launch_decode(h, stream, P, 1, head_dim, (long long)t_cur + 1);
}
extern "C" int mx230_attn_decode_dyn(mx230_handle *h, void *stream, float *out, const float *qkv,
                                     const float *kcache, const float *vcache, const int *pos_ptr,
                                     int n_head, int n_kv_head, int head_dim) {
    MX_REQUIRE(pos_ptr, MX230_ERR_INVALID_ARG, "attn_decode_dyn: null pos_ptr");
    DecodeParams P = base_params(out, n_head * 64, qkv, 0, n_head, n_kv_head);
    P.kcache = kcache, P.vcache = vcache, P.pos_kind = 1, P.pos_dev = pos_ptr;
    return launch_decode(h, stream, P, 1, head_dim, 0);
}
extern "C" int mx230_attn_decode_paged(mx230_handle *h, void *stream, float *out, const float *qkv,
                                       const float *kcache, const float *vcache, int t_cur,
                                       int n_head, int n_kv_head, int head_dim, const int *bt,
                                       int bs) {
    MX_REQUIRE(bt, MX230_ERR_INVALID_ARG, "attn_decode_paged: null block table");
    DecodeParams P = base_params(out, n_head * 64, qkv, 0, n_head, n_kv_head);
    P.kcache = kcache, P.vcache = vcache, P.pos_kind = 0, P.pos = t_cur, P.tables = bt, P.bs = bs;
    return launch_decode(h, stream, P, 1, head_dim, (long long)t_cur + 1);
}
extern "C" int mx230_attn_decode_paged_dyn(mx230_handle *h, void *stream, float *out,
                                           const float *qkv, const float *kcache,
                                           const float *vcache, const int *pos_ptr, int n_head,
                                           int n_kv_head, int head_dim, const int *bt, int bs) {
    MX_REQUIRE(pos_ptr && bt, MX230_ERR_INVALID_ARG, "attn_decode_paged_dyn: null argument");
    DecodeParams P = base_params(out, n_head * 64, qkv, 0, n_head, n_kv_head);
    P.kcache = kcache, P.vcache = vcache, P.pos_kind = 1, P.pos_dev = pos_ptr, P.tables = bt, P.bs = bs;
    return launch_decode(h, stream, P, 1, head_dim, 0);
}
extern "C" int mx230_attn_decode_batched(mx230_handle *h, void *stream, float *out,
                                         const float *qkv, const float *kcache,
                                         const float *vcache, const int *pos, int n_seq,
                                         int n_head, int n_kv_head, int head_dim,
                                         const int *tables, int block_size, int n_log,
                                         int qkv_stride, int out_stride) {
    MX_REQUIRE(pos && tables, MX230_ERR_INVALID_ARG, "attn_decode_batched: null argument");
    DecodeParams P = base_params(out, out_stride, qkv, qkv_stride, n_head, n_kv_head);
    P.kcache = kcache, P.vcache = vcache, P.pos_kind = 2, P.pos_dev = pos;
    P.tables = tables, P.bs = block_size, P.n_log = n_log;
    return launch_decode(h, stream, P, n_seq, head_dim, (long long)n_log * block_size);
}

// ---- int8 cache ----
#define Q8_ARGS kq, vq, ks, vs, kb, vb
static void set_q8(DecodeParams &P, const int8_t *kq, const int8_t *vq, const float *ks,
                   const float *vs, const float *kb, const float *vb) {
    P.kq = kq, P.vq = vq, P.ks = ks, P.vs = vs, P.kb = kb, P.vb = vb;
}
extern "C" int mx230_attn_decode_q8(mx230_handle *h, void *stream, float *out, const float *qkv,
                                    const int8_t *kq, const int8_t *vq, const float *ks,
                                    const float *vs, const float *kb, const float *vb, int t_cur,
                                    int n_head, int n_kv_head, int head_dim) {
    MX_REQUIRE(kq, MX230_ERR_INVALID_ARG, "attn_decode_q8: null kq");
    DecodeParams P = base_params(out, n_head * 64, qkv, 0, n_head, n_kv_head);
    set_q8(P, Q8_ARGS);
    P.pos_kind = 0, P.pos = t_cur;
    return launch_decode(h, stream, P, 1, head_dim, (long long)t_cur + 1);
}
extern "C" int mx230_attn_decode_q8_dyn(mx230_handle *h, void *stream, float *out,
                                        const float *qkv, const int8_t *kq, const int8_t *vq,
                                        const float *ks, const float *vs, const float *kb,
                                        const float *vb, const int *pos_ptr, int n_head,
                                        int n_kv_head, int head_dim) {
    MX_REQUIRE(kq && pos_ptr, MX230_ERR_INVALID_ARG, "attn_decode_q8_dyn: null argument");
    DecodeParams P = base_params(out, n_head * 64, qkv, 0, n_head, n_kv_head);
    set_q8(P, Q8_ARGS);
    P.pos_kind = 1, P.pos_dev = pos_ptr;
    return launch_decode(h, stream, P, 1, head_dim, 0);
}
extern "C" int mx230_attn_decode_q8_paged(mx230_handle *h, void *stream, float *out,
                                          const float *qkv, const int8_t *kq, const int8_t *vq,
                                          const float *ks, const float *vs, const float *kb,
                                          const float *vb, int t_cur, int n_head, int n_kv_head,
                                          int head_dim, const int *bt, int bs) {
    MX_REQUIRE(kq && bt, MX230_ERR_INVALID_ARG, "attn_decode_q8_paged: null argument");
    DecodeParams P = base_params(out, n_head * 64, qkv, 0, n_head, n_kv_head);
    set_q8(P, Q8_ARGS);
    P.pos_kind = 0, P.pos = t_cur, P.tables = bt, P.bs = bs;
    return launch_decode(h, stream, P, 1, head_dim, (long long)t_cur + 1);
}
extern "C" int mx230_attn_decode_q8_paged_dyn(mx230_handle *h, void *stream, float *out,
                                              const float *qkv, const int8_t *kq,
                                              const int8_t *vq, const float *ks, const float *vs,
                                              const float *kb, const float *vb, const int *pos_ptr,
                                              int n_head, int n_kv_head, int head_dim,
                                              const int *bt, int bs) {
    MX_REQUIRE(kq && pos_ptr && bt, MX230_ERR_INVALID_ARG, "attn_decode_q8_paged_dyn: null argument");
    DecodeParams P = base_params(out, n_head * 64, qkv, 0, n_head, n_kv_head);
    set_q8(P, Q8_ARGS);
    P.pos_kind = 1, P.pos_dev = pos_ptr, P.tables = bt, P.bs = bs;
    return launch_decode(h, stream, P, 1, head_dim, 0);
}
extern "C" int mx230_attn_decode_q8_batched(mx230_handle *h, void *stream, float *out,
                                            const float *qkv, const int8_t *kq, const int8_t *vq,
                                            const float *ks, const float *vs, const float *kb,
                                            const float *vb, const int *pos, int n_seq, int n_head,
                                            int n_kv_head, int head_dim, const int *tables,
                                            int block_size, int n_log, int qkv_stride,
                                            int out_stride) {
    MX_REQUIRE(kq && pos && tables, MX230_ERR_INVALID_ARG, "attn_decode_q8_batched: null argument");
    DecodeParams P = base_params(out, out_stride, qkv, qkv_stride, n_head, n_kv_head);
    set_q8(P, Q8_ARGS);
    P.pos_kind = 2, P.pos_dev = pos, P.tables = tables, P.bs = block_size, P.n_log = n_log;
    return launch_decode(h, stream, P, n_seq, head_dim, (long long)n_log * block_size);
}

// ---- contiguous per-sequence slabs, and split-KV partials ----
extern "C" int mx230_attn_decode_slab(mx230_handle *h, void *stream, float *out, const float *qkv,
                                      const float *kcache, const float *vcache, const int8_t *kq,
                                      const int8_t *vq, const float *ks, const float *vs,
                                      const float *kb, const float *vb, const int *pos, int n_seq,
                                      int n_head, int n_kv_head, int head_dim, long long seq_rows,
                                      int qkv_stride, int out_stride) {
    MX_REQUIRE(pos && seq_rows > 0, MX230_ERR_INVALID_ARG, "attn_decode_slab: null pos or bad seq_rows");
    DecodeParams P = base_params(out, out_stride, qkv, qkv_stride, n_head, n_kv_head);
    P.kcache = kcache, P.vcache = vcache;
    set_q8(P, Q8_ARGS);
    P.pos_kind = 2, P.pos_dev = pos, P.seq_rows = seq_rows;
    return launch_decode(h, stream, P, n_seq, head_dim, seq_rows);
}

extern "C" int mx230_attn_decode_partial(mx230_handle *h, void *stream, float *part_m,
                                         float *part_l, float *part_acc, const float *qkv,
                                         const float *kcache, const float *vcache,
                                         const int8_t *kq, const int8_t *vq, const float *ks,
                                         const float *vs, const float *kb, const float *vb, int t0,
                                         int t1, int n_seq, int n_head, int n_kv_head, int head_dim,
                                         long long seq_rows, int qkv_stride) {
    MX_REQUIRE(part_m && part_l && part_acc, MX230_ERR_INVALID_ARG,
               "attn_decode_partial: null partial output");
    MX_REQUIRE(seq_rows > 0 || n_seq == 1, MX230_ERR_INVALID_ARG, "attn_decode_partial: bad seq_rows");
    DecodeParams P = base_params(nullptr, 0, qkv, qkv_stride, n_head, n_kv_head);
    P.kcache = kcache, P.vcache = vcache;
    set_q8(P, Q8_ARGS);
    P.fin_m = part_m, P.fin_l = part_l, P.fin_acc = part_acc;
    P.range_mode = 1, P.t0 = t0, P.t1 = t1, P.seq_rows = seq_rows;
    return launch_decode(h, stream, P, n_seq, head_dim, (long long)t1 - t0);
}

int mx230_splitkv_push_neutral(mx230_splitkv_comm *c, void *stream, float *out);   // splitkv.cu

static int decode_push(mx230_handle *h, void *stream, mx230_splitkv_comm *c, float *out, const float *qkv,
                       const float *kcache, const float *vcache, const int8_t *kq, const int8_t *vq, const float *ks,
                       const float *vs, const float *kb, const float *vb, int t0, int t1, int n_seq, int n_head,
                       int n_kv_head, int head_dim, long long seq_rows, int qkv_stride) {
    MX_REQUIRE(h && c, MX230_ERR_INVALID_ARG, "split-KV decode: null argument");
    MX_REQUIRE(c->h == h, MX230_ERR_INVALID_ARG, "split-KV decode: the communicator belongs to another handle");
    MX_REQUIRE((long long)n_seq * n_head == c->rows, MX230_ERR_INVALID_ARG,
               "split-KV decode: n_seq * n_head = %lld, the communicator was made for %d rows",
               (long long)n_seq * n_head, c->rows);
    for (int p = 0; p < c->world; ++p)
        MX_REQUIRE(c->region[p], MX230_ERR_INVALID_ARG, "split-KV decode: rank %d is not connected", p);
    if (t1 <= t0) return mx230_splitkv_push_neutral(c, stream, out);   // an empty key range contributes (-inf, 0, 0)
    MX_REQUIRE(seq_rows > 0 || n_seq == 1, MX230_ERR_INVALID_ARG, "split-KV decode: bad seq_rows");
    DecodeParams P = base_params(nullptr, 0, qkv, qkv_stride, n_head, n_kv_head);
    P.kcache = kcache, P.vcache = vcache;
    set_q8(P, Q8_ARGS);
    P.fin_m = c->local, P.fin_l = c->local + c->rows, P.fin_acc = c->local + 2 * (size_t)c->rows;
    P.range_mode = 1, P.t0 = t0, P.t1 = t1, P.seq_rows = seq_rows;
    P.push_regions = c->region_dev;
    P.push_steps = (unsigned *)(c->region[c->rank] + c->step_offset_words);
    P.push_out = out;
    P.push_status = h->status_dev;
    P.push_part_words = c->part_words;
    P.push_rank = c->rank, P.push_world = c->world, P.push_rows = c->rows;
    return launch_decode(h, stream, P, n_seq, head_dim, (long long)t1 - t0, c);
}

extern "C" int mx230_attn_decode_partial_push(mx230_handle *h, void *stream, mx230_splitkv_comm *c, const float *qkv,
                                              const float *kcache, const float *vcache, const int8_t *kq,
                                              const int8_t *vq, const float *ks, const float *vs, const float *kb,
                                              const float *vb, int t0, int t1, int n_seq, int n_head, int n_kv_head,
                                              int head_dim, long long seq_rows, int qkv_stride) {
    return decode_push(h, stream, c, nullptr, qkv, kcache, vcache, Q8_ARGS, t0, t1, n_seq, n_head, n_kv_head, head_dim,
                       seq_rows, qkv_stride);
}

extern "C" int mx230_attn_decode_splitkv(mx230_handle *h, void *stream, mx230_splitkv_comm *c, float *out,
                                         const float *qkv, const float *kcache, const float *vcache, const int8_t *kq,
                                         const int8_t *vq, const float *ks, const float *vs, const float *kb,
                                         const float *vb, int t0, int t1, int n_seq, int n_head, int n_kv_head,
                                         int head_dim, long long seq_rows, int qkv_stride) {
    MX_REQUIRE(out && (((uintptr_t)out) & 15) == 0, MX230_ERR_INVALID_ARG,
               "attn_decode_splitkv: out must be a 16-byte aligned device pointer");
    return decode_push(h, stream, c, out, qkv, kcache, vcache, Q8_ARGS, t0, t1, n_seq, n_head, n_kv_head, head_dim,
                       seq_rows, qkv_stride);
}

extern "C" int mx230_merge_partials(mx230_handle *h, void *stream, float *out, const float *m,
                                    const float *l, const float *acc, int parts, int rows,
                                    int head_dim) {
    MX_REQUIRE(h && out && m && l && acc, MX230_ERR_INVALID_ARG, "merge_partials: null argument");
    MX_REQUIRE(head_dim == 64, MX230_ERR_UNSUPPORTED, "merge_partials: head_dim must be 64");
    MX_REQUIRE(parts > 0 && rows >= 0, MX230_ERR_INVALID_ARG, "merge_partials: bad sizes");
    if (rows == 0) return MX230_OK;
    mx230_device_guard guard(h->device);
    cudaStream_t st = (cudaStream_t)stream;
    MX_LAUNCH(h, st, MX230_K_MERGE,
              (merge_partials_kernel<<<(rows * 16 + 127) / 128, 128, 0, st>>>(out, m, l, acc, parts, rows, (size_t)rows,
                                                                              (size_t)rows * 64)));
    return MX230_OK;
}

extern "C" int mx230_merge_partials_packed(mx230_handle *h, void *stream, float *out, const float *gathered,
                                           int parts, int rows, int head_dim) {
    MX_REQUIRE(h && out && gathered, MX230_ERR_INVALID_ARG, "merge_partials_packed: null argument");
    MX_REQUIRE(head_dim == 64, MX230_ERR_UNSUPPORTED, "merge_partials_packed: head_dim must be 64");
    MX_REQUIRE(parts > 0 && rows >= 0, MX230_ERR_INVALID_ARG, "merge_partials_packed: bad sizes");
    MX_REQUIRE(rows % 2 == 0 && (((uintptr_t)gathered) & 15) == 0, MX230_ERR_INVALID_ARG,
               "merge_partials_packed: rows must be even and the buffer 16-byte aligned");
    if (rows == 0) return MX230_OK;
    mx230_device_guard guard(h->device);
    cudaStream_t st = (cudaStream_t)stream;
    const size_t f = (size_t)rows * 66;   // floats per part: [m | l | acc]
    MX_LAUNCH(h, st, MX230_K_MERGE,
              (merge_partials_kernel<<<(rows * 16 + 127) / 128, 128, 0, st>>>(out, gathered, gathered + rows,
                                                                              gathered + 2 * (size_t)rows, parts, rows, f, f)));
    return MX230_OK;
}

// ---------------------------------------------------------------------------
// Decode over an int8 cache for callers that must not allocate.
//
// Every other entry point works through a handle, and a handle's split-KV scratch (partial
// (m, l, acc) triples and arrival counters) comes from cudaMalloc.  Some hosts cannot do that
// at the point where they first need attention: an engine that has already handed every free
// byte of HBM to its KV-block pool (cudaMalloc would fail), or a component that is only
// allowed to enqueue work on a stream it was given and must not touch the allocator (cudaMalloc
// can block on the whole device).  For them this one entry point takes no handle and keeps its
// scratch in a fixed array inside the library image.
//
//  * The array is NOALLOC_SCRATCH_BYTES (1 MiB + 4 KiB) per GPU that loads the library and stays
//    resident until the process exits.  A call needs n_head * n_splits * 264 bytes of it
//    (n_splits <= 64) plus n_kv_head counters; a shape that does not fit is refused with
//    MX230_ERR_WORKSPACE.  Single sequence, contiguous cache, reference score mode.  It always runs the
//    CUDA-core kernel (decode_q8_kernel), not the tensor-core one that handle-based calls default to: the same
//    results as mx230_attn_decode_q8 to rounding, but for GQA groups a fraction of its bandwidth.
//  * The first call on each device resolves the array's device address (the name of a __device__
//    array is not a device pointer in host code) and reads the SM count, under a process-wide lock, so
//    first calls from several host threads are safe; make that first call outside of any stream capture.
//  * All calls on a device share the array.  It keeps what the previous call left there: the
//    counters are cleared on the stream before every launch, the partials are always rewritten
//    before they are read.  Two calls that overlap on the GPU (different streams) race on it.
//  * It calls no cudaMalloc / cudaFree and nothing that allocates.
// ---------------------------------------------------------------------------
namespace {

constexpr size_t NOALLOC_PARTIAL_BYTES = 1u << 20;
constexpr size_t NOALLOC_COUNTER_BYTES = 4096;
constexpr size_t NOALLOC_SCRATCH_BYTES = NOALLOC_PARTIAL_BYTES + NOALLOC_COUNTER_BYTES;
static __device__ __align__(256) unsigned char g_noalloc_scratch[NOALLOC_SCRATCH_BYTES];

constexpr int NOALLOC_MAX_DEVICES = 64;
struct NoallocDevice {
    void *scratch;  // device address of g_noalloc_scratch on this device
    int sm_count;
};
NoallocDevice g_noalloc_dev[NOALLOC_MAX_DEVICES];  // zero-initialised: scratch == nullptr means "not set up"
std::mutex g_noalloc_mutex;                       // guards the one-time set-up of an entry above

template <int G>
int noalloc_launch(int device, cudaStream_t st, const DecodeParams &P, dim3 grid) {
    const size_t sm = q8_smem_bytes<G>();
    MX_SMEM_ATTR_ONCE(device, (decode_q8_kernel<G, false>), sm);
    decode_q8_kernel<G, false><<<grid, Q8_THREADS, sm, st>>>(P);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess)
        return mx230_fail(MX230_ERR_CUDA, "attn_decode_q8_noalloc: launch failed: %s", cudaGetErrorString(e));
    return MX230_OK;
}

}  // namespace

extern "C" int mx230_attn_decode_q8_noalloc(void *stream, float *out, const float *qkv, const int8_t *kq,
                                            const int8_t *vq, const float *ks, const float *vs,
                                            const float *kb, const float *vb, int t_cur, int n_head,
                                            int n_kv_head, int head_dim) {
    const char *who = "attn_decode_q8_noalloc";
    MX_REQUIRE(out && qkv && kq && vq && ks && vs, MX230_ERR_INVALID_ARG, "%s: null argument", who);
    MX_REQUIRE((kb == nullptr) == (vb == nullptr), MX230_ERR_INVALID_ARG,
               "%s: kb and vb must both be given (affine) or both be null (absmax)", who);
    MX_REQUIRE(head_dim == 64, MX230_ERR_UNSUPPORTED, "%s: head_dim %d unsupported (must be 64)", who, head_dim);
    MX_REQUIRE(n_head > 0 && n_kv_head > 0 && n_head % n_kv_head == 0, MX230_ERR_UNSUPPORTED,
               "%s: n_head %d must be a positive multiple of n_kv_head %d", who, n_head, n_kv_head);
    MX_REQUIRE(t_cur >= 0, MX230_ERR_INVALID_ARG, "%s: negative position %d", who, t_cur);
    MX_REQUIRE((((uintptr_t)qkv | (uintptr_t)out | (uintptr_t)kq | (uintptr_t)vq) & 15) == 0,
               MX230_ERR_INVALID_ARG, "%s: buffers must be 16-byte aligned", who);

    int dev = -1;
    MX_CHECK_CUDA(cudaGetDevice(&dev));
    MX_REQUIRE(dev >= 0 && dev < NOALLOC_MAX_DEVICES, MX230_ERR_UNSUPPORTED, "%s: device %d out of range", who, dev);
    NoallocDevice &nd = g_noalloc_dev[dev];
    {
        // one-time set-up for this device, with this device current; host threads making their first calls
        // at the same time are serialised here (later calls only take the uncontended lock)
        std::lock_guard<std::mutex> lock(g_noalloc_mutex);
        if (nd.scratch == nullptr) {
            int major = 0;
            MX_CHECK_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
            MX_REQUIRE(major == 10, MX230_ERR_NO_DEVICE, "%s: device %d is not sm_100", who, dev);
            int sms = 0;
            MX_CHECK_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
            void *p = nullptr;
            cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
            if (e != cudaSuccess || p == nullptr)
                return mx230_fail(MX230_ERR_CUDA, "%s: cudaGetSymbolAddress failed: %s", who, cudaGetErrorString(e));
            nd.sm_count = sms;
            nd.scratch = p;
        }
    }

    DecodeParams P;
    memset(&P, 0, sizeof(P));
    P.out = out;
    P.out_stride = n_head * 64;
    P.qkv = qkv;
    P.n_head = n_head;
    P.n_kv_head = n_kv_head;
    P.kq = kq, P.vq = vq, P.ks = ks, P.vs = vs, P.kb = kb, P.vb = vb;
    P.pos_kind = 0;
    P.pos = t_cur;
    P.group = n_head / n_kv_head;
    P.head_groups = (P.group + 7) / 8;
    P.score_mode = MX230_Q8_SCORE_REF;
    const int gy = n_kv_head * P.head_groups;
    MX_REQUIRE((size_t)gy * sizeof(unsigned) <= NOALLOC_COUNTER_BYTES, MX230_ERR_WORKSPACE,
               "%s: %d kv-head groups exceed the %zu built-in counters", who, gy,
               NOALLOC_COUNTER_BYTES / sizeof(unsigned));

    // same split rule as the handle path: fill the machine in one wave, >= 256 keys per split
    const long long keys = (long long)t_cur + 1;
    int n_splits = (int)((2LL * nd.sm_count) / gy);
    const int max_by_len = (int)((keys + 255) / 256);
    if (n_splits > max_by_len) n_splits = max_by_len;
    if (n_splits > 64) n_splits = 64;
    if (n_splits < 1) n_splits = 1;
    const size_t rows = (size_t)n_head * n_splits;
    const size_t need = rows * 66 * sizeof(float);
    MX_REQUIRE(need <= NOALLOC_PARTIAL_BYTES, MX230_ERR_WORKSPACE,
               "%s: n_head %d x %d key splits needs %zu B of scratch, the built-in array holds %zu B", who,
               n_head, n_splits, need, NOALLOC_PARTIAL_BYTES);
    P.ws_acc = (float *)nd.scratch;
    P.ws_m = P.ws_acc + rows * 64;
    P.ws_l = P.ws_m + rows;
    P.counters = (unsigned *)((unsigned char *)nd.scratch + NOALLOC_PARTIAL_BYTES);

    cudaStream_t st = (cudaStream_t)stream;
    // the arrival counters must start at zero whatever an earlier call left behind
    MX_CHECK_CUDA(cudaMemsetAsync(P.counters, 0, (size_t)gy * sizeof(unsigned), st));
    dim3 grid(n_splits, gy, 1);
    const int g = P.group > 8 ? 8 : P.group;
    if (g == 1) return noalloc_launch<1>(dev, st, P, grid);
    if (g == 2) return noalloc_launch<2>(dev, st, P, grid);
    if (g <= 4) return noalloc_launch<4>(dev, st, P, grid);
    if (g <= 7) return noalloc_launch<7>(dev, st, P, grid);
    return noalloc_launch<8>(dev, st, P, grid);
}
