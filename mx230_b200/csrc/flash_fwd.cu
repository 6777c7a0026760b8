// Flash-attention forward for sm_100a: O = softmax(scale * Q K^T [+ causal]) V and
// the per-row log-sum-exp L = m + ln(l), never materialising the N x N scores.
//
// Reference semantics: flash_fwd / attn_flash / attn_flash_lse,
// 02-flash-attention/kernels/attention_flash.cu:17-100 (fp32 SIMT, one thread per
// query row).  This kernel keeps those semantics (scale 1/sqrt(64), key j <= query i
// when causal, any N, natural-log L) and maps the two contractions onto the 5th-gen
// tensor cores:
//
//   * a work item is 256 query rows of one head as two 128-row tiles; the kernel is persistent:
//     one CTA per SM walks a fixed share of the items (heaviest first, dealt out in snake order so
//     that every CTA gets the same number of key tiles), and every role runs ahead into the next
//     item on its own, so the next item's Q / K loads and first Q K^T run under the current
//     item's last softmax and its epilogue;
//   * warps 0-15 are four softmax warpgroups, two per query tile (tile t = warp / 8), each taking 64 of
//     the 128 key columns of every score tile, one thread per (query row, half): the thread pulls its
//     columns into registers 32 at a time (the second piece lands under the first one's exponentials),
//     which frees S_t for the next Q K^T, takes exp2 and the row sum, and writes bf16 P into its own
//     tensor-memory columns.  Usually without a row max (see the fixed-reference mode below: the
//     halves of a row then meet only once per item, to add their sums); otherwise the halves exchange
//     their part of the row max through shared memory and O_t is rescaled in tensor memory only when
//     the max grows by > 2^8;
//   * warp 16 streams Q (two buffers, alternating by item) and K/V tiles (128 keys) through a
//     4-stage shared-memory ring with plain per-CTA TMA tile loads (128-byte swizzle);
//   * warp 17 issues the tcgen05.mma stream S_t = Q_t K^T into tensor memory (128 fp32 columns
//     per tile), warp 18 the stream O_t += P_t V with P_t read from tensor memory as bf16 (each
//     stream has its own warp, which runs its loop warp-uniformly with one elected lane issuing).
//   The two tiles ping-pong and S, P, O never alias, so the tensor core computes the next
//   scores and the other tile's P V while a tile's softmax runs on the CUDA cores.
//
// Operands are bf16 (rounded once by the cast pre-pass), accumulation is fp32.
#include <math_constants.h>

#include <cstring>
#include <type_traits>

#include "common.cuh"

namespace {

constexpr int BM = 128;        // query rows per tile
constexpr int QT = 2;          // query tiles per CTA
constexpr int BN = 128;        // keys per K/V tile
constexpr int HD = 64;
constexpr int KV_STAGES = 4;
constexpr int TILE_BYTES = BN * HD * 2;  // 16 KB
constexpr int HALVES = 2;               // softmax groups per query tile: each takes half of the tile's key columns
constexpr int SOFT_WARPS = QT * HALVES * 4;   // 16
constexpr int FWD_THREADS = (SOFT_WARPS + 4) * 32;   // 640: four softmax warpgroups + {TMA, 2 MMA issuers, idle}
// setmaxnreg moves registers only inside the CTA's launch-time allocation (96 per thread for 640
// threads): what the softmax warps gain must have been released by the service warpgroup, or the
// increase would block for ever.
#ifndef FWD_REGS_SOFTMAX
#define FWD_REGS_SOFTMAX 104
#define FWD_REGS_SERVICE 64
#endif
static_assert(SOFT_WARPS * FWD_REGS_SOFTMAX + 4 * FWD_REGS_SERVICE <= (SOFT_WARPS + 4) * 96, "setmaxnreg budget exceeds the launch-time register allocation");

// build-time knobs of the softmax loop
#ifndef FWD_FAST
#define FWD_FAST 1        // fixed-reference mode (no row max, no subtraction) while the sums stay in range
#endif
#ifndef FWD_POLY
#define FWD_POLY 1        // of every FWD_POLY_DEN column pairs, how many take 2^x from the FMA-pipe polynomial (with four
                          // softmax warps per scheduler the loop is issue-bound: 1 of 4 beats 2 of 4 by 7-10 %, 0 of 4 loses 9 %)
#endif
#ifndef FWD_POLY_DEN
#define FWD_POLY_DEN 4
#endif
#ifndef FWD_ADD2
#define FWD_ADD2 1        // row sums with packed f32x2 adds
#endif

#ifndef FWD_UNIFORM_ISSUE
#define FWD_UNIFORM_ISSUE 1   // MMA issuer warps run warp-uniform with one elected lane (0: a lone lane in a divergent branch)
#endif
#if FWD_UNIFORM_ISSUE
#define ISSUER_WAIT(w) __all_sync(0xFFFFFFFFu, (w))
#define ISSUER_LANE mx::elect_one()
#else
#define ISSUER_WAIT(w) (w)
#define ISSUER_LANE true
#endif

constexpr int Q_BUFS = 2;                // Q of the next item lands while the current one is in use
constexpr int SMEM_Q = 0;
constexpr int SMEM_K = SMEM_Q + Q_BUFS * QT * TILE_BYTES;
constexpr int SMEM_V = SMEM_K + KV_STAGES * TILE_BYTES;
constexpr int SMEM_BAR = SMEM_V + KV_STAGES * TILE_BYTES;
constexpr int SMEM_XCH = SMEM_BAR + 512;   // [2 item parities][QT][2][BM] floats: row sums handed from the second half of a tile to the first
constexpr int SMEM_XMAX = SMEM_XCH + 2 * QT * 2 * BM * 4;   // [QT][2 tile parities][HALVES][BM] floats: row-max parts of the general mode
constexpr int SMEM_TOTAL = SMEM_XMAX + QT * 2 * HALVES * BM * 4;
constexpr int SMEM_ALLOC = SMEM_TOTAL + 1024;  // slack for 1024-byte alignment

// barrier slots (8 bytes each) inside SMEM_BAR
constexpr int BAR_Q_FULL = 0;                    // [Q_BUFS]
constexpr int BAR_Q_EMPTY = BAR_Q_FULL + Q_BUFS; // [Q_BUFS] softmax warps -> TMA: item done with its Q buffer
constexpr int BAR_K_FULL = BAR_Q_EMPTY + Q_BUFS; // [KV_STAGES]
constexpr int BAR_K_EMPTY = BAR_K_FULL + KV_STAGES;
constexpr int BAR_V_FULL = BAR_K_EMPTY + KV_STAGES;
constexpr int BAR_V_EMPTY = BAR_V_FULL + KV_STAGES;
constexpr int BAR_S_FULL = BAR_V_EMPTY + KV_STAGES;  // [QT] MMA -> softmax: S_t written
constexpr int BAR_S_FREE = BAR_S_FULL + QT;          // [QT] softmax -> MMA: S_t copied to registers
constexpr int BAR_P_FULL = BAR_S_FREE + QT;          // [QT] softmax -> MMA: P_t written
constexpr int BAR_O_DONE = BAR_P_FULL + QT;          // [QT] MMA -> softmax: O_t += P_t V complete
constexpr int BAR_XCH = BAR_O_DONE + QT;             // [QT] second half of tile t -> first half: its row sums are published
constexpr int BAR_XMAX = BAR_XCH + QT;               // [QT] general mode: both halves of tile t have published their part of the row max
constexpr int N_BARS = BAR_XMAX + QT;                // 32

// tensor-memory columns: nothing aliases, so S_t(j+1) can be produced while P_t(j) is consumed
constexpr int TM_S = 0;     // S_t at TM_S + t*128, fp32
constexpr int TM_P = 256;   // P_t at TM_P + t*64, bf16 pairs
constexpr int TM_O = 384;   // O_t at TM_O + t*64, fp32
constexpr int TM_COLS = 512;

// The running row max is only raised when it would grow by more than 2^RESCALE_LOG2 in the
// exponent; until then probabilities are taken against the stale max (they stay below
// 2^RESCALE_LOG2, harmless in bf16/fp32) and O needs no rescale.
constexpr float RESCALE_LOG2 = 8.0f;

struct FwdParams {
    float *O;             // row r of head h at O + h*o_head_stride + r*o_row_stride (floats)
    float *L;             // [heads][n_q] or null
    long long o_head_stride, o_row_stride;
    int n_q;              // query rows per head
    int n_k;              // keys per head
    int q_off;            // causal: query row r sees keys <= r + q_off (0 for self-attention)
    int kv_group;         // query heads per K/V head (K/V head of query head h is h / kv_group)
    int causal;
    int heads;            // query heads (items are (query block, head) pairs, heads fastest)
    int item_tiles;       // query tiles per work item: QT, or 1 when two-tile items would leave SMs without work
    int n_qblocks;        // blocks of item_tiles*BM query rows per head
    int n_items;          // heads * n_qblocks
    int tma_out;          // O leaves through staged TMA stores (strides and base 16-byte aligned) or per-thread stores
    int prescaled;        // Q was staged multiplied by scale * log2(e): the scores arrive in log2 units
    const float *q_norm2; // [heads][MX230_NORM_PARTS] largest squared row norm of the unscaled Q per head and part, or null
    const float *k_norm2; // [heads / kv_group][MX230_NORM_PARTS] the same for K
    int test_drop_tile;   // test hook: K/V tile (counted over the CTA's items) that CTA 0's producer never requests; -1 = off
    // int8 score mode (prefill over an int8 cache with the reference kernel's arithmetic): Q and K hold int8 CODES
    // (exact in bf16), so the MMA returns exact integer dots, and the score is rebuilt per element as
    // row_a[i] * (dot * ks[j] + row_qsum[i] * kb[j]) in log2 units (03-llm-engine/kernels/llm.cu:3774-3782)
    const float *row_a;      // [heads][n_q]   q scale * 1/sqrt(64) * log2(e), or null = mode off
    const float *row_qsum;   // [heads][n_q]   sum of the row's q codes
    const float2 *col_kskb;  // [heads / kv_group][n_k_pad] (scale, offset) of every key
    int n_k_pad;             // n_k rounded up to a multiple of BN
    int *status;
};

__device__ __forceinline__ float fmax3(float a, float b, float c) {
    float r;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}

// The CTA's `round`-th work item.  Items are listed heaviest first (when causal: the latest query block of
// every head, then the one before, ...) and dealt to the CTAs forwards in even rounds, backwards in odd ones.
__device__ __forceinline__ bool fwd_item(const FwdParams &P, int round, int &bh, int &q0) {
    const int G = (int)gridDim.x, c = (int)blockIdx.x;
    const int i = round * G + ((round & 1) ? G - 1 - c : c);
    if (i >= P.n_items) return false;
    const int rank = i / P.heads;
    bh = i - rank * P.heads;
    q0 = (P.causal ? P.n_qblocks - 1 - rank : rank) * (P.item_tiles * BM);
    return true;
}
// K/V tiles that query tile `t` of the block starting at row q0 has to see
__device__ __forceinline__ int fwd_tile_iters(const FwdParams &P, int q0, int t) {
    const int r0 = q0 + t * BM;
    if (r0 >= P.n_q || t >= P.item_tiles) return 0;
    const int n_kv_total = (P.n_k + BN - 1) / BN;
    return P.causal ? min(n_kv_total, (r0 + BM - 1 + P.q_off) / BN + 1) : n_kv_total;
}

__global__ void __launch_bounds__(FWD_THREADS, 1)
flash_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmO,
                 const FwdParams P) {
    extern __shared__ unsigned char smem_dyn[];
    const uint32_t smem_base = (mx::smem_u32(smem_dyn) + 1023u) & ~1023u;
    unsigned char *smem = smem_dyn + (smem_base - mx::smem_u32(smem_dyn));
    const uint32_t bar0 = smem_base + SMEM_BAR;
    auto bar = [&](int i) { return bar0 + 8u * (uint32_t)i; };
    volatile uint32_t *tmem_slot = (volatile uint32_t *)(smem + SMEM_BAR + 8 * N_BARS);
    volatile int *abort_flag = (volatile int *)(smem + SMEM_BAR + 8 * N_BARS + 8);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int NQ = P.n_q, N = P.n_k;  // N: keys (bounds the K/V loop and the key mask)

    if (tid == 0) {
        for (int b = 0; b < Q_BUFS; ++b) {
            mx::mbar_init(bar(BAR_Q_FULL + b), 1);
            mx::mbar_init(bar(BAR_Q_EMPTY + b), SOFT_WARPS);  // one elected lane per softmax warp arrives
        }
        for (int s = 0; s < KV_STAGES; ++s) {
            mx::mbar_init(bar(BAR_K_FULL + s), 1);
            mx::mbar_init(bar(BAR_K_EMPTY + s), 1);
            mx::mbar_init(bar(BAR_V_FULL + s), 1);
            mx::mbar_init(bar(BAR_V_EMPTY + s), 1);
        }
        for (int t = 0; t < QT; ++t) {
            mx::mbar_init(bar(BAR_S_FULL + t), 1);
            mx::mbar_init(bar(BAR_S_FREE + t), HALVES * BM / 32);  // one elected lane per warp of the tile's groups arrives
            mx::mbar_init(bar(BAR_P_FULL + t), HALVES * BM / 32);
            mx::mbar_init(bar(BAR_O_DONE + t), 1);
            mx::mbar_init(bar(BAR_XCH + t), BM / 32);
            mx::mbar_init(bar(BAR_XMAX + t), HALVES * BM / 32);
        }
        *abort_flag = 0;
        mx::mbar_fence_init();
    }
    if (warp == SOFT_WARPS + 1) mx::tmem_alloc(mx::smem_u32((const void *)tmem_slot), TM_COLS);
    mx::tc_fence_before();
    __syncthreads();
    mx::tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    // register budget: a softmax thread holds 64 score values and their packed probabilities, the
    // service warpgroup (TMA, two MMA issuers, one idle warp) needs few
    if (warp >= SOFT_WARPS) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(FWD_REGS_SERVICE));
        if (warp == SOFT_WARPS) {
        // ------------------------- TMA producer -------------------------
        if (lane == 0) {
            mx::tma_prefetch_desc(&tmQ);
            mx::tma_prefetch_desc(&tmK);
            mx::tma_prefetch_desc(&tmV);
            bool ok = true;
            uint32_t g = 0;  // K/V tiles loaded so far, over all items: ring slot g % KV_STAGES, use g / KV_STAGES
            int bh, q0;
            for (int it = 0; ok && fwd_item(P, it, bh, q0); ++it) {
                const int n_it1 = fwd_tile_iters(P, q0, 1);
                const int n_max = max(fwd_tile_iters(P, q0, 0), n_it1);
                const int qbuf = it & 1;
                // the buffer's previous item (two items ago) must have staged its last O piece out of it
                if (it >= Q_BUFS) ok = mx::mbar_wait(bar(BAR_Q_EMPTY + qbuf), ((it >> 1) - 1) & 1, abort_flag, P.status);
                if (!ok) break;
                const int nq = (n_it1 > 0) ? 2 : 1;
                mx::mbar_expect_tx(bar(BAR_Q_FULL + qbuf), nq * TILE_BYTES);
                for (int t = 0; t < nq; ++t)
                    mx::tma_load_3d(smem_base + SMEM_Q + (qbuf * QT + t) * TILE_BYTES, &tmQ, bar(BAR_Q_FULL + qbuf), 0,
                                    q0 + t * BM, bh);
                const int kvh = bh / P.kv_group;
                for (int j = 0; j < n_max; ++j, ++g) {
                    const int s = g % KV_STAGES;
                    const uint32_t r = g / KV_STAGES;
                    if (r > 0) ok = mx::mbar_wait(bar(BAR_K_EMPTY + s), (r - 1) & 1, abort_flag, P.status);
                    if (!ok) break;
                    if (P.test_drop_tile == (int)g && blockIdx.x == 0) continue;   // test hook: this tile never arrives
                    mx::mbar_expect_tx(bar(BAR_K_FULL + s), TILE_BYTES);
                    mx::tma_load_3d(smem_base + SMEM_K + s * TILE_BYTES, &tmK, bar(BAR_K_FULL + s), 0,
                                    j * BN, kvh);
                    if (r > 0) ok = mx::mbar_wait(bar(BAR_V_EMPTY + s), (r - 1) & 1, abort_flag, P.status);
                    if (!ok) break;
                    mx::mbar_expect_tx(bar(BAR_V_FULL + s), TILE_BYTES);
                    mx::tma_load_3d(smem_base + SMEM_V + s * TILE_BYTES, &tmV, bar(BAR_V_FULL + s), 0,
                                    j * BN, kvh);
                }
            }
        }
        __syncwarp();
        } else if (warp == SOFT_WARPS + 1) {
        // ------------------------- MMA issuer 1: S_t = Q_t K^T ----------
        // The whole warp runs the loop and the waits; one elected lane issues.  Control flow and descriptor
        // arithmetic stay warp-uniform that way (a lone thread inside a divergent branch pays several dependent
        // instructions per tcgen05.mma to move its operands to the uniform registers the instruction reads).
        if (FWD_UNIFORM_ISSUE || lane == 0) {
            constexpr uint32_t IDESC_S = mx::mma_idesc_bf16(BM, BN, false, false);
            bool ok = true;
            uint32_t g = 0;            // K/V tiles consumed so far, over all items
            uint32_t cs[QT] = {0, 0};  // score tiles issued so far per query tile, over all items
            int bh, q0;
            for (int it = 0; ok && fwd_item(P, it, bh, q0); ++it) {
                int n_it[QT];
#pragma unroll
                for (int t = 0; t < QT; ++t) n_it[t] = fwd_tile_iters(P, q0, t);
                const int n_max = max(n_it[0], n_it[1]);
                const int qbuf = it & 1;
                ok = ISSUER_WAIT(mx::mbar_wait(bar(BAR_Q_FULL + qbuf), (it >> 1) & 1, abort_flag, P.status));
                for (int j = 0; j < n_max && ok; ++j, ++g) {
                    const int s = g % KV_STAGES;
                    ok = ISSUER_WAIT(mx::mbar_wait(bar(BAR_K_FULL + s), (g / KV_STAGES) & 1, abort_flag, P.status));
                    const uint64_t b = mx::smem_desc_sw128(smem_base + SMEM_K + s * TILE_BYTES);
#pragma unroll
                    for (int t = 0; t < QT; ++t) {
                        if (!ok || j >= n_it[t]) continue;
                        // next scores as soon as the softmax group holds the previous ones in registers (the
                        // previous ones may be the last of the item before: this is where the items overlap)
                        if (cs[t] > 0) ok = ISSUER_WAIT(mx::mbar_wait(bar(BAR_S_FREE + t), (cs[t] - 1) & 1, abort_flag, P.status));
                        if (!ok) continue;
                        mx::tc_fence_after();
                        const uint64_t a = mx::smem_desc_sw128(smem_base + SMEM_Q + (qbuf * QT + t) * TILE_BYTES);
                        if (ISSUER_LANE) {
#pragma unroll
                            for (int k = 0; k < HD / 16; ++k)  // 32 bytes per 16-element step inside the swizzle span
                                mx::mma_ss(tmem + TM_S + t * BN, a + 2 * k, b + 2 * k, IDESC_S, k > 0);
                            mx::mma_commit(bar(BAR_S_FULL + t));
                        }
                        ++cs[t];
                    }
                    if (!ok) break;
                    if (ISSUER_LANE) mx::mma_commit(bar(BAR_K_EMPTY + s));
                }
            }
        }
        __syncwarp();
        } else if (warp == SOFT_WARPS + 2) {
        // ------------------------- MMA issuer 2: O_t += P_t V -----------
        if (FWD_UNIFORM_ISSUE || lane == 0) {
            constexpr uint32_t IDESC_O = mx::mma_idesc_bf16(BM, HD, false, true);
            bool ok = true;
            uint32_t g = 0;            // K/V tiles consumed so far, over all items
            uint32_t cp[QT] = {0, 0};  // P tiles consumed so far per query tile, over all items
            int bh, q0;
            for (int it = 0; ok && fwd_item(P, it, bh, q0); ++it) {
                int n_it[QT];
#pragma unroll
                for (int t = 0; t < QT; ++t) n_it[t] = fwd_tile_iters(P, q0, t);
                const int n_max = max(n_it[0], n_it[1]);
                for (int j = 0; j < n_max && ok; ++j, ++g) {
                    const int s = g % KV_STAGES;
                    ok = ISSUER_WAIT(mx::mbar_wait(bar(BAR_V_FULL + s), (g / KV_STAGES) & 1, abort_flag, P.status));
                    const uint64_t b = mx::smem_desc_sw128(smem_base + SMEM_V + s * TILE_BYTES);
#pragma unroll
                    for (int t = 0; t < QT; ++t) {
                        if (!ok || j >= n_it[t]) continue;
                        // an item's first P_t is written after the softmax group has taken the previous item's
                        // O_t out of tensor memory, so overwriting O_t (j == 0) needs no barrier of its own
                        ok = ISSUER_WAIT(mx::mbar_wait(bar(BAR_P_FULL + t), cp[t] & 1, abort_flag, P.status));
                        if (!ok) continue;
                        mx::tc_fence_after();
                        if (ISSUER_LANE) {
#pragma unroll
                            for (int k = 0; k < BN / 16; ++k)  // 16 keys: 8 packed columns of P, 2048 bytes of V
                                mx::mma_ts(tmem + TM_O + t * HD, tmem + TM_P + t * (BN / 2) + 8 * k, b + 128 * k,
                                           IDESC_O, (j > 0 || k > 0));
                            mx::mma_commit(bar(BAR_O_DONE + t));
                        }
                        ++cp[t];
                    }
                    if (!ok) break;
                    if (ISSUER_LANE) mx::mma_commit(bar(BAR_V_EMPTY + s));
                }
            }
        }
        __syncwarp();
        }
    } else {
        // ------------------------- softmax groups -----------------------
        // Four groups: tile t = warp / 8 has two, each taking 64 of the 128 key columns of every score tile (one thread
        // per query row and half).  Four softmax warps per scheduler instead of two hide each other's dependent-issue
        // latencies; without a row max (the usual mode) the halves never talk to each other inside the loop, and the
        // general mode has each half compute the full row's max redundantly rather than exchange it.
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(FWD_REGS_SOFTMAX));
        const int t = warp >> 3;             // query tile of this group
        const int half = (warp >> 2) & 1;    // which 64 key columns of every tile
        const int row_in_tile = (warp & 3) * 32 + lane;
        const uint32_t lane_off = (uint32_t)((warp & 3) * 32) << 16;
        const uint32_t tm_s_tile = tmem + lane_off + TM_S + t * BN;
        const uint32_t tm_s = tm_s_tile + half * (BN / 2);
        const uint32_t tm_p = tmem + lane_off + TM_P + t * (BN / 2) + half * (BN / 4);
        const uint32_t tm_o = tmem + lane_off + TM_O + t * HD;
        // Scores arrive in log2 units when Q was staged pre-multiplied by scale * log2(e) (c = 1), else raw (c = scale * log2(e)).
        const bool i8_scores = P.row_a != nullptr;   // scores rebuilt from integer dots: already in log2 units
        const float c = (P.prescaled || i8_scores) ? 1.0f : 0.125f * 1.4426950408889634f;
        const float l_scale = (P.prescaled || i8_scores) ? 0.6931471805599453f : 0.125f;   // running max -> natural-log units
        bool ok = true;
        uint32_t cnt = 0;  // score tiles this group has taken so far, over all items
        uint32_t xmc = 0;  // row-max exchanges this group has made so far (general-mode tiles only)
        int bh, q0;
        for (int it = 0; ok && fwd_item(P, it, bh, q0); ++it) {
        const int n_t = fwd_tile_iters(P, q0, t);
        const int row = q0 + t * BM + row_in_tile;
        const int qbuf = it & 1;
        const int last = P.causal ? min(N - 1, row + P.q_off) : N - 1;  // last visible key of this row
        // Fixed-reference mode, chosen per head: when |q . k| * scale * log2(e) <= 80 for every row pair of the head --
        // by Cauchy-Schwarz from the largest row norms of Q and K that the staging pass left -- the probabilities are
        // taken as 2^s against the reference 0: no row max, no subtraction, no rescale of O.  bf16 probabilities and
        // fp32 sums carry the same relative precision at 2^-80 .. 2^80 as around 1, every row sum stays inside
        // [2^-80, N 2^80], and the result is that of the max-subtracted form.  Heads with larger scores (and calls
        // without the norms) take the general path: running max, lazy rescale.
        bool fast = false;
        if (FWD_FAST && P.q_norm2 != nullptr) {
            float nq = 0.0f, nk = 0.0f;
            if (lane < MX230_NORM_PARTS) {
                nq = P.q_norm2[(size_t)bh * MX230_NORM_PARTS + lane];
                nk = P.k_norm2[(size_t)(bh / P.kv_group) * MX230_NORM_PARTS + lane];
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                nq = fmaxf(nq, __shfl_xor_sync(0xFFFFFFFFu, nq, o));
                nk = fmaxf(nk, __shfl_xor_sync(0xFFFFFFFFu, nk, o));
            }
            // the norms are those of the fp32 values; rounding to bf16 moves a norm by less than 0.4 %
            fast = nq * nk * (MX230_QK_LOG2_SCALE * MX230_QK_LOG2_SCALE) <= 80.0f * 80.0f;
        }
        float m = fast ? 0.0f : -CUDART_INF_F, l = 0.0f;   // l: this half's share of the row sum
        float l_norm = 0.0f;   // what O is divided by (fast mode: see below; general mode: l)
        uint32_t va[32], vb[32];
        if (fast) {
        // ---- max-free loop: the group's second 32 columns land under the exponentials of the first 32
        uint64_t rs2[2] = {0ull, 0ull};
        float rs[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        auto exp32 = [&](const uint32_t *src, uint32_t *pk, int key_base, bool need_mask) {
            uint32_t x[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) x[i] = src[i];
            if (need_mask) {   // diagonal and ragged tiles only (a warp-uniform branch: full tiles pay nothing)
#pragma unroll
                for (int i = 0; i < 32; ++i)
                    if (key_base + i > last) x[i] = (FWD_POLY > 0) ? 0xC2FC0000u : 0xFF800000u;  // -126 (2^-126 against sums >= 2^-80) | -inf
            }
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
                float p0, p1;
                if (((i >> 1) % FWD_POLY_DEN) < FWD_POLY) {
                    mx::ex2_poly2<false>(__uint_as_float(x[i]), __uint_as_float(x[i + 1]), p0, p1);
                } else {
                    p0 = mx::ex2(__uint_as_float(x[i]));
                    p1 = mx::ex2(__uint_as_float(x[i + 1]));
                }
                pk[i >> 1] = mx::pack_bf16(p0, p1);
                if (FWD_ADD2) {
                    rs2[(i >> 1) & 1] = mx::add2(rs2[(i >> 1) & 1], mx::pk2(p0, p1));
                } else {
                    rs[i & 2] += p0;
                    rs[(i & 2) + 1] += p1;
                }
            }
        };
        // First key tile only: the sum of the ROUNDED probabilities as well.  Rows that see a handful of keys live
        // there (the first rows of a causal head), and for them the output has to be normalised by what the tensor
        // core actually multiplies with V -- a row with one visible key must return that row of V, not V times
        // bf16(p) / p, or dO . O stops cancelling against dP in the backward.  Everywhere else a row sums so many
        // terms that the two sums differ far below the rounding of V itself, and the fp32 sum serves both uses.
        float rb[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        float l_first = 0.0f;   // fp32 sum of the first tile
        auto sum_rounded16 = [&](const uint32_t *pk) {
#pragma unroll
            for (int w = 0; w < 16; ++w) mx::add_bf16x2(pk[w], rb[(w & 1) * 2], rb[(w & 1) * 2 + 1]);
        };
        auto sum_now = [&]() {
            if (FWD_ADD2) {
                float a0, a1, a2, a3;
                mx::upk2(rs2[0], a0, a1);
                mx::upk2(rs2[1], a2, a3);
                return (a0 + a1) + (a2 + a3);
            }
            return (rs[0] + rs[1]) + (rs[2] + rs[3]);
        };
        // one score tile; FIRST (a compile-time flag: the loop below stays free of the first tile's extra work) also
        // takes the sums of the rounded probabilities
        auto tile = [&](auto first_c, int j) -> bool {
            constexpr bool FIRST = decltype(first_c)::value;
            bool good = __all_sync(0xFFFFFFFFu, mx::mbar_wait(bar(BAR_S_FULL + t), cnt & 1, abort_flag, P.status));
            if (!good) return false;
            mx::tc_fence_after();
            mx::tmem_ld32(tm_s, va);
            mx::tmem_wait_ld();                                       // va is in registers
            mx::tmem_ld32(tm_s + 32, vb);                             // lands under the first exponentials
            const int key0 = j * BN;
            const bool need_mask = (key0 + BN > N) || (P.causal && key0 + BN - 1 > q0 + t * BM + P.q_off);
            uint32_t pk[16];
            exp32(va, pk, key0 + half * (BN / 2), need_mask);
            mx::tmem_wait_ld();                                       // this group's columns have left S_t
            mx::tc_fence_before();
            __syncwarp();
            if (lane == 0) mx::mbar_arrive(bar(BAR_S_FREE + t));
            if (!FIRST) {
                // P_t is free once the previous P V has completed: that takes several hundred cycles from the end of the
                // previous softmax, which is why a quarter of the row is exponentiated before the first store
                good = __all_sync(0xFFFFFFFFu,
                                  mx::mbar_wait_fast(bar(BAR_O_DONE + t), (cnt - 1) & 1, abort_flag, P.status));
                if (!good) return false;
                mx::tc_fence_after();
            }
            mx::tmem_st16(tm_p, pk);
            if (FIRST) sum_rounded16(pk);
            exp32(vb, pk, key0 + half * (BN / 2) + 32, need_mask);
            mx::tmem_st16(tm_p + 16, pk);
            if (FIRST) {
                sum_rounded16(pk);
                l_first = sum_now();
            }
            mx::tmem_wait_st();
            mx::tc_fence_before();
            __syncwarp();
            if (lane == 0) mx::mbar_arrive(bar(BAR_P_FULL + t));
            return true;
        };
        if (n_t > 0) {
            ok = tile(std::true_type{}, 0);
            ++cnt;
            for (int j = 1; ok && j < n_t; ++j) {
                ok = tile(std::false_type{}, j);
                ++cnt;
            }
        }
        l = sum_now();
        l_norm = l - l_first + ((rb[0] + rb[1]) + (rb[2] + rb[3]));
        } else {
        // ---- general loop: running row max, raised lazily.  Each half takes the max of its own 64 columns and the two
        // exchange them through shared memory (one bounded barrier per tile and query tile); both then hold the same
        // row max and take the same decisions, exponentiate their own columns and rescale their own 32 columns of O.
        float row_a = 0.0f, row_qsum = 0.0f;
        if (i8_scores && row < NQ) {
            row_a = P.row_a[(size_t)bh * NQ + row];
            row_qsum = P.row_qsum[(size_t)bh * NQ + row];
        }
        float *xmax = (float *)(smem + SMEM_XMAX) + t * 2 * HALVES * BM;   // [2 tile parities][HALVES][BM]
        for (int j = 0; j < n_t; ++j, ++cnt) {
            ok = __all_sync(0xFFFFFFFFu, mx::mbar_wait(bar(BAR_S_FULL + t), cnt & 1, abort_flag, P.status));
            if (!ok) break;
            mx::tc_fence_after();
            mx::tmem_ld32(tm_s, va);
            mx::tmem_ld32(tm_s + 32, vb);
            mx::tmem_wait_ld();
            mx::tc_fence_before();
            __syncwarp();
            if (lane == 0) mx::mbar_arrive(bar(BAR_S_FREE + t));   // this group's columns have left S_t
            const int key0 = j * BN, col0 = half * (BN / 2);
            if (i8_scores) {
                // the tile holds exact integer dots of int8 codes: the reference kernel's score for them
                const float2 *cs = P.col_kskb + (size_t)(bh / P.kv_group) * P.n_k_pad + key0 + col0;
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const float2 k0 = __ldg(cs + i), k1 = __ldg(cs + 32 + i);
                    va[i] = __float_as_uint(row_a * fmaf(__uint_as_float(va[i]), k0.x, row_qsum * k0.y));
                    vb[i] = __float_as_uint(row_a * fmaf(__uint_as_float(vb[i]), k1.x, row_qsum * k1.y));
                }
            }
            if ((key0 + BN > N) || (P.causal && key0 + BN - 1 > q0 + t * BM + P.q_off)) {
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    if (key0 + col0 + i > last) va[i] = 0xFF800000u;  // -inf
                    if (key0 + col0 + 32 + i > last) vb[i] = 0xFF800000u;
                }
            }
            // four independent max chains (a single chain would serialise on the ALU latency)
            float mx4[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) mx4[u] = fmaxf(__uint_as_float(va[u]), __uint_as_float(vb[u]));
#pragma unroll
            for (int i = 4; i < 32; i += 4)
#pragma unroll
                for (int u = 0; u < 4; ++u) mx4[u] = fmax3(mx4[u], __uint_as_float(va[i + u]), __uint_as_float(vb[i + u]));
            float mx_ = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
            // exchange with the other half of the row
            float *xm = xmax + (cnt & 1) * HALVES * BM;
            xm[half * BM + row_in_tile] = mx_;
            __syncwarp();
            if (lane == 0) mx::mbar_arrive(bar(BAR_XMAX + t));
            ok = __all_sync(0xFFFFFFFFu, mx::mbar_wait(bar(BAR_XMAX + t), xmc & 1, abort_flag, P.status));
            ++xmc;
            if (!ok) break;
            mx_ = fmaxf(mx_, xm[(1 - half) * BM + row_in_tile]);
            // raise the running max only when it pays (always on the first tile)
            const bool raise = (j == 0) || ((mx_ - m) * c > RESCALE_LOG2);
            const float m_new = raise ? mx_ : m;
            const float alpha = (raise && j > 0) ? mx::ex2((m - m_new) * c) : 1.0f;
            const float nmc = -m_new * c;
            if (j > 0) {
                // P_t and O_t are stable once the previous P V has completed
                ok = __all_sync(0xFFFFFFFFu,
                                mx::mbar_wait(bar(BAR_O_DONE + t), (cnt - 1) & 1, abort_flag, P.status));
                if (!ok) break;
                mx::tc_fence_after();
                if (__any_sync(0xFFFFFFFFu, raise)) {
#pragma unroll 1
                    for (int cc = 0; cc < 2; ++cc) {
                        uint32_t o[16];
                        mx::tmem_ld16(tm_o + half * 32 + cc * 16, o);
                        mx::tmem_wait_ld();
#pragma unroll
                        for (int i = 0; i < 16; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                        mx::tmem_st16(tm_o + half * 32 + cc * 16, o);
                    }
                }
            }
            float rs[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            uint32_t pk[16];
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
                const float p0 = mx::ex2(fmaf(__uint_as_float(va[i]), c, nmc));
                const float p1 = mx::ex2(fmaf(__uint_as_float(va[i + 1]), c, nmc));
                rs[i & 2] += p0;
                rs[(i & 2) + 1] += p1;
                pk[i >> 1] = mx::pack_bf16(p0, p1);
            }
            mx::tmem_st16(tm_p, pk);
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
                const float p0 = mx::ex2(fmaf(__uint_as_float(vb[i]), c, nmc));
                const float p1 = mx::ex2(fmaf(__uint_as_float(vb[i + 1]), c, nmc));
                rs[i & 2] += p0;
                rs[(i & 2) + 1] += p1;
                pk[i >> 1] = mx::pack_bf16(p0, p1);
            }
            mx::tmem_st16(tm_p + 16, pk);
            l = l * alpha + ((rs[0] + rs[1]) + (rs[2] + rs[3]));
            m = m_new;
            mx::tmem_wait_st();
            mx::tc_fence_before();
            __syncwarp();
            if (lane == 0) mx::mbar_arrive(bar(BAR_P_FULL + t));
        }
        l_norm = l;
        }
        // The two halves of a row add their sums: half 1 publishes its pair and goes on to the next item, half 0 waits
        // for it (and for the tile's last P V) and does the tile's epilogue.
        float *xch = (float *)(smem + SMEM_XCH) + ((it & 1) * QT + t) * 2 * BM;
        if (half == 1) {
            // (the tile's last P V must have read this group's share of P_t before the next item's first tile overwrites it)
            if (ok && n_t > 0)
                ok = __all_sync(0xFFFFFFFFu, mx::mbar_wait(bar(BAR_O_DONE + t), (cnt - 1) & 1, abort_flag, P.status));
            if (ok) {
                xch[row_in_tile] = l;
                xch[BM + row_in_tile] = l_norm;
                __syncwarp();
                if (lane == 0) mx::mbar_arrive(bar(BAR_XCH + t));
            }
        } else if (ok) {
            ok = __all_sync(0xFFFFFFFFu, mx::mbar_wait(bar(BAR_XCH + t), it & 1, abort_flag, P.status));
            if (ok) {
                l += xch[row_in_tile];
                l_norm += xch[BM + row_in_tile];
            }
        }
        // epilogue: O / l and the log-sum-exp
        if (ok && n_t > 0 && half == 0) {
            ok = __all_sync(0xFFFFFFFFu,
                            mx::mbar_wait(bar(BAR_O_DONE + t), (cnt - 1) & 1, abort_flag, P.status));
            if (ok) {
                mx::tc_fence_after();
                const float inv = 1.0f / l_norm;
                float *orow = P.O + (size_t)bh * P.o_head_stride + (size_t)row * P.o_row_stride;
                if (P.tma_out) {
                    // each warp stages its 32 rows, 32 columns at a time, in a swizzled 4 KB piece of this tile's Q
                    // buffer (its last Q K^T has completed) and hands it to the TMA unit, which clips rows past the
                    // end: 16-byte stores from lane = row registers each touch a sector of their own
                    const int wrow0 = q0 + t * BM + (warp & 3) * 32;
                    const int st_off = SMEM_Q + (qbuf * QT + t) * TILE_BYTES + (warp & 3) * 4096;
#pragma unroll 1
                    for (int cc = 0; cc < HD / 32; ++cc) {
                        mx::tmem_ld32(tm_o + cc * 32, va);
                        mx::tmem_wait_ld();
                        unsigned char *srow = smem + st_off + lane * 128;
#pragma unroll
                        for (int cch = 0; cch < 8; ++cch)
                            *(float4 *)(srow + ((cch ^ (lane & 7)) << 4)) =
                                make_float4(__uint_as_float(va[4 * cch]) * inv, __uint_as_float(va[4 * cch + 1]) * inv,
                                            __uint_as_float(va[4 * cch + 2]) * inv, __uint_as_float(va[4 * cch + 3]) * inv);
                        mx::fence_proxy_async_smem();
                        __syncwarp();
                        if (lane == 0 && wrow0 < NQ) {
                            mx::tma_store_3d(&tmO, smem_base + st_off, cc * 32, wrow0, bh);
                            mx::bulk_commit_group();
                            mx::bulk_wait_group_read<0>();   // the piece is reused for the second half and must outlive the read
                        }
                        __syncwarp();
                    }
                } else
#pragma unroll 1
                for (int cc = 0; cc < HD / 32; ++cc) {
                    mx::tmem_ld32(tm_o + cc * 32, va);
                    mx::tmem_wait_ld();
                    if (row < NQ) {
#pragma unroll
                        for (int i = 0; i < 32; i += 4) {
                            float4 o4 = make_float4(__uint_as_float(va[i]) * inv, __uint_as_float(va[i + 1]) * inv,
                                                    __uint_as_float(va[i + 2]) * inv, __uint_as_float(va[i + 3]) * inv);
                            *(float4 *)(orow + cc * 32 + i) = o4;
                        }
                    }
                }
                if (P.L != nullptr && row < NQ) P.L[(size_t)bh * NQ + row] = m * l_scale + __logf(l);
            }
        }
        // this warp no longer touches the item's Q buffer (operand of its tile's Q K^T, then staging space)
        __syncwarp();
        if (ok && lane == 0) mx::mbar_arrive(bar(BAR_Q_EMPTY + qbuf));
        }  // items
    }

    // ------------------------- teardown ---------------------------------
    mx::tc_fence_before();
    __syncthreads();
    mx::tc_fence_after();
    if (warp == SOFT_WARPS + 1) mx::tmem_dealloc(tmem, TM_COLS);
}

// fp32 -> bf16 (round to nearest even) for up to four equally sized tensors of `heads` x `per_head4` float4s.
struct CastParams {
    const float *src[4];
    __nv_bfloat16 *dst[4];
    size_t per_head4;   // float4s per head (the whole tensor when heads == 1)
    float4 *zero;       // optional: a buffer of the tensors' size set to zero by one more slice of the grid (blockIdx.y = n_tensors)
    float *norm2[2];    // optional, tensors 0 and 1: [heads][MX230_NORM_PARTS] largest squared row norm seen by each grid part
    int n_tensors;
    float scale0;       // tensor 0 is multiplied by this before rounding (1 = plain cast)
};

// Grid (parts, tensors [+ 1], heads): a block converts every gridDim.x-th group of 256 float4s of its head.  Four
// coalesced 16-byte loads in flight per thread (streaming: the fp32 operands are not needed again and should not push
// the bf16 copies, which the attention kernels read next, out of L2), 8-byte stores.  A row of 64 values is 16
// neighbouring lanes, so its squared norm costs four shuffles on a kernel that waits for memory anyway.
__global__ void __launch_bounds__(256) cast_bf16_kernel(const CastParams P) {
    const size_t n4 = P.per_head4;
    const size_t base = (size_t)blockIdx.z * n4;
    const size_t step = (size_t)gridDim.x * blockDim.x;
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if ((int)blockIdx.y == P.n_tensors) {
        for (; i < n4; i += step) P.zero[base + i] = make_float4(0.f, 0.f, 0.f, 0.f);
        return;
    }
    const float4 *src = (const float4 *)P.src[blockIdx.y] + base;
    uint2 *dst = (uint2 *)P.dst[blockIdx.y] + base;
    const float sc = blockIdx.y == 0 ? P.scale0 : 1.0f;   // one rounding either way: fp32 product -> bf16
    float *norm_out = blockIdx.y < 2 ? P.norm2[blockIdx.y] : nullptr;
    const unsigned half_mask = 0xFFFFu << (threadIdx.x & 16);   // the 16 lanes that hold one row
    float mx = 0.0f;
    auto row_norm = [&](const float4 &a) {
        float q = a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) q += __shfl_xor_sync(half_mask, q, o);
        mx = fmaxf(mx, q);
    };
    for (; i + 3 * step < n4; i += 4 * step) {
        float4 a[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) a[u] = __ldcs(src + i + u * step);
#pragma unroll
        for (int u = 0; u < 4; ++u)
            dst[i + u * step] = make_uint2(mx::pack_bf16(a[u].x * sc, a[u].y * sc), mx::pack_bf16(a[u].z * sc, a[u].w * sc));
        if (norm_out != nullptr) {
#pragma unroll
            for (int u = 0; u < 4; ++u) row_norm(a[u]);
        }
    }
    for (; i < n4; i += step) {
        const float4 a = __ldcs(src + i);
        dst[i] = make_uint2(mx::pack_bf16(a.x * sc, a.y * sc), mx::pack_bf16(a.z * sc, a.w * sc));
        if (norm_out != nullptr) row_norm(a);
    }
    if (norm_out != nullptr) {   // block maximum -> this part's slot (parts the grid does not have are set to 0)
        __shared__ float red[8];
        __syncwarp();
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o));
        if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = mx;
        __syncthreads();
        if (threadIdx.x == 0) {
            for (int w = 1; w < 8; ++w) mx = fmaxf(mx, red[w]);
            norm_out[(size_t)blockIdx.z * MX230_NORM_PARTS + blockIdx.x] = mx;
            if (blockIdx.x == 0)
                for (int q = (int)gridDim.x; q < MX230_NORM_PARTS; ++q) norm_out[(size_t)blockIdx.z * MX230_NORM_PARTS + q] = 0.0f;
        }
    }
}

}  // namespace

int mx230_launch_cast(mx230_handle *h, cudaStream_t st, const float *const *src, void *const *dst,
                      int n_tensors, int heads, size_t per_head, float *zero, float scale0, float *const *norm2) {
    MX_REQUIRE(per_head % 8 == 0, MX230_ERR_INVALID_ARG, "cast: element count must be a multiple of 8");
    MX_REQUIRE(norm2 == nullptr || per_head % 64 == 0, MX230_ERR_INVALID_ARG, "cast: row norms need rows of 64 values");
    if (per_head == 0 || n_tensors == 0 || heads == 0) return MX230_OK;
    MX_REQUIRE(heads > 0 && heads <= 65535, MX230_ERR_UNSUPPORTED, "cast: %d heads", heads);
    CastParams P;
    for (int i = 0; i < 4; ++i) {
        P.src[i] = src[i < n_tensors ? i : 0];
        P.dst[i] = (__nv_bfloat16 *)dst[i < n_tensors ? i : 0];
        MX_REQUIRE((((uintptr_t)P.src[i] | (uintptr_t)P.dst[i]) & 15) == 0, MX230_ERR_INVALID_ARG,
                   "cast: buffers must be 16-byte aligned");
    }
    P.per_head4 = per_head / 4;
    P.zero = (float4 *)zero;
    P.n_tensors = n_tensors;
    P.scale0 = scale0;
    P.norm2[0] = norm2 ? norm2[0] : nullptr;
    P.norm2[1] = norm2 && n_tensors > 1 ? norm2[1] : nullptr;
    MX_REQUIRE(((uintptr_t)zero & 15) == 0, MX230_ERR_INVALID_ARG, "cast: buffers must be 16-byte aligned");
    // parts per head: every thread gets at least one round of four loads, the whole grid about eight blocks per SM
    const int slices = n_tensors + (zero ? 1 : 0);
    size_t want = (P.per_head4 + 1023) / 1024;
    size_t cap = ((size_t)h->sm_count * 8 + (size_t)slices * heads - 1) / ((size_t)slices * heads);
    size_t parts = want < cap ? want : cap;
    if (parts < 1) parts = 1;
    if (norm2 != nullptr && parts > MX230_NORM_PARTS) parts = MX230_NORM_PARTS;
    if (parts > 65535) parts = 65535;
    MX_LAUNCH(h, st, MX230_K_CAST, (cast_bf16_kernel<<<dim3((unsigned)parts, slices, heads), 256, 0, st>>>(P)));
    return MX230_OK;
}

// General launcher.  Q: bf16 [heads][n_q][64]; K, V: bf16 [heads / kv_group][n_k][64].
int mx230_launch_flash_fwd_ex(mx230_handle *h, cudaStream_t st, const void *Qb, const void *Kb,
                              const void *Vb, float *O, float *L, int heads, int n_q, int n_k, int q_off,
                              int kv_group, long long o_head_stride, long long o_row_stride, int causal,
                              int q_prescaled, const float *q_norm2, const float *k_norm2, const float *row_a,
                              const float *row_qsum, const float *col_kskb) {
    CUtensorMap tq, tk, tv, to;
    uint64_t rs = HD * 2;
    int rc;
    const bool tma_out = (((uintptr_t)O & 15) == 0) && o_row_stride % 4 == 0 && o_head_stride % 4 == 0 &&
                         o_row_stride > 0 && o_head_stride > 0;
    if (tma_out) {
        if ((rc = mx230_make_tmap_f32_half_rows_strided(h, &to, O, n_q, heads, (uint64_t)o_row_stride * 4,
                                                        (uint64_t)o_head_stride * 4)))
            return rc;
    } else {
        memset(&to, 0, sizeof(to));
    }
    if ((rc = mx230_make_tmap_bf16(h, &tq, Qb, n_q, heads, rs, (uint64_t)n_q * HD * 2, BM))) return rc;
    if ((rc = mx230_make_tmap_bf16(h, &tk, Kb, n_k, heads / kv_group, rs, (uint64_t)n_k * HD * 2, BN))) return rc;
    if ((rc = mx230_make_tmap_bf16(h, &tv, Vb, n_k, heads / kv_group, rs, (uint64_t)n_k * HD * 2, BN))) return rc;
    // function attributes are per device: one handle per GPU may live in the same process
    static bool attr_set[64] = {};
    MX_REQUIRE(h->device >= 0 && h->device < 64, MX230_ERR_UNSUPPORTED, "flash forward: device index %d", h->device);
    if (!attr_set[h->device]) {
        MX_CHECK_CUDA(cudaFuncSetAttribute(flash_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           SMEM_ALLOC));
        attr_set[h->device] = true;
    }
    FwdParams P;
    P.O = O;
    P.L = L;
    P.o_head_stride = o_head_stride;
    P.o_row_stride = o_row_stride;
    P.n_q = n_q;
    P.n_k = n_k;
    P.q_off = q_off;
    P.kv_group = kv_group;
    P.causal = causal ? 1 : 0;
    P.heads = heads;
    // Two query tiles per item keep both softmax groups of a CTA busy; a call so small that every 128-row tile can have
    // an SM of its own is cut into single-tile items instead (the second group idles, but twice as many SMs work).
    // With more tiles than SMs the single-tile form would need a second round at two thirds of the two-tile pace per
    // tile (measured: one head of 32768 rows, 0.51 ms against 0.37).
    P.item_tiles = ((long long)heads * ((n_q + BM - 1) / BM) <= h->sm_count) ? 1 : QT;
    P.n_qblocks = (n_q + P.item_tiles * BM - 1) / (P.item_tiles * BM);
    MX_REQUIRE((long long)heads * P.n_qblocks <= 0x7FFFFFFF, MX230_ERR_UNSUPPORTED, "flash forward: too many query blocks");
    P.n_items = heads * P.n_qblocks;
    P.tma_out = tma_out ? 1 : 0;
    P.prescaled = q_prescaled ? 1 : 0;
    P.q_norm2 = (q_prescaled && q_norm2 && k_norm2) ? q_norm2 : nullptr;
    P.k_norm2 = P.q_norm2 ? k_norm2 : nullptr;
    P.test_drop_tile = h->test_drop_tile;
    P.row_a = (row_a && row_qsum && col_kskb) ? row_a : nullptr;
    P.row_qsum = P.row_a ? row_qsum : nullptr;
    P.col_kskb = P.row_a ? (const float2 *)col_kskb : nullptr;
    P.n_k_pad = (n_k + BN - 1) / BN * BN;
    P.status = h->status_dev;
    // persistent: one CTA per SM (the kernel holds all of an SM's tensor memory), each walking its share of the items
    dim3 grid((unsigned)(P.n_items < h->sm_count ? P.n_items : h->sm_count));
    MX_LAUNCH(h, st, MX230_K_FLASH_FWD,
              (flash_fwd_kernel<<<grid, FWD_THREADS, SMEM_ALLOC, st>>>(tq, tk, tv, to, P)));
    return MX230_OK;
}

int mx230_launch_flash_fwd(mx230_handle *h, cudaStream_t st, const void *Qb, const void *Kb,
                           const void *Vb, float *O, float *L, int batch_heads, int n, int causal,
                           int q_prescaled, const float *q_norm2, const float *k_norm2) {
    return mx230_launch_flash_fwd_ex(h, st, Qb, Kb, Vb, O, L, batch_heads, n, n, 0, 1, (long long)n * HD, HD,
                                     causal, q_prescaled, q_norm2, k_norm2, nullptr, nullptr, nullptr);
}

static int check_flash_args(const char *who, mx230_handle *h, int batch_heads, int n) {
    MX_REQUIRE(h != nullptr, MX230_ERR_INVALID_ARG, "%s: null handle", who);
    MX_REQUIRE(batch_heads >= 0 && n >= 0, MX230_ERR_INVALID_ARG, "%s: negative size", who);
    MX_REQUIRE(batch_heads <= 65535, MX230_ERR_UNSUPPORTED, "%s: batch_heads %d > 65535", who,
               batch_heads);
    return MX230_OK;
}

extern "C" int mx230_cast_bf16(mx230_handle *h, void *stream, const float *src, void *dst_bf16,
                               size_t count) {
    MX_REQUIRE(h && (count == 0 || (src && dst_bf16)), MX230_ERR_INVALID_ARG, "cast_bf16: null argument");
    mx230_device_guard guard(h->device);
    const float *s[1] = {src};
    void *d[1] = {dst_bf16};
    return mx230_launch_cast(h, (cudaStream_t)stream, s, d, 1, 1, count, nullptr, 1.0f, nullptr);
}

extern "C" int mx230_attn_flash_bf16(mx230_handle *h, void *stream, const void *Qb, const void *Kb,
                                     const void *Vb, float *O, float *L_or_null, int batch_heads,
                                     int n, int causal) {
    int rc = check_flash_args("attn_flash_bf16", h, batch_heads, n);
    if (rc) return rc;
    if (batch_heads == 0 || n == 0) return MX230_OK;
    MX_REQUIRE(Qb && Kb && Vb && O, MX230_ERR_INVALID_ARG, "attn_flash_bf16: null tensor");
    MX_REQUIRE((((uintptr_t)O) & 15) == 0, MX230_ERR_INVALID_ARG, "attn_flash_bf16: O must be 16-byte aligned");
    mx230_device_guard guard(h->device);
    return mx230_launch_flash_fwd(h, (cudaStream_t)stream, Qb, Kb, Vb, O, L_or_null, batch_heads, n,
                                  causal, 0, nullptr, nullptr);
}

static int flash_fp32(mx230_handle *h, void *stream, const float *Q, const float *K, const float *V,
                      float *O, float *L, int batch_heads, int n, int causal, const char *who) {
    int rc = check_flash_args(who, h, batch_heads, n);
    if (rc) return rc;
    if (batch_heads == 0 || n == 0) return MX230_OK;
    MX_REQUIRE(Q && K && V && O, MX230_ERR_INVALID_ARG, "%s: null tensor", who);
    size_t need = mx230_flash_workspace_bytes(batch_heads, n, 0);
    MX_REQUIRE(h->ws && need <= h->ws_bytes, MX230_ERR_WORKSPACE,
               "%s: workspace %zu B < %zu B needed (call mx230_reserve)", who, h->ws_bytes, need);
    mx230_device_guard guard(h->device);
    const size_t one = mx230_flash_stage_bytes(batch_heads, n);
    void *qb = h->ws, *kb = (char *)h->ws + one, *vb = (char *)h->ws + 2 * one;
    float *qn = (float *)((char *)h->ws + 3 * one), *kn = qn + (size_t)batch_heads * MX230_NORM_PARTS;
    const float *src[3] = {Q, K, V};
    void *dst[3] = {qb, kb, vb};
    float *norms[2] = {qn, kn};
    // Q is staged as Q * (scale * log2 e), rounded once from the fp32 product: the kernel's scores are then
    // already in log2 units.  The same launch leaves the largest row norms of Q and K per head, from which the
    // kernel bounds |q . k| and, where the bound allows, runs its softmax loop without a row max.
    h->staged.valid = 0;
    rc = mx230_launch_cast(h, (cudaStream_t)stream, src, dst, 3, batch_heads, (size_t)n * HD, nullptr,
                           MX230_QK_LOG2_SCALE, norms);
    if (rc) return rc;
    h->staged = {Q, K, V, batch_heads, n, 1, nullptr};
    return mx230_launch_flash_fwd(h, (cudaStream_t)stream, qb, kb, vb, O, L, batch_heads, n, causal, 1, qn, kn);
}

extern "C" int mx230_attn_flash(mx230_handle *h, void *stream, const float *Q, const float *K,
                                const float *V, float *O, int batch_heads, int n, int causal) {
    return flash_fp32(h, stream, Q, K, V, O, nullptr, batch_heads, n, causal, "attn_flash");
}

extern "C" int mx230_attn_flash_lse(mx230_handle *h, void *stream, const float *Q, const float *K,
                                    const float *V, float *O, float *L, int batch_heads, int n,
                                    int causal) {
    MX_REQUIRE(L != nullptr || batch_heads == 0 || n == 0, MX230_ERR_INVALID_ARG,
               "attn_flash_lse: null L");
    return flash_fp32(h, stream, Q, K, V, O, L, batch_heads, n, causal, "attn_flash_lse");
}

