// Flash-attention backward for sm_100a: dQ, dK, dV of the scalar loss <O, dO>, with
// the probabilities recomputed from the saved log-sum-exp, never stored.
//
// Reference semantics: attn_bwd_preprocess, attn_bwd_dq, attn_bwd_dkv,
// 02-flash-attention/kernels/attention_bwd.cu:32-44,96-158,165-243 (fp32 SIMT):
//   Delta_i = sum_x dO[i,x] O[i,x]
//   p_ij  = exp(scale * q_i.k_j - L_i),  dP_ij = dO_i . v_j
//   dS_ij = p_ij (dP_ij - Delta_i) scale
//   dQ_i += dS_ij k_j ;  dK_j += dS_ij q_i ;  dV_j += p_ij dO_i
// Two ways through the same kernel template, all contractions on tcgen05 tensor cores (bf16 operands,
// fp32 accumulators in tensor memory):
//  * the reference's atomic-free split -- a dQ pass owned by query tiles (MODE 0) and a dK/dV pass owned
//    by key tiles (MODE 1), each output element written exactly once, bit-reproducible;
//  * one fused pass (MODE 2, the default of mx230_attn_bwd_flash): the dK/dV pass also forms every tile's
//    dQ contribution and adds it to global memory with fp32 reductions, so S and dP are computed once.
// A work item is ONE owned 128-row tile of one head (queries for dQ, keys otherwise) against the 128-row tiles
// of the other axis, streamed through a TMA ring.  The two-pass kernels run one item per CTA; the fused pass is
// persistent: one CTA per SM walks its share of the items (heaviest first, dealt out in snake order), ring
// positions and barrier parities run on from item to item, and the next item's owned and first streamed tiles
// are requested as soon as the current item's last MMAs have completed, while its dK / dV are still being stored.
// Per streamed tile:
//
//   X = A_own A_str^T, Y = B_own B_str^T      (S, dP   |  S^T, dP^T)   128 x 128, N = 128 MMAs
//   P = exp2(X c - L), E = P o (Y - Delta)    one thread per owned row and column half
//   acc0 += E A_str   (dQ += dS K | dK += dS^T Q),   acc1 += P B_str (dV += P^T dO)
//   fused pass only:  dQ_tile = E^T K  (fresh accumulator), drained to global memory by four warps
//
// Every MMA stream has its own issuing thread in the two-pass kernels: a thread issues an MMA about
// every 60 cycles and stalls on each commit until its MMAs have drained, so one thread cannot
// keep the tensor pipe busy with 32-cycle N = 64 MMAs.  The two compute warpgroups take the left
// and right 64 columns of X, Y: X, Y of the next tile are issued as soon as both hold the current
// ones in registers, and the accumulate MMAs of a tile run under the next tile's exponentials.
// In the dQ pass the owned Q and dO tiles are read as A operands from tensor memory (written there
// once by the compute threads), which leaves shared-memory bandwidth to the streamed operand; in
// the other passes tensor memory is full and they stay in shared memory.  The recomputed tiles go back
// to tensor memory as bf16 A operands; the fused pass has no columns left for E and keeps it in shared
// memory (two swizzled buffers written inside the exp loop), where the dQ contraction needs it anyway:
// the same bytes are read K-major for dK and MN-major (queries contiguous) for dQ.
// The 1/sqrt(d) factor of dS is applied to the fp32 accumulators on their way out (exact: 2^-3).
#include <math_constants.h>

#include <type_traits>

#include "common.cuh"

namespace {
constexpr int HD = 64;
constexpr int BT = 128;          // rows of the owned tile (queries in dQ, keys in dK/dV)
constexpr int BS = 128;          // rows of a streamed tile
constexpr int HS = BS / 2;       // columns of X, Y per compute warpgroup
constexpr int STAGES = 4;
constexpr int OWN_BYTES = BT * HD * 2;   // 16 KB
constexpr int STR_BYTES = BS * HD * 2;   // 16 KB
constexpr int BWD_THREADS = 512;
// warpgroups: compute left, compute right, {TMA, X, acc0, Y}, {acc1, 3 idle}; fused pass: {TMA, X+Y, dK, dV+dQ},
// {4 drain warps}.
// setmaxnreg moves registers only inside the CTA's launch-time allocation (128 per thread for 512 threads)
#ifndef BWD_REGS_COMPUTE
#define BWD_REGS_COMPUTE 192
#define BWD_REGS_SERVICE 64
#endif
#ifndef BWD_SPLIT_LOAD
#define BWD_SPLIT_LOAD 1   // X, Y of a tile are pulled in two 32-column pieces, the second under the first one's arithmetic (fused pass: 290 -> 281 us)
#endif
#ifndef BWD_POLY
#define BWD_POLY 0         // fused pass: of every four column pairs, how many take 2^x from the FMA-pipe polynomial
#endif
constexpr int REGS_COMPUTE = BWD_REGS_COMPUTE, REGS_SERVICE = BWD_REGS_SERVICE;
static_assert(8 * REGS_COMPUTE + 8 * REGS_SERVICE <= 16 * 128, "setmaxnreg budget exceeds the launch-time register allocation");

// shared memory map (after 1024-byte alignment)
constexpr int SM_OWN_A = 0;                              // K (dK/dV pass)
constexpr int SM_OWN_B = SM_OWN_A + OWN_BYTES;           // V (dK/dV pass)
constexpr int SM_STR_A = SM_OWN_B + OWN_BYTES;           // STAGES x 16 KB: K / Q
constexpr int SM_STR_B = SM_STR_A + STAGES * STR_BYTES;  // STAGES x 16 KB: V / dO
constexpr int SM_LD = SM_STR_B + STAGES * STR_BYTES;     // STAGES x 2 x 128 floats: -L*log2e, -Delta (dK/dV)
constexpr int SM_DS = SM_LD + STAGES * 2 * BS * 4;        // fused pass: dS^T as bf16, two [128 keys][64 queries] tiles
constexpr int DS_HALF_BYTES = BT * HS * 2;               // 16 KB
constexpr int SM_DS1_A = SM_STR_A + (STAGES - 1) * STR_BYTES;   // second E buffer: the last stage's slots
constexpr int SM_DS1_B = SM_STR_B + (STAGES - 1) * STR_BYTES;
constexpr int SM_DQ = SM_DS + 2 * DS_HALF_BYTES;          // fused pass: 4 x 4 KB, one staging tile per drain warp
constexpr int DQ_STAGE_BYTES = 32 * 32 * 4;              // 32 queries x 32 dims fp32, 128-byte rows
// fused pass: -8 L and -Delta of the streamed queries enter X and Y through a fifth K step of their MMAs
// (three bf16 terms each, against columns of ones), so the compute threads load nothing per element.
// Unswizzled K-major operands of 128 rows x 16 columns: the first 8 columns are a dense [128][8] bf16 tile,
// the second 8 columns of every operand are one shared block of zeros.
constexpr int AUG_BYTES = 128 * 16;                      // 2 KB
constexpr int SM_AUG_B = SM_DQ + 4 * DQ_STAGE_BYTES;     // (STAGES - 1) tiles: row q = {Lh, Lm, Ll, Dh, Dm, Dl, 0, 0}
constexpr int SM_AUG_AX = SM_AUG_B + (STAGES - 1) * AUG_BYTES;   // ones in columns 0..2
constexpr int SM_AUG_AY = SM_AUG_AX + AUG_BYTES;                 // ones in columns 3..5
constexpr int SM_AUG_Z = SM_AUG_AY + AUG_BYTES;                  // zeros (placed last: offsets to it are positive)
constexpr int SM_BAR = SM_AUG_Z + AUG_BYTES;
static_assert(SM_DS % 1024 == 0 && SM_DQ % 1024 == 0, "swizzled tiles start on 1024-byte boundaries");
constexpr int SM_TOTAL = SM_BAR + 256;
constexpr int SM_ALLOC = SM_TOTAL + 1024;
static_assert(SM_ALLOC <= 227 * 1024, "shared memory per CTA");

constexpr int BAR_OWN_FULL = 0;
constexpr int BAR_STR_FULL = 1;                          // [STAGES]
constexpr int BAR_STR_EMPTY = BAR_STR_FULL + STAGES;     // [STAGES] accumulate MMAs of the stage's tile done
constexpr int BAR_SDP_FULL = BAR_STR_EMPTY + STAGES;     // MMA -> compute: X, Y written
constexpr int BAR_SDP_FREE = BAR_SDP_FULL + 1;           // compute -> MMA: X, Y in registers
constexpr int BAR_DS_READY = BAR_SDP_FREE + 1;           // compute -> MMA: E, P written
constexpr int BAR_ACC_DONE = BAR_DS_READY + 1;
constexpr int BAR_DQ_FULL = BAR_ACC_DONE + 1;            // fused pass: MMA -> drain warps
constexpr int BAR_DQ_FREE = BAR_DQ_FULL + 1;             // drain warps -> MMA
constexpr int N_BARS = BAR_DQ_FREE + 1;

// tensor memory columns
constexpr int TM_X = 0, TM_Y = 128, TM_E = 256, TM_P = 320;   // E, P: bf16 pairs, 64 columns each
constexpr int TM_ACC0 = 384, TM_ACC1 = 448;
// dQ pass only (no second accumulator there): the owned Q and dO tiles as bf16 A operands, 32 columns each
constexpr int TM_OWN_A = 448, TM_OWN_B = 480;
// fused pass: E lives in shared memory (the dQ contraction needs it there), which frees 64 columns for dQ's tile
constexpr int TMF_P = 256, TMF_ACC0 = 320, TMF_ACC1 = 384, TMF_DQ = 448;
constexpr int TM_COLS = 512;
constexpr float LOG2E = 1.4426950408889634f;

struct BwdParams {
    const float *L;      // [BH][N]
    const float *Delta;  // [BH][N]
    float *out0;         // dQ (dQ pass) / dK (dK/dV pass)   [BH][N][64]
    float *out1;         // unused / dV
    float *dq;           // fused pass: dQ, zeroed before the launch, summed into with fp32 reductions
    const uint4 *own_a;  // dQ pass: bf16 Q  [BH][N][64], read straight into tensor memory
    const uint4 *own_b;  // dQ pass: bf16 dO [BH][N][64]
    int n;
    int causal;
    int *status;
    int heads;           // batch_heads
    int n_tiles;         // owned tiles per head
    int n_items;         // heads * n_tiles work items (owned tile, head), heads fastest, heaviest tiles first
    int test_drop_tile;  // test hook (fused pass): streamed tile (counted over the CTA's items) that CTA 0's producer never requests; -1 = off
};

// One CTA's `round`-th work item: an owned 128-row tile of one head and the range of streamed tiles it sees.
// Items are listed heaviest first (dQ: late query tiles see the most keys; dK/dV: early key tiles see the most
// queries) and dealt to the CTAs forwards in even rounds, backwards in odd ones, so that a persistent grid of
// one CTA per SM ends up with equal shares; a grid of n_items CTAs gives every CTA exactly one item.
struct BwdItem {
    int bh, own0, it_beg, n;   // head, first owned row, first streamed tile, streamed tiles (>= 1)
};
template <int MODE>
__device__ __forceinline__ bool bwd_item(const BwdParams &P, int round, BwdItem &I) {
    const int G = (int)gridDim.x, c = (int)blockIdx.x;
    const int i = round * G + ((round & 1) ? G - 1 - c : c);
    if (i >= P.n_items) return false;
    const int rank = i / P.heads;
    I.bh = i - rank * P.heads;
    const int tile = (MODE == 0 && P.causal) ? P.n_tiles - 1 - rank : rank;
    I.own0 = tile * BT;
    const int n_str_total = (P.n + BS - 1) / BS;
    int it_beg = 0, it_end = n_str_total;
    if (P.causal) {
        if (MODE == 0) it_end = min(n_str_total, (I.own0 + BT - 1) / BS + 1);
        else it_beg = I.own0 / BS;
    }
    I.it_beg = it_beg;
    I.n = it_end - it_beg;
    return true;
}

// MODE 0: dQ pass (own = Q, dO; stream = K, V).  MODE 1: dK/dV pass (own = K, V; stream = Q, dO).
// MODE 2: the dK/dV pass that also forms every tile's dQ contribution (dS K, a fifth MMA stream reading
// dS^T from shared memory as an MN-major A operand) and adds it to dQ in global memory.
// PRE: the bf16 Q holds Q * scale * log2(e) (what the fp32 entry points stage, and what the forward used for L): the
// scores X arrive in log2 units, and dK, a product with that Q, is scaled back on its way out.  The caller-staged
// bf16 entry point passes plain Q (PRE = false).
template <int MODE, bool PRE>
__global__ void __launch_bounds__(BWD_THREADS, 1)
bwd_kernel(const __grid_constant__ CUtensorMap tmOwnA, const __grid_constant__ CUtensorMap tmOwnB,
           const __grid_constant__ CUtensorMap tmStrA, const __grid_constant__ CUtensorMap tmStrB,
           const __grid_constant__ CUtensorMap tmDQ, const __grid_constant__ CUtensorMap tmOut0,
           const __grid_constant__ CUtensorMap tmOut1, const BwdParams P) {
    extern __shared__ unsigned char smem_dyn[];
    const uint32_t smem_base = (mx::smem_u32(smem_dyn) + 1023u) & ~1023u;
    unsigned char *smem = smem_dyn + (smem_base - mx::smem_u32(smem_dyn));
    const uint32_t bar0 = smem_base + SM_BAR;
    auto bar = [&](int i) { return bar0 + 8u * (uint32_t)i; };
    volatile uint32_t *tmem_slot = (volatile uint32_t *)(smem + SM_BAR + 8 * N_BARS);
    volatile int *abort_flag = (volatile int *)(smem + SM_BAR + 8 * N_BARS + 8);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int N = P.n;
    constexpr bool FUSED = MODE == 2;
    // the fused pass streams through three stages: the fourth one's two 16 KB slots hold its second E buffer
    constexpr int NST = FUSED ? STAGES - 1 : STAGES;
    constexpr int N_ACC = MODE == 0 ? 1 : 2;   // accumulate issuers: one commit each per tile
    constexpr int tP = FUSED ? TMF_P : TM_P, tACC0 = FUSED ? TMF_ACC0 : TM_ACC0, tACC1 = FUSED ? TMF_ACC1 : TM_ACC1;

    if (tid == 0) {
        mx::mbar_init(bar(BAR_OWN_FULL), MODE == 0 ? 2 * BT / 32 : 1);  // dQ: every compute warp; dK/dV: TMA
        for (int s = 0; s < STAGES; ++s) {
            mx::mbar_init(bar(BAR_STR_FULL + s), MODE >= 1 ? 33 : 1);
            mx::mbar_init(bar(BAR_STR_EMPTY + s), N_ACC);
        }
        mx::mbar_init(bar(BAR_SDP_FULL), FUSED ? 1 : 2);  // the X and the Y issuer (one thread in the fused pass)
        mx::mbar_init(bar(BAR_DQ_FULL), 1);
        mx::mbar_init(bar(BAR_DQ_FREE), 4);
        mx::mbar_init(bar(BAR_SDP_FREE), 2 * BT / 32);    // one elected lane per compute warp arrives
        mx::mbar_init(bar(BAR_DS_READY), 2 * BT / 32);
        mx::mbar_init(bar(BAR_ACC_DONE), N_ACC);
        *abort_flag = 0;
        mx::mbar_fence_init();
    }
    if (warp == 9) mx::tmem_alloc(mx::smem_u32((const void *)tmem_slot), TM_COLS);
    mx::tc_fence_before();
    __syncthreads();
    mx::tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    if (warp >= 8) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(REGS_SERVICE));
        if (warp == 8) {
            // ------------------------- producer -------------------------
            if (lane == 0) {
                mx::tma_prefetch_desc(&tmStrA);
                mx::tma_prefetch_desc(&tmStrB);
                if (MODE >= 1) {
                    mx::tma_prefetch_desc(&tmOwnA);
                    mx::tma_prefetch_desc(&tmOwnB);
                }
            }
            if (FUSED) {   // the constant operands: ones for X, ones for Y, zeros (ordered before the first arrive below)
                uint4 *ax = (uint4 *)(smem + SM_AUG_AX), *ay = (uint4 *)(smem + SM_AUG_AY), *az = (uint4 *)(smem + SM_AUG_Z);
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    ax[u * 32 + lane] = make_uint4(0x3F803F80u, 0x00003F80u, 0u, 0u);
                    ay[u * 32 + lane] = make_uint4(0u, 0x3F800000u, 0x3F803F80u, 0u);
                    az[u * 32 + lane] = make_uint4(0u, 0u, 0u, 0u);
                }
            }
            bool ok = true;
            uint32_t g = 0;   // streamed tiles so far, over all items: ring slot g % NST, use g / NST
            BwdItem I;
            for (int it = 0; ok && bwd_item<MODE>(P, it, I); ++it) {
                const int bh = I.bh;
                if (MODE >= 1) {
                    // the owned tiles are single-buffered: every MMA of the previous item must have completed
                    if (it > 0) ok = __all_sync(0xFFFFFFFFu, mx::mbar_wait(bar(BAR_ACC_DONE), (it - 1) & 1, abort_flag, P.status));
                    if (!ok) break;
                    if (lane == 0) {
                        mx::mbar_expect_tx(bar(BAR_OWN_FULL), 2 * OWN_BYTES);
                        mx::tma_load_3d(smem_base + SM_OWN_A, &tmOwnA, bar(BAR_OWN_FULL), 0, I.own0, bh);
                        mx::tma_load_3d(smem_base + SM_OWN_B, &tmOwnB, bar(BAR_OWN_FULL), 0, I.own0, bh);
                    }
                }
                for (int y = 0; y < I.n; ++y, ++g) {
                    const int s = g % NST;
                    const uint32_t r = g / NST;
                    const int row0 = (I.it_beg + y) * BS;
                    // -L*log2(e) and -Delta of the streamed queries: fetched before the wait, stored after it
                    float lv[4], dv[4];
                    if (MODE >= 1) {
#pragma unroll
                        for (int u = 0; u < 4; ++u) {
                            const int q = row0 + u * 32 + lane;
                            const bool v = q < N;
                            // fused pass over a plain Q: X + lv is multiplied by 0.125 log2(e) afterwards, hence -8 L (exact)
                            lv[u] = v ? -P.L[(size_t)bh * N + q] * ((FUSED && !PRE) ? 8.0f : LOG2E) : 0.0f;
                            dv[u] = v ? -P.Delta[(size_t)bh * N + q] : 0.0f;
                        }
                    }
                    if (r > 0)
                        ok = __all_sync(0xFFFFFFFFu,
                                        mx::mbar_wait(bar(BAR_STR_EMPTY + s), (r - 1) & 1, abort_flag, P.status));
                    if (!ok) break;
                    if (FUSED && P.test_drop_tile == (int)g && blockIdx.x == 0) continue;   // test hook: this tile never arrives
                    if (lane == 0) {
                        mx::mbar_expect_tx(bar(BAR_STR_FULL + s), 2 * STR_BYTES);
                        mx::tma_load_3d(smem_base + SM_STR_A + s * STR_BYTES, &tmStrA, bar(BAR_STR_FULL + s), 0, row0, bh);
                        mx::tma_load_3d(smem_base + SM_STR_B + s * STR_BYTES, &tmStrB, bar(BAR_STR_FULL + s), 0, row0, bh);
                    }
                    if (FUSED) {
                        uint4 *aug = (uint4 *)(smem + SM_AUG_B + s * AUG_BYTES);
#pragma unroll
                        for (int u = 0; u < 4; ++u) {
                            // value = hi + mid + lo, each a bf16: what is left over is below 2^-24 of it
                            const uint32_t lh = mx::pack_bf16(lv[u], 0.0f) & 0xFFFFu;
                            const float l1 = lv[u] - __uint_as_float(lh << 16);
                            const uint32_t lm = mx::pack_bf16(l1, 0.0f) & 0xFFFFu;
                            const float l2 = l1 - __uint_as_float(lm << 16);
                            const uint32_t dh = mx::pack_bf16(dv[u], 0.0f) & 0xFFFFu;
                            const float d1 = dv[u] - __uint_as_float(dh << 16);
                            const uint32_t dm = mx::pack_bf16(d1, 0.0f) & 0xFFFFu;
                            const float d2 = d1 - __uint_as_float(dm << 16);
                            aug[u * 32 + lane] = make_uint4(lh | (lm << 16), (mx::pack_bf16(l2, 0.0f) & 0xFFFFu) | (dh << 16),
                                                            dm | (mx::pack_bf16(d2, 0.0f) << 16), 0u);
                        }
                        mx::fence_proxy_async_smem();   // read by the MMAs
                        mx::mbar_arrive(bar(BAR_STR_FULL + s));
                    } else if (MODE >= 1) {
                        float *ld = (float *)(smem + SM_LD + s * (2 * BS * 4));
#pragma unroll
                        for (int u = 0; u < 4; ++u) {
                            ld[u * 32 + lane] = lv[u];
                            ld[BS + u * 32 + lane] = dv[u];
                        }
                        mx::mbar_arrive(bar(BAR_STR_FULL + s));
                    }
                }
            }
            __syncwarp();
        } else if (!FUSED && (warp == 9 || warp == 11)) {
            // ------------------------- MMA issuers 1, 2: X (warp 9) and Y (warp 11) ---------
            // (the loops are kept free of run-time choices between instruction forms, which slow
            // the issuing thread down)
            if (lane == 0) {
                const bool is_y = warp == 11;
                constexpr uint32_t IDESC_S = mx::mma_idesc_bf16(BT, BS, false, false);  // [128 x 128] = A B^T
                const uint64_t own = mx::smem_desc_sw128(smem_base + (is_y ? SM_OWN_B : SM_OWN_A));
                const uint32_t own_t = tmem + (is_y ? TM_OWN_B : TM_OWN_A);
                const uint32_t str_base = smem_base + (is_y ? SM_STR_B : SM_STR_A);
                const uint32_t dst = tmem + (is_y ? TM_Y : TM_X);
                bool ok = true;
                uint32_t g = 0;
                BwdItem I;
                for (int it = 0; ok && bwd_item<MODE>(P, it, I); ++it) {
                    ok = mx::mbar_wait(bar(BAR_OWN_FULL), it & 1, abort_flag, P.status);
                    for (int y = 0; y < I.n && ok; ++y, ++g) {
                        const int s = g % NST;
                        ok = mx::mbar_wait(bar(BAR_STR_FULL + s), (g / NST) & 1, abort_flag, P.status);
                        // as soon as both warpgroups hold the previous X, Y in registers
                        if (ok && g > 0) ok = mx::mbar_wait(bar(BAR_SDP_FREE), (g - 1) & 1, abort_flag, P.status);
                        if (!ok) break;
                        mx::tc_fence_after();
                        const uint64_t sd = mx::smem_desc_sw128(str_base + s * STR_BYTES);
                        if (MODE == 0) {
#pragma unroll
                            for (int k = 0; k < HD / 16; ++k) mx::mma_ts(dst, own_t + 8 * k, sd + 2 * k, IDESC_S, k > 0);
                        } else {
#pragma unroll
                            for (int k = 0; k < HD / 16; ++k) mx::mma_ss(dst, own + 2 * k, sd + 2 * k, IDESC_S, k > 0);
                        }
                        mx::mma_commit(bar(BAR_SDP_FULL));
                    }
                }
            }
            __syncwarp();
        } else if (!FUSED && (warp == 10 || (MODE == 1 && warp == 12))) {
            // ------------------------- MMA issuers 3, 4: accumulators ------------
            // warp 10: acc0 += E A_str (dQ += dS K | dK += dS^T Q); warp 12 (dK/dV pass): acc1 += P B_str
            // (dV += P^T dO).  One commit per tile and thread: it frees the stage for the producer and
            // tells the compute warpgroups that E, P have been consumed.
            if (lane == 0) {
                const bool second = warp == 12;
                constexpr uint32_t IDESC_G = mx::mma_idesc_bf16(BT, HD, false, true);   // acc += (tmem A) B
                const uint32_t acc = tmem + (second ? TM_ACC1 : TM_ACC0);
                const uint32_t a = tmem + (second ? TM_P : TM_E);
                const uint32_t str_base = smem_base + (second ? SM_STR_B : SM_STR_A);
                bool ok = true;
                uint32_t g = 0;
                BwdItem I;
                for (int it = 0; ok && bwd_item<MODE>(P, it, I); ++it) {
                    for (int y = 0; y < I.n && ok; ++y, ++g) {
                        const int s = g % NST;
                        // the streamed tile (read here as the MN-major B operand) and E, P
                        ok = mx::mbar_wait(bar(BAR_STR_FULL + s), (g / NST) & 1, abort_flag, P.status);
                        if (ok) ok = mx::mbar_wait(bar(BAR_DS_READY), g & 1, abort_flag, P.status);
                        if (!ok) break;
                        mx::tc_fence_after();
                        const uint64_t sd = mx::smem_desc_sw128(str_base + s * STR_BYTES);
#pragma unroll
                        for (int k = 0; k < BS / 16; ++k) mx::mma_ts(acc, a + 8 * k, sd + 128 * k, IDESC_G, (y > 0 || k > 0));
                        // X, Y of this tile were complete before its E, P could be formed, so this commit
                        // also covers every read of the stage
                        mx::mma_commit(bar(BAR_STR_EMPTY + s));
                        if (y == I.n - 1) mx::mma_commit(bar(BAR_ACC_DONE));
                    }
                }
            }
            __syncwarp();
        } else if (FUSED && warp == 9) {
            // ------------------------- fused pass, issuer 1: X = K Q^T, then Y = V dO^T ------------
            // (the compute warps are busy with the previous tile for far longer than both take)
            {
                constexpr uint32_t IDESC_S = mx::mma_idesc_bf16(BT, BS, false, false);
                const uint64_t own_k = mx::smem_desc_sw128(smem_base + SM_OWN_A);
                const uint64_t own_v = mx::smem_desc_sw128(smem_base + SM_OWN_B);
                const uint64_t aug_x = mx::smem_desc_kmajor_plain(smem_base + SM_AUG_AX, SM_AUG_Z - SM_AUG_AX);
                const uint64_t aug_y = mx::smem_desc_kmajor_plain(smem_base + SM_AUG_AY, SM_AUG_Z - SM_AUG_AY);
                bool ok = true;
                uint32_t g = 0;
                BwdItem I;
                for (int it = 0; ok && bwd_item<MODE>(P, it, I); ++it) {
                    ok = __all_sync(0xFFFFFFFFu, mx::mbar_wait(bar(BAR_OWN_FULL), it & 1, abort_flag, P.status));
                    for (int y = 0; y < I.n && ok; ++y, ++g) {
                        const int s = g % NST;
                        ok = __all_sync(0xFFFFFFFFu, mx::mbar_wait(bar(BAR_STR_FULL + s), (g / NST) & 1, abort_flag, P.status));
                        if (ok && g > 0) ok = __all_sync(0xFFFFFFFFu, mx::mbar_wait(bar(BAR_SDP_FREE), (g - 1) & 1, abort_flag, P.status));
                        if (!ok) break;
                        mx::tc_fence_after();
                        const uint64_t sq = mx::smem_desc_sw128(smem_base + SM_STR_A + s * STR_BYTES);
                        const uint64_t so = mx::smem_desc_sw128(smem_base + SM_STR_B + s * STR_BYTES);
                        const uint64_t bq = mx::smem_desc_kmajor_plain(smem_base + SM_AUG_B + s * AUG_BYTES,
                                                                       SM_AUG_Z - SM_AUG_B - s * AUG_BYTES);
                        if (mx::elect_one()) {
#pragma unroll
                            for (int k = 0; k < HD / 16; ++k) mx::mma_ss(tmem + TM_X, own_k + 2 * k, sq + 2 * k, IDESC_S, k > 0);
                            mx::mma_ss(tmem + TM_X, aug_x, bq, IDESC_S, 1);   // X -= L (in the units of X) of the query column
#pragma unroll
                            for (int k = 0; k < HD / 16; ++k) mx::mma_ss(tmem + TM_Y, own_v + 2 * k, so + 2 * k, IDESC_S, k > 0);
                            mx::mma_ss(tmem + TM_Y, aug_y, bq, IDESC_S, 1);   // Y -= Delta of the query column
                            mx::mma_commit(bar(BAR_SDP_FULL));
                        }
                    }
                }
            }
            __syncwarp();
        } else if (FUSED && warp == 10) {
            // ------------------------- fused pass, issuer 2: dK += E Q, E (K-major) and Q from shared memory ----
            {
                constexpr uint32_t IDESC_G = mx::mma_idesc_bf16(BT, HD, false, true);
                const uint64_t ds0 = mx::smem_desc_sw128(smem_base + SM_DS), ds1 = mx::smem_desc_sw128(smem_base + SM_DS1_A);
                bool ok = true;
                uint32_t g = 0;
                BwdItem I;
                for (int it = 0; ok && bwd_item<MODE>(P, it, I); ++it) {
                    for (int y = 0; y < I.n && ok; ++y, ++g) {
                        const int s = g % NST;
                        ok = __all_sync(0xFFFFFFFFu, mx::mbar_wait(bar(BAR_STR_FULL + s), (g / NST) & 1, abort_flag, P.status));
                        if (ok) ok = __all_sync(0xFFFFFFFFu, mx::mbar_wait(bar(BAR_DS_READY), g & 1, abort_flag, P.status));
                        if (!ok) break;
                        mx::tc_fence_after();
                        const uint64_t sd = mx::smem_desc_sw128(smem_base + SM_STR_A + s * STR_BYTES);
                        // 16 queries of contraction = 32 B inside a row; queries 64.. are the second half tile
                        const uint64_t lo = (g & 1) ? ds1 : ds0;
                        const uint64_t hi = lo + (uint64_t)(((g & 1) ? SM_DS1_B - SM_DS1_A : DS_HALF_BYTES) >> 4);
                        if (mx::elect_one()) {
#pragma unroll
                            for (int k = 0; k < BS / 16; ++k)
                                mx::mma_ss(tmem + TMF_ACC0, (k >> 2 ? hi : lo) + (uint64_t)(2 * (k & 3)), sd + 128 * k, IDESC_G,
                                           (y > 0 || k > 0));
                            mx::mma_commit(bar(BAR_STR_EMPTY + s));
                            if (y == I.n - 1) mx::mma_commit(bar(BAR_ACC_DONE));
                        }
                    }
                }
            }
            __syncwarp();
        } else if (FUSED && warp == 11) {
            // ------------------------- fused pass, issuer 3: dV += P dO, then this tile's dQ = E^T K ----------
            // dQ: A = E read with the queries contiguous (MN-major; the second 64 queries in the other half
            // tile), B = the owned K tile with its rows as the contraction; a fresh accumulator per tile,
            // taken over by the drain warps.
            {
                constexpr uint32_t IDESC_G = mx::mma_idesc_bf16(BT, HD, false, true);
                constexpr uint32_t IDESC_Q = mx::mma_idesc_bf16(BS, HD, true, true);
                const uint64_t ad0 = mx::smem_desc_sw128_mn(smem_base + SM_DS, DS_HALF_BYTES);
                const uint64_t ad1 = mx::smem_desc_sw128_mn(smem_base + SM_DS1_A, SM_DS1_B - SM_DS1_A);
                const uint64_t bd = mx::smem_desc_sw128(smem_base + SM_OWN_A);
                bool ok = true;
                uint32_t g = 0;
                BwdItem I;
                for (int it = 0; ok && bwd_item<MODE>(P, it, I); ++it) {
                    for (int y = 0; y < I.n && ok; ++y, ++g) {
                        const int s = g % NST;
                        ok = __all_sync(0xFFFFFFFFu, mx::mbar_wait(bar(BAR_STR_FULL + s), (g / NST) & 1, abort_flag, P.status));
                        if (ok) ok = __all_sync(0xFFFFFFFFu, mx::mbar_wait(bar(BAR_DS_READY), g & 1, abort_flag, P.status));
                        if (!ok) break;
                        mx::tc_fence_after();
                        const uint64_t sd = mx::smem_desc_sw128(smem_base + SM_STR_B + s * STR_BYTES);
                        if (mx::elect_one()) {
#pragma unroll
                            for (int k = 0; k < BS / 16; ++k)
                                mx::mma_ts(tmem + TMF_ACC1, tmem + TMF_P + 8 * k, sd + 128 * k, IDESC_G, (y > 0 || k > 0));
                        }
                        // the drain warps hold the previous dQ tile in registers
                        if (g > 0) ok = __all_sync(0xFFFFFFFFu, mx::mbar_wait(bar(BAR_DQ_FREE), (g - 1) & 1, abort_flag, P.status));
                        if (!ok) break;
                        mx::tc_fence_after();
                        const uint64_t ad = (g & 1) ? ad1 : ad0;
                        if (mx::elect_one()) {
#pragma unroll
                            for (int k = 0; k < BT / 16; ++k) mx::mma_ss(tmem + TMF_DQ, ad + 128 * k, bd + 128 * k, IDESC_Q, k > 0);
                            mx::mma_commit(bar(BAR_DQ_FULL));
                            mx::mma_commit(bar(BAR_STR_EMPTY + s));
                            if (y == I.n - 1) mx::mma_commit(bar(BAR_ACC_DONE));
                        }
                    }
                }
            }
            __syncwarp();
        } else if (FUSED && warp >= 12) {
            // ------------------------- fused pass, drain warps: dQ tile -> global memory -------------------
            // Warp 12 + j takes lanes 32j .. 32j+31 (queries) of the finished 128 x 64 tile, 0.125 applied, through
            // a 4 KB swizzled staging tile of its own (32 queries x 32 dims at a time) and hands it to the TMA
            // unit, which adds it to dQ in global memory (fp32 reductions at L2, whole 128-byte lines, rows past
            // the end of the sequence clipped).  Per-thread red instructions from the registers were slower: they
            // stall their warp on issue and, in any lane layout a tensor-memory load gives directly, split lines.
            const uint32_t ta = tmem + ((uint32_t)((warp & 3) * 32) << 16) + TMF_DQ;
            const uint32_t stage = smem_base + SM_DQ + (warp & 3) * DQ_STAGE_BYTES;
            unsigned char *stage_row = smem + SM_DQ + (warp & 3) * DQ_STAGE_BYTES + lane * 128;
            if (lane == 0) mx::tma_prefetch_desc(&tmDQ);
            bool ok = true;
            uint32_t g = 0;
            BwdItem I;
            for (int it = 0; ok && bwd_item<MODE>(P, it, I); ++it) {
                for (int y = 0; y < I.n; ++y, ++g) {
                    ok = __all_sync(0xFFFFFFFFu, mx::mbar_wait(bar(BAR_DQ_FULL), g & 1, abort_flag, P.status));
                    if (!ok) break;
                    mx::tc_fence_after();
                    const int qw = (I.it_beg + y) * BS + (warp & 3) * 32;   // first query of this warp's 32
#pragma unroll
                    for (int half = 0; half < 2; ++half) {
                        uint32_t v[32];
                        mx::tmem_ld32(ta + half * 32, v);
                        mx::tmem_wait_ld();
                        if (half == 1) {  // the whole tile has left tensor memory
                            mx::tc_fence_before();
                            __syncwarp();
                            if (lane == 0) mx::mbar_arrive(bar(BAR_DQ_FREE));
                        }
                        // the previous reduction has finished reading the staging tile
                        if (lane == 0) mx::bulk_wait_group_read<0>();
                        __syncwarp();
#pragma unroll
                        for (int cch = 0; cch < 8; ++cch)
                            *(float4 *)(stage_row + ((cch ^ (lane & 7)) << 4)) =
                                make_float4(__uint_as_float(v[4 * cch]) * 0.125f, __uint_as_float(v[4 * cch + 1]) * 0.125f,
                                            __uint_as_float(v[4 * cch + 2]) * 0.125f, __uint_as_float(v[4 * cch + 3]) * 0.125f);
                        mx::fence_proxy_async_smem();
                        __syncwarp();
                        if (lane == 0 && qw < N) {   // a tile wholly past the end has nothing to add
                            mx::tma_reduce_add_3d(&tmDQ, stage, half * 32, qw, I.bh);
                            mx::bulk_commit_group();
                        }
                    }
                }
            }
            // the staging tile must outlive the reads; the reductions themselves complete before the grid does
            if (lane == 0) mx::bulk_wait_group_read<0>();
            __syncwarp();
        }
    } else {
        // ------------------------- compute warpgroups -------------------
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(REGS_COMPUTE));
        const int h = warp >> 2;                        // column half of this warpgroup
        const uint32_t lane_off = (uint32_t)((warp & 3) * 32) << 16;
        const uint32_t tm_row = tmem + lane_off;
        const float c = 0.125f * LOG2E;
        // dK = scale * dS^T Q; with Q staged as Q * scale * log2(e) that is dS^T Q' / log2(e)
        constexpr float DK_SCALE = PRE ? 0.6931471805599453f : 0.125f;
        bool ok = true;
        uint32_t g = 0;   // streamed tiles so far, over all items
        BwdItem I;
        for (int it = 0; ok && bwd_item<MODE>(P, it, I); ++it) {
        const int bh = I.bh, own0 = I.own0, n = I.n, it_beg = I.it_beg;
        const int row = own0 + (tid & 127);             // owned row (query | key) of this thread
        const bool rv = row < N;
        float nl0 = 0.0f, nl1 = 0.0f, nd0 = 0.0f, nd1 = 0.0f;  // -L*log2e and -Delta (MODE 0: of this row)
        if (MODE == 0) {
            nl0 = nl1 = rv ? -P.L[(size_t)bh * N + row] * LOG2E : 0.0f;
            nd0 = nd1 = rv ? -P.Delta[(size_t)bh * N + row] : 0.0f;
            // this thread's row of Q (left warpgroup) or dO (right) as a bf16 A operand: 32 packed columns
            uint32_t w[32];
            const uint4 *src = (h == 0 ? P.own_a : P.own_b) + ((size_t)bh * N + row) * (HD * 2 / 16);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const uint4 x = rv ? src[i] : make_uint4(0u, 0u, 0u, 0u);
                w[4 * i] = x.x, w[4 * i + 1] = x.y, w[4 * i + 2] = x.z, w[4 * i + 3] = x.w;
            }
            mx::tmem_st32(tm_row + (h == 0 ? TM_OWN_A : TM_OWN_B), w);
            mx::tmem_wait_st();
            mx::tc_fence_before();
            __syncwarp();
            if (lane == 0) mx::mbar_arrive(bar(BAR_OWN_FULL));
        }
        for (int y = 0; y < n; ++y, ++g) {
            const int s = g % NST;
            const uint32_t r = g / NST;
            ok = __all_sync(0xFFFFFFFFu, mx::mbar_wait(bar(BAR_SDP_FULL), g & 1, abort_flag, P.status));
            if (MODE == 1 && ok)  // the stage's L / Delta slices were written with plain stores
                ok = __all_sync(0xFFFFFFFFu, mx::mbar_wait(bar(BAR_STR_FULL + s), r & 1, abort_flag, P.status));
            if (!ok) break;
            mx::tc_fence_after();
            uint32_t xv[HS], yv[HS];
#if BWD_SPLIT_LOAD
            // the second 32 columns are requested once the first have landed and arrive under their arithmetic
            mx::tmem_ld32(tm_row + TM_X + h * HS, *(uint32_t(*)[32])(xv));
            mx::tmem_ld32(tm_row + TM_Y + h * HS, *(uint32_t(*)[32])(yv));
            mx::tmem_wait_ld();
            mx::tmem_ld32(tm_row + TM_X + h * HS + 32, *(uint32_t(*)[32])(xv + 32));
            mx::tmem_ld32(tm_row + TM_Y + h * HS + 32, *(uint32_t(*)[32])(yv + 32));
#else
            mx::tmem_ld32(tm_row + TM_X + h * HS, *(uint32_t(*)[32])(xv));
            mx::tmem_ld32(tm_row + TM_X + h * HS + 32, *(uint32_t(*)[32])(xv + 32));
            mx::tmem_ld32(tm_row + TM_Y + h * HS, *(uint32_t(*)[32])(yv));
            mx::tmem_ld32(tm_row + TM_Y + h * HS + 32, *(uint32_t(*)[32])(yv + 32));
            mx::tmem_wait_ld();
            mx::tc_fence_before();
            __syncwarp();
            if (lane == 0) mx::mbar_arrive(bar(BAR_SDP_FREE));
#endif

            const int str0 = (it_beg + y) * BS + h * HS;    // first streamed row of this half
            const bool need_mask = (str0 + HS > N) ||
                                   (P.causal && (MODE == 0 ? (str0 + HS - 1 > own0) : (str0 < own0 + BT - 1)));
            const float *ld = (const float *)(smem + SM_LD + s * (2 * BS * 4)) + h * HS;
            auto mask_cols = [&](int i0, int i1) {
                // masked scores become -inf up front (p = 0, so E = 0): the main loop stays branch-free
#pragma unroll
                for (int i = i0; i < i1; ++i) {
                    const int c0 = str0 + i;
                    const bool v0 = c0 < N && (!P.causal || (MODE == 0 ? c0 <= row : c0 >= row));
                    if (!v0) xv[i] = 0xFF800000u;
                }
            };
            if (need_mask) mask_cols(0, BWD_SPLIT_LOAD ? 32 : HS);
            uint32_t pe[HS / 2], pp[MODE >= 1 ? HS / 2 : 1];
            // fused pass: E goes to shared memory as bf16, this thread's key row = one 128-byte swizzled line of
            // 64 queries.  Two buffers: the MMAs of tile y-1 may still read the other one (those of y-2 are
            // done: the previous iteration waited for them before its own tensor-memory stores).
            unsigned char *dsrow = smem + ((g & 1) ? SM_DS1_A + h * (SM_DS1_B - SM_DS1_A) : SM_DS + h * DS_HALF_BYTES) +
                                   (tid & 127) * 128;
#pragma unroll
            for (int i = 0; i < HS; i += 2) {
#if BWD_SPLIT_LOAD
                if (i == 32) {   // the second half of this thread's X, Y is in registers: the MMAs may overwrite them
                    mx::tmem_wait_ld();
                    mx::tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mx::mbar_arrive(bar(BAR_SDP_FREE));
                    if (need_mask) mask_cols(32, HS);
                }
#endif
                if (MODE == 1) {
                    const float2 l2 = *(const float2 *)(ld + i), d2 = *(const float2 *)(ld + BS + i);
                    nl0 = l2.x, nl1 = l2.y, nd0 = d2.x, nd1 = d2.y;
                }
                // (fused pass: X, Y arrive with -8 L and -Delta already added by the MMAs; nl, nd stay 0)
                float p0, p1;
                if (FUSED && PRE && ((i >> 1) & 3) < BWD_POLY) {
                    // a share of the exponentials on the FMA pipe (the exp unit is what the two compute warps of a
                    // scheduler queue for); the arguments are <= ~0 but unbounded below, masked ones -inf
                    mx::ex2_poly2<true>(__uint_as_float(xv[i]), __uint_as_float(xv[i + 1]), p0, p1);
                } else if (FUSED) {
                    p0 = PRE ? mx::ex2(__uint_as_float(xv[i])) : mx::ex2(__uint_as_float(xv[i]) * c);
                    p1 = PRE ? mx::ex2(__uint_as_float(xv[i + 1])) : mx::ex2(__uint_as_float(xv[i + 1]) * c);
                } else {
                    p0 = PRE ? mx::ex2(__uint_as_float(xv[i]) + nl0) : mx::ex2(fmaf(__uint_as_float(xv[i]), c, nl0));
                    p1 = PRE ? mx::ex2(__uint_as_float(xv[i + 1]) + nl1) : mx::ex2(fmaf(__uint_as_float(xv[i + 1]), c, nl1));
                }
                const float e0 = FUSED ? p0 * __uint_as_float(yv[i]) : p0 * (__uint_as_float(yv[i]) + nd0);
                const float e1 = FUSED ? p1 * __uint_as_float(yv[i + 1]) : p1 * (__uint_as_float(yv[i + 1]) + nd1);
                pe[i >> 1] = mx::pack_bf16(e0, e1);
                if (MODE >= 1) pp[i >> 1] = mx::pack_bf16(p0, p1);
                if (FUSED && (i & 7) == 6) {  // eight values = one 16-byte piece of this key row's swizzled line
                    const int cch = i >> 3;
                    *(uint4 *)(dsrow + ((cch ^ (tid & 7)) << 4)) =
                        make_uint4(pe[4 * cch], pe[4 * cch + 1], pe[4 * cch + 2], pe[4 * cch + 3]);
                }
            }
            if (g > 0) {  // the accumulate MMAs of the previous tile (of the previous item, at y == 0) have consumed E, P
                ok = __all_sync(0xFFFFFFFFu, mx::mbar_wait(bar(BAR_STR_EMPTY + (g - 1) % NST),
                                                           ((g - 1) / NST) & 1, abort_flag, P.status));
                if (!ok) break;
                mx::tc_fence_after();
            }
            if (FUSED) mx::fence_proxy_async_smem();   // E went to shared memory inside the loop above
            else mx::tmem_st32(tm_row + TM_E + h * (HS / 2), *(uint32_t(*)[32])(pe));
            if (MODE >= 1) mx::tmem_st32(tm_row + tP + h * (HS / 2), *(uint32_t(*)[32])(pp));
            mx::tmem_wait_st();
            mx::tc_fence_before();
            __syncwarp();
            if (lane == 0) mx::mbar_arrive(bar(BAR_DS_READY));
        }
        // ---- epilogue: accumulators -> global, dS's 1/sqrt(d) applied here ----
        if (ok) ok = __all_sync(0xFFFFFFFFu, mx::mbar_wait(bar(BAR_ACC_DONE), it & 1, abort_flag, P.status));
        if (ok) {
            mx::tc_fence_after();
            if (MODE == 0) {
                // both warpgroups hold the same 128 rows: the left one stores dims 0..31, the right one 32..63
                uint32_t v[32];
                mx::tmem_ld32(tm_row + TM_ACC0 + h * 32, v);
                mx::tmem_wait_ld();
                if (rv) {
                    float *dst = P.out0 + ((size_t)bh * N + row) * HD + h * 32;
#pragma unroll
                    for (int i = 0; i < 32; i += 4)
                        *(float4 *)(dst + i) = make_float4(__uint_as_float(v[i]) * 0.125f, __uint_as_float(v[i + 1]) * 0.125f,
                                                           __uint_as_float(v[i + 2]) * 0.125f, __uint_as_float(v[i + 3]) * 0.125f);
                }
            } else if (FUSED) {
                // the left warpgroup stores dK (scaled), the right one dV: each warp stages its 32 rows, 32 columns
                // at a time, in a swizzled 4 KB tile and hands it to the TMA unit -- 16-byte stores from lane = row
                // registers would each touch a sector of their own and took 3.2 us per CTA.  The two staging tiles
                // are this warp's own 32 rows of the two E buffers (every MMA of the item has completed, and no other
                // warp writes there), so the stream stages and the owned tiles are free for the next item's loads
                // meanwhile.
                const float sc = h == 0 ? DK_SCALE : 1.0f;
                const CUtensorMap *tm = h == 0 ? &tmOut0 : &tmOut1;
                const int wrow0 = own0 + (warp & 3) * 32;
                const int st_off[2] = {SM_DS + h * DS_HALF_BYTES + (warp & 3) * DQ_STAGE_BYTES,
                                       SM_DS1_A + h * (SM_DS1_B - SM_DS1_A) + (warp & 3) * DQ_STAGE_BYTES};
#pragma unroll
                for (int cc = 0; cc < 2; ++cc) {
                    uint32_t v[32];
                    mx::tmem_ld32(tm_row + (h == 0 ? tACC0 : tACC1) + cc * 32, v);
                    mx::tmem_wait_ld();
                    unsigned char *srow = smem + st_off[cc] + lane * 128;
#pragma unroll
                    for (int cch = 0; cch < 8; ++cch)
                        *(float4 *)(srow + ((cch ^ (lane & 7)) << 4)) =
                            make_float4(__uint_as_float(v[4 * cch]) * sc, __uint_as_float(v[4 * cch + 1]) * sc,
                                        __uint_as_float(v[4 * cch + 2]) * sc, __uint_as_float(v[4 * cch + 3]) * sc);
                }
                mx::fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0 && wrow0 < N) {
                    mx::tma_store_3d(tm, smem_base + st_off[0], 0, wrow0, bh);
                    mx::tma_store_3d(tm, smem_base + st_off[1], 32, wrow0, bh);
                    mx::bulk_commit_group();
                    mx::bulk_wait_group_read<0>();   // the staging tiles must outlive the reads
                }
                __syncwarp();
            } else {
                // the left warpgroup stores dK (scaled), the right one dV
                const float sc = h == 0 ? DK_SCALE : 1.0f;
                float *dst = (h == 0 ? P.out0 : P.out1) + ((size_t)bh * N + row) * HD;
#pragma unroll
                for (int cc = 0; cc < 2; ++cc) {
                    uint32_t v[32];
                    mx::tmem_ld32(tm_row + (h == 0 ? tACC0 : tACC1) + cc * 32, v);
                    mx::tmem_wait_ld();
                    if (rv) {
#pragma unroll
                        for (int i = 0; i < 32; i += 4)
                            *(float4 *)(dst + cc * 32 + i) =
                                make_float4(__uint_as_float(v[i]) * sc, __uint_as_float(v[i + 1]) * sc,
                                            __uint_as_float(v[i + 2]) * sc, __uint_as_float(v[i + 3]) * sc);
                    }
                }
            }
        }
        }  // items
    }
    mx::tc_fence_before();
    __syncthreads();
    mx::tc_fence_after();
    if (warp == 9) mx::tmem_dealloc(tmem, TM_COLS);
}

// Delta_i = sum_x dO[i,x] O[i,x]; 16 threads per row, one float4 each.  With `dOb` the bf16 copy of dO that the
// backward's tensor-core passes read is written on the way (the values are in registers here anyway).
__global__ void bwd_preprocess_kernel(const float *dO, const float *O, float *Delta, size_t rows, __nv_bfloat16 *dOb) {
    size_t gid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    size_t row = gid >> 4;
    int part = (int)(gid & 15);
    float d = 0.0f;
    if (row < rows) {
        float4 a = *(const float4 *)(dO + row * HD + part * 4);
        float4 b = *(const float4 *)(O + row * HD + part * 4);
        d = a.x * b.x + a.y * b.y + a.z * b.z + a.w * b.w;
        if (dOb) {
            __nv_bfloat162 lo = __floats2bfloat162_rn(a.x, a.y), hi = __floats2bfloat162_rn(a.z, a.w);
            uint2 w;
            w.x = *(const uint32_t *)&lo, w.y = *(const uint32_t *)&hi;
            *(uint2 *)(dOb + row * HD + part * 4) = w;
        }
    }
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) d += __shfl_xor_sync(0xFFFFFFFFu, d, o);
    if (row < rows && part == 0) Delta[row] = d;
}

// function attributes are per device: one handle per GPU may live in the same process
int set_attrs(int device) {
    static bool done[64] = {};
    MX_REQUIRE(device >= 0 && device < 64, MX230_ERR_UNSUPPORTED, "flash backward: device index %d", device);
    if (!done[device]) {
        MX_CHECK_CUDA(cudaFuncSetAttribute(bwd_kernel<0, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SM_ALLOC));
        MX_CHECK_CUDA(cudaFuncSetAttribute(bwd_kernel<1, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SM_ALLOC));
        MX_CHECK_CUDA(cudaFuncSetAttribute(bwd_kernel<2, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SM_ALLOC));
        MX_CHECK_CUDA(cudaFuncSetAttribute(bwd_kernel<0, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SM_ALLOC));
        MX_CHECK_CUDA(cudaFuncSetAttribute(bwd_kernel<1, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SM_ALLOC));
        MX_CHECK_CUDA(cudaFuncSetAttribute(bwd_kernel<2, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SM_ALLOC));
        done[device] = true;
    }
    return MX230_OK;
}

struct Maps {
    CUtensorMap box128[4];  // Q, K, V, dO with 128-row boxes (owned and streamed tiles alike)
    const void *ptr[4];     // the bf16 tensors themselves
};

int make_maps(mx230_handle *h, Maps &m, const void *Qb, const void *Kb, const void *Vb, const void *dOb,
              int batch_heads, int n) {
    const void *p[4] = {Qb, Kb, Vb, dOb};
    uint64_t rs = HD * 2, os = (uint64_t)n * HD * 2;
    for (int i = 0; i < 4; ++i) {
        int rc;
        m.ptr[i] = p[i];
        if ((rc = mx230_make_tmap_bf16(h, &m.box128[i], p[i], n, batch_heads, rs, os, BT))) return rc;
    }
    return MX230_OK;
}

// work-item fields of the parameters; returns the number of items
int set_items(BwdParams &P, int batch_heads, int n) {
    P.test_drop_tile = -1;
    P.heads = batch_heads;
    P.n_tiles = (n + BT - 1) / BT;
    P.n_items = batch_heads * P.n_tiles;
    return P.n_items;
}

int launch_dq(mx230_handle *h, cudaStream_t st, const Maps &m, const float *L, const float *Delta, float *dQ,
              int batch_heads, int n, int causal, bool pre) {
    BwdParams P{L, Delta, dQ, nullptr, nullptr, (const uint4 *)m.ptr[0], (const uint4 *)m.ptr[3], n, causal ? 1 : 0,
                h->status_dev};
    dim3 grid((unsigned)set_items(P, batch_heads, n));   // one item per CTA
    if (pre)
        MX_LAUNCH(h, st, MX230_K_BWD_DQ,
                  (bwd_kernel<0, true><<<grid, BWD_THREADS, SM_ALLOC, st>>>(m.box128[0], m.box128[3], m.box128[1], m.box128[2],
                                                                            m.box128[0], m.box128[0], m.box128[0], P)));
    else
        MX_LAUNCH(h, st, MX230_K_BWD_DQ,
                  (bwd_kernel<0, false><<<grid, BWD_THREADS, SM_ALLOC, st>>>(m.box128[0], m.box128[3], m.box128[1], m.box128[2],
                                                                             m.box128[0], m.box128[0], m.box128[0], P)));
    return MX230_OK;
}

int launch_dkv(mx230_handle *h, cudaStream_t st, const Maps &m, const float *L, const float *Delta, float *dK,
               float *dV, int batch_heads, int n, int causal, bool pre) {
    BwdParams P{L, Delta, dK, dV, nullptr, nullptr, nullptr, n, causal ? 1 : 0, h->status_dev};
    dim3 grid((unsigned)set_items(P, batch_heads, n));   // one item per CTA
    if (pre)
        MX_LAUNCH(h, st, MX230_K_BWD_DKV,
                  (bwd_kernel<1, true><<<grid, BWD_THREADS, SM_ALLOC, st>>>(m.box128[1], m.box128[2], m.box128[0], m.box128[3],
                                                                            m.box128[0], m.box128[0], m.box128[0], P)));
    else
        MX_LAUNCH(h, st, MX230_K_BWD_DKV,
                  (bwd_kernel<1, false><<<grid, BWD_THREADS, SM_ALLOC, st>>>(m.box128[1], m.box128[2], m.box128[0], m.box128[3],
                                                                             m.box128[0], m.box128[0], m.box128[0], P)));
    return MX230_OK;
}

// One pass over the (key tile, query tile) pairs for all three gradients: dK, dV written once by the
// CTA that owns the key tile, dQ zeroed here and summed into by every CTA (fp32 reductions at L2, so
// the order of dQ's partial sums is not fixed from run to run).
int launch_fused(mx230_handle *h, cudaStream_t st, const Maps &m, const float *L, const float *Delta, float *dQ,
                 float *dK, float *dV, int batch_heads, int n, int causal, bool dq_is_zero, bool pre) {
    CUtensorMap tm_dq, tm_dk, tm_dv;
    int rc = mx230_make_tmap_f32_half_rows(h, &tm_dq, dQ, n, batch_heads);
    if (!rc) rc = mx230_make_tmap_f32_half_rows(h, &tm_dk, dK, n, batch_heads);
    if (!rc) rc = mx230_make_tmap_f32_half_rows(h, &tm_dv, dV, n, batch_heads);
    if (rc) return rc;
    if (!dq_is_zero) MX_CHECK_CUDA(cudaMemsetAsync(dQ, 0, (size_t)batch_heads * n * HD * sizeof(float), st));
    BwdParams P{L, Delta, dK, dV, dQ, nullptr, nullptr, n, causal ? 1 : 0, h->status_dev};
    // persistent: one CTA per SM (the kernel holds all of an SM's tensor memory) walks its share of the items, the
    // next item's owned and first streamed tiles loading while the compute warps store the current item's dK, dV
    const int n_items = set_items(P, batch_heads, n);
    P.test_drop_tile = h->test_drop_tile;
    dim3 grid((unsigned)(n_items < h->sm_count ? n_items : h->sm_count));
    if (pre)
        MX_LAUNCH(h, st, MX230_K_BWD_FUSED,
                  (bwd_kernel<2, true><<<grid, BWD_THREADS, SM_ALLOC, st>>>(m.box128[1], m.box128[2], m.box128[0], m.box128[3],
                                                                            tm_dq, tm_dk, tm_dv, P)));
    else
        MX_LAUNCH(h, st, MX230_K_BWD_FUSED,
                  (bwd_kernel<2, false><<<grid, BWD_THREADS, SM_ALLOC, st>>>(m.box128[1], m.box128[2], m.box128[0], m.box128[3],
                                                                             tm_dq, tm_dk, tm_dv, P)));
    return MX230_OK;
}

int check_args(const char *who, mx230_handle *h, int batch_heads, int n) {
    MX_REQUIRE(h != nullptr, MX230_ERR_INVALID_ARG, "%s: null handle", who);
    MX_REQUIRE(batch_heads >= 0 && n >= 0, MX230_ERR_INVALID_ARG, "%s: negative size", who);
    MX_REQUIRE(batch_heads <= 65535, MX230_ERR_UNSUPPORTED, "%s: batch_heads %d > 65535", who, batch_heads);
    return MX230_OK;
}

// which: bit 0 = dQ pass, bit 1 = dK/dV pass
int bwd_bf16(mx230_handle *h, void *stream, const void *Qb, const void *Kb, const void *Vb, const void *dOb,
             const float *L, const float *Delta, float *dQ, float *dK, float *dV, int batch_heads, int n,
             int causal, int which, const char *who, bool dq_is_zero = false, bool pre = false) {
    MX_REQUIRE(Qb && Kb && Vb && dOb && L && Delta, MX230_ERR_INVALID_ARG, "%s: null input", who);
    MX_REQUIRE(!(which & 1) || dQ, MX230_ERR_INVALID_ARG, "%s: null dQ", who);
    MX_REQUIRE(!(which & 2) || (dK && dV), MX230_ERR_INVALID_ARG, "%s: null dK/dV", who);
    MX_REQUIRE((((uintptr_t)dQ | (uintptr_t)dK | (uintptr_t)dV) & 15) == 0, MX230_ERR_INVALID_ARG,
               "%s: outputs must be 16-byte aligned", who);
    int rc = set_attrs(h->device);
    if (rc) return rc;
    Maps m;
    if ((rc = make_maps(h, m, Qb, Kb, Vb, dOb, batch_heads, n))) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    if (which == 3 && !h->bwd_two_pass)
        return launch_fused(h, st, m, L, Delta, dQ, dK, dV, batch_heads, n, causal, dq_is_zero, pre);
    if ((which & 1) && (rc = launch_dq(h, st, m, L, Delta, dQ, batch_heads, n, causal, pre))) return rc;
    if ((which & 2) && (rc = launch_dkv(h, st, m, L, Delta, dK, dV, batch_heads, n, causal, pre))) return rc;
    return MX230_OK;
}

int bwd_fp32(mx230_handle *h, void *stream, const float *Q, const float *K, const float *V, const float *dO,
             const float *L, const float *Delta, float *dQ, float *dK, float *dV, int batch_heads, int n,
             int causal, int which, const char *who) {
    int rc = check_args(who, h, batch_heads, n);
    if (rc) return rc;
    if (batch_heads == 0 || n == 0) return MX230_OK;
    MX_REQUIRE(Q && K && V && dO, MX230_ERR_INVALID_ARG, "%s: null input", who);
    size_t need = mx230_flash_workspace_bytes(batch_heads, n, 1);
    MX_REQUIRE(h->ws && need <= h->ws_bytes, MX230_ERR_WORKSPACE,
               "%s: workspace %zu B < %zu B needed (call mx230_reserve)", who, h->ws_bytes, need);
    mx230_device_guard guard(h->device);
    size_t one = mx230_flash_stage_bytes(batch_heads, n);
    void *dst[4] = {h->ws, (char *)h->ws + one, (char *)h->ws + 2 * one, (char *)h->ws + 3 * one};
    const float *src[4] = {Q, K, V, dO};
    // the fused pass sums into dQ: the staging launch clears it on the way
    const bool fused = which == 3 && !h->bwd_two_pass;
    MX_REQUIRE(!fused || (dQ && ((uintptr_t)dQ & 15) == 0), MX230_ERR_INVALID_ARG, "%s: dQ null or not 16-byte aligned", who);
    // Q is staged as Q * scale * log2(e), bit for bit what the forward staged and took L from: the recomputed
    // probabilities then sum to one over a row whatever the rounding did to a single score.
    if (h->bwd_reuse_staged && h->staged.valid && h->staged.q == Q && h->staged.k == K && h->staged.v == V &&
        h->staged.batch_heads == batch_heads && h->staged.n == n) {
        // the forward's bf16 copies of these very tensors are still in the workspace: only dO is staged, and not even
        // that when the Delta pre-pass of this dO has left its bf16 copy in the fourth slot (dQ is then cleared by a memset)
        if (h->staged.d_o == dO) {
            if (fused) MX_CHECK_CUDA(cudaMemsetAsync(dQ, 0, (size_t)batch_heads * n * HD * sizeof(float), (cudaStream_t)stream));
        } else {
            h->staged.d_o = nullptr;   // the slot is about to hold another tensor's copy
            rc = mx230_launch_cast(h, (cudaStream_t)stream, src + 3, dst + 3, 1, batch_heads, (size_t)n * HD,
                                   fused ? dQ : nullptr, 1.0f, nullptr);
            if (!rc) h->staged.d_o = dO;
        }
    } else {
        h->staged.valid = 0;
        rc = mx230_launch_cast(h, (cudaStream_t)stream, src, dst, 4, batch_heads, (size_t)n * HD, fused ? dQ : nullptr,
                               MX230_QK_LOG2_SCALE, nullptr);
        if (!rc) h->staged = {Q, K, V, batch_heads, n, 1, dO};
    }
    if (rc) return rc;
    return bwd_bf16(h, stream, dst[0], dst[1], dst[2], dst[3], L, Delta, dQ, dK, dV, batch_heads, n, causal,
                    which, who, fused, true);
}

}  // namespace

extern "C" int mx230_attn_bwd_preprocess(mx230_handle *h, void *stream, const float *dO, const float *O,
                                         float *Delta, int batch_heads, int n) {
    int rc = check_args("attn_bwd_preprocess", h, batch_heads, n);
    if (rc) return rc;
    size_t rows = (size_t)batch_heads * n;
    if (rows == 0) return MX230_OK;
    MX_REQUIRE(dO && O && Delta, MX230_ERR_INVALID_ARG, "attn_bwd_preprocess: null tensor");
    MX_REQUIRE((((uintptr_t)dO | (uintptr_t)O) & 15) == 0, MX230_ERR_INVALID_ARG,
               "attn_bwd_preprocess: inputs must be 16-byte aligned");
    mx230_device_guard guard(h->device);
    size_t threads = rows * 16;
    cudaStream_t st = (cudaStream_t)stream;
    // With the reuse option, and the forward's staged Q, K, V of this very shape still in the workspace, the backward
    // that follows will look for dO's bf16 copy in the fourth staging slot: leave it there now.
    __nv_bfloat16 *dOb = nullptr;
    if (h->bwd_reuse_staged && h->staged.valid && h->staged.batch_heads == batch_heads && h->staged.n == n && h->ws &&
        mx230_flash_workspace_bytes(batch_heads, n, 1) <= h->ws_bytes) {
        dOb = (__nv_bfloat16 *)((char *)h->ws + 3 * mx230_flash_stage_bytes(batch_heads, n));
        h->staged.d_o = nullptr;
    }
    MX_LAUNCH(h, st, MX230_K_BWD_PREPROCESS,
              (bwd_preprocess_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, st>>>(dO, O, Delta, rows, dOb)));
    if (dOb) h->staged.d_o = dO;
    return MX230_OK;
}

extern "C" int mx230_attn_bwd_dq(mx230_handle *h, void *stream, const float *Q, const float *K, const float *V,
                                 const float *dO, const float *L, const float *Delta, float *dQ,
                                 int batch_heads, int n, int causal) {
    return bwd_fp32(h, stream, Q, K, V, dO, L, Delta, dQ, nullptr, nullptr, batch_heads, n, causal, 1,
                    "attn_bwd_dq");
}

extern "C" int mx230_attn_bwd_dkv(mx230_handle *h, void *stream, const float *Q, const float *K, const float *V,
                                  const float *dO, const float *L, const float *Delta, float *dK, float *dV,
                                  int batch_heads, int n, int causal) {
    return bwd_fp32(h, stream, Q, K, V, dO, L, Delta, nullptr, dK, dV, batch_heads, n, causal, 2,
                    "attn_bwd_dkv");
}

extern "C" int mx230_attn_bwd_flash(mx230_handle *h, void *stream, const float *Q, const float *K,
                                    const float *V, const float *dO, const float *L, const float *Delta,
                                    float *dQ, float *dK, float *dV, int batch_heads, int n, int causal) {
    return bwd_fp32(h, stream, Q, K, V, dO, L, Delta, dQ, dK, dV, batch_heads, n, causal, 3, "attn_bwd_flash");
}

extern "C" int mx230_attn_bwd_flash_bf16(mx230_handle *h, void *stream, const void *Qb, const void *Kb,
                                         const void *Vb, const void *dOb, const float *L, const float *Delta,
                                         float *dQ, float *dK, float *dV, int batch_heads, int n, int causal) {
    int rc = check_args("attn_bwd_flash_bf16", h, batch_heads, n);
    if (rc) return rc;
    if (batch_heads == 0 || n == 0) return MX230_OK;
    mx230_device_guard guard(h->device);
    return bwd_bf16(h, stream, Qb, Kb, Vb, dOb, L, Delta, dQ, dK, dV, batch_heads, n, causal, 3,
                    "attn_bwd_flash_bf16");
}

