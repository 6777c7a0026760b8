// Flash-attention backward for sm_100a: dQ, dK, dV of the scalar loss <O, dO>, with
// the probabilities recomputed from the saved log-sum-exp, never stored.
//
// Reference semantics: attn_bwd_preprocess, attn_bwd_dq, attn_bwd_dkv,
// 02-flash-attention/kernels/attention_bwd.cu:32-44,96-158,165-243 (fp32 SIMT):
//   Delta_i = sum_x dO[i,x] O[i,x]
//   p_ij  = exp(scale * q_i.k_j - L_i),  dP_ij = dO_i . v_j
//   dS_ij = p_ij (dP_ij - Delta_i) scale
//   dQ_i += dS_ij k_j ;  dK_j += dS_ij q_i ;  dV_j += p_ij dO_i
// The same atomic-free split is kept -- a dQ pass owned by query tiles and a dK/dV pass
// owned by key tiles, each output element written exactly once -- with all contractions on
// tcgen05 tensor cores (bf16 operands, fp32 accumulators in tensor memory).  Both passes are
// one kernel template: a CTA owns ONE 128-row tile (queries for dQ, keys for dK/dV) and
// streams 64-row tiles of the other axis through a TMA ring:
//
//   X = A_own A_str^T, Y = B_own B_str^T      (S, dP   |  S^T, dP^T)      SS MMAs into TMEM
//   P = exp2(X c - L), E = P o (Y - Delta)    one thread per owned row, registers
//   acc0 += E A_str   (dQ += dS K | dK += dS^T Q),   acc1 += P B_str (dV += P^T dO)   TS MMAs
//
// Two streamed tiles are in flight at once ("slots" = even / odd iteration), each with its own
// X, Y, E, P columns in tensor memory and its own compute warpgroup, so nothing aliases: the
// MMA warp issues X, Y of iteration j+2 as soon as the warpgroup has pulled iteration j into
// registers, and the accumulate MMAs of j when E, P are written.  The recomputed tiles go back
// to tensor memory as bf16 A operands; no operand is ever written to shared memory by a thread.
// The 1/sqrt(d) factor of dS is applied to the fp32 accumulators in the epilogue (exact: 2^-3).
#include <math_constants.h>

#include "common.cuh"

namespace {

constexpr int HD = 64;
constexpr int BT = 128;          // rows of the owned tile (queries in dQ, keys in dK/dV)
constexpr int BS = 64;           // rows of a streamed tile
constexpr int STAGES = 6;
constexpr int OWN_BYTES = BT * HD * 2;   // 16 KB
constexpr int STR_BYTES = BS * HD * 2;   // 8 KB
constexpr int BWD_THREADS = 384;
// setmaxnreg moves registers only inside the CTA's launch-time allocation (168 per thread)
static_assert(8 * 216 + 4 * 72 <= 12 * 168, "setmaxnreg budget exceeds the launch-time register allocation");         // warpgroups: compute slot 0, compute slot 1, {TMA, MMA, 2 idle}

// shared memory map (after 1024-byte alignment)
constexpr int SM_OWN_A = 0;                              // Q (dQ pass) / K (dK/dV pass)
constexpr int SM_OWN_B = SM_OWN_A + OWN_BYTES;           // dO / V
constexpr int SM_STR_A = SM_OWN_B + OWN_BYTES;           // STAGES x 8 KB: K / Q
constexpr int SM_STR_B = SM_STR_A + STAGES * STR_BYTES;  // STAGES x 8 KB: V / dO
constexpr int SM_LD = SM_STR_B + STAGES * STR_BYTES;     // STAGES x 2 x 64 floats: -L*log2e, -Delta (dK/dV)
constexpr int SM_BAR = SM_LD + STAGES * 2 * BS * 4;
constexpr int SM_TOTAL = SM_BAR + 256;
constexpr int SM_ALLOC = SM_TOTAL + 1024;

constexpr int BAR_OWN_FULL = 0;
constexpr int BAR_STR_FULL = 1;                          // [STAGES]
constexpr int BAR_STR_EMPTY = BAR_STR_FULL + STAGES;     // [STAGES]
constexpr int BAR_SDP_FULL = BAR_STR_EMPTY + STAGES;     // [2] MMA -> compute: X, Y written
constexpr int BAR_SDP_FREE = BAR_SDP_FULL + 2;           // [2] compute -> MMA: X, Y in registers
constexpr int BAR_DS_READY = BAR_SDP_FREE + 2;           // [2] compute -> MMA: E, P written
constexpr int BAR_DS_FREE = BAR_DS_READY + 2;            // [2] MMA -> compute: E, P consumed
constexpr int BAR_ACC_DONE = BAR_DS_FREE + 2;
constexpr int N_BARS = BAR_ACC_DONE + 1;

// tensor memory columns: slot u at u*192: X [0,64) Y [64,128) E [128,160) P [160,192)
constexpr int TM_SLOT = 192, TM_X = 0, TM_Y = 64, TM_E = 128, TM_P = 160;
constexpr int TM_ACC0 = 384, TM_ACC1 = 448;
constexpr int TM_COLS = 512;
constexpr float LOG2E = 1.4426950408889634f;

struct BwdParams {
    const float *L;      // [BH][N]
    const float *Delta;  // [BH][N]
    float *out0;         // dQ (dQ pass) / dK (dK/dV pass)   [BH][N][64]
    float *out1;         // unused / dV
    int n;
    int causal;
    int *status;
};

// MODE 0: dQ pass (own = Q, dO; stream = K, V).  MODE 1: dK/dV pass (own = K, V; stream = Q, dO).
template <int MODE>
__global__ void __launch_bounds__(BWD_THREADS, 1)
bwd_kernel(const __grid_constant__ CUtensorMap tmOwnA, const __grid_constant__ CUtensorMap tmOwnB,
           const __grid_constant__ CUtensorMap tmStrA, const __grid_constant__ CUtensorMap tmStrB,
           const BwdParams P) {
    extern __shared__ unsigned char smem_dyn[];
    const uint32_t smem_base = (mx::smem_u32(smem_dyn) + 1023u) & ~1023u;
    unsigned char *smem = smem_dyn + (smem_base - mx::smem_u32(smem_dyn));
    const uint32_t bar0 = smem_base + SM_BAR;
    auto bar = [&](int i) { return bar0 + 8u * (uint32_t)i; };
    volatile uint32_t *tmem_slot = (volatile uint32_t *)(smem + SM_BAR + 8 * N_BARS);
    volatile int *abort_flag = (volatile int *)(smem + SM_BAR + 8 * N_BARS + 8);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int N = P.n, bh = blockIdx.x;
    const int n_str_total = (N + BS - 1) / BS;
    // dQ: late query tiles see the most keys; dK/dV: early key tiles see the most queries.
    // Either way the heaviest tiles of every head are dispatched first.
    const int tile = (MODE == 0 && P.causal) ? (int)(gridDim.y - 1 - blockIdx.y) : (int)blockIdx.y;
    const int own0 = tile * BT;
    int it_beg = 0, it_end = n_str_total;
    if (P.causal) {
        if (MODE == 0) it_end = min(n_str_total, (own0 + BT - 1) / BS + 1);
        else it_beg = own0 / BS;
    }
    const int n = it_end - it_beg;  // >= 1

    if (tid == 0) {
        mx::mbar_init(bar(BAR_OWN_FULL), 1);
        for (int s = 0; s < STAGES; ++s) {
            mx::mbar_init(bar(BAR_STR_FULL + s), MODE == 1 ? 33 : 1);
            mx::mbar_init(bar(BAR_STR_EMPTY + s), 1);
        }
        for (int u = 0; u < 2; ++u) {
            mx::mbar_init(bar(BAR_SDP_FULL + u), 1);
            mx::mbar_init(bar(BAR_SDP_FREE + u), BT / 32);  // one elected lane per warp arrives
            mx::mbar_init(bar(BAR_DS_READY + u), BT / 32);
            mx::mbar_init(bar(BAR_DS_FREE + u), 1);
        }
        mx::mbar_init(bar(BAR_ACC_DONE), 1);
        *abort_flag = 0;
        mx::mbar_fence_init();
    }
    if (warp == 9) mx::tmem_alloc(mx::smem_u32((const void *)tmem_slot), TM_COLS);
    mx::tc_fence_before();
    __syncthreads();
    mx::tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    if (warp >= 8) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 72;");
        if (warp == 8) {
            // ------------------------- producer -------------------------
            if (lane == 0) {
                mx::tma_prefetch_desc(&tmOwnA);
                mx::tma_prefetch_desc(&tmOwnB);
                mx::tma_prefetch_desc(&tmStrA);
                mx::tma_prefetch_desc(&tmStrB);
                mx::mbar_expect_tx(bar(BAR_OWN_FULL), 2 * OWN_BYTES);
                mx::tma_load_3d(smem_base + SM_OWN_A, &tmOwnA, bar(BAR_OWN_FULL), 0, own0, bh);
                mx::tma_load_3d(smem_base + SM_OWN_B, &tmOwnB, bar(BAR_OWN_FULL), 0, own0, bh);
            }
            bool ok = true;
            for (int y = 0; y < n; ++y) {
                const int s = y % STAGES, r = y / STAGES;
                const int row0 = (it_beg + y) * BS;
                if (r > 0)
                    ok = __all_sync(0xFFFFFFFFu,
                                    mx::mbar_wait(bar(BAR_STR_EMPTY + s), (r - 1) & 1, abort_flag, P.status));
                if (!ok) break;
                if (lane == 0) {
                    mx::mbar_expect_tx(bar(BAR_STR_FULL + s), 2 * STR_BYTES);
                    mx::tma_load_3d(smem_base + SM_STR_A + s * STR_BYTES, &tmStrA, bar(BAR_STR_FULL + s), 0, row0, bh);
                    mx::tma_load_3d(smem_base + SM_STR_B + s * STR_BYTES, &tmStrB, bar(BAR_STR_FULL + s), 0, row0, bh);
                }
                if (MODE == 1) {
                    // -L*log2(e) and -Delta of the 64 streamed queries
                    float *ld = (float *)(smem + SM_LD + s * (2 * BS * 4));
#pragma unroll
                    for (int u = 0; u < 2; ++u) {
                        int q = row0 + u * 32 + lane;
                        bool v = q < N;
                        ld[u * 32 + lane] = v ? -P.L[(size_t)bh * N + q] * LOG2E : 0.0f;
                        ld[BS + u * 32 + lane] = v ? -P.Delta[(size_t)bh * N + q] : 0.0f;
                    }
                    mx::mbar_arrive(bar(BAR_STR_FULL + s));
                }
            }
            __syncwarp();
        } else if (warp == 9) {
            // ------------------------- MMA issuer 1: X, Y --------------------
            // (issuing one tcgen05.mma costs the issuing thread ~65 cycles, twice what a
            // 128x64x16 MMA takes to execute: the two MMA streams get a thread each)
            if (lane == 0) {
                constexpr uint32_t IDESC_S = mx::mma_idesc_bf16(BT, BS, false, false);  // [128 x 64] = A B^T
                const uint64_t own_a = mx::smem_desc_sw128(smem_base + SM_OWN_A);
                const uint64_t own_b = mx::smem_desc_sw128(smem_base + SM_OWN_B);
                auto issue_sdp = [&](int y) {
                    const int s = y % STAGES, u = y & 1;
                    const uint64_t sa = mx::smem_desc_sw128(smem_base + SM_STR_A + s * STR_BYTES);
                    const uint64_t sb = mx::smem_desc_sw128(smem_base + SM_STR_B + s * STR_BYTES);
#pragma unroll
                    for (int k = 0; k < HD / 16; ++k)
                        mx::mma_ss(tmem + u * TM_SLOT + TM_X, own_a + 2 * k, sa + 2 * k, IDESC_S, k > 0);
#pragma unroll
                    for (int k = 0; k < HD / 16; ++k)
                        mx::mma_ss(tmem + u * TM_SLOT + TM_Y, own_b + 2 * k, sb + 2 * k, IDESC_S, k > 0);
                    mx::mma_commit(bar(BAR_SDP_FULL + u));
                };
                bool ok = mx::mbar_wait(bar(BAR_OWN_FULL), 0, abort_flag, P.status);
                for (int y = 0; y < 2 && y < n && ok; ++y) {
                    ok = mx::mbar_wait(bar(BAR_STR_FULL + y), 0, abort_flag, P.status);
                    if (!ok) break;
                    mx::tc_fence_after();
                    issue_sdp(y);
                }
                // X, Y two iterations ahead, as soon as the slot's registers hold the current ones
                for (int y = 0; y + 2 < n && ok; ++y) {
                    const int s2 = (y + 2) % STAGES, r2 = (y + 2) / STAGES;
                    ok = mx::mbar_wait(bar(BAR_STR_FULL + s2), r2 & 1, abort_flag, P.status);
                    if (ok) ok = mx::mbar_wait(bar(BAR_SDP_FREE + (y & 1)), (y >> 1) & 1, abort_flag, P.status);
                    if (!ok) break;
                    mx::tc_fence_after();
                    issue_sdp(y + 2);
                }
            }
            __syncwarp();
        } else if (warp == 10) {
            // ------------------------- MMA issuer 2: accumulators ------------
            if (lane == 0) {
                constexpr uint32_t IDESC_G = mx::mma_idesc_bf16(BT, HD, false, true);   // acc += (tmem A) B
                bool ok = true;
                for (int y = 0; y < n && ok; ++y) {
                    const int s = y % STAGES, r = y / STAGES, u = y & 1;
                    // the streamed tile (read here as the MN-major B operand) and E, P of this slot
                    ok = mx::mbar_wait(bar(BAR_STR_FULL + s), r & 1, abort_flag, P.status);
                    if (ok) ok = mx::mbar_wait(bar(BAR_DS_READY + u), (y >> 1) & 1, abort_flag, P.status);
                    if (!ok) break;
                    mx::tc_fence_after();
                    const uint64_t sa = mx::smem_desc_sw128(smem_base + SM_STR_A + s * STR_BYTES);
                    const uint64_t sb = mx::smem_desc_sw128(smem_base + SM_STR_B + s * STR_BYTES);
                    if (MODE == 1) {
#pragma unroll
                        for (int k = 0; k < BS / 16; ++k)  // dV += P^T dO
                            mx::mma_ts(tmem + TM_ACC1, tmem + u * TM_SLOT + TM_P + 8 * k, sb + 128 * k, IDESC_G,
                                       (y > 0 || k > 0));
                    }
#pragma unroll
                    for (int k = 0; k < BS / 16; ++k)      // dQ += dS K  |  dK += dS^T Q
                        mx::mma_ts(tmem + TM_ACC0, tmem + u * TM_SLOT + TM_E + 8 * k, sa + 128 * k, IDESC_G,
                                   (y > 0 || k > 0));
                    mx::mma_commit(bar(BAR_DS_FREE + u));
                    // X, Y of this iteration were complete before its E, P could be formed, so this
                    // commit also covers every read of the stage
                    mx::mma_commit(bar(BAR_STR_EMPTY + s));
                    if (y == n - 1) mx::mma_commit(bar(BAR_ACC_DONE));
                }
            }
            __syncwarp();
        }
    } else {
        // ------------------------- compute warpgroups -------------------
        asm volatile("setmaxnreg.inc.sync.aligned.u32 216;");
        const int u = warp >> 2;                        // slot of this warpgroup
        const int row = own0 + (tid & 127);             // owned row (query | key) of this thread
        const uint32_t lane_off = (uint32_t)((warp & 3) * 32) << 16;
        const uint32_t tm_slot = tmem + lane_off + u * TM_SLOT;
        const float c = 0.125f * LOG2E;
        const bool rv = row < N;
        float nl0 = 0.0f, nl1 = 0.0f, nd0 = 0.0f, nd1 = 0.0f;  // -L*log2e and -Delta (MODE 0: of this row)
        if (MODE == 0) {
            nl0 = nl1 = rv ? -P.L[(size_t)bh * N + row] * LOG2E : 0.0f;
            nd0 = nd1 = rv ? -P.Delta[(size_t)bh * N + row] : 0.0f;
        }
        bool ok = true;
        for (int y = u; y < n; y += 2) {
            const int q = y >> 1;
            const int s = y % STAGES, r = y / STAGES;
            ok = __all_sync(0xFFFFFFFFu, mx::mbar_wait(bar(BAR_SDP_FULL + u), q & 1, abort_flag, P.status));
            if (MODE == 1 && ok)  // the stage's L / Delta slices were written with plain stores
                ok = __all_sync(0xFFFFFFFFu, mx::mbar_wait(bar(BAR_STR_FULL + s), r & 1, abort_flag, P.status));
            if (!ok) break;
            mx::tc_fence_after();
            uint32_t xv[BS], yv[BS];
            mx::tmem_ld32(tm_slot + TM_X, *(uint32_t(*)[32])(xv));
            mx::tmem_ld32(tm_slot + TM_X + 32, *(uint32_t(*)[32])(xv + 32));
            mx::tmem_ld32(tm_slot + TM_Y, *(uint32_t(*)[32])(yv));
            mx::tmem_ld32(tm_slot + TM_Y + 32, *(uint32_t(*)[32])(yv + 32));
            mx::tmem_wait_ld();
            mx::tc_fence_before();
            __syncwarp();
            if (lane == 0) mx::mbar_arrive(bar(BAR_SDP_FREE + u));

            const int str0 = (it_beg + y) * BS;
            const bool need_mask = (str0 + BS > N) ||
                                   (P.causal && (MODE == 0 ? (str0 + BS - 1 > own0) : (str0 < own0 + BT - 1)));
            const float *ld = (const float *)(smem + SM_LD + s * (2 * BS * 4));
            if (need_mask) {
                // masked scores become -inf up front (p = 0, so E = 0): the main loop stays branch-free
#pragma unroll
                for (int i = 0; i < BS; ++i) {
                    const int c0 = str0 + i;
                    const bool v0 = c0 < N && (!P.causal || (MODE == 0 ? c0 <= row : c0 >= row));
                    if (!v0) xv[i] = 0xFF800000u;
                }
            }
            uint32_t pe[BS / 2], pp[MODE == 1 ? BS / 2 : 1];
#pragma unroll
            for (int i = 0; i < BS; i += 2) {
                if (MODE == 1) {
                    const float2 l2 = *(const float2 *)(ld + i), d2 = *(const float2 *)(ld + BS + i);
                    nl0 = l2.x, nl1 = l2.y, nd0 = d2.x, nd1 = d2.y;
                }
                const float p0 = mx::ex2(fmaf(__uint_as_float(xv[i]), c, nl0));
                const float p1 = mx::ex2(fmaf(__uint_as_float(xv[i + 1]), c, nl1));
                const float e0 = p0 * (__uint_as_float(yv[i]) + nd0);
                const float e1 = p1 * (__uint_as_float(yv[i + 1]) + nd1);
                pe[i >> 1] = mx::pack_bf16(e0, e1);
                if (MODE == 1) pp[i >> 1] = mx::pack_bf16(p0, p1);
            }
            if (q > 0) {  // the accumulate MMAs of this slot's previous iteration have consumed E, P
                ok = __all_sync(0xFFFFFFFFu, mx::mbar_wait(bar(BAR_DS_FREE + u), (q - 1) & 1, abort_flag, P.status));
                if (!ok) break;
                mx::tc_fence_after();
            }
            mx::tmem_st32(tm_slot + TM_E, *(uint32_t(*)[32])(pe));
            if (MODE == 1) mx::tmem_st32(tm_slot + TM_P, *(uint32_t(*)[32])(pp));
            mx::tmem_wait_st();
            mx::tc_fence_before();
            __syncwarp();
            if (lane == 0) mx::mbar_arrive(bar(BAR_DS_READY + u));
        }
        // ---- epilogue: accumulators -> global, dS's 1/sqrt(d) applied here ----
        if (ok) ok = __all_sync(0xFFFFFFFFu, mx::mbar_wait(bar(BAR_ACC_DONE), 0, abort_flag, P.status));
        if (ok) {
            mx::tc_fence_after();
            const uint32_t tm_row = tmem + lane_off;
            if (MODE == 0) {
                // both warpgroups hold the same 128 rows: slot 0 stores dims 0..31, slot 1 dims 32..63
                uint32_t v[32];
                mx::tmem_ld32(tm_row + TM_ACC0 + u * 32, v);
                mx::tmem_wait_ld();
                if (rv) {
                    float *dst = P.out0 + ((size_t)bh * N + row) * HD + u * 32;
#pragma unroll
                    for (int i = 0; i < 32; i += 4)
                        *(float4 *)(dst + i) = make_float4(__uint_as_float(v[i]) * 0.125f, __uint_as_float(v[i + 1]) * 0.125f,
                                                           __uint_as_float(v[i + 2]) * 0.125f, __uint_as_float(v[i + 3]) * 0.125f);
                }
            } else {
                // slot 0 stores dK (scaled), slot 1 stores dV
                const float sc = u == 0 ? 0.125f : 1.0f;
                float *dst = (u == 0 ? P.out0 : P.out1) + ((size_t)bh * N + row) * HD;
#pragma unroll
                for (int cc = 0; cc < 2; ++cc) {
                    uint32_t v[32];
                    mx::tmem_ld32(tm_row + (u == 0 ? TM_ACC0 : TM_ACC1) + cc * 32, v);
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
    }
    mx::tc_fence_before();
    __syncthreads();
    mx::tc_fence_after();
    if (warp == 9) mx::tmem_dealloc(tmem, TM_COLS);
}

// Delta_i = sum_x dO[i,x] O[i,x]; 16 threads per row, one float4 each.
__global__ void bwd_preprocess_kernel(const float *dO, const float *O, float *Delta, size_t rows) {
    size_t gid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    size_t row = gid >> 4;
    int part = (int)(gid & 15);
    float d = 0.0f;
    if (row < rows) {
        float4 a = *(const float4 *)(dO + row * HD + part * 4);
        float4 b = *(const float4 *)(O + row * HD + part * 4);
        d = a.x * b.x + a.y * b.y + a.z * b.z + a.w * b.w;
    }
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) d += __shfl_xor_sync(0xFFFFFFFFu, d, o);
    if (row < rows && part == 0) Delta[row] = d;
}

int set_attrs() {
    static bool done = false;
    if (!done) {
        MX_CHECK_CUDA(cudaFuncSetAttribute(bwd_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, SM_ALLOC));
        MX_CHECK_CUDA(cudaFuncSetAttribute(bwd_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, SM_ALLOC));
        done = true;
    }
    return MX230_OK;
}

struct Maps {
    CUtensorMap own128[4];  // Q, K, V, dO with 128-row boxes
    CUtensorMap str64[4];   // Q, K, V, dO with 64-row boxes
};

int make_maps(mx230_handle *h, Maps &m, const void *Qb, const void *Kb, const void *Vb, const void *dOb,
              int batch_heads, int n) {
    const void *p[4] = {Qb, Kb, Vb, dOb};
    uint64_t rs = HD * 2, os = (uint64_t)n * HD * 2;
    for (int i = 0; i < 4; ++i) {
        int rc;
        if ((rc = mx230_make_tmap_bf16(h, &m.own128[i], p[i], n, batch_heads, rs, os, BT))) return rc;
        if ((rc = mx230_make_tmap_bf16(h, &m.str64[i], p[i], n, batch_heads, rs, os, BS))) return rc;
    }
    return MX230_OK;
}

int launch_dq(mx230_handle *h, cudaStream_t st, const Maps &m, const float *L, const float *Delta, float *dQ,
              int batch_heads, int n, int causal) {
    BwdParams P{L, Delta, dQ, nullptr, n, causal ? 1 : 0, h->status_dev};
    dim3 grid(batch_heads, (n + BT - 1) / BT);
    MX_LAUNCH(h, st, MX230_K_BWD_DQ,
              (bwd_kernel<0><<<grid, BWD_THREADS, SM_ALLOC, st>>>(m.own128[0], m.own128[3], m.str64[1],
                                                                  m.str64[2], P)));
    return MX230_OK;
}

int launch_dkv(mx230_handle *h, cudaStream_t st, const Maps &m, const float *L, const float *Delta, float *dK,
               float *dV, int batch_heads, int n, int causal) {
    BwdParams P{L, Delta, dK, dV, n, causal ? 1 : 0, h->status_dev};
    dim3 grid(batch_heads, (n + BT - 1) / BT);
    MX_LAUNCH(h, st, MX230_K_BWD_DKV,
              (bwd_kernel<1><<<grid, BWD_THREADS, SM_ALLOC, st>>>(m.own128[1], m.own128[2], m.str64[0],
                                                                  m.str64[3], P)));
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
             int causal, int which, const char *who) {
    MX_REQUIRE(Qb && Kb && Vb && dOb && L && Delta, MX230_ERR_INVALID_ARG, "%s: null input", who);
    MX_REQUIRE(!(which & 1) || dQ, MX230_ERR_INVALID_ARG, "%s: null dQ", who);
    MX_REQUIRE(!(which & 2) || (dK && dV), MX230_ERR_INVALID_ARG, "%s: null dK/dV", who);
    MX_REQUIRE((((uintptr_t)dQ | (uintptr_t)dK | (uintptr_t)dV) & 15) == 0, MX230_ERR_INVALID_ARG,
               "%s: outputs must be 16-byte aligned", who);
    int rc = set_attrs();
    if (rc) return rc;
    Maps m;
    if ((rc = make_maps(h, m, Qb, Kb, Vb, dOb, batch_heads, n))) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    if ((which & 1) && (rc = launch_dq(h, st, m, L, Delta, dQ, batch_heads, n, causal))) return rc;
    if ((which & 2) && (rc = launch_dkv(h, st, m, L, Delta, dK, dV, batch_heads, n, causal))) return rc;
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
    size_t one = need / 4;
    size_t count = (size_t)batch_heads * n * HD;
    void *dst[4] = {h->ws, (char *)h->ws + one, (char *)h->ws + 2 * one, (char *)h->ws + 3 * one};
    const float *src[4] = {Q, K, V, dO};
    rc = mx230_launch_cast(h, (cudaStream_t)stream, src, dst, 4, count);
    if (rc) return rc;
    return bwd_bf16(h, stream, dst[0], dst[1], dst[2], dst[3], L, Delta, dQ, dK, dV, batch_heads, n, causal,
                    which, who);
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
    MX_LAUNCH(h, st, MX230_K_BWD_PREPROCESS,
              (bwd_preprocess_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, st>>>(dO, O, Delta, rows)));
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

