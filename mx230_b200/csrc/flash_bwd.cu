// Flash-attention backward for sm_100a: dQ, dK, dV of the scalar loss <O, dO>, with
// the probabilities recomputed from the saved log-sum-exp, never stored.
//
// Reference semantics: attn_bwd_preprocess, attn_bwd_dq, attn_bwd_dkv,
// 02-flash-attention/kernels/attention_bwd.cu:32-44,96-158,165-243 (fp32 SIMT):
//   Delta_i = sum_x dO[i,x] O[i,x]
//   p_ij  = exp(scale * q_i.k_j - L_i),  dP_ij = dO_i . v_j
//   dS_ij = p_ij (dP_ij - Delta_i) scale
//   dQ_i += dS_ij k_j ;  dK_j += dS_ij q_i ;  dV_j += p_ij dO_i
// The same atomic-free split is kept -- a dQ pass owned by query tiles and a dK/dV
// pass owned by key tiles, each output element written exactly once -- with all
// contractions on tcgen05 tensor cores (bf16 operands, fp32 accumulators in tensor
// memory).  In both passes the recomputed P / dS tiles go back into tensor memory as
// bf16 and are consumed from there as the A operand, so no operand is ever written
// to shared memory by a thread.
//
// dQ pass:    CTA = two 128-query tiles; streams 64-key K/V tiles.
//             S = Q K^T, dP = dO V^T  ->  dS  ->  dQ += dS K
// dK/dV pass: CTA = two 128-key tiles; streams 64-query Q/dO tiles (+ their L, Delta).
//             S^T = K Q^T, dP^T = V dO^T  ->  P^T, dS^T  ->  dV += P^T dO, dK += dS^T Q
// Warp roles as in the forward: warps 0-3 / 4-7 compute tile 0 / 1 (one thread per
// row), warp 8 is the TMA producer, warp 9 issues the MMAs; the two tiles ping-pong.
#include <math_constants.h>

#include "common.cuh"

namespace {

constexpr int HD = 64;
constexpr int BT = 128;          // rows of an owned tile (queries in dQ, keys in dK/dV)
constexpr int BS = 64;           // rows of a streamed tile
constexpr int NT = 2;            // owned tiles per CTA
constexpr int STAGES = 4;
constexpr int OWN_BYTES = BT * HD * 2;   // 16 KB
constexpr int STR_BYTES = BS * HD * 2;   // 8 KB
constexpr int BWD_THREADS = 320;

// shared memory map (after 1024-byte alignment)
constexpr int SM_OWN_A = 0;                              // NT x 16 KB: Q (dQ pass) / K (dK/dV pass)
constexpr int SM_OWN_B = SM_OWN_A + NT * OWN_BYTES;      // NT x 16 KB: dO / V
constexpr int SM_STR_A = SM_OWN_B + NT * OWN_BYTES;      // STAGES x 8 KB: K / Q
constexpr int SM_STR_B = SM_STR_A + STAGES * STR_BYTES;  // STAGES x 8 KB: V / dO
constexpr int SM_LD = SM_STR_B + STAGES * STR_BYTES;     // STAGES x 2 x 64 floats: L, Delta (dK/dV)
constexpr int SM_BAR = SM_LD + STAGES * 2 * BS * 4;
constexpr int SM_TOTAL = SM_BAR + 256;
constexpr int SM_ALLOC = SM_TOTAL + 1024;

constexpr int BAR_OWN_FULL = 0;
constexpr int BAR_STR_FULL = 1;                          // [STAGES]
constexpr int BAR_STR_EMPTY = BAR_STR_FULL + STAGES;     // [STAGES]
constexpr int BAR_SDP_FULL = BAR_STR_EMPTY + STAGES;     // [NT]
constexpr int BAR_DS_READY = BAR_SDP_FULL + NT;          // [NT]
constexpr int BAR_ACC_DONE = BAR_DS_READY + NT;          // [NT]
constexpr int N_BARS = BAR_ACC_DONE + NT;

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

struct Ctx {
    uint32_t smem_base;
    unsigned char *smem;
    uint32_t bar0;
    volatile uint32_t *tmem_slot;
    volatile int *abort_flag;
    __device__ uint32_t bar(int i) const { return bar0 + 8u * (uint32_t)i; }
};

__device__ __forceinline__ Ctx make_ctx(unsigned char *smem_dyn) {
    Ctx c;
    c.smem_base = (mx::smem_u32(smem_dyn) + 1023u) & ~1023u;
    c.smem = smem_dyn + (c.smem_base - mx::smem_u32(smem_dyn));
    c.bar0 = c.smem_base + SM_BAR;
    c.tmem_slot = (volatile uint32_t *)(c.smem + SM_BAR + 8 * N_BARS);
    c.abort_flag = (volatile int *)(c.smem + SM_BAR + 8 * N_BARS + 8);
    return c;
}

__device__ __forceinline__ void init_barriers(const Ctx &c, int str_full_count) {
    mx::mbar_init(c.bar(BAR_OWN_FULL), 1);
    for (int s = 0; s < STAGES; ++s) {
        mx::mbar_init(c.bar(BAR_STR_FULL + s), str_full_count);
        mx::mbar_init(c.bar(BAR_STR_EMPTY + s), 1);
    }
    for (int t = 0; t < NT; ++t) {
        mx::mbar_init(c.bar(BAR_SDP_FULL + t), 1);
        mx::mbar_init(c.bar(BAR_DS_READY + t), BT);
        mx::mbar_init(c.bar(BAR_ACC_DONE + t), 1);
    }
    *c.abort_flag = 0;
    mx::mbar_fence_init();
}

// Stores one 64-column fp32 accumulator row from tensor memory to global memory.
__device__ __forceinline__ void store_acc_row(uint32_t taddr, float *dst, bool valid) {
#pragma unroll
    for (int cc = 0; cc < HD / 32; ++cc) {
        uint32_t v[32];
        mx::tmem_ld32(taddr + cc * 32, v);
        mx::tmem_wait_ld();
        if (valid) {
#pragma unroll
            for (int i = 0; i < 32; i += 4)
                *(float4 *)(dst + cc * 32 + i) =
                    make_float4(__uint_as_float(v[i]), __uint_as_float(v[i + 1]),
                                __uint_as_float(v[i + 2]), __uint_as_float(v[i + 3]));
        }
    }
}

// ===========================================================================
// dQ pass.  tensor memory per query tile t (192 columns): S [0,64), dP [64,128)
// (dS overlays the first 32 columns of dP as packed bf16), dQ [128,192).
// ===========================================================================
__global__ void __launch_bounds__(BWD_THREADS, 1)
bwd_dq_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmdO,
              const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
              const BwdParams P) {
    extern __shared__ unsigned char smem_dyn[];
    const Ctx cx = make_ctx(smem_dyn);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int N = P.n, bh = blockIdx.y;
    const int qb = P.causal ? (int)(gridDim.x - 1 - blockIdx.x) : (int)blockIdx.x;
    const int q0 = qb * (NT * BT);
    const int n_kv_total = (N + BS - 1) / BS;
    int n_it[NT];
#pragma unroll
    for (int t = 0; t < NT; ++t) {
        int r0 = q0 + t * BT;
        if (r0 >= N) n_it[t] = 0;
        else n_it[t] = P.causal ? min(n_kv_total, (r0 + BT - 1) / BS + 1) : n_kv_total;
    }
    const int n_max = max(n_it[0], n_it[1]);

    if (tid == 0) init_barriers(cx, 1);
    if (warp == 9) mx::tmem_alloc(mx::smem_u32((const void *)cx.tmem_slot), TM_COLS);
    mx::tc_fence_before();
    __syncthreads();
    mx::tc_fence_after();
    const uint32_t tmem = *cx.tmem_slot;

    if (warp == 8) {
        if (lane == 0) {
            mx::tma_prefetch_desc(&tmQ);
            mx::tma_prefetch_desc(&tmdO);
            mx::tma_prefetch_desc(&tmK);
            mx::tma_prefetch_desc(&tmV);
            int nq = (n_it[1] > 0) ? 2 : 1;
            mx::mbar_expect_tx(cx.bar(BAR_OWN_FULL), nq * 2 * OWN_BYTES);
            for (int t = 0; t < nq; ++t) {
                mx::tma_load_3d(cx.smem_base + SM_OWN_A + t * OWN_BYTES, &tmQ, cx.bar(BAR_OWN_FULL), 0,
                                q0 + t * BT, bh);
                mx::tma_load_3d(cx.smem_base + SM_OWN_B + t * OWN_BYTES, &tmdO, cx.bar(BAR_OWN_FULL), 0,
                                q0 + t * BT, bh);
            }
            for (int j = 0; j < n_max; ++j) {
                int s = j % STAGES, r = j / STAGES;
                if (r > 0 && !mx::mbar_wait(cx.bar(BAR_STR_EMPTY + s), (r - 1) & 1, cx.abort_flag, P.status))
                    break;
                mx::mbar_expect_tx(cx.bar(BAR_STR_FULL + s), 2 * STR_BYTES);
                mx::tma_load_3d(cx.smem_base + SM_STR_A + s * STR_BYTES, &tmK, cx.bar(BAR_STR_FULL + s), 0,
                                j * BS, bh);
                mx::tma_load_3d(cx.smem_base + SM_STR_B + s * STR_BYTES, &tmV, cx.bar(BAR_STR_FULL + s), 0,
                                j * BS, bh);
            }
        }
        __syncwarp();
    } else if (warp == 9) {
        if (lane == 0) {
            constexpr uint32_t IDESC_S = mx::mma_idesc_bf16(BT, BS, false, false);  // [128 x 64] += A B^T
            constexpr uint32_t IDESC_G = mx::mma_idesc_bf16(BT, HD, false, true);   // dQ += dS K
            auto issue_sdp = [&](int t, int stage) {
                uint64_t aq = mx::smem_desc_sw128(cx.smem_base + SM_OWN_A + t * OWN_BYTES);
                uint64_t ad = mx::smem_desc_sw128(cx.smem_base + SM_OWN_B + t * OWN_BYTES);
                uint64_t bk = mx::smem_desc_sw128(cx.smem_base + SM_STR_A + stage * STR_BYTES);
                uint64_t bv = mx::smem_desc_sw128(cx.smem_base + SM_STR_B + stage * STR_BYTES);
#pragma unroll
                for (int k = 0; k < HD / 16; ++k)
                    mx::mma_ss(tmem + t * 192, aq + 2 * k, bk + 2 * k, IDESC_S, k > 0);
#pragma unroll
                for (int k = 0; k < HD / 16; ++k)
                    mx::mma_ss(tmem + t * 192 + 64, ad + 2 * k, bv + 2 * k, IDESC_S, k > 0);
                mx::mma_commit(cx.bar(BAR_SDP_FULL + t));
            };
            bool ok = mx::mbar_wait(cx.bar(BAR_OWN_FULL), 0, cx.abort_flag, P.status);
            if (ok) ok = mx::mbar_wait(cx.bar(BAR_STR_FULL + 0), 0, cx.abort_flag, P.status);
            if (ok) {
                mx::tc_fence_after();
                for (int t = 0; t < NT; ++t)
                    if (n_it[t] > 0) issue_sdp(t, 0);
            }
            for (int j = 0; j < n_max && ok; ++j) {
                int s = j % STAGES;
                int s1 = (j + 1) % STAGES, r1 = (j + 1) / STAGES;
                if (j + 1 < n_max) ok = mx::mbar_wait(cx.bar(BAR_STR_FULL + s1), r1 & 1, cx.abort_flag, P.status);
                for (int t = 0; t < NT && ok; ++t) {
                    if (j >= n_it[t]) continue;
                    ok = mx::mbar_wait(cx.bar(BAR_DS_READY + t), j & 1, cx.abort_flag, P.status);
                    if (!ok) break;
                    mx::tc_fence_after();
                    uint64_t bk = mx::smem_desc_sw128(cx.smem_base + SM_STR_A + s * STR_BYTES);
#pragma unroll
                    for (int k = 0; k < BS / 16; ++k)
                        mx::mma_ts(tmem + t * 192 + 128, tmem + t * 192 + 64 + 8 * k, bk + 128 * k, IDESC_G,
                                   (j > 0 || k > 0));
                    if (j + 1 == n_it[t]) mx::mma_commit(cx.bar(BAR_ACC_DONE + t));
                    if (j + 1 < n_it[t]) issue_sdp(t, s1);
                }
                if (!ok) break;
                mx::mma_commit(cx.bar(BAR_STR_EMPTY + s));
            }
        }
        __syncwarp();
    } else {
        const int t = warp >> 2;
        const int row = q0 + t * BT + (tid & 127);
        const uint32_t lane_off = (uint32_t)((warp & 3) * 32) << 16;
        const uint32_t tm_s = tmem + lane_off + t * 192;
        const uint32_t tm_dp = tm_s + 64;
        const uint32_t tm_dq = tm_s + 128;
        const float c = 0.125f * LOG2E;
        const int n_t = n_it[t];
        const bool rv = row < N;
        const float Li = rv ? P.L[(size_t)bh * N + row] * LOG2E : 0.0f;
        const float Di = rv ? P.Delta[(size_t)bh * N + row] : 0.0f;
        bool ok = true;
        for (int j = 0; j < n_t; ++j) {
            ok = __all_sync(0xFFFFFFFFu, mx::mbar_wait(cx.bar(BAR_SDP_FULL + t), j & 1, cx.abort_flag, P.status));
            if (!ok) break;
            mx::tc_fence_after();
            const int key0 = j * BS;
            const bool need_mask = (key0 + BS > N) || (P.causal && key0 + BS - 1 > q0 + t * BT);
#pragma unroll
            for (int cc = 0; cc < BS / 32; ++cc) {
                uint32_t sv[32], dv[32];
                mx::tmem_ld32(tm_s + cc * 32, sv);
                mx::tmem_ld32(tm_dp + cc * 32, dv);
                mx::tmem_wait_ld();
                uint32_t pk[16];
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    float p0 = mx::ex2(fmaf(__uint_as_float(sv[i]), c, -Li));
                    float p1 = mx::ex2(fmaf(__uint_as_float(sv[i + 1]), c, -Li));
                    if (need_mask) {
                        int key = key0 + cc * 32 + i;
                        if (!(key < N && (!P.causal || key <= row))) p0 = 0.0f;
                        if (!(key + 1 < N && (!P.causal || key + 1 <= row))) p1 = 0.0f;
                    }
                    float d0 = p0 * (__uint_as_float(dv[i]) - Di) * 0.125f;
                    float d1 = p1 * (__uint_as_float(dv[i + 1]) - Di) * 0.125f;
                    pk[i >> 1] = mx::pack_bf16(d0, d1);
                }
                mx::tmem_st16(tm_dp + cc * 16, pk);
            }
            mx::tmem_wait_st();
            mx::tc_fence_before();
            mx::mbar_arrive(cx.bar(BAR_DS_READY + t));
        }
        if (ok && n_t > 0) {
            ok = __all_sync(0xFFFFFFFFu, mx::mbar_wait(cx.bar(BAR_ACC_DONE + t), 0, cx.abort_flag, P.status));
            if (ok) {
                mx::tc_fence_after();
                store_acc_row(tm_dq, P.out0 + ((size_t)bh * N + row) * HD, rv);
            }
        }
    }
    mx::tc_fence_before();
    __syncthreads();
    mx::tc_fence_after();
    if (warp == 9) mx::tmem_dealloc(tmem, TM_COLS);
}

// ===========================================================================
// dK/dV pass.  tensor memory per key tile t (256 columns): S^T [0,64) (P^T overlays
// its first 32 columns), dP^T [64,128) (dS^T overlays), dK [128,192), dV [192,256).
// ===========================================================================
__global__ void __launch_bounds__(BWD_THREADS, 1)
bwd_dkv_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
               const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmdO,
               const BwdParams P) {
    extern __shared__ unsigned char smem_dyn[];
    const Ctx cx = make_ctx(smem_dyn);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int N = P.n, bh = blockIdx.y;
    const int k0 = blockIdx.x * (NT * BT);  // causal: early key blocks see the most queries
    const int n_q_total = (N + BS - 1) / BS;
    int i_beg[NT];
    bool act[NT];
#pragma unroll
    for (int t = 0; t < NT; ++t) {
        int r0 = k0 + t * BT;
        act[t] = r0 < N;
        i_beg[t] = P.causal ? r0 / BS : 0;  // first query tile that can see this key tile
    }
    const int i0 = i_beg[0];
    const int n_iter = n_q_total - i0;  // query tiles i0 .. n_q_total-1 (tile 0 is always active)

    if (tid == 0) init_barriers(cx, 1 + 32);
    if (warp == 9) mx::tmem_alloc(mx::smem_u32((const void *)cx.tmem_slot), TM_COLS);
    mx::tc_fence_before();
    __syncthreads();
    mx::tc_fence_after();
    const uint32_t tmem = *cx.tmem_slot;

    if (warp == 8) {
        if (lane == 0) {
            mx::tma_prefetch_desc(&tmQ);
            mx::tma_prefetch_desc(&tmdO);
            mx::tma_prefetch_desc(&tmK);
            mx::tma_prefetch_desc(&tmV);
            int nk = act[1] ? 2 : 1;
            mx::mbar_expect_tx(cx.bar(BAR_OWN_FULL), nk * 2 * OWN_BYTES);
            for (int t = 0; t < nk; ++t) {
                mx::tma_load_3d(cx.smem_base + SM_OWN_A + t * OWN_BYTES, &tmK, cx.bar(BAR_OWN_FULL), 0,
                                k0 + t * BT, bh);
                mx::tma_load_3d(cx.smem_base + SM_OWN_B + t * OWN_BYTES, &tmV, cx.bar(BAR_OWN_FULL), 0,
                                k0 + t * BT, bh);
            }
        }
        bool ok = true;
        for (int it = 0; it < n_iter; ++it) {
            int s = it % STAGES, r = it / STAGES;
            int qrow0 = (i0 + it) * BS;
            if (r > 0)
                ok = __all_sync(0xFFFFFFFFu,
                                mx::mbar_wait(cx.bar(BAR_STR_EMPTY + s), (r - 1) & 1, cx.abort_flag, P.status));
            if (!ok) break;
            if (lane == 0) {
                mx::mbar_expect_tx(cx.bar(BAR_STR_FULL + s), 2 * STR_BYTES);
                mx::tma_load_3d(cx.smem_base + SM_STR_A + s * STR_BYTES, &tmQ, cx.bar(BAR_STR_FULL + s), 0,
                                qrow0, bh);
                mx::tma_load_3d(cx.smem_base + SM_STR_B + s * STR_BYTES, &tmdO, cx.bar(BAR_STR_FULL + s), 0,
                                qrow0, bh);
            }
            // L (pre-multiplied by log2 e) and Delta of the 64 streamed queries
            float *ld = (float *)(cx.smem + SM_LD + s * (2 * BS * 4));
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                int q = qrow0 + u * 32 + lane;
                bool v = q < N;
                ld[u * 32 + lane] = v ? P.L[(size_t)bh * N + q] * LOG2E : 0.0f;
                ld[BS + u * 32 + lane] = v ? P.Delta[(size_t)bh * N + q] : 0.0f;
            }
            mx::mbar_arrive(cx.bar(BAR_STR_FULL + s));
        }
        __syncwarp();
    } else if (warp == 9) {
        if (lane == 0) {
            constexpr uint32_t IDESC_S = mx::mma_idesc_bf16(BT, BS, false, false);
            constexpr uint32_t IDESC_G = mx::mma_idesc_bf16(BT, HD, false, true);
            auto issue_sdp = [&](int t, int stage) {
                uint64_t ak = mx::smem_desc_sw128(cx.smem_base + SM_OWN_A + t * OWN_BYTES);
                uint64_t av = mx::smem_desc_sw128(cx.smem_base + SM_OWN_B + t * OWN_BYTES);
                uint64_t bq = mx::smem_desc_sw128(cx.smem_base + SM_STR_A + stage * STR_BYTES);
                uint64_t bd = mx::smem_desc_sw128(cx.smem_base + SM_STR_B + stage * STR_BYTES);
#pragma unroll
                for (int k = 0; k < HD / 16; ++k)
                    mx::mma_ss(tmem + t * 256, ak + 2 * k, bq + 2 * k, IDESC_S, k > 0);
#pragma unroll
                for (int k = 0; k < HD / 16; ++k)
                    mx::mma_ss(tmem + t * 256 + 64, av + 2 * k, bd + 2 * k, IDESC_S, k > 0);
                mx::mma_commit(cx.bar(BAR_SDP_FULL + t));
            };
            // iteration `it` of tile t is active when the query tile can see the key tile
            auto active = [&](int t, int it) { return act[t] && (i0 + it) >= i_beg[t]; };
            int cnt[NT] = {0, 0};  // active iterations issued so far per tile (accumulate flag)
            bool ok = mx::mbar_wait(cx.bar(BAR_OWN_FULL), 0, cx.abort_flag, P.status);
            if (ok && n_iter > 0) ok = mx::mbar_wait(cx.bar(BAR_STR_FULL + 0), 0, cx.abort_flag, P.status);
            if (ok && n_iter > 0) {
                mx::tc_fence_after();
                for (int t = 0; t < NT; ++t)
                    if (active(t, 0)) issue_sdp(t, 0);
            }
            for (int it = 0; it < n_iter && ok; ++it) {
                int s = it % STAGES;
                int s1 = (it + 1) % STAGES, r1 = (it + 1) / STAGES;
                if (it + 1 < n_iter)
                    ok = mx::mbar_wait(cx.bar(BAR_STR_FULL + s1), r1 & 1, cx.abort_flag, P.status);
                for (int t = 0; t < NT && ok; ++t) {
                    if (!active(t, it)) {
                        // the tile joins at the next query tile: its first S^T/dP^T go out now
                        if (it + 1 < n_iter && active(t, it + 1)) {
                            mx::tc_fence_after();
                            issue_sdp(t, s1);
                        }
                        continue;
                    }
                    ok = mx::mbar_wait(cx.bar(BAR_DS_READY + t), cnt[t] & 1, cx.abort_flag, P.status);
                    if (!ok) break;
                    mx::tc_fence_after();
                    uint64_t bq = mx::smem_desc_sw128(cx.smem_base + SM_STR_A + s * STR_BYTES);
                    uint64_t bd = mx::smem_desc_sw128(cx.smem_base + SM_STR_B + s * STR_BYTES);
#pragma unroll
                    for (int k = 0; k < BS / 16; ++k)  // dV += P^T dO
                        mx::mma_ts(tmem + t * 256 + 192, tmem + t * 256 + 8 * k, bd + 128 * k, IDESC_G,
                                   (cnt[t] > 0 || k > 0));
#pragma unroll
                    for (int k = 0; k < BS / 16; ++k)  // dK += dS^T Q
                        mx::mma_ts(tmem + t * 256 + 128, tmem + t * 256 + 64 + 8 * k, bq + 128 * k, IDESC_G,
                                   (cnt[t] > 0 || k > 0));
                    ++cnt[t];
                    if (it + 1 == n_iter) mx::mma_commit(cx.bar(BAR_ACC_DONE + t));
                    else issue_sdp(t, s1);
                }
                if (!ok) break;
                mx::mma_commit(cx.bar(BAR_STR_EMPTY + s));
            }
        }
        __syncwarp();
    } else {
        const int t = warp >> 2;
        const int krow = k0 + t * BT + (tid & 127);  // this thread's key
        const uint32_t lane_off = (uint32_t)((warp & 3) * 32) << 16;
        const uint32_t tm_s = tmem + lane_off + t * 256;
        const uint32_t tm_dp = tm_s + 64;
        const float c = 0.125f * LOG2E;
        const bool kvalid = krow < N;
        bool ok = true;
        int cnt = 0;
        if (act[t]) {
            for (int it = 0; it < n_iter; ++it) {
                if (i0 + it < i_beg[t]) continue;
                ok = __all_sync(0xFFFFFFFFu,
                                mx::mbar_wait(cx.bar(BAR_SDP_FULL + t), cnt & 1, cx.abort_flag, P.status));
                if (!ok) break;
                // the streamed stage's L/Delta became visible with the same full barrier the
                // MMA warp waited on before issuing; wait on it here too for the plain loads
                int s = it % STAGES, r = it / STAGES;
                ok = __all_sync(0xFFFFFFFFu,
                                mx::mbar_wait(cx.bar(BAR_STR_FULL + s), r & 1, cx.abort_flag, P.status));
                if (!ok) break;
                mx::tc_fence_after();
                const float *ld = (const float *)(cx.smem + SM_LD + s * (2 * BS * 4));
                const int qrow0 = (i0 + it) * BS;
                const bool need_mask = (qrow0 + BS > N) || (P.causal && qrow0 < k0 + t * BT + BT - 1);
#pragma unroll
                for (int cc = 0; cc < BS / 32; ++cc) {
                    uint32_t sv[32], dv[32];
                    mx::tmem_ld32(tm_s + cc * 32, sv);
                    mx::tmem_ld32(tm_dp + cc * 32, dv);
                    mx::tmem_wait_ld();
                    uint32_t pp[16], pd[16];
#pragma unroll
                    for (int i = 0; i < 32; i += 2) {
                        float2 l2 = *(const float2 *)(ld + cc * 32 + i);
                        float2 d2 = *(const float2 *)(ld + BS + cc * 32 + i);
                        float p0 = mx::ex2(fmaf(__uint_as_float(sv[i]), c, -l2.x));
                        float p1 = mx::ex2(fmaf(__uint_as_float(sv[i + 1]), c, -l2.y));
                        if (need_mask) {
                            int q = qrow0 + cc * 32 + i;
                            if (!(q < N && (!P.causal || q >= krow))) p0 = 0.0f;
                            if (!(q + 1 < N && (!P.causal || q + 1 >= krow))) p1 = 0.0f;
                        }
                        float e0 = p0 * (__uint_as_float(dv[i]) - d2.x) * 0.125f;
                        float e1 = p1 * (__uint_as_float(dv[i + 1]) - d2.y) * 0.125f;
                        pp[i >> 1] = mx::pack_bf16(p0, p1);
                        pd[i >> 1] = mx::pack_bf16(e0, e1);
                    }
                    mx::tmem_st16(tm_s + cc * 16, pp);
                    mx::tmem_st16(tm_dp + cc * 16, pd);
                }
                mx::tmem_wait_st();
                mx::tc_fence_before();
                mx::mbar_arrive(cx.bar(BAR_DS_READY + t));
                ++cnt;
            }
            if (ok && cnt > 0) {
                ok = __all_sync(0xFFFFFFFFu, mx::mbar_wait(cx.bar(BAR_ACC_DONE + t), 0, cx.abort_flag, P.status));
                if (ok) {
                    mx::tc_fence_after();
                    store_acc_row(tm_s + 128, P.out0 + ((size_t)bh * N + krow) * HD, kvalid);
                    store_acc_row(tm_s + 192, P.out1 + ((size_t)bh * N + krow) * HD, kvalid);
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
        MX_CHECK_CUDA(cudaFuncSetAttribute(bwd_dq_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SM_ALLOC));
        MX_CHECK_CUDA(cudaFuncSetAttribute(bwd_dkv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SM_ALLOC));
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
    dim3 grid((n + NT * BT - 1) / (NT * BT), batch_heads);
    MX_LAUNCH(h, st, MX230_K_BWD_DQ,
              (bwd_dq_kernel<<<grid, BWD_THREADS, SM_ALLOC, st>>>(m.own128[0], m.own128[3], m.str64[1],
                                                                  m.str64[2], P)));
    return MX230_OK;
}

int launch_dkv(mx230_handle *h, cudaStream_t st, const Maps &m, const float *L, const float *Delta, float *dK,
               float *dV, int batch_heads, int n, int causal) {
    BwdParams P{L, Delta, dK, dV, n, causal ? 1 : 0, h->status_dev};
    dim3 grid((n + NT * BT - 1) / (NT * BT), batch_heads);
    MX_LAUNCH(h, st, MX230_K_BWD_DKV,
              (bwd_dkv_kernel<<<grid, BWD_THREADS, SM_ALLOC, st>>>(m.own128[1], m.own128[2], m.str64[0],
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
