// Batched projections either side of prefill attention: C[m][n] = A[m][k] . W[k][n] + bias[n]
// (the reference's `gemm`, 03-llm-engine/src/gpu.rs:1291-1420, called at gpu.rs:3187-3198 for qkv and
// gpu.rs:3354-3365 for the output projection; kernels gemm_f32* / gemm_half*, llm.cu).  fp32 activations in and
// out, weights fp32 or fp16 in the reference's [k][n] layout.
//
// tcgen05 with 16-bit operands and fp32 accumulation in tensor memory:
//   * fp16 weights are the B operand as they lie in memory (rows = contraction index: an MN-major operand, the
//     same descriptor form as V in the attention kernels); A is staged to fp16 once per call;
//   * fp32 weights would lose their low mantissa bits in one 16-bit operand, so both sides are staged as a
//     (high, low) pair of bf16 values, x = hi + lo to 16 bits of mantissa, and three products are accumulated:
//     A_hi W_hi + A_hi W_lo + A_lo W_hi.  The tensor cores have the time: these GEMMs are launch-bound.
// CTA = one 128 x 64 tile of C; k in steps of 64 through a 4-stage TMA ring (out-of-range rows and columns are
// zero-filled by the TMA unit, so m, n, k need no padding); one TMA warp, one MMA-issuing warp, four epilogue
// warps that add the bias and store fp32 rows.
#include "common.cuh"

namespace {

constexpr int GM = 128, GN = 64, GK = 64;
constexpr int STAGES = 4;
constexpr int A_TILE = GM * GK * 2;   // 16 KB
constexpr int W_TILE = GK * GN * 2;   // 8 KB
constexpr int THREADS = 256;

template <bool SPLIT>
struct Smem {
    static constexpr int PARTS = SPLIT ? 2 : 1;
    static constexpr int STAGE = PARTS * (A_TILE + W_TILE);
    static constexpr int BAR = STAGES * STAGE;
    static constexpr int TOTAL = BAR + 128;
    static constexpr int ALLOC = TOTAL + 1024;
};

struct GemmParams {
    float *C;
    const float *bias;
    int m, n, k;
    int *status;
};

// kind::f16 instruction descriptor: fp32 accumulate, A K-major, B MN-major, both operands fp16 or both bf16
__host__ __device__ constexpr uint32_t idesc(bool bf16) {
    return (1u << 4) | ((bf16 ? 1u : 0u) << 7) | ((bf16 ? 1u : 0u) << 10) | (0u << 15) | (1u << 16) |
           ((uint32_t)(GN >> 3) << 17) | ((uint32_t)(GM >> 4) << 24);
}

template <bool SPLIT>
__global__ void __launch_bounds__(THREADS, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmA0, const __grid_constant__ CUtensorMap tmA1,
            const __grid_constant__ CUtensorMap tmW0, const __grid_constant__ CUtensorMap tmW1, const GemmParams P) {
    using S = Smem<SPLIT>;
    extern __shared__ unsigned char smem_dyn[];
    const uint32_t smem_base = (mx::smem_u32(smem_dyn) + 1023u) & ~1023u;
    unsigned char *smem = smem_dyn + (smem_base - mx::smem_u32(smem_dyn));
    const uint32_t bar0 = smem_base + S::BAR;
    auto bar = [&](int i) { return bar0 + 8u * (uint32_t)i; };   // FULL[s] = s, EMPTY[s] = STAGES + s, ACC = 2 * STAGES
    volatile uint32_t *tmem_slot = (volatile uint32_t *)(smem + S::BAR + 8 * (2 * STAGES + 1));
    volatile int *abort_flag = (volatile int *)(smem + S::BAR + 8 * (2 * STAGES + 1) + 8);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int m0 = blockIdx.y * GM, n0 = blockIdx.x * GN;
    const int n_steps = (P.k + GK - 1) / GK;

    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mx::mbar_init(bar(s), 1);
            mx::mbar_init(bar(STAGES + s), 1);
        }
        mx::mbar_init(bar(2 * STAGES), 1);
        *abort_flag = 0;
        mx::mbar_fence_init();
    }
    if (warp == 1) mx::tmem_alloc(mx::smem_u32((const void *)tmem_slot), GN);
    mx::tc_fence_before();
    __syncthreads();
    mx::tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    if (warp == 0) {
        // ------------------------- TMA producer -------------------------
        if (lane == 0) {
            mx::tma_prefetch_desc(&tmA0);
            mx::tma_prefetch_desc(&tmW0);
            bool ok = true;
            for (int i = 0; i < n_steps && ok; ++i) {
                const int s = i % STAGES;
                if (i >= STAGES) ok = mx::mbar_wait(bar(STAGES + s), (i / STAGES - 1) & 1, abort_flag, P.status);
                if (!ok) break;
                const uint32_t base = smem_base + s * S::STAGE;
                mx::mbar_expect_tx(bar(s), S::STAGE);
                mx::tma_load_3d(base, &tmA0, bar(s), i * GK, m0, 0);
                mx::tma_load_3d(base + S::PARTS * A_TILE, &tmW0, bar(s), n0, i * GK, 0);
                if (SPLIT) {
                    mx::tma_load_3d(base + A_TILE, &tmA1, bar(s), i * GK, m0, 0);
                    mx::tma_load_3d(base + 2 * A_TILE + W_TILE, &tmW1, bar(s), n0, i * GK, 0);
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------- MMA issuer (warp-uniform, one elected lane issues) --------------------
        constexpr uint32_t IDESC = idesc(SPLIT);
        bool ok = true;
        for (int i = 0; i < n_steps && ok; ++i) {
            const int s = i % STAGES;
            ok = __all_sync(0xFFFFFFFFu, mx::mbar_wait(bar(s), (i / STAGES) & 1, abort_flag, P.status));
            if (!ok) break;
            mx::tc_fence_after();
            const uint32_t base = smem_base + s * S::STAGE;
            const uint64_t a0 = mx::smem_desc_sw128(base), w0 = mx::smem_desc_sw128(base + S::PARTS * A_TILE);
            const uint64_t a1 = mx::smem_desc_sw128(base + A_TILE), w1 = mx::smem_desc_sw128(base + 2 * A_TILE + W_TILE);
            if (mx::elect_one()) {
#pragma unroll
                for (int kk = 0; kk < GK / 16; ++kk) {   // A: 32 bytes per 16-element step inside the swizzle span; W: 16 rows of 128 bytes
                    mx::mma_ss(tmem, a0 + 2 * kk, w0 + 128 * kk, IDESC, (i > 0 || kk > 0));
                    if (SPLIT) {
                        mx::mma_ss(tmem, a0 + 2 * kk, w1 + 128 * kk, IDESC, 1);
                        mx::mma_ss(tmem, a1 + 2 * kk, w0 + 128 * kk, IDESC, 1);
                    }
                }
                mx::mma_commit(bar(STAGES + s));
                if (i == n_steps - 1) mx::mma_commit(bar(2 * STAGES));
            }
            __syncwarp();
        }
    } else if (warp >= 4) {
        // ------------------------- epilogue: bias, fp32 rows out -------------------------
        const int q = warp & 3;
        bool ok = __all_sync(0xFFFFFFFFu, mx::mbar_wait(bar(2 * STAGES), 0, abort_flag, P.status));
        if (ok) {
            mx::tc_fence_after();
            const int row = m0 + q * 32 + lane;
            const uint32_t ta = tmem + ((uint32_t)(q * 32) << 16);
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                uint32_t v[32];
                mx::tmem_ld32(ta + half * 32, v);
                mx::tmem_wait_ld();
                if (row < P.m) {
                    float *crow = P.C + (size_t)row * P.n + n0 + half * 32;
#pragma unroll
                    for (int c = 0; c < 32; c += 4) {
                        const int col = n0 + half * 32 + c;
                        if (col < P.n) {   // n is a multiple of 4: a float4 is inside or outside as a whole
                            float4 b4 = P.bias ? *(const float4 *)(P.bias + col) : make_float4(0.f, 0.f, 0.f, 0.f);
                            *(float4 *)(crow + c) = make_float4(__uint_as_float(v[c]) + b4.x, __uint_as_float(v[c + 1]) + b4.y,
                                                                __uint_as_float(v[c + 2]) + b4.z, __uint_as_float(v[c + 3]) + b4.w);
                        }
                    }
                }
            }
        }
    }
    mx::tc_fence_before();
    __syncthreads();
    mx::tc_fence_after();
    if (warp == 1) mx::tmem_dealloc(tmem, GN);
}

// Staging.  SPLIT: x -> (hi, lo) bf16 with hi = bf16(x), lo = bf16(x - hi); else x -> fp16.  Two tensors per launch
// (blockIdx.y selects): the activations, and with fp32 weights the weight matrix.
struct StageParams {
    const float *src[2];
    void *hi[2];
    void *lo[2];
    size_t n4[2];   // float4s per tensor
};

template <bool SPLIT>
__global__ void gemm_stage_kernel(StageParams P) {
    const int t = blockIdx.y;
    const float4 *src = (const float4 *)P.src[t];
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < P.n4[t]; i += (size_t)gridDim.x * blockDim.x) {
        const float4 x = src[i];
        if (SPLIT) {
            const __nv_bfloat16 h0 = __float2bfloat16_rn(x.x), h1 = __float2bfloat16_rn(x.y), h2 = __float2bfloat16_rn(x.z),
                                h3 = __float2bfloat16_rn(x.w);
            const __nv_bfloat16 l0 = __float2bfloat16_rn(x.x - __bfloat162float(h0)),
                                l1 = __float2bfloat16_rn(x.y - __bfloat162float(h1)),
                                l2 = __float2bfloat16_rn(x.z - __bfloat162float(h2)),
                                l3 = __float2bfloat16_rn(x.w - __bfloat162float(h3));
            __nv_bfloat162 hv[2] = {__halves2bfloat162(h0, h1), __halves2bfloat162(h2, h3)};
            __nv_bfloat162 lv[2] = {__halves2bfloat162(l0, l1), __halves2bfloat162(l2, l3)};
            ((uint2 *)P.hi[t])[i] = *(const uint2 *)hv;
            ((uint2 *)P.lo[t])[i] = *(const uint2 *)lv;
        } else {
            __half2 hv[2] = {__floats2half2_rn(x.x, x.y), __floats2half2_rn(x.z, x.w)};
            ((uint2 *)P.hi[t])[i] = *(const uint2 *)hv;
        }
    }
}

size_t align256(size_t x) { return (x + 255) & ~(size_t)255; }

}  // namespace

extern "C" size_t mx230_gemm_workspace_bytes(int m, int n, int k, int weights_fp16) {
    if (m <= 0 || n <= 0 || k <= 0) return 0;
    const size_t a = align256((size_t)m * k * 2), w = align256((size_t)k * n * 2);
    return weights_fp16 ? a : 2 * a + 2 * w;
}

extern "C" int mx230_gemm(mx230_handle *h, void *stream, float *C, const float *A, const void *w, int w_fp16,
                          const float *bias, int m, int n, int k) {
    MX_REQUIRE(h && C && A && w, MX230_ERR_INVALID_ARG, "gemm: null argument");
    const float *W = w_fp16 ? nullptr : (const float *)w;
    const void *W_fp16 = w_fp16 ? w : nullptr;
    MX_REQUIRE(m >= 0 && n > 0 && k > 0, MX230_ERR_INVALID_ARG, "gemm: bad sizes %d x %d x %d", m, n, k);
    MX_REQUIRE(k % 16 == 0 && n % 8 == 0, MX230_ERR_UNSUPPORTED, "gemm: k must be a multiple of 16 and n of 8 (got k %d, n %d)", k, n);
    MX_REQUIRE((((uintptr_t)C | (uintptr_t)A | (uintptr_t)W | (uintptr_t)W_fp16 | (uintptr_t)bias) & 15) == 0,
               MX230_ERR_INVALID_ARG, "gemm: buffers must be 16-byte aligned");
    if (m == 0) return MX230_OK;
    const bool split = W != nullptr;
    const size_t need = mx230_gemm_workspace_bytes(m, n, k, split ? 0 : 1);
    MX_REQUIRE(h->ws && need <= h->ws_bytes, MX230_ERR_WORKSPACE, "gemm: workspace %zu B < %zu B needed", h->ws_bytes, need);
    h->staged.valid = 0;   // the workspace is about to hold something else
    mx230_device_guard guard(h->device);
    cudaStream_t st = (cudaStream_t)stream;
    const size_t a_bytes = align256((size_t)m * k * 2), w_bytes = align256((size_t)k * n * 2);
    unsigned char *ws = (unsigned char *)h->ws;
    void *a_hi = ws, *a_lo = ws + a_bytes, *w_hi = ws + 2 * a_bytes, *w_lo = ws + 2 * a_bytes + w_bytes;

    StageParams SP;
    SP.src[0] = A, SP.hi[0] = a_hi, SP.lo[0] = a_lo, SP.n4[0] = (size_t)m * k / 4;
    SP.src[1] = W, SP.hi[1] = w_hi, SP.lo[1] = w_lo, SP.n4[1] = split ? (size_t)k * n / 4 : 0;
    const size_t big = SP.n4[0] > SP.n4[1] ? SP.n4[0] : SP.n4[1];
    unsigned blocks = (unsigned)((big + 255) / 256);
    if (blocks > (unsigned)h->sm_count * 8) blocks = (unsigned)h->sm_count * 8;
    if (split) {
        MX_LAUNCH(h, st, MX230_K_CAST, (gemm_stage_kernel<true><<<dim3(blocks, 2), 256, 0, st>>>(SP)));
    } else {
        MX_LAUNCH(h, st, MX230_K_CAST, (gemm_stage_kernel<false><<<dim3(blocks, 1), 256, 0, st>>>(SP)));
    }

    CUtensorMap tA0, tA1, tW0, tW1;
    const int f16 = split ? 0 : 1;
    int rc = mx230_make_tmap_2d_16bit(h, &tA0, a_hi, f16, (uint64_t)k, (uint64_t)m, (uint64_t)k * 2, GK, GM);
    if (rc) return rc;
    rc = mx230_make_tmap_2d_16bit(h, &tA1, split ? a_lo : a_hi, f16, (uint64_t)k, (uint64_t)m, (uint64_t)k * 2, GK, GM);
    if (rc) return rc;
    rc = mx230_make_tmap_2d_16bit(h, &tW0, split ? w_hi : W_fp16, f16, (uint64_t)n, (uint64_t)k, (uint64_t)n * 2, GN, GK);
    if (rc) return rc;
    rc = mx230_make_tmap_2d_16bit(h, &tW1, split ? w_lo : W_fp16, f16, (uint64_t)n, (uint64_t)k, (uint64_t)n * 2, GN, GK);
    if (rc) return rc;

    GemmParams P;
    P.C = C, P.bias = bias, P.m = m, P.n = n, P.k = k, P.status = h->status_dev;
    dim3 grid((unsigned)((n + GN - 1) / GN), (unsigned)((m + GM - 1) / GM));
    if (split) {
        MX_SMEM_ATTR_ONCE(h->device, (gemm_kernel<true>), Smem<true>::ALLOC);
        MX_LAUNCH(h, st, MX230_K_GEMV, (gemm_kernel<true><<<grid, THREADS, Smem<true>::ALLOC, st>>>(tA0, tA1, tW0, tW1, P)));
    } else {
        MX_SMEM_ATTR_ONCE(h->device, (gemm_kernel<false>), Smem<false>::ALLOC);
        MX_LAUNCH(h, st, MX230_K_GEMV, (gemm_kernel<false><<<grid, THREADS, Smem<false>::ALLOC, st>>>(tA0, tA1, tW0, tW1, P)));
    }
    MX_CHECK_CUDA(cudaGetLastError());
    return MX230_OK;
}
