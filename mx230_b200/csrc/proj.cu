// The projections either side of the attention step, for one decode token:
//   gemv:            y[o] (+)= sum_i x[i] w[i*n_out + o] + b[o]     (gemv / gemv_half, the output
//                    projection with its fused residual add, 03-llm-engine/kernels/llm.cu:144-177,
//                    host gemv() src/gpu.rs:1158-1198, call site :2676-2686)
//   qkv step, fused: qkv = x W + b, RoPE on the Q and K heads, K and V rows written to the cache
//                    (fp32 copy or int8 quantize-on-write), the rotated q left in qkv for the decode
//                    attention -- one launch for the reference's gemv + rope + KV write
//                    (gpu.rs:2558-2646; rope llm.cu:1072-1100, quant_affine :1137-1149).
//
//   gemv_int8:       the same with int8 weights and on-the-fly int8 activations (llm.cu:226-316): the
//                    activation row is quantised per group of AG values (absmax / 127, round to nearest
//                    even), weights are int32 words of four consecutive input rows, w32[(i/4)*n_out + o],
//                    integer dots by dp4a, one float multiply-add per group, one scale per output column.
//
// HBM-bound on the weight matrix (n_in x n_out fp32, fp16 or int8, each byte read once).  The reference
// gives one thread a whole output column, which leaves most of a B200 idle for a 1152-column
// matrix; here a CTA owns a 64-column block (one attention head) and a slice of the input rows, so
// that the grid covers the machine: 16 lanes x 128-bit loads across the columns, 8 row lanes down
// the slice.  Slices leave partial sums in the workspace; the last CTA to arrive for a column block
// adds them in slice order (deterministic), adds the bias and runs the epilogue on its 64 values.
#include <cuda_fp16.h>

#include "common.cuh"

namespace {

constexpr int PJ_THREADS = 128;
constexpr int PJ_COLS = 64;     // columns per CTA = one head
constexpr int PJ_ROWLANES = 8;
#ifndef PJ_CTAS_PER_SM
#define PJ_CTAS_PER_SM 6
#endif

struct QkvEpilogue {
    int enabled;
    int pos;                 // host position, unless pos_dev
    const int *pos_dev;
    int n_head, n_kv_head;
    float theta;
    float *kcache, *vcache;  // fp32 cache, or null
    int8_t *kq, *vq;         // int8 cache, or null
    float *ks, *vs, *kb, *vb;
    const int *bt;           // block table or null
    int bs;
};

struct GemvParams {
    float *y;
    const float *x;
    const void *w;
    const float *b;
    int n_in, n_out, accum;
    const float *scales;     // int8 weights: one scale per output column
    int ag;                  // int8 weights: activations are quantised in groups of `ag` values (4 or 8)
    int rows_per_slice;
    float *partials;         // [n_slices][n_out]
    unsigned *counters;      // one per column block, self-resetting
    QkvEpilogue e;
};

__device__ __forceinline__ float4 load_w4(const float *w, size_t idx) { return *(const float4 *)(w + idx); }
__device__ __forceinline__ float4 load_w4(const __half *w, size_t idx) {
    const uint2 raw = *(const uint2 *)(w + idx);
    const float2 a = __half22float2(*(const __half2 *)&raw.x), c = __half22float2(*(const __half2 *)&raw.y);
    return make_float4(a.x, a.y, c.x, c.y);
}

__device__ __forceinline__ float wmax(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
    return v;
}

template <typename WT>
__global__ void __launch_bounds__(PJ_THREADS)
gemv_heads_kernel(const GemvParams P) {
    __shared__ float red[PJ_ROWLANES][PJ_COLS];
    __shared__ float val[PJ_COLS];
    __shared__ int is_last;
    extern __shared__ float xs[];                      // this slice of x (int8: packed codes, then group scales)
    constexpr bool I8 = sizeof(WT) == 1;
    const int tid = threadIdx.x;
    const int col0 = blockIdx.x * PJ_COLS;
    const int k0 = blockIdx.y * P.rows_per_slice;
    const int k1 = min(P.n_in, k0 + P.rows_per_slice);
    int *xq = (int *)xs;                               // int8: (k1 - k0) / 4 words
    float *xsc = xs + P.rows_per_slice / 4;            // int8: (k1 - k0) / ag scales
    if (!I8) {
        for (int i = tid; i < k1 - k0; i += PJ_THREADS) xs[i] = P.x[k0 + i];
    } else {
        // quantise this slice of the activations exactly as the reference kernel does
        const int ag = P.ag;
        for (int g = tid; g < (k1 - k0) / ag; g += PJ_THREADS) {
            const float *xg = P.x + k0 + g * ag;
            float amax = 0.0f;
            for (int j = 0; j < ag; ++j) amax = fmaxf(amax, fabsf(xg[j]));
            const float id = amax > 0.0f ? __fdiv_rn(127.0f, amax) : 0.0f;
            for (int q = 0; q < ag / 4; ++q) {
                int packed = 0;
                for (int j = 0; j < 4; ++j) {
                    const int v = max(-127, min(127, __float2int_rn(xg[4 * q + j] * id)));
                    packed |= (v & 0xFF) << (8 * j);
                }
                xq[g * (ag / 4) + q] = packed;
            }
            xsc[g] = amax > 0.0f ? __fdiv_rn(amax, 127.0f) : 1.0f;
        }
    }
    __syncthreads();

    const int cq = tid & 15, rl = tid >> 4;
    const int col = col0 + 4 * cq;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    if (col + 3 < P.n_out) {
        if constexpr (!I8) {
            const WT *w = (const WT *)P.w;
#pragma unroll 8
            for (int i = k0 + rl; i < k1; i += PJ_ROWLANES) {
                const float4 w4 = load_w4(w, (size_t)i * P.n_out + col);
                const float xv = xs[i - k0];
                acc.x = fmaf(xv, w4.x, acc.x);
                acc.y = fmaf(xv, w4.y, acc.y);
                acc.z = fmaf(xv, w4.z, acc.z);
                acc.w = fmaf(xv, w4.w, acc.w);
            }
        } else {
            // word q holds input rows 4q .. 4q+3 of a column; its group scale is xsc[q / (ag / 4)]
            const int *w32 = (const int *)P.w;
            const int wpg = P.ag / 4;
#pragma unroll 8
            for (int q = k0 / 4 + rl; q < k1 / 4; q += PJ_ROWLANES) {
                const int4 wv = *(const int4 *)(w32 + (size_t)q * P.n_out + col);
                const int xv = xq[q - k0 / 4];
                const float sx = xsc[(q - k0 / 4) / wpg];
                acc.x = fmaf((float)__dp4a(wv.x, xv, 0), sx, acc.x);
                acc.y = fmaf((float)__dp4a(wv.y, xv, 0), sx, acc.y);
                acc.z = fmaf((float)__dp4a(wv.z, xv, 0), sx, acc.z);
                acc.w = fmaf((float)__dp4a(wv.w, xv, 0), sx, acc.w);
            }
        }
    }
    *(float4 *)&red[rl][4 * cq] = acc;
    __syncthreads();
    const int n_slices = gridDim.y;
    if (tid < PJ_COLS) {
        float s = 0.0f;
#pragma unroll
        for (int r = 0; r < PJ_ROWLANES; ++r) s += red[r][tid];
        if (n_slices == 1) val[tid] = s;
        else if (col0 + tid < P.n_out) P.partials[(size_t)blockIdx.y * P.n_out + col0 + tid] = s;
    }
    if (n_slices > 1) {
        __threadfence();
        __syncthreads();
        if (tid == 0) is_last = atomicInc(&P.counters[blockIdx.x], n_slices - 1) == (unsigned)(n_slices - 1);
        __syncthreads();
        if (!is_last) return;
        __threadfence();
        if (tid < PJ_COLS && col0 + tid < P.n_out) {
            float s = 0.0f;
            for (int sl = 0; sl < n_slices; ++sl) s += P.partials[(size_t)sl * P.n_out + col0 + tid];
            val[tid] = s;
        }
    }
    __syncthreads();
    // ---- epilogue on the 64 finished sums of this column block ----
    if (tid < PJ_COLS) {
        const int o = col0 + tid;
        if (o < P.n_out) val[tid] = (I8 ? val[tid] * P.scales[o] : val[tid]) + (P.b ? P.b[o] : 0.0f);
    }
    __syncthreads();
    if (!P.e.enabled) {
        if (tid < PJ_COLS && col0 + tid < P.n_out) {
            const int o = col0 + tid;
            P.y[o] = P.accum ? P.y[o] + val[tid] : val[tid];
        }
        return;
    }
    // qkv step: this block is head `hb` of the row [Q heads | K heads | V heads]
    const QkvEpilogue &E = P.e;
    const int hb = blockIdx.x;
    const int pos = E.pos_dev ? *E.pos_dev : E.pos;
    const bool is_v = hb >= E.n_head + E.n_kv_head;
    if (tid < 32) {   // one warp: lane l owns the rotation pair (l, l + 32), then elements 2l, 2l+1
        if (!is_v) {
            // HF rotate_half RoPE with precise powf / sincosf (the reference's CPU semantics, cpu.rs:25-37)
            const float freq = powf(E.theta, -2.0f * (float)tid / 64.0f);
            float sn, cs;
            sincosf((float)pos * freq, &sn, &cs);
            const float x1 = val[tid], x2 = val[tid + 32];
            val[tid] = x1 * cs - x2 * sn;
            val[tid + 32] = x1 * sn + x2 * cs;
        }
        __syncwarp();
        const float2 xv = make_float2(val[2 * tid], val[2 * tid + 1]);
        *(float2 *)(P.y + (size_t)hb * 64 + 2 * tid) = xv;
        if (hb >= E.n_head) {   // K or V head: the cache row of this position
            const int kvh = is_v ? hb - E.n_head - E.n_kv_head : hb - E.n_head;
            const size_t row = E.bt ? (size_t)(E.bt[pos / E.bs] * E.bs + pos % E.bs) : (size_t)pos;
            const int kvd = E.n_kv_head * 64;
            if (E.kq == nullptr) {
                float *dst = (is_v ? E.vcache : E.kcache) + row * kvd + kvh * 64;
                *(float2 *)(dst + 2 * tid) = xv;
            } else {
                int8_t *dst = (is_v ? E.vq : E.kq) + row * kvd + kvh * 64;
                float *sc = is_v ? E.vs : E.ks, *be = is_v ? E.vb : E.kb;
                const size_t sd = row * E.n_kv_head + kvh;
                int c0, c1;
                if (be != nullptr) {   // affine, IEEE division and round-to-nearest-even as quant_affine
                    const float hi = wmax(fmaxf(xv.x, xv.y));
                    const float lo = -wmax(fmaxf(-xv.x, -xv.y));
                    const float scale = (hi > lo) ? __fdiv_rn(hi - lo, 255.0f) : 1.0f;
                    const float beta = __fmaf_rn(128.0f, scale, lo);
                    c0 = max(-128, min(127, __float2int_rn(__fdiv_rn(xv.x - beta, scale))));
                    c1 = max(-128, min(127, __float2int_rn(__fdiv_rn(xv.y - beta, scale))));
                    if (tid == 0) sc[sd] = scale, be[sd] = beta;
                } else {               // symmetric absmax
                    const float amax = wmax(fmaxf(fabsf(xv.x), fabsf(xv.y)));
                    const float id = amax > 0.0f ? __fdiv_rn(127.0f, amax) : 0.0f;
                    c0 = max(-127, min(127, __float2int_rn(xv.x * id)));
                    c1 = max(-127, min(127, __float2int_rn(xv.y * id)));
                    if (tid == 0) sc[sd] = amax > 0.0f ? __fdiv_rn(amax, 127.0f) : 0.0f;
                }
                *(unsigned short *)(dst + 2 * tid) = (unsigned short)((c0 & 0xFF) | ((c1 & 0xFF) << 8));
            }
        }
    }
}

// w_kind: 0 fp32, 1 fp16, 2 int8 (packed words, P.scales and P.ag set)
int launch_gemv(mx230_handle *h, void *stream, GemvParams P, int w_kind, const char *who) {
    MX_REQUIRE(h && P.y && P.x && P.w, MX230_ERR_INVALID_ARG, "%s: null argument", who);
    MX_REQUIRE(P.n_in > 0 && P.n_out > 0 && P.n_out % 4 == 0, MX230_ERR_INVALID_ARG,
               "%s: n_in %d, n_out %d (n_out must be a positive multiple of 4)", who, P.n_in, P.n_out);
    MX_REQUIRE((((uintptr_t)P.w | (uintptr_t)P.y) & 15) == 0, MX230_ERR_INVALID_ARG, "%s: y and w must be 16-byte aligned", who);
    const int n_blocks = (P.n_out + PJ_COLS - 1) / PJ_COLS;
    // enough input slices for PJ_CTAS_PER_SM CTAs on every SM (bytes in flight, not arithmetic, set the
    // pace), at least 16 rows each
    int n_slices = (PJ_CTAS_PER_SM * h->sm_count + n_blocks - 1) / n_blocks;
    const int max_slices = (P.n_in + 15) / 16;
    if (n_slices > max_slices) n_slices = max_slices;
    if (n_slices < 1) n_slices = 1;
    // int8: a slice holds whole activation groups and whole passes of the eight row lanes over 4-row words
    const int gran = w_kind == 2 ? 4 * PJ_ROWLANES : PJ_ROWLANES;
    if (w_kind == 2) {
        MX_REQUIRE(P.scales && (P.ag == 4 || P.ag == 8) && P.n_in % 8 == 0, MX230_ERR_INVALID_ARG,
                   "%s: int8 weights need scales, an activation group of 4 or 8 and n_in %% 8 == 0 (n_in %d)", who, P.n_in);
    }
    P.rows_per_slice = ((P.n_in + n_slices - 1) / n_slices + gran - 1) / gran * gran;
    n_slices = (P.n_in + P.rows_per_slice - 1) / P.rows_per_slice;
    if (n_slices > 1) {
        const size_t need = (size_t)n_slices * P.n_out * sizeof(float);
        MX_REQUIRE(h->ws && need <= h->ws_bytes, MX230_ERR_WORKSPACE, "%s: workspace %zu B < %zu B needed", who,
                   h->ws_bytes, need);
        MX_REQUIRE((size_t)n_blocks <= h->n_counters, MX230_ERR_UNSUPPORTED, "%s: %d column blocks exceed %zu counters",
                   who, n_blocks, h->n_counters);
        h->staged.valid = 0;   // the workspace is about to hold something else
        P.partials = (float *)h->ws;
        P.counters = h->counters;
    }
    mx230_device_guard guard(h->device);
    cudaStream_t st = (cudaStream_t)stream;
    dim3 grid(n_blocks, n_slices);
    const size_t sm = (size_t)P.rows_per_slice * sizeof(float);   // int8: n/4 words + n/ag scales <= n floats
    if (w_kind == 2) MX_LAUNCH(h, st, MX230_K_GEMV, (gemv_heads_kernel<int8_t><<<grid, PJ_THREADS, sm, st>>>(P)));
    else if (w_kind == 1) MX_LAUNCH(h, st, MX230_K_GEMV, (gemv_heads_kernel<__half><<<grid, PJ_THREADS, sm, st>>>(P)));
    else MX_LAUNCH(h, st, MX230_K_GEMV, (gemv_heads_kernel<float><<<grid, PJ_THREADS, sm, st>>>(P)));
    return MX230_OK;
}

}  // namespace

extern "C" int mx230_gemv(mx230_handle *h, void *stream, float *y, const float *x, const void *w, int w_fp16,
                          const float *b, int n_in, int n_out, int accum) {
    GemvParams P{};
    P.y = y, P.x = x, P.w = w, P.b = b, P.n_in = n_in, P.n_out = n_out, P.accum = accum ? 1 : 0;
    return launch_gemv(h, stream, P, w_fp16 ? 1 : 0, "gemv");
}

extern "C" int mx230_gemv_int8(mx230_handle *h, void *stream, float *y, const float *x, const void *w_packed,
                               const float *scales, const float *b, int n_in, int n_out, int accum, int act_group) {
    GemvParams P{};
    P.y = y, P.x = x, P.w = w_packed, P.b = b, P.n_in = n_in, P.n_out = n_out, P.accum = accum ? 1 : 0;
    P.scales = scales, P.ag = act_group;
    return launch_gemv(h, stream, P, 2, "gemv_int8");
}

extern "C" int mx230_qkv_rope_kvwrite(mx230_handle *h, void *stream, float *qkv, const float *x, const void *w,
                                      int w_kind, const float *w_scales, int act_group, const float *b, int n_in,
                                      int pos, const int *pos_ptr,
                                      int n_head, int n_kv_head, int head_dim, float theta, float *kcache,
                                      float *vcache, int8_t *kq, int8_t *vq, float *ks, float *vs, float *kb,
                                      float *vb, const int *bt, int bs) {
    MX_REQUIRE(head_dim == 64, MX230_ERR_UNSUPPORTED, "qkv_rope_kvwrite: head_dim %d unsupported (must be 64)", head_dim);
    MX_REQUIRE(n_head > 0 && n_kv_head > 0, MX230_ERR_INVALID_ARG, "qkv_rope_kvwrite: bad head counts %d/%d", n_head, n_kv_head);
    MX_REQUIRE((kq != nullptr) ? (vq && ks && vs && ((kb == nullptr) == (vb == nullptr))) : (kcache && vcache),
               MX230_ERR_INVALID_ARG, "qkv_rope_kvwrite: missing cache array");
    MX_REQUIRE(pos_ptr || pos >= 0, MX230_ERR_INVALID_ARG, "qkv_rope_kvwrite: negative position %d", pos);
    MX_REQUIRE(bt == nullptr || bs > 0, MX230_ERR_INVALID_ARG, "qkv_rope_kvwrite: block size %d", bs);
    GemvParams P{};
    MX_REQUIRE(w_kind >= 0 && w_kind <= 2, MX230_ERR_INVALID_ARG, "qkv_rope_kvwrite: weight kind %d", w_kind);
    P.y = qkv, P.x = x, P.w = w, P.b = b, P.n_in = n_in, P.n_out = (n_head + 2 * n_kv_head) * 64, P.accum = 0;
    P.scales = w_scales, P.ag = act_group;
    P.e.enabled = 1, P.e.pos = pos, P.e.pos_dev = pos_ptr, P.e.n_head = n_head, P.e.n_kv_head = n_kv_head;
    P.e.theta = theta, P.e.kcache = kcache, P.e.vcache = vcache, P.e.kq = kq, P.e.vq = vq;
    P.e.ks = ks, P.e.vs = vs, P.e.kb = kb, P.e.vb = vb, P.e.bt = bt, P.e.bs = bs;
    return launch_gemv(h, stream, P, w_kind, "qkv_rope_kvwrite");
}
