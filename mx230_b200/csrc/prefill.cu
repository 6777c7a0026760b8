// Per-layer attention step, part 3: prefill attention of n_tok new rows at absolute
// positions pos0+qi over the KV cache (keys 0..=pos0+qi), grouped-query aware.
//
// Reference semantics: attn_prefill_body<KIND, PAGED> and its wrappers,
// 03-llm-engine/kernels/llm.cu:3657-3872 -- a flash-style fp32 SIMT kernel per
// (64-query tile, head) that reads q strided from the qkv buffer and K/V only from the
// cache (so under an int8 cache a token attends the *quantised* K/V of itself and of
// its batch-mates, exactly as decode does).
//
// This design: two HBM-bound staging kernels bring the operands into the bf16 head-major
// layout of the tcgen05 forward kernel (Q gathered from the strided qkv rows; K and V
// gathered from the cache through the optional block table, int8 codes dequantised as
// code*scale + beta first), then the same tensor-core flash kernel as the stage-2 forward
// runs with the GQA head mapping (K/V head = h / group), the causal offset pos0 and the
// reference's strided output layout.  KIND 2 of the reference (scores through on-the-fly
// int8 K, an opt-in speed approximation on sm_61) is served by the exact-score path.
#include "common.cuh"

namespace {

constexpr int HD = 64;

// Largest value of `v` over the block (v >= 0), returned to thread 0
__device__ __forceinline__ float block_max256(float v) {
    __shared__ float part[8];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = v;
    __syncthreads();
    if (threadIdx.x < 8) {
        v = part[threadIdx.x];
#pragma unroll
        for (int o = 4; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFu, v, o));
    }
    return v;
}

// out[h][r][0..63] (bf16) <- qkv[r*stride + h*64 + 0..63] * 1/sqrt(64) * log2(e), so that the attention
// kernel's scores arrive in log2 units (one rounding, from the fp32 product).  Grid (MX230_NORM_PARTS, n_head): block
// (p, h) stages the rows r = p (mod 32) of head h, eight threads per row, and leaves the largest squared norm of its
// (unscaled) rows in norm2[h][p]: with the keys' norms that bounds every score of the head, which lets the attention
// kernel run without a row max.
__global__ void stage_q_kernel(__nv_bfloat16 *out, float *norm2, const float *qkv, int n_tok, int n_head, int stride) {
    const int p = blockIdx.x, h = blockIdx.y;
    const int c = threadIdx.x & 7, slot = threadIdx.x >> 3;
    const float sc = MX230_QK_LOG2_SCALE;
    float best = 0.0f;
    for (int r0 = p; r0 < n_tok; r0 += MX230_NORM_PARTS * 32) {
        const int r = r0 + MX230_NORM_PARTS * slot;
        float ss = 0.0f;
        if (r < n_tok) {
            const float4 *src = (const float4 *)(qkv + (size_t)r * stride + h * HD + c * 8);
            const float4 a = src[0], b = src[1];
            ss = a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w + b.x * b.x + b.y * b.y + b.z * b.z + b.w * b.w;
            uint4 o;
            o.x = mx::pack_bf16(a.x * sc, a.y * sc);
            o.y = mx::pack_bf16(a.z * sc, a.w * sc);
            o.z = mx::pack_bf16(b.x * sc, b.y * sc);
            o.w = mx::pack_bf16(b.z * sc, b.w * sc);
            *(uint4 *)(out + ((size_t)h * n_tok + r) * HD + c * 8) = o;
        }
#pragma unroll
        for (int o = 4; o > 0; o >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, o);   // the row's eight threads
        best = fmaxf(best, ss);
    }
    best = block_max256(best);
    if (threadIdx.x == 0) norm2[h * MX230_NORM_PARTS + p] = best;
}

struct StageKv {
    __nv_bfloat16 *kout, *vout;      // [n_kv_head][n_keys][64]
    const float *kcache, *vcache;    // fp32 cache, or
    const int8_t *kq, *vq;           // int8 cache with
    const float *ks, *vs, *kb, *vb;  // per-(row, head) scale and (optional) beta
    const int *bt;
    int bs;
    int n_keys, n_kv_head;
};

// Grid (MX230_NORM_PARTS, n_kv_head): block (p, h) stages the keys t = p (mod 32) of K/V head h, eight threads per key (8
// consecutive dims of K and of V each), and leaves the largest squared norm of its staged K rows in norm2[h][p].
__global__ void stage_kv_kernel(const StageKv P, float *norm2) {
    const int p = blockIdx.x, h = blockIdx.y;
    const int c = threadIdx.x & 7, slot = threadIdx.x >> 3;
    const size_t kvd = (size_t)P.n_kv_head * HD;
    float best = 0.0f;
    for (int t0 = p; t0 < P.n_keys; t0 += MX230_NORM_PARTS * 32) {
        const int t = t0 + MX230_NORM_PARTS * slot;
        float ss = 0.0f;
        if (t < P.n_keys) {
            const size_t row = P.bt ? (size_t)(P.bt[t / P.bs] * P.bs + t % P.bs) : (size_t)t;
            const size_t dst = ((size_t)h * P.n_keys + t) * HD + c * 8;
            float k[8], v[8];
            if (P.kq) {
                int2 kw = *(const int2 *)(P.kq + row * kvd + h * HD + c * 8);
                int2 vw = *(const int2 *)(P.vq + row * kvd + h * HD + c * 8);
                float ksc = P.ks[row * P.n_kv_head + h], vsc = P.vs[row * P.n_kv_head + h];
                float kbe = P.kb ? P.kb[row * P.n_kv_head + h] : 0.0f, vbe = P.vb ? P.vb[row * P.n_kv_head + h] : 0.0f;
                const int kk[2] = {kw.x, kw.y}, vv[2] = {vw.x, vw.y};
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    // dequantise as the reference does into its V tile: code * scale + beta (llm.cu:3759-3764)
                    k[i] = (float)(int8_t)((kk[i >> 2] >> (8 * (i & 3))) & 0xFF) * ksc + kbe;
                    v[i] = (float)(int8_t)((vv[i >> 2] >> (8 * (i & 3))) & 0xFF) * vsc + vbe;
                }
            } else {
                const float4 *kp = (const float4 *)(P.kcache + row * kvd + h * HD + c * 8);
                const float4 *vp = (const float4 *)(P.vcache + row * kvd + h * HD + c * 8);
                float4 a = kp[0], b = kp[1], e = vp[0], f = vp[1];
                k[0] = a.x, k[1] = a.y, k[2] = a.z, k[3] = a.w, k[4] = b.x, k[5] = b.y, k[6] = b.z, k[7] = b.w;
                v[0] = e.x, v[1] = e.y, v[2] = e.z, v[3] = e.w, v[4] = f.x, v[5] = f.y, v[6] = f.z, v[7] = f.w;
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) ss += k[i] * k[i];
            uint4 ko, vo;
            ko.x = mx::pack_bf16(k[0], k[1]), ko.y = mx::pack_bf16(k[2], k[3]);
            ko.z = mx::pack_bf16(k[4], k[5]), ko.w = mx::pack_bf16(k[6], k[7]);
            vo.x = mx::pack_bf16(v[0], v[1]), vo.y = mx::pack_bf16(v[2], v[3]);
            vo.z = mx::pack_bf16(v[4], v[5]), vo.w = mx::pack_bf16(v[6], v[7]);
            *(uint4 *)(P.kout + dst) = ko;
            *(uint4 *)(P.vout + dst) = vo;
        }
#pragma unroll
        for (int o = 4; o > 0; o >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, o);   // the key's eight threads
        best = fmaxf(best, ss);
    }
    best = block_max256(best);
    if (threadIdx.x == 0) norm2[h * MX230_NORM_PARTS + p] = best;
}

// ---- int8 score mode (the reference kernels' own arithmetic, llm.cu:3700-3716,3737-3754,3774-3782) ----
// q row -> int8 codes per (row, head): id = 127 / amax, code = clamp(rne(q * id), +-127); the codes go out as bf16
// (exact), with the row's score factor (amax / 127) * 1/sqrt(64) * log2(e) and the sum of its codes.
// One warp per (head, row); lane l holds dims l and l + 32.
__global__ void stage_q_codes_kernel(__nv_bfloat16 *out, float *row_a, float *row_qsum, const float *qkv, int n_tok,
                                     int n_head, int stride) {
    const int w = (int)(((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5), lane = threadIdx.x & 31;
    if (w >= n_head * n_tok) return;
    const int h = w / n_tok, r = w - h * n_tok;
    const float *src = qkv + (size_t)r * stride + h * HD;
    const float a = src[lane], b = src[lane + 32];
    float amax = fmaxf(fabsf(a), fabsf(b));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
    const float id = amax > 0.0f ? __fdiv_rn(127.0f, amax) : 0.0f;
    const int ca = max(-127, min(127, __float2int_rn(a * id))), cb = max(-127, min(127, __float2int_rn(b * id)));
    int sum = ca + cb;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, o);
    __nv_bfloat16 *dst = out + ((size_t)h * n_tok + r) * HD;
    dst[lane] = __float2bfloat16((float)ca);
    dst[lane + 32] = __float2bfloat16((float)cb);
    if (lane == 0) {
        const float qs = amax > 0.0f ? __fdiv_rn(amax, 127.0f) : 0.0f;
        row_a[(size_t)h * n_tok + r] = qs * 0.125f * 1.4426950408889634f;
        row_qsum[(size_t)h * n_tok + r] = (float)sum;
    }
}

// K as int8 codes in bf16 (exact) with its per-key (scale, offset) pair, V dequantised to bf16.  Over an int8
// cache the codes and pairs are the cache's own (absmax format: offset 0); over an fp32 cache (the reference's
// opt-in attn_prefill_dp4a) every K row is quantised on the fly, symmetric absmax, and V is the fp32 row.
// One thread stages 8 consecutive dims of one (key, kv head); the 8 threads of a row are neighbouring lanes.
__global__ void stage_kv_codes_kernel(const StageKv P, float2 *kskb, int n_k_pad) {
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;  // over n_keys*n_kv_head*8
    size_t total = (size_t)P.n_keys * P.n_kv_head * 8;
    const bool live = idx < total;
    if (!live) idx = total - 1;   // keep the row's lanes together for the shuffles below
    int c = (int)(idx & 7);
    size_t th = idx >> 3;
    int h = (int)(th % P.n_kv_head);
    int t = (int)(th / P.n_kv_head);
    size_t row = P.bt ? (size_t)(P.bt[t / P.bs] * P.bs + t % P.bs) : (size_t)t;
    size_t kvd = (size_t)P.n_kv_head * HD;
    size_t dst = ((size_t)h * P.n_keys + t) * HD + c * 8;
    float k[8], v[8];
    float ksc, kbe;
    if (P.kq) {
        int2 kw = *(const int2 *)(P.kq + row * kvd + h * HD + c * 8);
        int2 vw = *(const int2 *)(P.vq + row * kvd + h * HD + c * 8);
        ksc = P.ks[row * P.n_kv_head + h];
        kbe = P.kb ? P.kb[row * P.n_kv_head + h] : 0.0f;
        float vsc = P.vs[row * P.n_kv_head + h], vbe = P.vb ? P.vb[row * P.n_kv_head + h] : 0.0f;
        const int kk[2] = {kw.x, kw.y}, vv[2] = {vw.x, vw.y};
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            k[i] = (float)(int8_t)((kk[i >> 2] >> (8 * (i & 3))) & 0xFF);
            v[i] = (float)(int8_t)((vv[i >> 2] >> (8 * (i & 3))) & 0xFF) * vsc + vbe;
        }
    } else {
        const float4 *kp = (const float4 *)(P.kcache + row * kvd + h * HD + c * 8);
        const float4 *vp = (const float4 *)(P.vcache + row * kvd + h * HD + c * 8);
        float4 a = kp[0], b = kp[1], e = vp[0], f = vp[1];
        k[0] = a.x, k[1] = a.y, k[2] = a.z, k[3] = a.w, k[4] = b.x, k[5] = b.y, k[6] = b.z, k[7] = b.w;
        v[0] = e.x, v[1] = e.y, v[2] = e.z, v[3] = e.w, v[4] = f.x, v[5] = f.y, v[6] = f.z, v[7] = f.w;
        float amax = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(k[i]));
        const unsigned m8 = 0xFFu << ((threadIdx.x & 31) & ~7);   // the 8 lanes of this row
#pragma unroll
        for (int o = 4; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(m8, amax, o));
        const float id = amax > 0.0f ? __fdiv_rn(127.0f, amax) : 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) k[i] = (float)max(-127, min(127, __float2int_rn(k[i] * id)));
        ksc = amax > 0.0f ? __fdiv_rn(amax, 127.0f) : 0.0f;
        kbe = 0.0f;
    }
    if (!live) return;
    uint4 ko, vo;
    ko.x = mx::pack_bf16(k[0], k[1]), ko.y = mx::pack_bf16(k[2], k[3]);
    ko.z = mx::pack_bf16(k[4], k[5]), ko.w = mx::pack_bf16(k[6], k[7]);
    vo.x = mx::pack_bf16(v[0], v[1]), vo.y = mx::pack_bf16(v[2], v[3]);
    vo.z = mx::pack_bf16(v[4], v[5]), vo.w = mx::pack_bf16(v[6], v[7]);
    *(uint4 *)(P.kout + dst) = ko;
    *(uint4 *)(P.vout + dst) = vo;
    if (c == 0) kskb[(size_t)h * n_k_pad + t] = make_float2(ksc, kbe);
}

size_t align1k(size_t x) { return (x + 1023) & ~(size_t)1023; }

int prefill(mx230_handle *h, void *stream, float *out, const float *qkv, const float *kcache,
            const float *vcache, const int8_t *kq, const int8_t *vq, const float *ks, const float *vs,
            const float *kb, const float *vb, int pos0, int n_tok, int n_head, int n_kv_head, int qkv_stride,
            int out_stride, const int *bt, int bs, const char *who, bool dp4a = false) {
    MX_REQUIRE(h != nullptr, MX230_ERR_INVALID_ARG, "%s: null handle", who);
    MX_REQUIRE(pos0 >= 0 && n_tok >= 0, MX230_ERR_INVALID_ARG, "%s: negative pos0/n_tok", who);
    if (n_tok == 0) return MX230_OK;
    MX_REQUIRE(out && qkv, MX230_ERR_INVALID_ARG, "%s: null out/qkv", who);
    MX_REQUIRE(n_head > 0 && n_kv_head > 0 && n_head % n_kv_head == 0, MX230_ERR_UNSUPPORTED,
               "%s: n_head %d must be a positive multiple of n_kv_head %d", who, n_head, n_kv_head);
    if (kq)
        MX_REQUIRE(vq && ks && vs && ((kb == nullptr) == (vb == nullptr)), MX230_ERR_INVALID_ARG,
                   "%s: missing int8 cache array", who);
    else
        MX_REQUIRE(kcache && vcache, MX230_ERR_INVALID_ARG, "%s: null cache", who);
    MX_REQUIRE(bt == nullptr || bs > 0, MX230_ERR_INVALID_ARG, "%s: block size %d", who, bs);
    MX_REQUIRE(qkv_stride % 4 == 0 && out_stride % 4 == 0 &&
                   (((uintptr_t)qkv | (uintptr_t)out | (uintptr_t)kcache | (uintptr_t)vcache | (uintptr_t)kq |
                     (uintptr_t)vq) & 15) == 0,
               MX230_ERR_INVALID_ARG, "%s: buffers must be 16-byte aligned, strides multiples of 4", who);
    const int n_keys = pos0 + n_tok;
    const int n_k_pad = (n_keys + 127) / 128 * 128;
    size_t qbytes = align1k((size_t)n_head * n_tok * HD * 2);
    size_t kbytes = align1k((size_t)n_kv_head * n_keys * HD * 2);
    size_t rbytes = align1k((size_t)n_head * n_tok * 4);
    size_t cbytes = align1k((size_t)n_kv_head * n_k_pad * 8);
    size_t nbytes = align1k((size_t)(n_head + n_kv_head) * MX230_NORM_PARTS * 4);
    size_t need = qbytes + 2 * kbytes + 2 * rbytes + cbytes + nbytes;
    MX_REQUIRE(h->ws && need <= h->ws_bytes, MX230_ERR_WORKSPACE,
               "%s: workspace %zu B < %zu B needed (call mx230_reserve)", who, h->ws_bytes, need);
    mx230_device_guard guard(h->device);
    cudaStream_t st = (cudaStream_t)stream;
    h->staged.valid = 0;   // the workspace is about to hold something else
    __nv_bfloat16 *qb = (__nv_bfloat16 *)h->ws;
    __nv_bfloat16 *kbuf = (__nv_bfloat16 *)((char *)h->ws + qbytes);
    __nv_bfloat16 *vbuf = (__nv_bfloat16 *)((char *)h->ws + qbytes + kbytes);
    float *row_a = (float *)((char *)h->ws + qbytes + 2 * kbytes);
    float *row_qsum = (float *)((char *)row_a + rbytes);
    float2 *kskb = (float2 *)((char *)row_qsum + rbytes);
    float *q_norm2 = (float *)((char *)kskb + cbytes);
    float *k_norm2 = q_norm2 + (size_t)n_head * MX230_NORM_PARTS;
    StageKv S{kbuf, vbuf, kcache, vcache, kq, vq, ks, vs, kb, vb, bt, bs, n_keys, n_kv_head};
    size_t tk = (size_t)n_keys * n_kv_head * 8;
    // Which score arithmetic: over an int8 cache the handle's MX230_OPT_Q8_SCORE_MODE decides, as for decode
    // (REF, the default: q quantised per (row, head) to int8 and integer dots, what attn_prefill_q8 computes;
    // EXACT: fp32 q against dequantised K); the _dp4a entry points are the reference's int8-score approximation
    // over an fp32 cache by definition.
    const bool i8_scores = dp4a || (kq && h->q8_score_mode == MX230_Q8_SCORE_REF);
    if (i8_scores) {
        size_t warps = (size_t)n_head * n_tok;
        MX_LAUNCH(h, st, MX230_K_PREFILL,
                  (stage_q_codes_kernel<<<(unsigned)((warps * 32 + 255) / 256), 256, 0, st>>>(qb, row_a, row_qsum, qkv, n_tok,
                                                                                              n_head, qkv_stride)));
        MX_LAUNCH(h, st, MX230_K_PREFILL, (stage_kv_codes_kernel<<<(unsigned)((tk + 255) / 256), 256, 0, st>>>(S, kskb, n_k_pad)));
        return mx230_launch_flash_fwd_ex(h, st, qb, kbuf, vbuf, out, nullptr, n_head, n_tok, n_keys, pos0,
                                         n_head / n_kv_head, HD, out_stride, 1, 0, nullptr, nullptr, row_a, row_qsum,
                                         (const float *)kskb);
    }
    // values (fp32 cache, or an int8 cache in the exact score mode): the staging kernels also leave the row norms that
    // let the attention kernel take its max-free path whenever the head's scores are bounded
    MX_LAUNCH(h, st, MX230_K_PREFILL,
              (stage_q_kernel<<<dim3(MX230_NORM_PARTS, n_head), 256, 0, st>>>(qb, q_norm2, qkv, n_tok, n_head, qkv_stride)));
    MX_LAUNCH(h, st, MX230_K_PREFILL, (stage_kv_kernel<<<dim3(MX230_NORM_PARTS, n_kv_head), 256, 0, st>>>(S, k_norm2)));
    return mx230_launch_flash_fwd_ex(h, st, qb, kbuf, vbuf, out, nullptr, n_head, n_tok, n_keys, pos0,
                                     n_head / n_kv_head, HD, out_stride, 1, 1, q_norm2, k_norm2, nullptr, nullptr, nullptr);
}

}  // namespace

extern "C" size_t mx230_prefill_workspace_bytes(int n_tok, int n_keys, int n_head, int n_kv_head) {
    if (n_tok <= 0 || n_keys <= 0 || n_head <= 0 || n_kv_head <= 0) return 0;
    // staged bf16 Q, K, V, then (int8 score mode) the per-row q factors and the per-key (scale, offset) pairs
    return align1k((size_t)n_head * n_tok * HD * 2) + 2 * align1k((size_t)n_kv_head * n_keys * HD * 2) +
           2 * align1k((size_t)n_head * n_tok * 4) + align1k((size_t)n_kv_head * ((n_keys + 127) / 128 * 128) * 8) +
           align1k((size_t)(n_head + n_kv_head) * MX230_NORM_PARTS * 4);
}

extern "C" int mx230_attn_prefill(mx230_handle *h, void *stream, float *out, const float *qkv,
                                  const float *kcache, const float *vcache, int pos0, int n_tok, int n_head,
                                  int n_kv_head, int qkv_stride, int out_stride) {
    return prefill(h, stream, out, qkv, kcache, vcache, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr,
                   pos0, n_tok, n_head, n_kv_head, qkv_stride, out_stride, nullptr, 0, "attn_prefill");
}
extern "C" int mx230_attn_prefill_paged(mx230_handle *h, void *stream, float *out, const float *qkv,
                                        const float *kcache, const float *vcache, int pos0, int n_tok,
                                        int n_head, int n_kv_head, int qkv_stride, int out_stride,
                                        const int *bt, int bs) {
    MX_REQUIRE(bt, MX230_ERR_INVALID_ARG, "attn_prefill_paged: null block table");
    return prefill(h, stream, out, qkv, kcache, vcache, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr,
                   pos0, n_tok, n_head, n_kv_head, qkv_stride, out_stride, bt, bs, "attn_prefill_paged");
}
extern "C" int mx230_attn_prefill_q8(mx230_handle *h, void *stream, float *out, const float *qkv,
                                     const int8_t *kq, const int8_t *vq, const float *ks, const float *vs,
                                     const float *kb, const float *vb, int pos0, int n_tok, int n_head,
                                     int n_kv_head, int qkv_stride, int out_stride) {
    MX_REQUIRE(kq, MX230_ERR_INVALID_ARG, "attn_prefill_q8: null kq");
    return prefill(h, stream, out, qkv, nullptr, nullptr, kq, vq, ks, vs, kb, vb, pos0, n_tok, n_head,
                   n_kv_head, qkv_stride, out_stride, nullptr, 0, "attn_prefill_q8");
}
extern "C" int mx230_attn_prefill_q8_paged(mx230_handle *h, void *stream, float *out, const float *qkv,
                                           const int8_t *kq, const int8_t *vq, const float *ks,
                                           const float *vs, const float *kb, const float *vb, int pos0,
                                           int n_tok, int n_head, int n_kv_head, int qkv_stride,
                                           int out_stride, const int *bt, int bs) {
    MX_REQUIRE(kq && bt, MX230_ERR_INVALID_ARG, "attn_prefill_q8_paged: null argument");
    return prefill(h, stream, out, qkv, nullptr, nullptr, kq, vq, ks, vs, kb, vb, pos0, n_tok, n_head,
                   n_kv_head, qkv_stride, out_stride, bt, bs, "attn_prefill_q8_paged");
}
extern "C" int mx230_attn_prefill_dp4a(mx230_handle *h, void *stream, float *out, const float *qkv,
                                       const float *kcache, const float *vcache, int pos0, int n_tok,
                                       int n_head, int n_kv_head, int qkv_stride, int out_stride) {
    return prefill(h, stream, out, qkv, kcache, vcache, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr,
                   pos0, n_tok, n_head, n_kv_head, qkv_stride, out_stride, nullptr, 0, "attn_prefill_dp4a", true);
}
extern "C" int mx230_attn_prefill_dp4a_paged(mx230_handle *h, void *stream, float *out, const float *qkv,
                                             const float *kcache, const float *vcache, int pos0, int n_tok,
                                             int n_head, int n_kv_head, int qkv_stride, int out_stride,
                                             const int *bt, int bs) {
    MX_REQUIRE(bt, MX230_ERR_INVALID_ARG, "attn_prefill_dp4a_paged: null block table");
    return prefill(h, stream, out, qkv, kcache, vcache, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr,
                   pos0, n_tok, n_head, n_kv_head, qkv_stride, out_stride, bt, bs, "attn_prefill_dp4a_paged", true);
}
