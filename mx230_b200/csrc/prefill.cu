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

// out[h][r][0..63] (bf16) <- qkv[r*stride + h*64 + 0..63] * 1/sqrt(64) * log2(e), so that the attention
// kernel's scores arrive in log2 units (one rounding, from the fp32 product); 8 elements per thread
__global__ void stage_q_kernel(__nv_bfloat16 *out, const float *qkv, int n_tok, int n_head, int stride) {
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;  // over n_head*n_tok*8
    size_t total = (size_t)n_head * n_tok * 8;
    if (idx >= total) return;
    int c = (int)(idx & 7);
    size_t hr = idx >> 3;
    int r = (int)(hr % n_tok);
    int h = (int)(hr / n_tok);
    const float4 *src = (const float4 *)(qkv + (size_t)r * stride + h * HD + c * 8);
    float4 a = src[0], b = src[1];
    const float sc = MX230_QK_LOG2_SCALE;
    uint4 o;
    o.x = mx::pack_bf16(a.x * sc, a.y * sc);
    o.y = mx::pack_bf16(a.z * sc, a.w * sc);
    o.z = mx::pack_bf16(b.x * sc, b.y * sc);
    o.w = mx::pack_bf16(b.z * sc, b.w * sc);
    *(uint4 *)(out + ((size_t)h * n_tok + r) * HD + c * 8) = o;
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

// one thread stages 8 consecutive dims of one (key, kv head) for K and V
__global__ void stage_kv_kernel(const StageKv P) {
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;  // over n_keys*n_kv_head*8
    size_t total = (size_t)P.n_keys * P.n_kv_head * 8;
    if (idx >= total) return;
    int c = (int)(idx & 7);
    size_t th = idx >> 3;
    int h = (int)(th % P.n_kv_head);
    int t = (int)(th / P.n_kv_head);
    size_t row = P.bt ? (size_t)(P.bt[t / P.bs] * P.bs + t % P.bs) : (size_t)t;
    size_t kvd = (size_t)P.n_kv_head * HD;
    size_t dst = ((size_t)h * P.n_keys + t) * HD + c * 8;
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
    uint4 ko, vo;
    ko.x = mx::pack_bf16(k[0], k[1]), ko.y = mx::pack_bf16(k[2], k[3]);
    ko.z = mx::pack_bf16(k[4], k[5]), ko.w = mx::pack_bf16(k[6], k[7]);
    vo.x = mx::pack_bf16(v[0], v[1]), vo.y = mx::pack_bf16(v[2], v[3]);
    vo.z = mx::pack_bf16(v[4], v[5]), vo.w = mx::pack_bf16(v[6], v[7]);
    *(uint4 *)(P.kout + dst) = ko;
    *(uint4 *)(P.vout + dst) = vo;
}

size_t align1k(size_t x) { return (x + 1023) & ~(size_t)1023; }

int prefill(mx230_handle *h, void *stream, float *out, const float *qkv, const float *kcache,
            const float *vcache, const int8_t *kq, const int8_t *vq, const float *ks, const float *vs,
            const float *kb, const float *vb, int pos0, int n_tok, int n_head, int n_kv_head, int qkv_stride,
            int out_stride, const int *bt, int bs, const char *who) {
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
    size_t qbytes = align1k((size_t)n_head * n_tok * HD * 2);
    size_t kbytes = align1k((size_t)n_kv_head * n_keys * HD * 2);
    size_t need = qbytes + 2 * kbytes;
    MX_REQUIRE(h->ws && need <= h->ws_bytes, MX230_ERR_WORKSPACE,
               "%s: workspace %zu B < %zu B needed (call mx230_reserve)", who, h->ws_bytes, need);
    mx230_device_guard guard(h->device);
    cudaStream_t st = (cudaStream_t)stream;
    h->staged.valid = 0;   // the workspace is about to hold something else
    __nv_bfloat16 *qb = (__nv_bfloat16 *)h->ws;
    __nv_bfloat16 *kbuf = (__nv_bfloat16 *)((char *)h->ws + qbytes);
    __nv_bfloat16 *vbuf = (__nv_bfloat16 *)((char *)h->ws + qbytes + kbytes);
    size_t tq = (size_t)n_head * n_tok * 8;
    MX_LAUNCH(h, st, MX230_K_PREFILL,
              (stage_q_kernel<<<(unsigned)((tq + 255) / 256), 256, 0, st>>>(qb, qkv, n_tok, n_head, qkv_stride)));
    StageKv S{kbuf, vbuf, kcache, vcache, kq, vq, ks, vs, kb, vb, bt, bs, n_keys, n_kv_head};
    size_t tk = (size_t)n_keys * n_kv_head * 8;
    MX_LAUNCH(h, st, MX230_K_PREFILL, (stage_kv_kernel<<<(unsigned)((tk + 255) / 256), 256, 0, st>>>(S)));
    return mx230_launch_flash_fwd_ex(h, st, qb, kbuf, vbuf, out, nullptr, n_head, n_tok, n_keys, pos0,
                                     n_head / n_kv_head, HD, out_stride, 1, 1, nullptr, nullptr);
}

}  // namespace

extern "C" size_t mx230_prefill_workspace_bytes(int n_tok, int n_keys, int n_head, int n_kv_head) {
    if (n_tok <= 0 || n_keys <= 0 || n_head <= 0 || n_kv_head <= 0) return 0;
    return align1k((size_t)n_head * n_tok * HD * 2) + 2 * align1k((size_t)n_kv_head * n_keys * HD * 2);
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
                   pos0, n_tok, n_head, n_kv_head, qkv_stride, out_stride, nullptr, 0, "attn_prefill_dp4a");
}
extern "C" int mx230_attn_prefill_dp4a_paged(mx230_handle *h, void *stream, float *out, const float *qkv,
                                             const float *kcache, const float *vcache, int pos0, int n_tok,
                                             int n_head, int n_kv_head, int qkv_stride, int out_stride,
                                             const int *bt, int bs) {
    MX_REQUIRE(bt, MX230_ERR_INVALID_ARG, "attn_prefill_dp4a_paged: null block table");
    return prefill(h, stream, out, qkv, kcache, vcache, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr,
                   pos0, n_tok, n_head, n_kv_head, qkv_stride, out_stride, bt, bs, "attn_prefill_dp4a_paged");
}
