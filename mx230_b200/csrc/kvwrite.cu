// Per-layer attention step, part 1: RoPE and the KV-cache write (fp32 copy or int8
// quantize-on-write).  HBM-bound elementwise work; one kernel family per op, the
// reference's single / device-position / batch / per-sequence variants differ only
// in where a row's position comes from.
//
// Reference: 03-llm-engine/kernels/llm.cu:959-986 (kv_row, copy_kv_*), 1072-1117 and
// 1513-1530 (rope*), 1137-1240 and 1503-1510 (quant_affine, quantize_kv*),
// 3635-3655 (copy_kv_batch*).
#include "common.cuh"

namespace {

// Where the position of row r comes from.
//   kind 0: host scalar, row r sits at pos + r        (rope, rope_batch, *_batch)
//   kind 1: *pos_dev (one row)                        (*_dyn, graph-captured decode)
//   kind 2: pos_dev[r], block table row r of `tables` (*_seqpos, batched decode)
struct RowPos {
    int kind;
    int pos;
    const int *pos_dev;
    const int *bt;   // block table (kind 0/1) or packed tables (kind 2); null = linear
    int bs;          // block size
    int n_log;       // table row length (kind 2)
};

__device__ __forceinline__ int row_position(const RowPos &rp, int r) {
    if (rp.kind == 0) return rp.pos + r;
    if (rp.kind == 1) return *rp.pos_dev;
    return rp.pos_dev[r];
}

__device__ __forceinline__ size_t phys_row(const RowPos &rp, int r, int t) {
    const int *bt = rp.bt;
    if (bt == nullptr) return (size_t)t;
    if (rp.kind == 2) bt += (size_t)r * rp.n_log;
    return (size_t)(bt[t / rp.bs] * rp.bs + t % rp.bs);
}

// HF rotate_half RoPE, pairs (d, d + hd/2), on the Q heads then the K heads of each row.
__global__ void rope_kernel(float *qkv, RowPos rp, int n_rows, int n_head, int n_kv_head,
                            int head_dim, int stride, float theta) {
    int half = head_dim / 2;
    int per_row = (n_head + n_kv_head) * half;
    int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n_rows * per_row) return;
    int r = idx / per_row;
    int i = idx - r * per_row;
    int h = i / half;
    int d = i - h * half;
    float *base = qkv + (size_t)r * stride + h * head_dim;
    // precise powf / sincosf: the reference's CPU path (03-llm-engine/src/cpu.rs:25-37);
    // its GPU kernel uses the fast intrinsics, which lose accuracy at large angles
    float freq = powf(theta, -2.0f * (float)d / (float)head_dim);
    float sn, cs;
    sincosf((float)row_position(rp, r) * freq, &sn, &cs);
    float x1 = base[d], x2 = base[d + half];
    base[d] = x1 * cs - x2 * sn;
    base[d + half] = x1 * sn + x2 * cs;
}

__global__ void copy_kv_kernel(float *kcache, float *vcache, const float *qkv, RowPos rp,
                               int q_dim, int kv_dim, int stride) {
    int r = blockIdx.y;
    int i = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (i >= kv_dim) return;
    size_t row = phys_row(rp, r, row_position(rp, r)) * kv_dim;
    const float *src = qkv + (size_t)r * stride + q_dim;
    *(float4 *)(kcache + row + i) = *(const float4 *)(src + i);
    *(float4 *)(vcache + row + i) = *(const float4 *)(src + kv_dim + i);
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
    return v;
}

// One warp quantises one 64-value head row (K or V) of one qkv row: lane l owns
// elements 2l, 2l+1.  IEEE division and round-to-nearest-even exactly as quant_affine.
__global__ void quantize_kv_kernel(int8_t *kq, int8_t *vq, float *ks, float *vs, float *kb,
                                   float *vb, const float *qkv, RowPos rp, int n_rows, int q_dim,
                                   int n_kv_head, int stride) {
    int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    int lane = threadIdx.x & 31;
    int total = n_rows * n_kv_head * 2;
    if (warp >= total) return;
    int which = warp & 1;  // 0 = K, 1 = V
    int h = (warp >> 1) % n_kv_head;
    int r = (warp >> 1) / n_kv_head;
    int kv_dim = n_kv_head * 64;
    const float *src = qkv + (size_t)r * stride + q_dim + which * kv_dim + h * 64;
    float2 x = *(const float2 *)(src + 2 * lane);
    size_t pr = phys_row(rp, r, row_position(rp, r));
    int8_t *dst = (which ? vq : kq) + pr * kv_dim + h * 64;
    float *sc = which ? vs : ks;
    float *be = which ? vb : kb;
    size_t sd = pr * n_kv_head + h;
    int c0, c1;
    if (be != nullptr) {
        float hi = warp_max(fmaxf(x.x, x.y));
        float lo = -warp_max(fmaxf(-x.x, -x.y));
        float scale = (hi > lo) ? __fdiv_rn(hi - lo, 255.0f) : 1.0f;
        float beta = __fmaf_rn(128.0f, scale, lo);  // exact: 128*scale is a power-of-two scaling
        c0 = max(-128, min(127, __float2int_rn(__fdiv_rn(x.x - beta, scale))));
        c1 = max(-128, min(127, __float2int_rn(__fdiv_rn(x.y - beta, scale))));
        if (lane == 0) {
            sc[sd] = scale;
            be[sd] = beta;
        }
    } else {
        float amax = warp_max(fmaxf(fabsf(x.x), fabsf(x.y)));
        float id = amax > 0.0f ? __fdiv_rn(127.0f, amax) : 0.0f;
        c0 = max(-127, min(127, __float2int_rn(x.x * id)));
        c1 = max(-127, min(127, __float2int_rn(x.y * id)));
        if (lane == 0) sc[sd] = amax > 0.0f ? __fdiv_rn(amax, 127.0f) : 0.0f;
    }
    unsigned short packed = (unsigned short)((c0 & 0xFF) | ((c1 & 0xFF) << 8));
    *(unsigned short *)(dst + 2 * lane) = packed;
}

int check_heads(const char *who, int n_head, int n_kv_head, int head_dim) {
    MX_REQUIRE(head_dim == 64, MX230_ERR_UNSUPPORTED, "%s: head_dim %d unsupported (must be 64)",
               who, head_dim);
    MX_REQUIRE(n_kv_head > 0 && n_head >= 0, MX230_ERR_INVALID_ARG, "%s: bad head counts %d/%d", who,
               n_head, n_kv_head);
    return MX230_OK;
}

int launch_rope(mx230_handle *h, void *stream, float *qkv, RowPos rp, int n_rows, int n_head,
                int n_kv_head, int head_dim, int stride, float theta) {
    MX_REQUIRE(h && qkv, MX230_ERR_INVALID_ARG, "rope: null argument");
    MX_REQUIRE(head_dim > 0 && head_dim % 2 == 0, MX230_ERR_UNSUPPORTED, "rope: odd head_dim");
    MX_REQUIRE(n_rows >= 0 && n_head >= 0 && n_kv_head >= 0, MX230_ERR_INVALID_ARG,
               "rope: negative size");
    long long total = (long long)n_rows * (n_head + n_kv_head) * (head_dim / 2);
    if (total == 0) return MX230_OK;
    mx230_device_guard guard(h->device);
    cudaStream_t st = (cudaStream_t)stream;
    MX_LAUNCH(h, st, MX230_K_ROPE, (rope_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(
        qkv, rp, n_rows, n_head, n_kv_head, head_dim, stride, theta)));
    return MX230_OK;
}

int launch_copy(mx230_handle *h, void *stream, float *kcache, float *vcache, const float *qkv,
                RowPos rp, int n_rows, int q_dim, int kv_dim, int stride) {
    MX_REQUIRE(h && kcache && vcache && qkv, MX230_ERR_INVALID_ARG, "copy_kv: null argument");
    MX_REQUIRE(kv_dim > 0 && kv_dim % 4 == 0 && q_dim % 4 == 0 && stride % 4 == 0,
               MX230_ERR_UNSUPPORTED, "copy_kv: q_dim, kv_dim and stride must be multiples of 4");
    MX_REQUIRE((((uintptr_t)kcache | (uintptr_t)vcache | (uintptr_t)qkv) & 15) == 0,
               MX230_ERR_INVALID_ARG, "copy_kv: buffers must be 16-byte aligned");
    if (n_rows <= 0) return n_rows == 0 ? MX230_OK
                                        : mx230_fail(MX230_ERR_INVALID_ARG, "copy_kv: negative rows");
    mx230_device_guard guard(h->device);
    dim3 grid((kv_dim / 4 + 127) / 128, n_rows);
    cudaStream_t st = (cudaStream_t)stream;
    MX_LAUNCH(h, st, MX230_K_COPY_KV,
              (copy_kv_kernel<<<grid, 128, 0, st>>>(kcache, vcache, qkv, rp, q_dim, kv_dim, stride)));
    return MX230_OK;
}

int launch_quant(mx230_handle *h, void *stream, int8_t *kq, int8_t *vq, float *ks, float *vs,
                 float *kb, float *vb, const float *qkv, RowPos rp, int n_rows, int q_dim,
                 int n_kv_head, int head_dim, int stride) {
    MX_REQUIRE(h && kq && vq && ks && vs && qkv, MX230_ERR_INVALID_ARG,
               "quantize_kv: null argument");
    MX_REQUIRE((kb == nullptr) == (vb == nullptr), MX230_ERR_INVALID_ARG,
               "quantize_kv: kb and vb must both be given (affine) or both be null (absmax)");
    int rc = check_heads("quantize_kv", 0, n_kv_head, head_dim);
    if (rc) return rc;
    MX_REQUIRE(q_dim % 2 == 0 && stride % 2 == 0 && (((uintptr_t)qkv) & 7) == 0 &&
                   ((((uintptr_t)kq) | ((uintptr_t)vq)) & 1) == 0,
               MX230_ERR_INVALID_ARG, "quantize_kv: misaligned qkv or cache");
    if (n_rows <= 0) return n_rows == 0 ? MX230_OK
                                        : mx230_fail(MX230_ERR_INVALID_ARG, "quantize_kv: negative rows");
    mx230_device_guard guard(h->device);
    long long warps = (long long)n_rows * n_kv_head * 2;
    cudaStream_t st = (cudaStream_t)stream;
    MX_LAUNCH(h, st, MX230_K_QUANTIZE_KV,
              (quantize_kv_kernel<<<(unsigned)((warps + 3) / 4), 128, 0, st>>>(
                  kq, vq, ks, vs, kb, vb, qkv, rp, n_rows, q_dim, n_kv_head, stride)));
    return MX230_OK;
}

RowPos host_pos(int pos, const int *bt = nullptr, int bs = 0) { return RowPos{0, pos, nullptr, bt, bs, 0}; }
RowPos dev_pos(const int *p, const int *bt = nullptr, int bs = 0) { return RowPos{1, 0, p, bt, bs, 0}; }
RowPos seq_pos(const int *p, const int *tables, int bs, int n_log) {
    return RowPos{2, 0, p, tables, bs, n_log};
}

}  // namespace

// ---- rope ----
extern "C" int mx230_rope(mx230_handle *h, void *stream, float *qkv, int pos, int n_head,
                          int n_kv_head, int head_dim, float theta) {
    return launch_rope(h, stream, qkv, host_pos(pos), 1, n_head, n_kv_head, head_dim, 0, theta);
}
extern "C" int mx230_rope_dyn(mx230_handle *h, void *stream, float *qkv, const int *pos_ptr,
                              int n_head, int n_kv_head, int head_dim, float theta) {
    MX_REQUIRE(pos_ptr, MX230_ERR_INVALID_ARG, "rope_dyn: null pos_ptr");
    return launch_rope(h, stream, qkv, dev_pos(pos_ptr), 1, n_head, n_kv_head, head_dim, 0, theta);
}
extern "C" int mx230_rope_batch(mx230_handle *h, void *stream, float *qkv, int pos0, int n_tok,
                                int n_head, int n_kv_head, int head_dim, int stride, float theta) {
    return launch_rope(h, stream, qkv, host_pos(pos0), n_tok, n_head, n_kv_head, head_dim, stride,
                       theta);
}
extern "C" int mx230_rope_seqpos(mx230_handle *h, void *stream, float *qkv, const int *pos,
                                 int n_seq, int n_head, int n_kv_head, int head_dim, int stride,
                                 float theta) {
    MX_REQUIRE(pos, MX230_ERR_INVALID_ARG, "rope_seqpos: null pos");
    return launch_rope(h, stream, qkv, seq_pos(pos, nullptr, 0, 0), n_seq, n_head, n_kv_head,
                       head_dim, stride, theta);
}

// ---- fp32 KV write ----
extern "C" int mx230_copy_kv(mx230_handle *h, void *stream, float *kcache, float *vcache,
                             const float *qkv, int pos, int q_dim, int kv_dim) {
    return launch_copy(h, stream, kcache, vcache, qkv, host_pos(pos), 1, q_dim, kv_dim, 0);
}
extern "C" int mx230_copy_kv_dyn(mx230_handle *h, void *stream, float *kcache, float *vcache,
                                 const float *qkv, const int *pos_ptr, int q_dim, int kv_dim) {
    MX_REQUIRE(pos_ptr, MX230_ERR_INVALID_ARG, "copy_kv_dyn: null pos_ptr");
    return launch_copy(h, stream, kcache, vcache, qkv, dev_pos(pos_ptr), 1, q_dim, kv_dim, 0);
}
extern "C" int mx230_copy_kv_paged_dyn(mx230_handle *h, void *stream, float *kcache, float *vcache,
                                       const float *qkv, const int *pos_ptr, int q_dim, int kv_dim,
                                       const int *bt, int bs) {
    MX_REQUIRE(pos_ptr && bt && bs > 0, MX230_ERR_INVALID_ARG, "copy_kv_paged_dyn: bad table");
    return launch_copy(h, stream, kcache, vcache, qkv, dev_pos(pos_ptr, bt, bs), 1, q_dim, kv_dim, 0);
}
extern "C" int mx230_copy_kv_batch(mx230_handle *h, void *stream, float *kcache, float *vcache,
                                   const float *qkv, int pos0, int n_tok, int q_dim, int kv_dim,
                                   int stride) {
    return launch_copy(h, stream, kcache, vcache, qkv, host_pos(pos0), n_tok, q_dim, kv_dim, stride);
}
extern "C" int mx230_copy_kv_batch_paged(mx230_handle *h, void *stream, float *kcache,
                                         float *vcache, const float *qkv, int pos0, int n_tok,
                                         int q_dim, int kv_dim, int stride, const int *bt, int bs) {
    MX_REQUIRE(bt && bs > 0, MX230_ERR_INVALID_ARG, "copy_kv_batch_paged: bad table");
    return launch_copy(h, stream, kcache, vcache, qkv, host_pos(pos0, bt, bs), n_tok, q_dim, kv_dim,
                       stride);
}
extern "C" int mx230_copy_kv_seqpos(mx230_handle *h, void *stream, float *kcache, float *vcache,
                                    const float *qkv, const int *pos, int n_seq, int q_dim,
                                    int kv_dim, int qkv_stride, const int *tables, int block_size,
                                    int n_log) {
    MX_REQUIRE(pos && tables && block_size > 0, MX230_ERR_INVALID_ARG, "copy_kv_seqpos: bad table");
    return launch_copy(h, stream, kcache, vcache, qkv, seq_pos(pos, tables, block_size, n_log), n_seq,
                       q_dim, kv_dim, qkv_stride);
}

// ---- int8 quantize-on-write ----
extern "C" int mx230_quantize_kv(mx230_handle *h, void *stream, int8_t *kq, int8_t *vq, float *ks,
                                 float *vs, float *kb, float *vb, const float *qkv, int pos,
                                 int q_dim, int n_kv_head, int head_dim) {
    return launch_quant(h, stream, kq, vq, ks, vs, kb, vb, qkv, host_pos(pos), 1, q_dim, n_kv_head,
                        head_dim, 0);
}
extern "C" int mx230_quantize_kv_dyn(mx230_handle *h, void *stream, int8_t *kq, int8_t *vq,
                                     float *ks, float *vs, float *kb, float *vb, const float *qkv,
                                     const int *pos_ptr, int q_dim, int n_kv_head, int head_dim) {
    MX_REQUIRE(pos_ptr, MX230_ERR_INVALID_ARG, "quantize_kv_dyn: null pos_ptr");
    return launch_quant(h, stream, kq, vq, ks, vs, kb, vb, qkv, dev_pos(pos_ptr), 1, q_dim,
                        n_kv_head, head_dim, 0);
}
extern "C" int mx230_quantize_kv_paged_dyn(mx230_handle *h, void *stream, int8_t *kq, int8_t *vq,
                                           float *ks, float *vs, float *kb, float *vb,
                                           const float *qkv, const int *pos_ptr, int q_dim,
                                           int n_kv_head, int head_dim, const int *bt, int bs) {
    MX_REQUIRE(pos_ptr && bt && bs > 0, MX230_ERR_INVALID_ARG, "quantize_kv_paged_dyn: bad table");
    return launch_quant(h, stream, kq, vq, ks, vs, kb, vb, qkv, dev_pos(pos_ptr, bt, bs), 1, q_dim,
                        n_kv_head, head_dim, 0);
}
extern "C" int mx230_quantize_kv_batch(mx230_handle *h, void *stream, int8_t *kq, int8_t *vq,
                                       float *ks, float *vs, float *kb, float *vb,
                                       const float *qkv, int pos0, int n_tok, int q_dim,
                                       int n_kv_head, int head_dim, int stride) {
    return launch_quant(h, stream, kq, vq, ks, vs, kb, vb, qkv, host_pos(pos0), n_tok, q_dim,
                        n_kv_head, head_dim, stride);
}
extern "C" int mx230_quantize_kv_batch_paged(mx230_handle *h, void *stream, int8_t *kq, int8_t *vq,
                                             float *ks, float *vs, float *kb, float *vb,
                                             const float *qkv, int pos0, int n_tok, int q_dim,
                                             int n_kv_head, int head_dim, int stride,
                                             const int *bt, int bs) {
    MX_REQUIRE(bt && bs > 0, MX230_ERR_INVALID_ARG, "quantize_kv_batch_paged: bad table");
    return launch_quant(h, stream, kq, vq, ks, vs, kb, vb, qkv, host_pos(pos0, bt, bs), n_tok, q_dim,
                        n_kv_head, head_dim, stride);
}
extern "C" int mx230_quantize_kv_seqpos(mx230_handle *h, void *stream, int8_t *kq, int8_t *vq,
                                        float *ks, float *vs, float *kb, float *vb,
                                        const float *qkv, const int *pos, int n_seq, int q_dim,
                                        int n_kv_head, int head_dim, int qkv_stride,
                                        const int *tables, int block_size, int n_log) {
    MX_REQUIRE(pos && tables && block_size > 0, MX230_ERR_INVALID_ARG,
               "quantize_kv_seqpos: bad table");
    return launch_quant(h, stream, kq, vq, ks, vs, kb, vb, qkv,
                        seq_pos(pos, tables, block_size, n_log), n_seq, q_dim, n_kv_head, head_dim,
                        qkv_stride);
}
