/*
 * mx230_attn.h -- C ABI of the B200 (sm_100a) attention library.
 *
 * Drop-in boundary for the attention path of glaucomaa/mx230.  The reference has
 * no FFI layer: its Rust host looks CUDA kernels up by C symbol name in embedded
 * PTX and launches them with cudarc.  Each entry point below therefore replaces
 * one reference kernel symbol (plus its Rust launch wrapper) and keeps that
 * kernel's argument list, in order, after two leading arguments:
 *
 *     handle  per-device library state (workspace, status words); replaces the
 *             CudaFunction handle tables (02-flash-attention/src/main.rs:24-28,
 *             92-98, 392-415; 03-llm-engine/src/gpu.rs:982-1098)
 *     stream  the caller's CUstream / cudaStream_t, as void*; replaces
 *             `stream.launch_builder(..)` (02-flash-attention/src/main.rs:47-64)
 *
 * Conventions
 *  - every pointer argument is a DEVICE pointer unless named `*_host`;
 *  - all work is enqueued on `stream`; no entry point synchronises, allocates or
 *    frees on the launch path (mx230_create / mx230_reserve / mx230_destroy /
 *    mx230_check_status are the only calls that do), so the decode step stays
 *    capturable in a CUDA graph as in 03-llm-engine/src/gpu.rs:4024-4054;
 *  - the caller owns every buffer it passes; head_dim must be 64;
 *  - return value: MX230_OK or an MX230_ERR_* code; mx230_last_error() returns a
 *    message for the calling thread.  The reference panics on a failed launch
 *    (02-flash-attention/src/main.rs:50,87); a binding should `.expect()` the code.
 *  - one handle is used by one host thread at a time; one handle per device.
 */
#ifndef MX230_ATTN_H
#define MX230_ATTN_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MX230_ABI_VERSION 1

enum {
    MX230_OK = 0,
    MX230_ERR_INVALID_ARG = 1,   /* null pointer, negative size, misalignment */
    MX230_ERR_UNSUPPORTED = 2,   /* e.g. head_dim != 64, n_head % n_kv_head != 0 */
    MX230_ERR_WORKSPACE = 3,     /* workspace too small: call mx230_reserve first */
    MX230_ERR_CUDA = 4,          /* a CUDA runtime/driver call failed */
    MX230_ERR_DEVICE_STATUS = 5, /* a kernel reported a bounded-wait timeout */
    MX230_ERR_NO_DEVICE = 6      /* no usable sm_100 device */
};

/* int8 KV score arithmetic of the decode/prefill kernels over an int8 cache */
enum {
    MX230_Q8_SCORE_REF = 0,  /* q quantised per head to int8 and integer dots, exactly the
                                reference kernel's arithmetic (llm.cu:1349-1386) */
    MX230_Q8_SCORE_EXACT = 1 /* fp32 q against dequantised K (scale*code + beta) */
};

enum {
    MX230_OPT_Q8_SCORE_MODE = 1, /* MX230_Q8_SCORE_* (default REF) */
    MX230_OPT_DECODE_CHUNK = 2,  /* keys per decode CTA; 0 = automatic */
    MX230_OPT_DECODE_TENSOR = 3, /* int8 decode in the reference score mode: 1 (default) = the GQA group's two
                                    contractions on warp-level tensor-core tiles, 0 = CUDA cores only */
    MX230_OPT_BWD_TWO_PASS = 4,  /* mx230_attn_bwd_flash*: 0 (default) = one fused pass, dK/dV written once and dQ
                                    summed with fp32 reductions (order of the partial sums not fixed);
                                    1 = the reference's atomic-free split, a dQ pass and a dK/dV pass,
                                    bit-reproducible */
    MX230_OPT_BWD_REUSE_STAGED = 5, /* mx230_attn_bwd_{dq,dkv,flash}: 1 = when the workspace still holds the bf16 copies
                                    of Q, K, V that mx230_attn_flash[_lse] staged for the SAME pointers and shape
                                    (no other workspace-using call in between, same stream, tensor contents
                                    unchanged -- the caller's promise), stage only dO; and when
                                    mx230_attn_bwd_preprocess ran in between for the SAME dO pointer (contents
                                    unchanged since), it has left dO's bf16 copy there as well and nothing is
                                    staged.  0 (default) = always stage all four */
    MX230_OPT_WAIT_LIMIT = 6,    /* bound of every device-side barrier wait, in thousands of SM cycles (default
                                    4000000 = 4e9 cycles, about 2 s); on expiry the kernel records a status and
                                    returns (mx230_check_status -> MX230_ERR_DEVICE_STATUS).  Synchronises the device */
    MX230_OPT_TEST_DROP_TILE = 7 /* test hook, default -1 = off: while set, the TMA producer of CTA 0 of a flash forward /
                                    fused backward launch never requests its value-th streamed tile, so that the
                                    bounded wait of its consumer runs out and the abort path executes */
};

/* kernel ids of the profiling interface */
enum {
    MX230_K_CAST = 0,
    MX230_K_FLASH_FWD = 1,
    MX230_K_BWD_PREPROCESS = 2,
    MX230_K_BWD_DQ = 3,
    MX230_K_BWD_DKV = 4,
    MX230_K_ROPE = 5,
    MX230_K_COPY_KV = 6,
    MX230_K_QUANTIZE_KV = 7,
    MX230_K_DECODE_F32 = 8,
    MX230_K_DECODE_Q8 = 9,
    MX230_K_MERGE = 10,
    MX230_K_PREFILL = 11,
    MX230_K_GEMV = 12,
    MX230_K_BWD_FUSED = 13,
    MX230_K_COUNT = 14
};

typedef struct mx230_handle mx230_handle;

/* ---- library / handle ------------------------------------------------------ */
int mx230_abi_version(void);
const char *mx230_last_error(void);
const char *mx230_status_string(int code);

/* Creates the per-device state and a workspace of `workspace_bytes` on `device`.
 * Replaces CudaContext::new + load_ptx (common/src/lib.rs:11-18). */
int mx230_create(mx230_handle **out, int device, size_t workspace_bytes);
int mx230_destroy(mx230_handle *h);
/* Grows the workspace to at least `bytes` (synchronises the device; not for the launch path). */
int mx230_reserve(mx230_handle *h, size_t bytes);
int mx230_set_option(mx230_handle *h, int option, int value);
/* Workspace needed by the fp32-in/fp32-out flash entry points (bf16 operand staging). */
size_t mx230_flash_workspace_bytes(int batch_heads, int n, int with_backward);
/* Workspace needed by decode (split-KV partial triples). */
size_t mx230_decode_workspace_bytes(int n_seq, int n_head, int max_splits);
/* Synchronises `stream`, reads and clears the device status words. */
int mx230_check_status(mx230_handle *h, void *stream);
/* Number of kernels launched through this handle so far. */
long long mx230_launch_count(const mx230_handle *h);

/* Seeded host-side input generators (no CUDA call; `out_host` is host memory).
 * mx230_pseudo_rand: pseudo_rand of common/src/lib.rs:67-78 -- xorshift64* from `seed`, uniform in [-1, 1).
 * mx230_fill_normal: N(0,1) values for benchmark and test inputs (the reference has no normal generator): the same
 * xorshift64* stream, started at splitmix64(seed * 16 + tensor_index) (0 is a fixed point of xorshift, so a seed
 * cannot be the state itself), through a Box-Muller transform in double precision, rounded to float. */
int mx230_pseudo_rand(float *out_host, size_t n, uint64_t seed);
int mx230_fill_normal(float *out_host, size_t n, uint64_t seed, uint64_t tensor_index);

/* Per-kernel device timing (the role of the reference's opt-in prof_attn_us attribution,
 * 03-llm-engine/src/gpu.rs:1922-1928): while enabled, every launch is bracketed by a CUDA
 * event pair on the caller's stream.  mx230_profile_read synchronises the recorded events
 * and returns, for kernel id `kernel` (MX230_K_*), the launch count and the summed device
 * milliseconds since the last mx230_profile_reset. */
int mx230_profile_enable(mx230_handle *h, int on);
int mx230_profile_reset(mx230_handle *h);
int mx230_profile_read(mx230_handle *h, int kernel, long long *launches, double *total_ms);
const char *mx230_kernel_name(int kernel);

/* ---- 02-flash-attention ----------------------------------------------------
 * Tensors are `batch_heads` independent heads laid out [batch_heads][n][64] fp32,
 * contiguous; batch_heads = 1 is exactly the reference call.  Scale = 1/sqrt(64).
 * Operands are rounded to bf16, products accumulate in fp32 on the tensor cores. */

/* attn_flash(Q,K,V,O,N,causal): 02-flash-attention/kernels/attention_flash.cu:91-94,
 * run_flash 02-flash-attention/src/main.rs:68-88 */
int mx230_attn_flash(mx230_handle *h, void *stream, const float *Q, const float *K,
                     const float *V, float *O, int batch_heads, int n, int causal);
/* attn_flash_lse(Q,K,V,O,L,N,causal): attention_flash.cu:97-100, run_flash_lse
 * main.rs:102-123.  L[i] = m_i + ln(l_i) (natural log of the scaled scores). */
int mx230_attn_flash_lse(mx230_handle *h, void *stream, const float *Q, const float *K,
                         const float *V, float *O, float *L, int batch_heads, int n, int causal);
/* attn_bwd_preprocess(dO,O,Delta,N): attention_bwd.cu:32-44, run_preprocess main.rs:126-143 */
int mx230_attn_bwd_preprocess(mx230_handle *h, void *stream, const float *dO, const float *O,
                              float *Delta, int batch_heads, int n);
/* attn_bwd_dq(Q,K,V,dO,L,Delta,dQ,N,causal): attention_bwd.cu:96-158 */
int mx230_attn_bwd_dq(mx230_handle *h, void *stream, const float *Q, const float *K,
                      const float *V, const float *dO, const float *L, const float *Delta,
                      float *dQ, int batch_heads, int n, int causal);
/* attn_bwd_dkv(Q,K,V,dO,L,Delta,dK,dV,N,causal): attention_bwd.cu:165-243 */
int mx230_attn_bwd_dkv(mx230_handle *h, void *stream, const float *Q, const float *K,
                       const float *V, const float *dO, const float *L, const float *Delta,
                       float *dK, float *dV, int batch_heads, int n, int causal);
/* run_bwd_flash (main.rs:179-210): the dQ pass then the dK/dV pass, one operand staging. */
int mx230_attn_bwd_flash(mx230_handle *h, void *stream, const float *Q, const float *K,
                         const float *V, const float *dO, const float *L, const float *Delta,
                         float *dQ, float *dK, float *dV, int batch_heads, int n, int causal);

/* bf16-resident forms (no counterpart in the reference, whose tensors are fp32):
 * operands already rounded to bf16 [batch_heads][n][64]; outputs stay fp32. */
int mx230_cast_bf16(mx230_handle *h, void *stream, const float *src, void *dst_bf16, size_t count);
int mx230_attn_flash_bf16(mx230_handle *h, void *stream, const void *Qb, const void *Kb,
                          const void *Vb, float *O, float *L_or_null, int batch_heads, int n,
                          int causal);
int mx230_attn_bwd_flash_bf16(mx230_handle *h, void *stream, const void *Qb, const void *Kb,
                              const void *Vb, const void *dOb, const float *L, const float *Delta,
                              float *dQ, float *dK, float *dV, int batch_heads, int n, int causal);

/* ---- 03-llm-engine: per-layer attention step (RoPE -> KV write -> attention) --
 * qkv row layout: [n_head*64 Q | n_kv_head*64 K | n_kv_head*64 V] fp32
 * (03-llm-engine/src/model.rs:95-103).  Cache layouts as the reference:
 * fp32  k,v   [slot][n_kv_head*64]
 * int8  kq,vq [slot][n_kv_head*64] codes; ks,vs,kb,vb [slot][n_kv_head] fp32
 * (03-llm-engine/src/gpu.rs:188-205).  kb == vb == NULL selects the symmetric
 * absmax/127 format (scale only) instead of the reference's affine (scale, beta).
 * Paged variants translate position t to row bt[t/bs]*bs + t%bs (llm.cu:959-963). */

/* rope / rope_dyn / rope_batch / rope_seqpos: llm.cu:1072-1117,1513-1530 */
int mx230_rope(mx230_handle *h, void *stream, float *qkv, int pos, int n_head, int n_kv_head,
               int head_dim, float theta);
int mx230_rope_dyn(mx230_handle *h, void *stream, float *qkv, const int *pos_ptr, int n_head,
                   int n_kv_head, int head_dim, float theta);
int mx230_rope_batch(mx230_handle *h, void *stream, float *qkv, int pos0, int n_tok, int n_head,
                     int n_kv_head, int head_dim, int stride, float theta);
int mx230_rope_seqpos(mx230_handle *h, void *stream, float *qkv, const int *pos, int n_seq,
                      int n_head, int n_kv_head, int head_dim, int stride, float theta);

/* fp32 KV write: copy_kv_dyn / copy_kv_paged_dyn (llm.cu:965-986), copy_kv_batch /
 * copy_kv_batch_paged (llm.cu:3635-3655), copy_kv_seqpos (llm.cu:1491-1501);
 * mx230_copy_kv replaces the two memcpy_dtod of 03-llm-engine/src/gpu.rs:2594-2605. */
int mx230_copy_kv(mx230_handle *h, void *stream, float *kcache, float *vcache, const float *qkv,
                  int pos, int q_dim, int kv_dim);
int mx230_copy_kv_dyn(mx230_handle *h, void *stream, float *kcache, float *vcache,
                      const float *qkv, const int *pos_ptr, int q_dim, int kv_dim);
int mx230_copy_kv_paged_dyn(mx230_handle *h, void *stream, float *kcache, float *vcache,
                            const float *qkv, const int *pos_ptr, int q_dim, int kv_dim,
                            const int *bt, int bs);
int mx230_copy_kv_batch(mx230_handle *h, void *stream, float *kcache, float *vcache,
                        const float *qkv, int pos0, int n_tok, int q_dim, int kv_dim, int stride);
int mx230_copy_kv_batch_paged(mx230_handle *h, void *stream, float *kcache, float *vcache,
                              const float *qkv, int pos0, int n_tok, int q_dim, int kv_dim,
                              int stride, const int *bt, int bs);
int mx230_copy_kv_seqpos(mx230_handle *h, void *stream, float *kcache, float *vcache,
                         const float *qkv, const int *pos, int n_seq, int q_dim, int kv_dim,
                         int qkv_stride, const int *tables, int block_size, int n_log);

/* int8 quantize-on-write, bit-exact with quant_affine (llm.cu:1137-1149):
 * quantize_kv / _dyn / _paged_dyn (llm.cu:1176-1203), _batch / _batch_paged
 * (llm.cu:1205-1240), _seqpos (llm.cu:1503-1510).  n_tok / n_seq are the grid.y
 * of the reference launches (gpu.rs:3292-3296,3585-3589). */
int mx230_quantize_kv(mx230_handle *h, void *stream, int8_t *kq, int8_t *vq, float *ks, float *vs,
                      float *kb, float *vb, const float *qkv, int pos, int q_dim, int n_kv_head,
                      int head_dim);
int mx230_quantize_kv_dyn(mx230_handle *h, void *stream, int8_t *kq, int8_t *vq, float *ks,
                          float *vs, float *kb, float *vb, const float *qkv, const int *pos_ptr,
                          int q_dim, int n_kv_head, int head_dim);
int mx230_quantize_kv_paged_dyn(mx230_handle *h, void *stream, int8_t *kq, int8_t *vq, float *ks,
                                float *vs, float *kb, float *vb, const float *qkv,
                                const int *pos_ptr, int q_dim, int n_kv_head, int head_dim,
                                const int *bt, int bs);
int mx230_quantize_kv_batch(mx230_handle *h, void *stream, int8_t *kq, int8_t *vq, float *ks,
                            float *vs, float *kb, float *vb, const float *qkv, int pos0, int n_tok,
                            int q_dim, int n_kv_head, int head_dim, int stride);
int mx230_quantize_kv_batch_paged(mx230_handle *h, void *stream, int8_t *kq, int8_t *vq, float *ks,
                                  float *vs, float *kb, float *vb, const float *qkv, int pos0,
                                  int n_tok, int q_dim, int n_kv_head, int head_dim, int stride,
                                  const int *bt, int bs);
int mx230_quantize_kv_seqpos(mx230_handle *h, void *stream, int8_t *kq, int8_t *vq, float *ks,
                             float *vs, float *kb, float *vb, const float *qkv, const int *pos,
                             int n_seq, int q_dim, int n_kv_head, int head_dim, int qkv_stride,
                             const int *tables, int block_size, int n_log);

/* decode attention over an fp32 cache, keys 0..=t_cur: attn_decode / _dyn / _paged /
 * _paged_dyn (llm.cu:1296-1325), attn_decode_batched (llm.cu:1468-1476).
 * Unlike the reference (shared s[2048], llm.cu:1251) the context is unbounded. */
int mx230_attn_decode(mx230_handle *h, void *stream, float *out, const float *qkv,
                      const float *kcache, const float *vcache, int t_cur, int n_head,
                      int n_kv_head, int head_dim);
int mx230_attn_decode_dyn(mx230_handle *h, void *stream, float *out, const float *qkv,
                          const float *kcache, const float *vcache, const int *pos_ptr,
                          int n_head, int n_kv_head, int head_dim);
int mx230_attn_decode_paged(mx230_handle *h, void *stream, float *out, const float *qkv,
                            const float *kcache, const float *vcache, int t_cur, int n_head,
                            int n_kv_head, int head_dim, const int *bt, int bs);
int mx230_attn_decode_paged_dyn(mx230_handle *h, void *stream, float *out, const float *qkv,
                                const float *kcache, const float *vcache, const int *pos_ptr,
                                int n_head, int n_kv_head, int head_dim, const int *bt, int bs);
int mx230_attn_decode_batched(mx230_handle *h, void *stream, float *out, const float *qkv,
                              const float *kcache, const float *vcache, const int *pos, int n_seq,
                              int n_head, int n_kv_head, int head_dim, const int *tables,
                              int block_size, int n_log, int qkv_stride, int out_stride);

/* the same over an int8 cache: attn_decode_q8 / _dyn / _paged / _paged_dyn
 * (llm.cu:1420-1458), attn_decode_q8_batched (llm.cu:1478-1487) */
int mx230_attn_decode_q8(mx230_handle *h, void *stream, float *out, const float *qkv,
                         const int8_t *kq, const int8_t *vq, const float *ks, const float *vs,
                         const float *kb, const float *vb, int t_cur, int n_head, int n_kv_head,
                         int head_dim);
int mx230_attn_decode_q8_dyn(mx230_handle *h, void *stream, float *out, const float *qkv,
                             const int8_t *kq, const int8_t *vq, const float *ks, const float *vs,
                             const float *kb, const float *vb, const int *pos_ptr, int n_head,
                             int n_kv_head, int head_dim);
int mx230_attn_decode_q8_paged(mx230_handle *h, void *stream, float *out, const float *qkv,
                               const int8_t *kq, const int8_t *vq, const float *ks,
                               const float *vs, const float *kb, const float *vb, int t_cur,
                               int n_head, int n_kv_head, int head_dim, const int *bt, int bs);
int mx230_attn_decode_q8_paged_dyn(mx230_handle *h, void *stream, float *out, const float *qkv,
                                   const int8_t *kq, const int8_t *vq, const float *ks,
                                   const float *vs, const float *kb, const float *vb,
                                   const int *pos_ptr, int n_head, int n_kv_head, int head_dim,
                                   const int *bt, int bs);
int mx230_attn_decode_q8_batched(mx230_handle *h, void *stream, float *out, const float *qkv,
                                 const int8_t *kq, const int8_t *vq, const float *ks,
                                 const float *vs, const float *kb, const float *vb, const int *pos,
                                 int n_seq, int n_head, int n_kv_head, int head_dim,
                                 const int *tables, int block_size, int n_log, int qkv_stride,
                                 int out_stride);

/* Decode over an int8 cache without a handle and without any allocation (no counterpart in
 * the reference, whose kernels use no scratch memory at all).  For hosts that cannot call
 * cudaMalloc when they need attention -- all free HBM already given to their KV pool, or only
 * allowed to enqueue on a stream they were handed -- the split-KV scratch lives in a fixed
 * 1 MiB + 4 KiB __device__ array inside the library image (resident per GPU until exit).
 * Single sequence, contiguous cache, keys 0..=t_cur, reference score mode, current device.
 * It runs the CUDA-core decode kernel, not the tensor-core one that mx230_attn_decode_q8 defaults to:
 * the same result to rounding, at a fraction of the bandwidth for GQA groups.
 * Shapes needing more than n_head * n_splits * 264 B <= 1 MiB are refused (MX230_ERR_WORKSPACE).
 * The first call on a device resolves the array's address (serialised against other host threads'
 * first calls): make it before any stream capture.
 * Calls share the array; calls that overlap on the GPU race on it. */
int mx230_attn_decode_q8_noalloc(void *stream, float *out, const float *qkv, const int8_t *kq,
                                 const int8_t *vq, const float *ks, const float *vs, const float *kb,
                                 const float *vb, int t_cur, int n_head, int n_kv_head, int head_dim);

/* Batched decode over per-sequence contiguous cache slabs (no counterpart in the
 * reference, which batches only through block tables): sequence s reads cache
 * rows [s*seq_rows, s*seq_rows + pos[s]].  fp32 cache when kq == NULL. */
int mx230_attn_decode_slab(mx230_handle *h, void *stream, float *out, const float *qkv,
                           const float *kcache, const float *vcache, const int8_t *kq,
                           const int8_t *vq, const float *ks, const float *vs, const float *kb,
                           const float *vb, const int *pos, int n_seq, int n_head, int n_kv_head,
                           int head_dim, long long seq_rows, int qkv_stride, int out_stride);

/* Split-KV decode across GPUs (no counterpart in the reference, which is single
 * device): each rank attends its own key range [t0, t1) of every sequence slab
 * and emits the unnormalised triple per (sequence, query head):
 *   part_m [n_seq][n_head], part_l [n_seq][n_head], part_acc [n_seq][n_head][64]
 * with acc = sum_j exp(s_j - m) v_j.  After an all-gather of the triples,
 * mx230_merge_partials combines `parts` of them by log-sum-exp:
 *   m = max m_r, l = sum l_r e^(m_r-m), out = sum acc_r e^(m_r-m) / l.
 * Gathered layout: m,l [parts][rows]; acc [parts][rows][64]; out [rows][64]. */
int mx230_attn_decode_partial(mx230_handle *h, void *stream, float *part_m, float *part_l,
                              float *part_acc, const float *qkv, const float *kcache,
                              const float *vcache, const int8_t *kq, const int8_t *vq,
                              const float *ks, const float *vs, const float *kb, const float *vb,
                              int t0, int t1, int n_seq, int n_head, int n_kv_head, int head_dim,
                              long long seq_rows, int qkv_stride);
int mx230_merge_partials(mx230_handle *h, void *stream, float *out, const float *m,
                         const float *l, const float *acc, int parts, int rows, int head_dim);
/* the same merge straight from the all-gathered buffer [parts][m[rows] | l[rows] | acc[rows][64]]
 * (rows even, so that every part's accumulators stay 16-byte aligned) */
int mx230_merge_partials_packed(mx230_handle *h, void *stream, float *out, const float *gathered,
                                int parts, int rows, int head_dim);

/* Split-KV exchange and merge in ONE kernel over peer memory (no reference counterpart: the reference
 * runs on one device).  Each rank (one process, one GPU) creates a communicator for `rows` =
 * n_seq * n_head rows; the library allocates an exchange region with cudaMalloc and exports it as a
 * 64-byte CUDA IPC handle, which the host passes to the other ranks by its own transport
 * (`_export` on the owner, `_import` on every other rank; `_attach` instead of `_import` for a region
 * whose device address is already valid in this process).  After mx230_attn_decode_partial has
 * written the rank's packed triples [m | l | acc] to `local`, mx230_splitkv_exchange_merge launches
 * one kernel that stores them into every rank's region over NVLink, publishes a step number, waits
 * (bounded by MX230_OPT_WAIT_LIMIT; expiry -> device status, the output is then not written) for the
 * other ranks' step numbers and merges all triples into out[rows][64].  Every rank must call it the
 * same number of times; ranks must not share a GPU (their kernels wait on one another).  Teardown in
 * two phases with a host barrier between them: every rank calls `_disconnect` (synchronises the
 * device, closes its imports), then, once all have, `_destroy` (frees its own region). */
typedef struct mx230_splitkv_comm mx230_splitkv_comm;
int mx230_splitkv_comm_create(mx230_handle *h, int rank, int world, int rows, int head_dim,
                              mx230_splitkv_comm **out);
int mx230_splitkv_comm_export(mx230_splitkv_comm *c, unsigned char *handle64);
int mx230_splitkv_comm_import(mx230_splitkv_comm *c, int peer, const unsigned char *handle64);
int mx230_splitkv_comm_region(mx230_splitkv_comm *c, void **base, size_t *bytes);
int mx230_splitkv_comm_attach(mx230_splitkv_comm *c, int peer, void *region);
int mx230_splitkv_exchange_merge(mx230_splitkv_comm *c, void *stream, float *out, const float *local);
/* The same step with the stores issued by the partial-attention kernel itself: the CTA that finishes a
 * (sequence, KV head) group stores its triples into every rank's region at once (arguments as
 * mx230_attn_decode_partial, n_seq * n_head = the communicator's rows; an empty range t1 <= t0 stores the
 * neutral triple), and mx230_splitkv_wait_merge, on the same stream, waits for all ranks' triples and merges
 * them into out[rows][64].  One _partial_push and one _wait_merge make a step. */
int mx230_attn_decode_partial_push(mx230_handle *h, void *stream, mx230_splitkv_comm *c, const float *qkv,
                                   const float *kcache, const float *vcache, const int8_t *kq,
                                   const int8_t *vq, const float *ks, const float *vs, const float *kb,
                                   const float *vb, int t0, int t1, int n_seq, int n_head, int n_kv_head,
                                   int head_dim, long long seq_rows, int qkv_stride);
int mx230_splitkv_wait_merge(mx230_splitkv_comm *c, void *stream, float *out);
/* The whole step in ONE kernel: the CTA that finishes a (sequence, KV head) group stores the group's triples
 * into every other rank's region, waits (bounded, as above) for their triples of the same rows and writes the
 * merged, normalised rows to out[rows][64].  The three forms of a step (_exchange_merge, _partial_push +
 * _wait_merge, _decode_splitkv) give bit-identical results and may be mixed from step to step, as long as every
 * rank makes one step per step. */
int mx230_attn_decode_splitkv(mx230_handle *h, void *stream, mx230_splitkv_comm *c, float *out,
                              const float *qkv, const float *kcache, const float *vcache, const int8_t *kq,
                              const int8_t *vq, const float *ks, const float *vs, const float *kb,
                              const float *vb, int t0, int t1, int n_seq, int n_head, int n_kv_head,
                              int head_dim, long long seq_rows, int qkv_stride);
int mx230_splitkv_comm_disconnect(mx230_splitkv_comm *c);
void mx230_splitkv_comm_destroy(mx230_splitkv_comm *c);

/* prefill attention of n_tok new rows at absolute positions pos0+qi over cache keys
 * 0..=pos0+qi: attn_prefill / _q8 / _paged / _q8_paged / _dp4a / _dp4a_paged
 * (llm.cu:3806-3872).  q row qi of head h is read at qkv[qi*qkv_stride + h*64], the result
 * goes to out[qi*out_stride + h*64]; K and V come only from the cache, which must already
 * hold positions pos0..pos0+n_tok-1 (the reference writes them first, gpu.rs:3243-3320).
 * Operands are rounded to bf16 for the tensor cores.  Over an int8 cache MX230_OPT_Q8_SCORE_MODE selects the score
 * arithmetic as for decode: REF (default) quantises q per (row, head) to int8 and rebuilds the score from the exact
 * integer dot as attn_prefill_q8 does (llm.cu:3700-3716,3774-3782; the codes pass through the tensor cores exactly);
 * EXACT scores with fp32 q on the dequantised K.  The _dp4a forms are the reference's opt-in int8-score
 * approximation over an fp32 cache: every K row quantised on the fly, symmetric absmax (llm.cu:3737-3754). */
size_t mx230_prefill_workspace_bytes(int n_tok, int n_keys, int n_head, int n_kv_head);
int mx230_attn_prefill(mx230_handle *h, void *stream, float *out, const float *qkv,
                       const float *kcache, const float *vcache, int pos0, int n_tok, int n_head,
                       int n_kv_head, int qkv_stride, int out_stride);
int mx230_attn_prefill_paged(mx230_handle *h, void *stream, float *out, const float *qkv,
                             const float *kcache, const float *vcache, int pos0, int n_tok,
                             int n_head, int n_kv_head, int qkv_stride, int out_stride,
                             const int *bt, int bs);
int mx230_attn_prefill_q8(mx230_handle *h, void *stream, float *out, const float *qkv,
                          const int8_t *kq, const int8_t *vq, const float *ks, const float *vs,
                          const float *kb, const float *vb, int pos0, int n_tok, int n_head,
                          int n_kv_head, int qkv_stride, int out_stride);
int mx230_attn_prefill_q8_paged(mx230_handle *h, void *stream, float *out, const float *qkv,
                                const int8_t *kq, const int8_t *vq, const float *ks,
                                const float *vs, const float *kb, const float *vb, int pos0,
                                int n_tok, int n_head, int n_kv_head, int qkv_stride,
                                int out_stride, const int *bt, int bs);
int mx230_attn_prefill_dp4a(mx230_handle *h, void *stream, float *out, const float *qkv,
                            const float *kcache, const float *vcache, int pos0, int n_tok, int n_head,
                            int n_kv_head, int qkv_stride, int out_stride);
int mx230_attn_prefill_dp4a_paged(mx230_handle *h, void *stream, float *out, const float *qkv,
                                  const float *kcache, const float *vcache, int pos0, int n_tok,
                                  int n_head, int n_kv_head, int qkv_stride, int out_stride,
                                  const int *bt, int bs);

/* ---- the projections either side of the attention step (one decode token) --------------------
 * gemv / gemv_half, 03-llm-engine/kernels/llm.cu:144-177 (host gemv(), src/gpu.rs:1158-1198):
 * y[o] (+)= sum_i x[i] w[i*n_out + o] + b[o], w row-major [n_in][n_out] in fp32 (w_fp16 = 0) or
 * fp16 (1), b may be null, accum != 0 adds into y (the residual add fused into the output
 * projection, gpu.rs:2676-2686).  n_out a multiple of 4; uses the handle's workspace
 * (n_slices * n_out floats, at most ceil(n_in / 16) slices). */
int mx230_gemv(mx230_handle *h, void *stream, float *y, const float *x, const void *w, int w_fp16,
               const float *b, int n_in, int n_out, int accum);
/* The same projections for a batch of rows (prefill): gemm(), src/gpu.rs:1291-1420, called for qkv at
 * gpu.rs:3187-3198 and for the output projection at gpu.rs:3354-3365 (kernels gemm_f32* / gemm_half*,
 * llm.cu:1632-1733): C[r][o] = sum_i A[r][i] w[i*n + o] + bias[o], A [m][k] and C [m][n] fp32 contiguous,
 * w [k][n] fp32 (w_fp16 = 0) or fp16 (1), bias may be null.  Any m; k % 16 == 0 (as the reference asserts),
 * n % 8 == 0.  Tensor cores with 16-bit operands and fp32 accumulation: fp16 weights are used as they lie, A is
 * rounded to fp16; fp32 weights and A are each split into two bf16 terms (16 bits of mantissa) and three
 * products are summed.  Workspace: mx230_gemm_workspace_bytes.  Int8 / int4 weight formats: not built. */
size_t mx230_gemm_workspace_bytes(int m, int n, int k, int w_fp16);
int mx230_gemm(mx230_handle *h, void *stream, float *C, const float *A, const void *w, int w_fp16,
               const float *bias, int m, int n, int k);
/* gemv_int8, llm.cu:226-316 (host gemv() Weights::Int8, gpu.rs:1200-1211): int8 weights packed as int32
 * words of four consecutive input rows, w_packed[(i/4)*n_out + o]; activations quantised inside the
 * kernel per group of act_group (4 or 8: the reference's compile-time AG) values, absmax/127, round to
 * nearest even; integer dots by dp4a; y[o] (+)= (sum_g dot_g * xs_g) * scales[o] + b[o].  n_in % 8 == 0. */
int mx230_gemv_int8(mx230_handle *h, void *stream, float *y, const float *x, const void *w_packed,
                    const float *scales, const float *b, int n_in, int n_out, int accum, int act_group);
/* The qkv step in one launch: qkv = x W + b (W [n_in][(n_head + 2 n_kv_head) * 64]; w_kind 0 fp32, 1 fp16,
 * 2 int8 packed with w_scales and act_group as for mx230_gemv_int8), RoPE at `pos` (or *pos_ptr when
 * non-null: the graph-captured decode) on the Q and K heads, K and V rows written to cache row pos
 * (through bt/bs when paged) as fp32 (kcache, vcache) or int8 quantize-on-write (kq .. vb; kb == vb == NULL
 * selects absmax), the rotated q left in qkv for mx230_attn_decode*.  Replaces gemv + rope[_dyn] +
 * memcpy / copy_kv_* / quantize_kv_* of gpu.rs:2558-2646, :2808-2893. */
int mx230_qkv_rope_kvwrite(mx230_handle *h, void *stream, float *qkv, const float *x, const void *w,
                           int w_kind, const float *w_scales, int act_group, const float *b, int n_in,
                           int pos, const int *pos_ptr, int n_head, int n_kv_head, int head_dim,
                           float theta, float *kcache, float *vcache, int8_t *kq, int8_t *vq, float *ks,
                           float *vs, float *kb, float *vb, const int *bt, int bs);

/* ---- host side of paged attention: KV block pool with a block-granular prefix tree ----------
 * Paging and RadixCache, 03-llm-engine/src/gpu.rs:211-343,372-539; the request protocol is that
 * of prefill_cached, gpu.rs:2273-2345.  Pure host state (no CUDA call): the table it keeps is what
 * the *_paged entry points above take as `bt`.  prefix_cache = 0 (Paging::new): one sequence owns
 * every block, logical block i -> physical block n_blocks-1-i.  prefix_cache = 1 (Paging::new_pool):
 * blocks start free, are reference-counted per request and by the tree, and a request whose token
 * prefix is resident reuses those blocks; when the free list is empty the least recently used tree
 * leaf that no live request borrows is evicted.  One pool is used by one thread at a time. */
typedef struct mx230_kv_pool mx230_kv_pool;
int mx230_kv_pool_create(mx230_kv_pool **out, int n_slots, int block_size, int prefix_cache);
void mx230_kv_pool_destroy(mx230_kv_pool *p);
int mx230_kv_pool_n_blocks(const mx230_kv_pool *p);
int mx230_kv_pool_block_size(const mx230_kv_pool *p);
int mx230_kv_pool_free_blocks(const mx230_kv_pool *p);
int mx230_kv_pool_cached_blocks(const mx230_kv_pool *p);
long long mx230_kv_pool_evictions(const mx230_kv_pool *p);            /* Engine::pool_evictions, gpu.rs:2259 */
int mx230_kv_pool_refcount(const mx230_kv_pool *p, int block);
int mx230_kv_pool_table(const mx230_kv_pool *p, int *table_out, int n); /* first n logical blocks */
int mx230_kv_pool_phys_row(const mx230_kv_pool *p, int t);             /* Paging::phys_row, gpu.rs:536 */
int mx230_kv_pool_alloc(mx230_kv_pool *p, int *block_out);             /* Paging::alloc, gpu.rs:443 */
int mx230_kv_pool_incref(mx230_kv_pool *p, int block);
int mx230_kv_pool_decref(mx230_kv_pool *p, int block);
int mx230_kv_pool_evict(mx230_kv_pool *p, int *freed_block);           /* Paging::evict; -1 = nothing reclaimable */
int mx230_kv_pool_lookup(mx230_kv_pool *p, const uint32_t *tokens, int n, int *blocks_out, int cap,
                         int *n_matched);                               /* RadixCache::lookup, gpu.rs:254 */
int mx230_kv_pool_insert(mx230_kv_pool *p, const uint32_t *tokens, int n, const int *blocks,
                         int n_blk, int *created_out, int cap, int *n_created); /* RadixCache::insert */
/* prefill_cached steps 1-2 (match, borrow, claim; *reused_tokens = positions already resident) and
 * step 4 (the tree takes over the new full chunks, the request's borrow is released). */
int mx230_kv_pool_begin_request(mx230_kv_pool *p, const uint32_t *tokens, int n, int *reused_tokens);
int mx230_kv_pool_end_request(mx230_kv_pool *p, const uint32_t *tokens, int n);
/* Gives the open request up instead of ending it (its attention step failed to enqueue): the borrow of
 * every table block is released and the tree adopts nothing, so the never-written blocks cannot be matched
 * by a later request.  The reference panics at this point (gpu.rs:2273-2345). */
int mx230_kv_pool_abort_request(mx230_kv_pool *p);
int mx230_kv_pool_audit(const mx230_kv_pool *p);                        /* Paging::audit, gpu.rs:476 */

/* ---- continuous-batching scheduler over batched decode ---------------------------------------
 * The state machine of Engine::run_continuous, 03-llm-engine/src/gpu.rs:3800-3915, without the
 * model: admission (a request reserves ceil((prompt + max_new) / block) blocks for its whole life
 * from the pool, so a running sequence never fails to allocate), the active batch of each decode
 * step (tokens, positions, packed tables = the arguments of the *_batched entry points) and
 * retirement.  Driver loop:
 *   for (;;) {
 *     while (mx230_sched_admit(s, &r, table), r >= 0) { first = prefill(prompt[r], table); mx230_sched_admitted(s, r, first); }
 *     mx230_sched_batch(s, &n, cur, pos, tables); if (n == 0) break;
 *     decode_batched(cur, pos, tables, n) -> next; mx230_sched_step_done(s, next);
 *   }
 * The pool must be a prefix_cache = 1 pool (only its reference-counted allocator is used). */
typedef struct mx230_sched mx230_sched;
int mx230_sched_create(mx230_sched **out, mx230_kv_pool *pool, int n_ctx, int max_batch,
                       const int *prompt_len, const int *max_new, int n_requests);
void mx230_sched_destroy(mx230_sched *s);
int mx230_sched_n_log(const mx230_sched *s);
int mx230_sched_admit(mx230_sched *s, int *request, int *table_out);
int mx230_sched_admitted(mx230_sched *s, int request, uint32_t first_token);
int mx230_sched_batch(mx230_sched *s, int *n_active, uint32_t *cur, int *pos, int *tables);
int mx230_sched_step_done(mx230_sched *s, const uint32_t *next_tokens);
int mx230_sched_result(const mx230_sched *s, int request, uint32_t *out, int cap, int *n);
long long mx230_sched_stat(const mx230_sched *s, int which); /* ServeStats gpu.rs:366: 0 decode_steps, 1 seq_decodes, 2 admitted */

#ifdef __cplusplus
}
#endif
#endif /* MX230_ATTN_H */
