/*
 * CPU oracle for the attention path of glaucomaa/mx230 -- TEST INFRASTRUCTURE ONLY.
 *
 * A plain-C restatement (written fresh, scalar loops, sequential fp32 sums in
 * index order, no fast-math, no FMA contraction) of the reference's own CPU and
 * kernel arithmetic.  It is the checker for the CUDA library and the timed CPU
 * baseline; the product never links or calls it.
 *
 * Parity status: the fp32 attention forward/backward follows the reference's
 * Rust CPU code and is additionally pinned on the GPU box against the
 * reference's own unmodified CUDA kernels (compiled out of tree into
 * oracle/_ref by build_ref() of oracle/build.py).  The int8 KV quantiser has no CPU
 * implementation and no test vector in the reference ("parity unpinned" by
 * reference fixtures); its ground truth is the reference kernel source, and it
 * too is pinned against that kernel run on the GPU box when oracle/_ref exists.
 *
 * Each function cites the reference file:line it follows.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define HD 64 /* head dim of the whole path: 02-flash-attention/src/main.rs:12,
                 03-llm-engine/src/gpu.rs:3148-3151 */

/* ------------------------------------------------------------------ */
/* common/src/lib.rs                                                   */
/* ------------------------------------------------------------------ */

/* xorshift64* uniform in [-1, 1): common/src/lib.rs:67-78 */
void orc_pseudo_rand(float *out, size_t n, uint64_t seed) {
    for (size_t i = 0; i < n; ++i) {
        seed ^= seed >> 12;
        seed ^= seed << 25;
        seed ^= seed >> 27;
        uint64_t r = seed * 0x2545F4914F6CDD1DULL;
        out[i] = (float)(r >> 40) / (float)(1ULL << 23) - 1.0f;
    }
}

/* N(0,1) inputs for the benchmark configurations.  Not in the reference (its
 * tests use the uniform generator above): the same xorshift64* stream feeds a
 * Box-Muller transform in f64.  State 0 is a fixed point of xorshift, so the
 * state is splitmix64(seed * 16 + tensor_index), forced non-zero. */
static uint64_t splitmix64(uint64_t x) {
    x += 0x9E3779B97F4A7C15ULL;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ULL;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBULL;
    return x ^ (x >> 31);
}
static inline double xs_unit(uint64_t *s) { /* (0, 1] */
    *s ^= *s >> 12;
    *s ^= *s << 25;
    *s ^= *s >> 27;
    uint64_t r = *s * 0x2545F4914F6CDD1DULL;
    return ((double)(r >> 11) + 1.0) / 9007199254740992.0;
}
void orc_normal(float *out, size_t n, uint64_t seed, uint64_t tensor_index) {
    uint64_t s = splitmix64(seed * 16u + tensor_index);
    if (s == 0) s = 0x9E3779B97F4A7C15ULL;
    for (size_t i = 0; i < n; i += 2) {
        double u1 = xs_unit(&s), u2 = xs_unit(&s);
        double r = sqrt(-2.0 * log(u1));
        double a = 6.283185307179586476925 * u2;
        out[i] = (float)(r * cos(a));
        if (i + 1 < n) out[i + 1] = (float)(r * sin(a));
    }
}

/* common/src/lib.rs:46-53 */
float orc_max_rel_err(const float *got, const float *want, size_t n) {
    float worst = 0.0f;
    for (size_t i = 0; i < n; ++i) {
        float d = fabsf(want[i]);
        if (d < 1e-6f) d = 1e-6f;
        float e = fabsf(got[i] - want[i]) / d;
        if (e > worst || e != e) worst = e;
    }
    return worst;
}

/* common/src/lib.rs:58-64 */
float orc_allclose_err(const float *got, const float *want, size_t n, float rtol, float atol) {
    float worst = 0.0f;
    for (size_t i = 0; i < n; ++i) {
        float e = fabsf(got[i] - want[i]) / (atol + rtol * fabsf(want[i]));
        if (e > worst || e != e) worst = e;
    }
    return worst;
}

/* ------------------------------------------------------------------ */
/* 02-flash-attention: one head [n][64]                                */
/* ------------------------------------------------------------------ */

/* cpu_attention, 02-flash-attention/src/main.rs:213-241.  lse (may be NULL)
 * is not returned by the reference CPU code; it is m + ln(l) from the same
 * m and l, the definition of the reference kernel
 * (02-flash-attention/kernels/attention_flash.cu:85-87). `s` is n floats. */
static void attn_fwd_head(const float *q, const float *k, const float *v, float *o, float *lse,
                          int n, int causal, float *s) {
    const float scale = 1.0f / sqrtf((float)HD);
    memset(o, 0, (size_t)n * HD * sizeof(float));
    for (int i = 0; i < n; ++i) {
        int cols = causal ? i + 1 : n;
        float m = -INFINITY;
        for (int j = 0; j < cols; ++j) {
            float dot = 0.0f;
            for (int x = 0; x < HD; ++x) dot += q[(size_t)i * HD + x] * k[(size_t)j * HD + x];
            s[j] = dot * scale;
            m = fmaxf(m, s[j]);
        }
        float l = 0.0f;
        for (int j = 0; j < cols; ++j) {
            s[j] = expf(s[j] - m);
            l += s[j];
        }
        for (int j = 0; j < cols; ++j) {
            float p = s[j] / l;
            for (int x = 0; x < HD; ++x) o[(size_t)i * HD + x] += p * v[(size_t)j * HD + x];
        }
        if (lse) lse[i] = m + logf(l);
    }
}

/* cpu_attention_bwd, 02-flash-attention/src/main.rs:246-300.  p, dp: n floats. */
static void attn_bwd_head(const float *q, const float *k, const float *v, const float *dout,
                          float *dq, float *dk, float *dv, int n, int causal, float *p,
                          float *dp) {
    const float scale = 1.0f / sqrtf((float)HD);
    memset(dq, 0, (size_t)n * HD * sizeof(float));
    memset(dk, 0, (size_t)n * HD * sizeof(float));
    memset(dv, 0, (size_t)n * HD * sizeof(float));
    for (int i = 0; i < n; ++i) {
        int cols = causal ? i + 1 : n;
        float m = -INFINITY;
        for (int j = 0; j < cols; ++j) {
            float dot = 0.0f;
            for (int x = 0; x < HD; ++x) dot += q[(size_t)i * HD + x] * k[(size_t)j * HD + x];
            p[j] = dot * scale;
            m = fmaxf(m, p[j]);
        }
        float l = 0.0f;
        for (int j = 0; j < cols; ++j) {
            p[j] = expf(p[j] - m);
            l += p[j];
        }
        for (int j = 0; j < cols; ++j) p[j] /= l;
        float delta = 0.0f;
        for (int j = 0; j < cols; ++j) {
            float d = 0.0f;
            for (int x = 0; x < HD; ++x) d += dout[(size_t)i * HD + x] * v[(size_t)j * HD + x];
            dp[j] = d;
            delta += p[j] * d;
        }
        for (int j = 0; j < cols; ++j) {
            float ds = p[j] * (dp[j] - delta) * scale;
            for (int x = 0; x < HD; ++x) {
                dv[(size_t)j * HD + x] += p[j] * dout[(size_t)i * HD + x];
                dk[(size_t)j * HD + x] += ds * q[(size_t)i * HD + x];
                dq[(size_t)i * HD + x] += ds * k[(size_t)j * HD + x];
            }
        }
    }
}

static int pick_threads(int threads) {
#ifdef _OPENMP
    if (threads <= 0) threads = omp_get_max_threads();
    return threads;
#else
    (void)threads;
    return 1;
#endif
}

int orc_max_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* `heads` independent heads laid out [heads][n][64]; the reference is one head
 * per call, the configurations add the (batch, head) dimension.  Heads run on
 * `threads` OpenMP threads (<=0: all); each head's arithmetic is unchanged. */
void orc_attn_fwd(const float *q, const float *k, const float *v, float *o, float *lse, int heads,
                  int n, int causal, int threads) {
    int nt = pick_threads(threads);
    (void)nt;
#pragma omp parallel num_threads(nt)
    {
        float *s = (float *)malloc((size_t)(n > 0 ? n : 1) * sizeof(float));
#pragma omp for schedule(dynamic, 1)
        for (int h = 0; h < heads; ++h) {
            size_t off = (size_t)h * n * HD;
            attn_fwd_head(q + off, k + off, v + off, o + off, lse ? lse + (size_t)h * n : NULL, n,
                          causal, s);
        }
        free(s);
    }
}

void orc_attn_bwd(const float *q, const float *k, const float *v, const float *dout, float *dq,
                  float *dk, float *dv, int heads, int n, int causal, int threads) {
    int nt = pick_threads(threads);
    (void)nt;
#pragma omp parallel num_threads(nt)
    {
        float *p = (float *)malloc((size_t)(n > 0 ? n : 1) * sizeof(float));
        float *dp = (float *)malloc((size_t)(n > 0 ? n : 1) * sizeof(float));
#pragma omp for schedule(dynamic, 1)
        for (int h = 0; h < heads; ++h) {
            size_t off = (size_t)h * n * HD;
            attn_bwd_head(q + off, k + off, v + off, dout + off, dq + off, dk + off, dv + off, n,
                          causal, p, dp);
        }
        free(p);
        free(dp);
    }
}

/* Row-sampled forward for the bounded CPU-baseline timing of very long
 * sequences: computes only query rows row0, row0+stride, ... of each head with
 * exactly the per-row arithmetic of attn_fwd_head.  Returns rows done per head. */
int orc_attn_fwd_rows(const float *q, const float *k, const float *v, float *o, int heads, int n,
                      int causal, int row0, int stride, int threads) {
    int nt = pick_threads(threads);
    (void)nt;
    int rows = 0;
    for (int i = row0; i < n; i += stride) ++rows;
    const float scale = 1.0f / sqrtf((float)HD);
#pragma omp parallel num_threads(nt)
    {
        float *s = (float *)malloc((size_t)(n > 0 ? n : 1) * sizeof(float));
#pragma omp for schedule(dynamic, 1) collapse(2)
        for (int h = 0; h < heads; ++h) {
            for (int r = 0; r < rows; ++r) {
                int i = row0 + r * stride;
                const float *qh = q + (size_t)h * n * HD, *kh = k + (size_t)h * n * HD,
                            *vh = v + (size_t)h * n * HD;
                float *oh = o + ((size_t)h * rows + r) * HD;
                int cols = causal ? i + 1 : n;
                float m = -INFINITY;
                for (int j = 0; j < cols; ++j) {
                    float dot = 0.0f;
                    for (int x = 0; x < HD; ++x) dot += qh[(size_t)i * HD + x] * kh[(size_t)j * HD + x];
                    s[j] = dot * scale;
                    m = fmaxf(m, s[j]);
                }
                float l = 0.0f;
                for (int j = 0; j < cols; ++j) {
                    s[j] = expf(s[j] - m);
                    l += s[j];
                }
                for (int x = 0; x < HD; ++x) oh[x] = 0.0f;
                for (int j = 0; j < cols; ++j) {
                    float p = s[j] / l;
                    for (int x = 0; x < HD; ++x) oh[x] += p * vh[(size_t)j * HD + x];
                }
            }
        }
        free(s);
    }
    return rows;
}

/* attn_bwd_preprocess, 02-flash-attention/kernels/attention_bwd.cu:32-44 */
void orc_bwd_preprocess(const float *dout, const float *o, float *delta, size_t rows) {
    for (size_t i = 0; i < rows; ++i) {
        float d = 0.0f;
        for (int x = 0; x < HD; ++x) d += dout[i * HD + x] * o[i * HD + x];
        delta[i] = d;
    }
}

/* attn_loss, 02-flash-attention/src/main.rs:304-333 (f64 forward, <O,dO>) */
double orc_attn_loss(const float *q, const float *k, const float *v, const float *dout, int n,
                     int causal) {
    const double scale = 1.0 / sqrt((double)HD);
    double loss = 0.0;
    double *s = (double *)malloc((size_t)(n > 0 ? n : 1) * sizeof(double));
    for (int i = 0; i < n; ++i) {
        int cols = causal ? i + 1 : n;
        double m = -INFINITY;
        for (int j = 0; j < cols; ++j) {
            double dot = 0.0;
            for (int x = 0; x < HD; ++x)
                dot += (double)q[(size_t)i * HD + x] * (double)k[(size_t)j * HD + x];
            s[j] = dot * scale;
            m = fmax(m, s[j]);
        }
        double l = 0.0;
        for (int j = 0; j < cols; ++j) {
            s[j] = exp(s[j] - m);
            l += s[j];
        }
        for (int x = 0; x < HD; ++x) {
            double o = 0.0;
            for (int j = 0; j < cols; ++j) o += s[j] / l * (double)v[(size_t)j * HD + x];
            loss += o * (double)dout[(size_t)i * HD + x];
        }
    }
    free(s);
    return loss;
}

/* ------------------------------------------------------------------ */
/* 03-llm-engine: per-layer attention step                             */
/* ------------------------------------------------------------------ */

/* rope, 03-llm-engine/src/cpu.rs:25-37 (HF rotate_half, precise libm) */
void orc_rope(float *x, int n_heads, int head_dim, int pos, float theta) {
    int half = head_dim / 2;
    for (int h = 0; h < n_heads; ++h) {
        int base = h * head_dim;
        for (int d = 0; d < half; ++d) {
            float freq = powf(theta, -2.0f * (float)d / (float)head_dim);
            float a = (float)pos * freq;
            float sn = sinf(a), cs = cosf(a);
            float x1 = x[base + d], x2 = x[base + d + half];
            x[base + d] = x1 * cs - x2 * sn;
            x[base + d + half] = x1 * sn + x2 * cs;
        }
    }
}

/* kv_row, 03-llm-engine/kernels/llm.cu:959-963 */
static inline size_t kv_row(const int *table, int block_size, int t) {
    if (table) return (size_t)(table[t / block_size] * block_size + t % block_size);
    return (size_t)t;
}

static inline int rne_clamp(float x, int lo, int hi) {
    /* __float2int_rn: round to nearest even (default rounding mode) */
    float r = nearbyintf(x);
    if (r < (float)lo) return lo;
    if (r > (float)hi) return hi;
    return (int)r;
}

/* quant_affine, 03-llm-engine/kernels/llm.cu:1137-1149 */
void orc_quant_affine(const float *src, int8_t *dst, float *scale_out, float *beta_out, int d) {
    float hi = -INFINITY, lo = INFINITY;
    for (int i = 0; i < d; ++i) {
        hi = fmaxf(hi, src[i]);
        lo = fminf(lo, src[i]); /* -max(-x) == min(x) exactly */
    }
    float scale = (hi > lo) ? (hi - lo) / 255.0f : 1.0f;
    float beta = lo + 128.0f * scale;
    for (int i = 0; i < d; ++i) dst[i] = (int8_t)rne_clamp((src[i] - beta) / scale, -128, 127);
    *scale_out = scale;
    *beta_out = beta;
}

/* Symmetric absmax int8, the reference's in-kernel convention for q and for
 * on-the-fly K: 03-llm-engine/kernels/llm.cu:1353-1364, 3743-3753. */
void orc_quant_absmax(const float *src, int8_t *dst, float *scale_out, int d) {
    float amax = 0.0f;
    for (int i = 0; i < d; ++i) amax = fmaxf(amax, fabsf(src[i]));
    float id = amax > 0.0f ? 127.0f / amax : 0.0f;
    for (int i = 0; i < d; ++i) dst[i] = (int8_t)rne_clamp(src[i] * id, -127, 127);
    *scale_out = amax > 0.0f ? amax / 127.0f : 0.0f;
}

/* quantize_kv_impl / quantize_kv_batch_impl / quantize_kv_seqpos:
 * 03-llm-engine/kernels/llm.cu:1154-1240,1503-1510.  Writes the K and V
 * sections of one qkv row into logical position `pos` (physical row through
 * the optional block table).  fmt 0 = affine (scale, beta), the reference's
 * cache format; fmt 1 = symmetric absmax (beta arrays untouched, may be NULL). */
void orc_quantize_kv_row(int8_t *kq, int8_t *vq, float *ks, float *vs, float *kb, float *vb,
                         const float *qkv_row, int pos, int q_dim, int n_kv_head, int head_dim,
                         const int *table, int block_size, int fmt) {
    int kv_dim = n_kv_head * head_dim;
    size_t pr = kv_row(table, block_size, pos);
    for (int h = 0; h < n_kv_head; ++h) {
        const float *k = qkv_row + q_dim + h * head_dim;
        const float *v = qkv_row + q_dim + kv_dim + h * head_dim;
        size_t row = pr * kv_dim + (size_t)h * head_dim;
        size_t sd = pr * n_kv_head + h;
        if (fmt == 0) {
            orc_quant_affine(k, kq + row, &ks[sd], &kb[sd], head_dim);
            orc_quant_affine(v, vq + row, &vs[sd], &vb[sd], head_dim);
        } else {
            orc_quant_absmax(k, kq + row, &ks[sd], head_dim);
            orc_quant_absmax(v, vq + row, &vs[sd], head_dim);
        }
    }
}

/* fp32 KV write: 03-llm-engine/src/gpu.rs:2594-2605,
 * 03-llm-engine/kernels/llm.cu:965-986,1491-1501,3635-3655 */
void orc_copy_kv_row(float *kcache, float *vcache, const float *qkv_row, int pos, int q_dim,
                     int kv_dim, const int *table, int block_size) {
    size_t row = kv_row(table, block_size, pos) * kv_dim;
    for (int i = 0; i < kv_dim; ++i) {
        kcache[row + i] = qkv_row[q_dim + i];
        vcache[row + i] = qkv_row[q_dim + kv_dim + i];
    }
}

/* Grouped-query attention of one query row over cache positions 0..=t_cur:
 * 03-llm-engine/src/cpu.rs:222-247 (and :130-154 with n_kv_head == n_head). */
void orc_gqa_decode_f32(float *out, const float *q, const float *kcache, const float *vcache,
                        int t_cur, int n_head, int n_kv_head, int head_dim, const int *table,
                        int block_size) {
    int kvd = n_kv_head * head_dim;
    int group = n_head / n_kv_head;
    float scale = 1.0f / sqrtf((float)head_dim);
    float *s = (float *)malloc((size_t)(t_cur + 1) * sizeof(float));
    for (int h = 0; h < n_head; ++h) {
        int kvh = h / group;
        const float *qh = q + h * head_dim;
        float m = -INFINITY;
        for (int j = 0; j <= t_cur; ++j) {
            const float *kr = kcache + kv_row(table, block_size, j) * kvd + kvh * head_dim;
            float dot = 0.0f;
            for (int d = 0; d < head_dim; ++d) dot += qh[d] * kr[d];
            s[j] = dot * scale;
            m = fmaxf(m, s[j]);
        }
        float sum = 0.0f;
        for (int j = 0; j <= t_cur; ++j) {
            s[j] = expf(s[j] - m);
            sum += s[j];
        }
        float *o = out + h * head_dim;
        for (int d = 0; d < head_dim; ++d) o[d] = 0.0f;
        for (int j = 0; j <= t_cur; ++j) {
            float p = s[j] / sum;
            const float *vr = vcache + kv_row(table, block_size, j) * kvd + kvh * head_dim;
            for (int d = 0; d < head_dim; ++d) o[d] += p * vr[d];
        }
    }
    free(s);
}

/* int8-cache decode.  mode 0 ("dequant-exact"): K^ = ks*code + kb,
 * V^ = vs*code + vb in fp32, then the cpu.rs attention above.  mode 1
 * ("kernel-faithful"): additionally quantises q per head and recombines exactly
 * as attn_decode_q8_impl does, 03-llm-engine/kernels/llm.cu:1332-1417
 * (integer dots, qs*(ks*dot + kb*sum_q), V beta folded through sum p*vb; the
 * GPU's parallel reduction order is replaced by index order).
 * kb/vb NULL = symmetric cache (beta 0). */
void orc_gqa_decode_q8(float *out, const float *q, const int8_t *kq, const int8_t *vq,
                       const float *ks, const float *vs, const float *kb, const float *vb,
                       int t_cur, int n_head, int n_kv_head, int head_dim, const int *table,
                       int block_size, int mode) {
    int kvd = n_kv_head * head_dim;
    int group = n_head / n_kv_head;
    float scale = 1.0f / sqrtf((float)head_dim);
    float *s = (float *)malloc((size_t)(t_cur + 1) * sizeof(float));
    int8_t qq[256];
    for (int h = 0; h < n_head; ++h) {
        int kvh = h / group;
        const float *qh = q + h * head_dim;
        float *o = out + h * head_dim;
        float m = -INFINITY;
        if (mode == 0) {
            for (int j = 0; j <= t_cur; ++j) {
                size_t r = kv_row(table, block_size, j);
                const int8_t *kr = kq + r * kvd + kvh * head_dim;
                float sc = ks[r * n_kv_head + kvh], be = kb ? kb[r * n_kv_head + kvh] : 0.0f;
                float dot = 0.0f;
                for (int d = 0; d < head_dim; ++d) dot += qh[d] * ((float)kr[d] * sc + be);
                s[j] = dot * scale;
                m = fmaxf(m, s[j]);
            }
            float sum = 0.0f;
            for (int j = 0; j <= t_cur; ++j) {
                s[j] = expf(s[j] - m);
                sum += s[j];
            }
            for (int d = 0; d < head_dim; ++d) o[d] = 0.0f;
            for (int j = 0; j <= t_cur; ++j) {
                float p = s[j] / sum;
                size_t r = kv_row(table, block_size, j);
                const int8_t *vr = vq + r * kvd + kvh * head_dim;
                float sc = vs[r * n_kv_head + kvh], be = vb ? vb[r * n_kv_head + kvh] : 0.0f;
                for (int d = 0; d < head_dim; ++d) o[d] += p * ((float)vr[d] * sc + be);
            }
        } else {
            float qmax = 0.0f;
            for (int d = 0; d < head_dim; ++d) qmax = fmaxf(qmax, fabsf(qh[d]));
            float qid = qmax > 0.0f ? 127.0f / qmax : 0.0f;
            int qsum_i = 0;
            for (int d = 0; d < head_dim; ++d) {
                qq[d] = (int8_t)rne_clamp(qh[d] * qid, -127, 127);
                qsum_i += qq[d];
            }
            float qs = (qmax > 0.0f ? qmax / 127.0f : 0.0f) * scale;
            float qsum = (float)qsum_i;
            for (int j = 0; j <= t_cur; ++j) {
                size_t r = kv_row(table, block_size, j);
                const int8_t *kr = kq + r * kvd + kvh * head_dim;
                int dot = 0;
                for (int d = 0; d < head_dim; ++d) dot += (int)kr[d] * (int)qq[d];
                float be = kb ? kb[r * n_kv_head + kvh] : 0.0f;
                s[j] = qs * (ks[r * n_kv_head + kvh] * (float)dot + be * qsum);
                m = fmaxf(m, s[j]);
            }
            float l = 0.0f;
            for (int j = 0; j <= t_cur; ++j) {
                s[j] = expf(s[j] - m);
                l += s[j];
            }
            float inv = 1.0f / l;
            float vbsum = 0.0f;
            if (vb)
                for (int j = 0; j <= t_cur; ++j)
                    vbsum += s[j] * vb[kv_row(table, block_size, j) * n_kv_head + kvh];
            for (int d = 0; d < head_dim; ++d) {
                float a = 0.0f;
                for (int j = 0; j <= t_cur; ++j) {
                    size_t r = kv_row(table, block_size, j);
                    float st = s[j] * vs[r * n_kv_head + kvh];
                    a += st * (float)vq[r * kvd + kvh * head_dim + d];
                }
                o[d] = (a + vbsum) * inv;
            }
        }
    }
    free(s);
}

/* Partial attention of one query row over cache positions [t0, t1): the
 * unnormalised triple (m, l, acc[hd]) with acc = sum_j exp(s_j - m) v_j, the
 * unit the split-KV decode exchanges.  Not in the reference (new for the
 * multi-GPU long-context decode).  mode as orc_gqa_decode_q8 mode 0 when
 * kq != NULL, fp32 cache otherwise. */
void orc_gqa_partial(float *m_out, float *l_out, float *acc_out, const float *q,
                     const float *kcache, const float *vcache, const int8_t *kq, const int8_t *vq,
                     const float *ks, const float *vs, const float *kb, const float *vb, int t0,
                     int t1, int n_head, int n_kv_head, int head_dim) {
    int kvd = n_kv_head * head_dim;
    int group = n_head / n_kv_head;
    float scale = 1.0f / sqrtf((float)head_dim);
    int n = t1 - t0;
    float *s = (float *)malloc((size_t)(n > 0 ? n : 1) * sizeof(float));
    for (int h = 0; h < n_head; ++h) {
        int kvh = h / group;
        const float *qh = q + h * head_dim;
        float m = -INFINITY;
        for (int j = t0; j < t1; ++j) {
            float dot = 0.0f;
            if (kq) {
                const int8_t *kr = kq + (size_t)j * kvd + kvh * head_dim;
                float sc = ks[(size_t)j * n_kv_head + kvh];
                float be = kb ? kb[(size_t)j * n_kv_head + kvh] : 0.0f;
                for (int d = 0; d < head_dim; ++d) dot += qh[d] * ((float)kr[d] * sc + be);
            } else {
                const float *kr = kcache + (size_t)j * kvd + kvh * head_dim;
                for (int d = 0; d < head_dim; ++d) dot += qh[d] * kr[d];
            }
            s[j - t0] = dot * scale;
            m = fmaxf(m, s[j - t0]);
        }
        float l = 0.0f;
        float *acc = acc_out + h * head_dim;
        for (int d = 0; d < head_dim; ++d) acc[d] = 0.0f;
        for (int j = t0; j < t1; ++j) {
            float p = expf(s[j - t0] - m);
            l += p;
            if (vq) {
                const int8_t *vr = vq + (size_t)j * kvd + kvh * head_dim;
                float sc = vs[(size_t)j * n_kv_head + kvh];
                float be = vb ? vb[(size_t)j * n_kv_head + kvh] : 0.0f;
                for (int d = 0; d < head_dim; ++d) acc[d] += p * ((float)vr[d] * sc + be);
            } else {
                const float *vr = vcache + (size_t)j * kvd + kvh * head_dim;
                for (int d = 0; d < head_dim; ++d) acc[d] += p * vr[d];
            }
        }
        m_out[h] = m;
        l_out[h] = l;
    }
    free(s);
}

/* Log-sum-exp merge of `parts` partial triples per row (new; no reference
 * code): m = max m_r, l = sum l_r e^{m_r - m}, out = sum acc_r e^{m_r - m} / l.
 * Layout: m,l [parts][rows]; acc [parts][rows][hd]; out [rows][hd]. */
void orc_merge_partials(float *out, const float *m, const float *l, const float *acc, int parts,
                        int rows, int head_dim) {
    for (int r = 0; r < rows; ++r) {
        float mm = -INFINITY;
        for (int p = 0; p < parts; ++p) mm = fmaxf(mm, m[(size_t)p * rows + r]);
        float ll = 0.0f;
        for (int d = 0; d < head_dim; ++d) out[(size_t)r * head_dim + d] = 0.0f;
        for (int p = 0; p < parts; ++p) {
            float mp = m[(size_t)p * rows + r];
            float w = (mp == -INFINITY) ? 0.0f : expf(mp - mm);
            ll += l[(size_t)p * rows + r] * w;
            for (int d = 0; d < head_dim; ++d)
                out[(size_t)r * head_dim + d] += acc[((size_t)p * rows + r) * head_dim + d] * w;
        }
        for (int d = 0; d < head_dim; ++d) out[(size_t)r * head_dim + d] /= ll;
    }
}

/* Batched decode over n_seq sequences, OpenMP over sequences: the arithmetic
 * per sequence is orc_gqa_decode_f32 / orc_gqa_decode_q8; mirrors the grid.y
 * dimension of attn_decode_batched, 03-llm-engine/kernels/llm.cu:1468-1487.
 * Caches are per-sequence slabs of `seq_rows` rows here (tables == NULL) or one
 * shared pool addressed through tables[s*n_log ..]. */
void orc_gqa_decode_batched(float *out, const float *qkv, const float *kcache, const float *vcache,
                            const int8_t *kq, const int8_t *vq, const float *ks, const float *vs,
                            const float *kb, const float *vb, const int *pos, int n_seq,
                            int n_head, int n_kv_head, int head_dim, const int *tables,
                            int block_size, int n_log, size_t seq_rows, int qkv_stride,
                            int out_stride, int mode, int threads) {
    int nt = pick_threads(threads);
    (void)nt;
    size_t kvd = (size_t)n_kv_head * head_dim;
#pragma omp parallel for num_threads(nt) schedule(dynamic, 1)
    for (int s = 0; s < n_seq; ++s) {
        const int *tb = tables ? tables + (size_t)s * n_log : NULL;
        size_t ro = tables ? 0 : (size_t)s * seq_rows;
        if (kq)
            orc_gqa_decode_q8(out + (size_t)s * out_stride, qkv + (size_t)s * qkv_stride,
                              kq + ro * kvd, vq + ro * kvd, ks + ro * n_kv_head,
                              vs + ro * n_kv_head, kb ? kb + ro * n_kv_head : NULL,
                              vb ? vb + ro * n_kv_head : NULL, pos[s], n_head, n_kv_head, head_dim,
                              tb, block_size, mode);
        else
            orc_gqa_decode_f32(out + (size_t)s * out_stride, qkv + (size_t)s * qkv_stride,
                               kcache + ro * kvd, vcache + ro * kvd, pos[s], n_head, n_kv_head,
                               head_dim, tb, block_size);
    }
}

/* One query row over an fp32 cache with int8 scores formed on the fly: KIND 2 of attn_prefill_body
 * (03-llm-engine/kernels/llm.cu:3700-3716 for q, :3737-3754 for K, :3774-3782 for the score).  q is quantised per
 * (row, head): id = 127/amax, codes clamp(rne(q*id), +-127), qs = amax/127; every K row symmetrically the same way
 * (Ks = amax/127, no offset); s = qs * scale * ((float)dot * Ks).  V stays fp32; softmax per row as in cpu.rs. */
static void orc_gqa_row_dp4a(float *out, const float *q, const float *kcache, const float *vcache, int t_cur,
                             int n_head, int n_kv_head, const int *table, int block_size) {
    int kvd = n_kv_head * HD;
    int group = n_head / n_kv_head;
    float scale = 1.0f / sqrtf((float)HD);
    float *s = (float *)malloc((size_t)(t_cur + 1) * sizeof(float));
    for (int h = 0; h < n_head; ++h) {
        int kvh = h / group;
        const float *qh = q + h * HD;
        float *o = out + h * HD;
        int qq[HD];
        float amax = 0.0f;
        for (int d = 0; d < HD; ++d) amax = fmaxf(amax, fabsf(qh[d]));
        float id = amax > 0.0f ? 127.0f / amax : 0.0f;
        for (int d = 0; d < HD; ++d) qq[d] = rne_clamp(qh[d] * id, -127, 127);
        float qs = amax > 0.0f ? amax / 127.0f : 0.0f;
        float m = -INFINITY;
        for (int j = 0; j <= t_cur; ++j) {
            const float *kr = kcache + kv_row(table, block_size, j) * kvd + kvh * HD;
            float kmax = 0.0f;
            for (int d = 0; d < HD; ++d) kmax = fmaxf(kmax, fabsf(kr[d]));
            float kid = kmax > 0.0f ? 127.0f / kmax : 0.0f;
            int dot = 0;
            for (int d = 0; d < HD; ++d) dot += qq[d] * rne_clamp(kr[d] * kid, -127, 127);
            float ksj = kmax > 0.0f ? kmax / 127.0f : 0.0f;
            s[j] = qs * scale * ((float)dot * ksj + 0.0f);
            m = fmaxf(m, s[j]);
        }
        float sum = 0.0f;
        for (int j = 0; j <= t_cur; ++j) {
            s[j] = expf(s[j] - m);
            sum += s[j];
        }
        for (int d = 0; d < HD; ++d) o[d] = 0.0f;
        for (int j = 0; j <= t_cur; ++j) {
            float p = s[j] / sum;
            const float *vr = vcache + kv_row(table, block_size, j) * kvd + kvh * HD;
            for (int d = 0; d < HD; ++d) o[d] += p * vr[d];
        }
    }
    free(s);
}

/* Prefill attention of n_tok new rows at absolute positions pos0+qi over cache
 * keys 0..=pos0+qi: the semantics of attn_prefill_body,
 * 03-llm-engine/kernels/llm.cu:3674-3804, evaluated with the cpu.rs per-row
 * softmax (max, exp/sum, normalise, PV) instead of the kernel's online form.
 * kind 0: fp32 cache, fp32 scores (KIND 0).  kind 1: int8 cache, dequant-exact (K^, V^ as above).
 * kind 2: int8 cache with the reference kernel's own score arithmetic (its KIND 1: q quantised per (row, head),
 * integer dots, llm.cu:3700-3716,3774-3782 -- the same arithmetic as its decode kernel).
 * kind 3: fp32 cache, K quantised on the fly (the reference's opt-in KIND 2, attn_prefill_dp4a).
 * q rows are read at qkv[qi*qkv_stride + h*64 ..], out at out[qi*out_stride + h*64 ..]. */
void orc_prefill(float *out, const float *qkv, const float *kcache, const float *vcache,
                 const int8_t *kq, const int8_t *vq, const float *ks, const float *vs,
                 const float *kb, const float *vb, int pos0, int n_tok, int n_head, int n_kv_head,
                 int qkv_stride, int out_stride, const int *table, int block_size, int kind,
                 int threads) {
    int nt = pick_threads(threads);
    (void)nt;
#pragma omp parallel for num_threads(nt) schedule(dynamic, 4)
    for (int qi = 0; qi < n_tok; ++qi) {
        if (kind == 0)
            orc_gqa_decode_f32(out + (size_t)qi * out_stride, qkv + (size_t)qi * qkv_stride, kcache,
                               vcache, pos0 + qi, n_head, n_kv_head, HD, table, block_size);
        else if (kind == 3)
            orc_gqa_row_dp4a(out + (size_t)qi * out_stride, qkv + (size_t)qi * qkv_stride, kcache, vcache,
                             pos0 + qi, n_head, n_kv_head, table, block_size);
        else
            orc_gqa_decode_q8(out + (size_t)qi * out_stride, qkv + (size_t)qi * qkv_stride, kq, vq,
                              ks, vs, kb, vb, pos0 + qi, n_head, n_kv_head, HD, table, block_size,
                              kind == 2 ? 1 : 0);
    }
}

/* y[o] (+)= sum_i x[i] w[i*n_out + o] + b[o]: the reference's gemv, one sequential fp32 sum per
 * output column (03-llm-engine/kernels/llm.cu:144-160; gemv_half :162-177 widens fp16 weights to
 * fp32 first, which the caller does before calling this).  b may be null. */
void orc_gemv(float *y, const float *x, const float *w, const float *b, int n_in, int n_out, int accum) {
    for (int o = 0; o < n_out; ++o) {
        float acc = 0.0f;
        for (int i = 0; i < n_in; ++i) acc += x[i] * w[(size_t)i * n_out + o];
        float r = acc + (b ? b[o] : 0.0f);
        y[o] = accum ? y[o] + r : r;
    }
}

/* gemv_int8 (03-llm-engine/kernels/llm.cu:226-316): the activation row is quantised per group of `ag`
 * values (absmax / 127, codes clamp(rne(x * (127 / amax)), +-127), group scale amax / 127, or 1 when the
 * group is all zero); weights are int32 words of four consecutive input rows, w32[(i/4)*n_out + o];
 * per output column: acc += (float)(integer dot of the group) * xs[g] over the groups in order, then
 * y[o] (+)= acc * scales[o] + b[o]. */
void orc_gemv_int8(float *y, const float *x, const int *w32, const float *scales, const float *b, int n_in,
                   int n_out, int accum, int ag) {
    int n_groups = n_in / ag;
    signed char *xq = (signed char *)malloc((size_t)n_in);
    float *xs = (float *)malloc(sizeof(float) * (size_t)n_groups);
    for (int g = 0; g < n_groups; ++g) {
        const float *xg = x + (size_t)g * ag;
        float amax = 0.0f;
        for (int j = 0; j < ag; ++j) amax = fmaxf(amax, fabsf(xg[j]));
        float id = amax > 0.0f ? 127.0f / amax : 0.0f;
        for (int j = 0; j < ag; ++j) {
            int v = (int)nearbyintf(xg[j] * id);
            v = v > 127 ? 127 : (v < -127 ? -127 : v);
            xq[(size_t)g * ag + j] = (signed char)v;
        }
        xs[g] = amax > 0.0f ? amax / 127.0f : 1.0f;
    }
    for (int o = 0; o < n_out; ++o) {
        float acc = 0.0f;
        for (int g = 0; g < n_groups; ++g) {
            int ig = 0;
            for (int q = 0; q < ag / 4; ++q) {
                int word = w32[(size_t)((ag / 4) * g + q) * n_out + o];
                for (int j = 0; j < 4; ++j)
                    ig += (int)(signed char)((word >> (8 * j)) & 0xFF) * (int)xq[(size_t)g * ag + 4 * q + j];
            }
            acc += (float)ig * xs[g];
        }
        float r = acc * scales[o] + (b ? b[o] : 0.0f);
        y[o] = accum ? y[o] + r : r;
    }
    free(xq);
    free(xs);
}
