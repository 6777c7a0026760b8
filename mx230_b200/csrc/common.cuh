// Shared declarations for the mx230 attention library (sm_100a only).
//
// Host side: status codes, the per-device handle, error plumbing.
// Device side: thin inline-PTX wrappers for mbarrier, TMA (cp.async.bulk.tensor,
// plain per-CTA loads only), tensor memory (tcgen05.alloc/ld/st) and the 5th-gen
// tensor-core MMA (tcgen05.mma + tcgen05.commit).
//
// Every device-side wait is bounded: a waiter polls for at most WAIT_LIMIT_CYCLES SM cycles
// and then records an error in the handle's status word and abandons the tile,
// so a protocol bug shows up as a status code, never as a hung GPU.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/mx230_attn.h"

// ---------------------------------------------------------------------------
// host
// ---------------------------------------------------------------------------
typedef CUresult (*mx230_encode_tiled_fn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                          const cuuint64_t *, const cuuint64_t *,
                                          const cuuint32_t *, const cuuint32_t *,
                                          CUtensorMapInterleave, CUtensorMapSwizzle,
                                          CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

struct mx230_handle {
    int device;
    int sm_count;
    void *ws;              // workspace: bf16 operand staging / split-KV partials
    size_t ws_bytes;
    int *status_dev;       // [8] device words: [0..3] status (0 = ok), [4..5] the wait limit in SM cycles (64-bit)
    int test_drop_tile;    // test hook: streamed tile that CTA 0's producer never requests (-1 = off)
    unsigned *counters;    // split-KV arrival counters (self-resetting)
    size_t n_counters;
    int q8_score_mode;     // MX230_Q8_SCORE_*
    int decode_chunk;      // keys per decode CTA (0 = automatic)
    int decode_tensor;     // int8 decode, reference score mode: tensor-core tiles (1) or CUDA cores (0)
    int bwd_two_pass;      // flash backward: two atomic-free passes (1) or one fused pass with dQ reductions (0)
    int bwd_reuse_staged;  // flash backward: skip re-staging Q, K, V when the workspace still holds the forward's copies
    // which fp32 tensors the workspace's staged bf16 Q (pre-scaled), K, V currently belong to; cleared by every
    // entry point that writes the workspace for something else
    struct {
        const void *q, *k, *v;
        int batch_heads, n;
        int valid;
        const void *d_o;   // the fp32 dO whose bf16 copy the Delta pre-pass left in the fourth staging slot (null: none)
    } staged;
    long long launches;    // kernels launched through this handle
    mx230_encode_tiled_fn encode_tiled;
    // per-kernel timing: event pairs recorded around launches while enabled
    int prof_on;
    int prof_used;                 // event pairs in flight
    cudaEvent_t *prof_ev;          // [2 * PROF_CAP]
    int *prof_kid;                 // [PROF_CAP]
    long long prof_count[MX230_K_COUNT];
    double prof_ms[MX230_K_COUNT];
};

constexpr int MX230_PROF_CAP = 8192;
int mx230_prof_begin(mx230_handle *h, cudaStream_t st, int kid);  // returns slot or -1
void mx230_prof_end(mx230_handle *h, cudaStream_t st, int slot);

// Brackets one kernel launch: optional event pair, launch check, launch count.
#define MX_LAUNCH(h, st, kid, ...)                                                          \
    do {                                                                                    \
        int _slot = (h)->prof_on ? mx230_prof_begin((h), (st), (kid)) : -1;                 \
        __VA_ARGS__;                                                                        \
        if (_slot >= 0) mx230_prof_end((h), (st), _slot);                                   \
        MX_LAUNCHED(h);                                                                     \
    } while (0)

void mx230_set_error(const char *fmt, ...);
int mx230_fail(int code, const char *fmt, ...);

#define MX_CHECK_CUDA(expr)                                                                  \
    do {                                                                                     \
        cudaError_t _e = (expr);                                                             \
        if (_e != cudaSuccess)                                                               \
            return mx230_fail(MX230_ERR_CUDA, "%s: %s (%s:%d)", #expr, cudaGetErrorString(_e), \
                              __FILE__, __LINE__);                                           \
    } while (0)

#define MX_REQUIRE(cond, code, ...)                        \
    do {                                                   \
        if (!(cond)) return mx230_fail(code, __VA_ARGS__); \
    } while (0)

// Raises a kernel's dynamic shared-memory limit once per device and call site (function attributes are per
// device; setting one costs a driver call, which has no place in front of every launch of a microsecond kernel).
#define MX_SMEM_ATTR_ONCE(device, kernel, bytes)                                                         \
    do {                                                                                                 \
        static bool _done[64] = {};                                                                      \
        const int _d = (device);                                                                         \
        if (_d < 0 || _d >= 64 || !_done[_d]) {                                                          \
            MX_CHECK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,      \
                                               (int)(bytes)));                                           \
            if (_d >= 0 && _d < 64) _done[_d] = true;                                                    \
        }                                                                                                \
    } while (0)

// Checks the launch and counts it on the handle.
#define MX_LAUNCHED(h)                                                                      \
    do {                                                                                    \
        cudaError_t _e = cudaGetLastError();                                                \
        if (_e != cudaSuccess)                                                              \
            return mx230_fail(MX230_ERR_CUDA, "kernel launch: %s (%s:%d)",                  \
                              cudaGetErrorString(_e), __FILE__, __LINE__);                  \
        (h)->launches++;                                                                    \
    } while (0)

// RAII-free "make this handle's device current" used at the top of every entry point.
struct mx230_device_guard {
    int prev;
    bool switched;
    explicit mx230_device_guard(int dev) : prev(-1), switched(false) {
        if (cudaGetDevice(&prev) == cudaSuccess && prev != dev) {
            cudaSetDevice(dev);
            switched = true;
        }
    }
    ~mx230_device_guard() {
        if (switched) cudaSetDevice(prev);
    }
};

// Split-KV exchange over peer memory (splitkv.cu; the partial-attention kernels of decode.cu push into it).
// A region holds, per step parity and source rank, rows*66 words {value, step number} in the packed order
// [m (rows) | l (rows) | acc (rows x 64)], then one step number per 16-row slice.
constexpr int MX230_SPLITKV_MAX_WORLD = 16;
struct mx230_splitkv_comm {
    mx230_handle *h;
    int rank, world, rows, slices;
    size_t part_words, step_offset_words, region_bytes;
    uint2 *region[MX230_SPLITKV_MAX_WORLD];   // [rank] is the own allocation, the others are peers' regions mapped here
    bool imported[MX230_SPLITKV_MAX_WORLD];   // opened from an IPC handle (closed again on disconnect)
    uint2 **region_dev;                       // the same table in device memory, for kernels that take it by pointer
    float *local;                             // packed triples of this rank, kept beside what is pushed
};

// 2-D/3-D bf16 tensor map over [outer][rows][64] with a {64, box_rows, 1} box and
// 128-byte swizzle (one 64-element bf16 row is exactly one 128-byte swizzle span).
int mx230_make_tmap_bf16(mx230_handle *h, CUtensorMap *out, const void *base, uint64_t rows,
                         uint64_t outer, uint64_t row_stride_bytes, uint64_t outer_stride_bytes,
                         uint32_t box_rows);
// 16-bit matrix [rows][inner] (bf16, or fp16 when `fp16`), {box_inner, box_rows, 1} boxes, 128-byte swizzle, zero fill.
int mx230_make_tmap_2d_16bit(mx230_handle *h, CUtensorMap *out, const void *base, int fp16, uint64_t inner,
                             uint64_t rows, uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_rows);
// fp32 tensor map over [outer][rows][64] with a {32, 32, 1} box (half rows of 128 bytes) and 128-byte swizzle.
int mx230_make_tmap_f32_half_rows(mx230_handle *h, CUtensorMap *out, const void *base, uint64_t rows,
                                  uint64_t outer);
int mx230_make_tmap_f32_half_rows_strided(mx230_handle *h, CUtensorMap *out, const void *base, uint64_t rows,
                                          uint64_t outer, uint64_t row_stride_bytes, uint64_t outer_stride_bytes);

// fp32 -> bf16 staging of up to four equally sized tensors of `heads` x `per_head` elements in one launch
// (flash_fwd.cu).  `zero`, if not null, is a buffer of the same size cleared by the same launch.  Tensor 0 is
// multiplied by `scale0` before rounding (1 = plain cast).  norm2[t] (t = 0, 1; may be null): receives, per head
// and grid part, the largest squared row norm (rows of 64 values) of tensor t as given, [heads][MX230_NORM_PARTS]
// floats with unused parts set to 0 -- what the forward kernel needs for its bound on |q . k|.
constexpr int MX230_NORM_PARTS = 32;
int mx230_launch_cast(mx230_handle *h, cudaStream_t st, const float *const *src, void *const *dst,
                      int n_tensors, int heads, size_t per_head, float *zero, float scale0, float *const *norm2);
// 1/sqrt(64) * log2(e): Q staged times this gives scores in log2 units
#define MX230_QK_LOG2_SCALE (0.125f * 1.4426950408889634f)
// layout of the flash entry points' workspace: `k` staged bf16 tensors of mx230_flash_stage_bytes each, then the
// row-norm partials of Q and K
inline size_t mx230_flash_stage_bytes(int batch_heads, int n) {
    size_t one = (size_t)batch_heads * (size_t)n * 64 * 2;
    return (one + 1023) & ~(size_t)1023;
}
inline size_t mx230_flash_norm_bytes(int batch_heads) {
    size_t b = (size_t)2 * batch_heads * MX230_NORM_PARTS * sizeof(float);
    return (b + 1023) & ~(size_t)1023;
}

// tcgen05 flash forward over staged bf16 operands (flash_fwd.cu).  Q [heads][n_q][64]; K, V
// [heads / kv_group][n_k][64]; causal row r sees keys <= r + q_off; output row r of head h at
// O + h*o_head_stride + r*o_row_stride.  q_prescaled: Qb holds Q * MX230_QK_LOG2_SCALE.  q_norm2 / k_norm2 (both or
// neither): largest squared row norm per head of the unscaled Q [heads][MX230_NORM_PARTS] and of K
// [heads / kv_group][MX230_NORM_PARTS]; with them (and q_prescaled) a head whose scores are provably small takes the
// kernel's max-free softmax loop.  row_a / row_qsum / col_kskb (all or none; with them q_prescaled must be 0 and Qb, Kb
// hold int8 codes as bf16): the int8 score mode -- score = row_a[h][i] * (dot * ks[j] + row_qsum[h][i] * kb[j]), with
// col_kskb [heads / kv_group][n_k rounded up to 128] pairs (ks, kb).
int mx230_launch_flash_fwd_ex(mx230_handle *h, cudaStream_t st, const void *Qb, const void *Kb,
                              const void *Vb, float *O, float *L, int heads, int n_q, int n_k, int q_off,
                              int kv_group, long long o_head_stride, long long o_row_stride, int causal,
                              int q_prescaled, const float *q_norm2, const float *k_norm2, const float *row_a,
                              const float *row_qsum, const float *col_kskb);

// ---------------------------------------------------------------------------
// device
// ---------------------------------------------------------------------------
#ifdef __CUDACC__

namespace mx {

constexpr long long WAIT_LIMIT_CYCLES = 4000000000ll;  // default bound of a wait: about 2 s of SM cycles
constexpr int STATUS_LIMIT_WORD = 4;                   // status[4..5]: the bound in force (64-bit), set by the host
constexpr int STATUS_WAIT_TIMEOUT = 1;

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}


// ---- mbarrier ----
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
                 : "memory");
}
// The suspend-time hint lets the hardware park the polling thread until the phase completes (or the
// hint runs out) instead of re-issuing the poll: a spinning single-lane issuer warp otherwise takes
// issue slots from the compute warp that shares its scheduler.
constexpr uint32_t TRY_WAIT_SUSPEND_HINT = 0x989680u;
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity), "r"(TRY_WAIT_SUSPEND_HINT)
        : "memory");
    return ok != 0;
}

// Bounded wait.  `abort_flag` is a CTA-shared word: once any role of the CTA gave
// up, everybody else leaves its waits at the next check.  Returns false on abort.
// The bound is counted on the SM's own cycle counter (cheap to read; reading the global
// nanosecond timer on every contended wait costs far more than the wait itself).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag,
                                          int *status) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    unsigned polls = 0;
    while (true) {
        if (mbar_try_wait(bar, parity)) return true;
        // A poll that finds the phase incomplete may have been parked by the hardware for up to the suspend hint,
        // so the abort flag and the clock are first looked at after 8 polls, then after 16, 32, ... (every 256 from
        // there on): early for a wait that is going to run out, rare for the short waits of the steady state, whose
        // polling warps share a scheduler with the compute warps.
        ++polls;
        if (polls >= 8u && (polls < 256u ? (polls & (polls - 1u)) == 0u : (polls & 255u) == 0u)) {
            if (*abort_flag) return false;
            if (clock64() - t0 > *(const volatile long long *)(status + STATUS_LIMIT_WORD)) {
                *abort_flag = 1;
                atomicExch(status, STATUS_WAIT_TIMEOUT);
                return false;
            }
        }
    }
}

// One lane of the (converged) warp: the branch it guards leaves the rest of the warp's code warp-uniform, so
// that operands of the guarded instructions (descriptors, addresses) can live on the uniform datapath.
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "elect.sync _|p, 0xFFFFFFFF;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(pred));
    return pred != 0;
}

// Non-blocking look at a barrier phase (no suspend, no retry): costs a fraction of a try_wait that passes.
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait with the cheap look first: for phases that have normally completed long before.
__device__ __forceinline__ bool mbar_wait_fast(uint32_t bar, uint32_t parity, volatile int *abort_flag, int *status) {
    if (mbar_test(bar, parity)) return true;
    return mbar_wait(bar, parity, abort_flag, status);
}

// ---- TMA: plain (per-CTA) tiled loads into this CTA's shared memory ----
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap *tmap, uint32_t bar,
                                            int x, int y, int z) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst), "l"(tmap), "r"(bar), "r"(x), "r"(y), "r"(z)
        : "memory");
}
// Tile in shared memory added (fp32) to the tensor in global memory; rows outside the tensor are
// clipped.  x must keep the 16-byte rule; never start a reduce at a negative coordinate.
__device__ __forceinline__ void tma_reduce_add_3d(const CUtensorMap *tmap, uint32_t src, int x, int y, int z) {
    asm volatile(
        "cp.reduce.async.bulk.tensor.3d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3, %4}], [%1];"
        ::"l"(tmap), "r"(src), "r"(x), "r"(y), "r"(z)
        : "memory");
}
// Tile in shared memory stored to the tensor in global memory (rows outside the tensor are clipped).
__device__ __forceinline__ void tma_store_3d(const CUtensorMap *tmap, uint32_t src, int x, int y, int z) {
    asm volatile(
        "cp.async.bulk.tensor.3d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4}], [%1];"
        ::"l"(tmap), "r"(src), "r"(x), "r"(y), "r"(z)
        : "memory");
}
__device__ __forceinline__ void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// all but the newest `N` groups of this thread have finished READING their shared-memory source
template <int N>
__device__ __forceinline__ void bulk_wait_group_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void bulk_wait_group() {
    asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap *tmap) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(tmap) : "memory");
}

// ---- proxy / tcgen05 fences ----
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_before() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// ---- tensor memory ----
// Whole-warp calls.  `slot` is a shared-memory word that receives the base address.
__device__ __forceinline__ void tmem_alloc(uint32_t slot, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot),
                 "r"(ncols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
                 : "memory");
}

// 32 lanes x 32 columns of 32-bit: thread i of the warp gets lane (base_lane + i).
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
          "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
          "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
// 16 lanes x 32 columns of 32-bit in the 256-bit pattern: for each group k of 8 columns, thread i gets
// columns 8k + 2(i%4) + {0,1} of lane base + i/4 in r[4k], r[4k+1] and of lane base + i/4 + 8 in
// r[4k+2], r[4k+3] -- four threads share a 32-byte piece of one row.
__device__ __forceinline__ void tmem_ld_16x256b_x4(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.16x256b.x4.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
          "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]),
          "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]),
          "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
          "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
          "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]),
          "r"(r[14]), "r"(r[15])
        : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() {
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_wait_st() {
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// ---- MMA descriptors ----
// Shared-memory operand descriptor, 128-byte swizzle, tile rows of 64 bf16 (128 B),
// 8-row groups 1024 B apart.  The same bytes serve as a K-major operand (contraction
// over the 64-element row) and as an MN-major operand (contraction over the rows).
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t saddr) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);   // start address, 16-byte units
    d |= (uint64_t)1 << 16;                     // leading-dim byte offset (unused here)
    d |= (uint64_t)(1024 >> 4) << 32;           // stride between 8-row groups
    d |= (uint64_t)1 << 46;                     // descriptor version of this architecture
    d |= (uint64_t)2 << 61;                     // 128-byte swizzle
    return d;
}

// The same tile layout read as an MN-major operand wider than one 64-element row: the next 64
// elements of the MN axis start `mn_chunk_bytes` further on (a second tile of the same shape).
__device__ __forceinline__ uint64_t smem_desc_sw128_mn(uint32_t saddr, uint32_t mn_chunk_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
    d |= (uint64_t)(mn_chunk_bytes >> 4) << 16;  // leading-dim byte offset: between 64-element chunks of the MN axis
    d |= (uint64_t)(1024 >> 4) << 32;            // stride between 8-row groups of the contraction axis
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

// Unswizzled K-major operand of 16 bf16 columns: 8 x 16-byte core matrices, the 8-row groups of the first
// 8 columns packed densely (128 B apart), the second 8 columns `k_chunk_bytes` after the first.
__device__ __forceinline__ uint64_t smem_desc_kmajor_plain(uint32_t saddr, uint32_t k_chunk_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
    d |= (uint64_t)(k_chunk_bytes >> 4) << 16;   // leading-dim byte offset: between the core matrices of the K axis
    d |= (uint64_t)(128 >> 4) << 32;             // stride between 8-row groups
    d |= (uint64_t)1 << 46;
    return d;                                    // swizzle field 0: none
}

// Vector fp32 reduction into global memory (no return value).  L2 works on 32-byte sectors: a warp
// instruction should cover whole sectors (four neighbouring lanes with 8 bytes each).
__device__ __forceinline__ void red_add_f32x2(float *dst, float a, float b) {
    asm volatile("red.global.add.v2.f32 [%0], {%1, %2};" ::"l"(dst), "f"(a), "f"(b) : "memory");
}

// Instruction descriptor for kind::f16 with bf16 operands and fp32 accumulation.
// b_mn_major: B operand is contraction-strided (rows are the contraction index).
__host__ __device__ constexpr uint32_t mma_idesc_bf16(int m, int n, bool a_mn_major,
                                                      bool b_mn_major) {
    return (1u << 4)                      // D = f32
           | (1u << 7)                    // A = bf16
           | (1u << 10)                   // B = bf16
           | ((a_mn_major ? 1u : 0u) << 15)
           | ((b_mn_major ? 1u : 0u) << 16)
           | ((uint32_t)(n >> 3) << 17)
           | ((uint32_t)(m >> 4) << 24);
}

// D[tmem] (+)= A[smem] * B[smem]
__device__ __forceinline__ void mma_ss(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc,
                                       uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]
__device__ __forceinline__ void mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc,
                                       uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Arrives on `bar` once every MMA issued so far by this thread has completed.
__device__ __forceinline__ void mma_commit(uint32_t bar) {
    asm volatile(
        "tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
        : "memory");
}

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// Packed pairs of fp32 (one 64-bit register pair per operand): half the instructions of the scalar forms.
__device__ __forceinline__ uint64_t pk2(float a, float b) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
    return r;
}
__device__ __forceinline__ void upk2(uint64_t v, float &a, float &b) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v));
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
    uint64_t r;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ uint64_t add2_rm(uint64_t a, uint64_t b) {   // round towards minus infinity
    uint64_t r;
    asm("add.rm.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
// a += lo(w), b += hi(w) for a packed pair of bf16 (fp32 sums of the ROUNDED probabilities)
__device__ __forceinline__ void add_bf16x2(uint32_t w, float &a, float &b) {
    asm("{\n\t.reg .b16 lo, hi;\n\tmov.b32 {lo, hi}, %2;\n\t"
        "add.rn.f32.bf16 %0, lo, %0;\n\tadd.rn.f32.bf16 %1, hi, %1;\n\t}"
        : "+f"(a), "+f"(b)
        : "r"(w));
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}

// 2^x for two values on the FMA and integer pipes, leaving the exp unit to the other columns: x = n + f
// with n = floor(x) (the magic-number add, rounded down, leaves n in the low mantissa bits), 2^f by a
// degree-3 polynomial (relative error 7.9e-5, far below the bf16 rounding of the probabilities), and n
// added to the exponent field.  Valid for -126 <= x < 128 and nothing else (no clamp): the caller uses it
// only where the scores are bounded, and never on masked (-inf) entries; CLAMP_LOW lifts the lower restriction
// (two more instructions per pair).
template <bool CLAMP_LOW>
__device__ __forceinline__ void ex2_poly2(float x0, float x1, float &p0, float &p1) {
    if (CLAMP_LOW) {   // for callers whose arguments are bounded above but not below (-inf included)
        x0 = fmaxf(x0, -126.0f);
        x1 = fmaxf(x1, -126.0f);
    }
    const uint64_t x = pk2(x0, x1);
    const uint64_t t = add2_rm(x, pk2(12582912.0f, 12582912.0f));          // 1.5 * 2^23 + floor(x)
    const uint64_t fl = add2(t, pk2(-12582912.0f, -12582912.0f));         // floor(x), exact
    const uint64_t f = fma2(fl, pk2(-1.0f, -1.0f), x);                    // x - floor(x) in [0, 1)
    uint64_t p = fma2(pk2(0.07806939631700516f, 0.07806939631700516f), f, pk2(0.22593535482883453f, 0.22593535482883453f));
    p = fma2(p, f, pk2(0.6959162950515747f, 0.6959162950515747f));
    p = fma2(p, f, pk2(0.9999210238456726f, 0.9999210238456726f));
    float a, b, ta, tb;
    upk2(p, a, b);
    upk2(t, ta, tb);
    p0 = __int_as_float(__float_as_int(a) + (__float_as_int(ta) << 23));
    p1 = __int_as_float(__float_as_int(b) + (__float_as_int(tb) << 23));
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}

// ---- {value, step} words of the split-KV exchange: 8-byte accesses are single-copy atomic, so a reader that
// finds the current step number in a word also has that word's value ----
__device__ __forceinline__ void st_words2(uint2 *p, float a, float b, unsigned step) {
    asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %2};" ::"l"(p), "r"(__float_as_uint(a)), "r"(step),
                 "r"(__float_as_uint(b))
                 : "memory");
}
__device__ __forceinline__ void st_word(uint2 *p, float a, unsigned step) {
    asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(__float_as_uint(a)), "r"(step) : "memory");
}
__device__ __forceinline__ uint4 ld_words2(const uint2 *p) {
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p)
                 : "memory");
    return v;
}
__device__ __forceinline__ uint2 ld_word(const uint2 *p) {
    uint2 v;
    asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
    return v;
}

}  // namespace mx
#endif  // __CUDACC__
