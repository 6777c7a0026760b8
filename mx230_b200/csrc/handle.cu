// Library state: per-device handle, workspace, status words, error strings and
// TMA tensor-map construction.  Replaces the reference's context / module plumbing
// (common/src/lib.rs:11-18, 02-flash-attention/src/main.rs:392-415).
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include <math.h>

#include "common.cuh"

static thread_local char g_err[512] = "";

void mx230_set_error(const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

int mx230_fail(int code, const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

extern "C" int mx230_abi_version(void) { return MX230_ABI_VERSION; }

extern "C" const char *mx230_last_error(void) { return g_err; }

extern "C" const char *mx230_status_string(int code) {
    switch (code) {
        case MX230_OK: return "ok";
        case MX230_ERR_INVALID_ARG: return "invalid argument";
        case MX230_ERR_UNSUPPORTED: return "unsupported shape or option";
        case MX230_ERR_WORKSPACE: return "workspace too small";
        case MX230_ERR_CUDA: return "CUDA call failed";
        case MX230_ERR_DEVICE_STATUS: return "device-side bounded wait timed out";
        case MX230_ERR_NO_DEVICE: return "no sm_100 device";
        default: return "unknown status";
    }
}

static const size_t N_COUNTERS = 1 << 16;

extern "C" int mx230_create(mx230_handle **out, int device, size_t workspace_bytes) {
    MX_REQUIRE(out != nullptr, MX230_ERR_INVALID_ARG, "mx230_create: out is null");
    *out = nullptr;
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || count == 0) {
        cudaGetLastError();
        return mx230_fail(MX230_ERR_NO_DEVICE, "mx230_create: no CUDA device visible");
    }
    MX_REQUIRE(device >= 0 && device < count, MX230_ERR_INVALID_ARG,
               "mx230_create: device %d out of range (0..%d)", device, count - 1);
    cudaDeviceProp prop;
    MX_CHECK_CUDA(cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10)
        return mx230_fail(MX230_ERR_NO_DEVICE,
                          "mx230_create: device %d is sm_%d%d; this library is built for sm_100a only",
                          device, prop.major, prop.minor);
    mx230_device_guard guard(device);
    MX_CHECK_CUDA(cudaSetDevice(device));

    mx230_handle *h = new mx230_handle();
    memset(h, 0, sizeof(*h));
    h->device = device;
    h->sm_count = prop.multiProcessorCount;
    h->q8_score_mode = MX230_Q8_SCORE_REF;
    h->decode_tensor = 1;
    h->n_counters = N_COUNTERS;

    void *fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
    if (e != cudaSuccess || fn == nullptr || qres != cudaDriverEntryPointSuccess) {
        delete h;
        return mx230_fail(MX230_ERR_CUDA, "mx230_create: cuTensorMapEncodeTiled unavailable");
    }
    h->encode_tiled = (mx230_encode_tiled_fn)fn;

    if (cudaMalloc(&h->status_dev, 8 * sizeof(int)) != cudaSuccess ||
        cudaMalloc(&h->counters, N_COUNTERS * sizeof(unsigned)) != cudaSuccess) {
        delete h;
        return mx230_fail(MX230_ERR_CUDA, "mx230_create: cudaMalloc of status words failed");
    }
    cudaMemset(h->status_dev, 0, 8 * sizeof(int));
    {
        const long long limit = 4000000000ll;   // bound of a device-side wait in SM cycles (mx::WAIT_LIMIT_CYCLES)
        cudaMemcpy(h->status_dev + 4, &limit, sizeof(limit), cudaMemcpyHostToDevice);
    }
    h->test_drop_tile = -1;
    cudaMemset(h->counters, 0, N_COUNTERS * sizeof(unsigned));
    if (workspace_bytes > 0) {
        if (cudaMalloc(&h->ws, workspace_bytes) != cudaSuccess) {
            cudaGetLastError();
            cudaFree(h->status_dev);
            cudaFree(h->counters);
            delete h;
            return mx230_fail(MX230_ERR_CUDA, "mx230_create: cudaMalloc(%zu) for the workspace failed",
                              workspace_bytes);
        }
        h->ws_bytes = workspace_bytes;
    }
    MX_CHECK_CUDA(cudaDeviceSynchronize());
    *out = h;
    return MX230_OK;
}

extern "C" int mx230_destroy(mx230_handle *h) {
    if (h == nullptr) return MX230_OK;
    mx230_device_guard guard(h->device);
    cudaDeviceSynchronize();
    if (h->ws) cudaFree(h->ws);
    if (h->status_dev) cudaFree(h->status_dev);
    if (h->counters) cudaFree(h->counters);
    if (h->prof_ev) {
        for (int i = 0; i < 2 * MX230_PROF_CAP; ++i)
            if (h->prof_ev[i]) cudaEventDestroy(h->prof_ev[i]);
        delete[] h->prof_ev;
        delete[] h->prof_kid;
    }
    delete h;
    return MX230_OK;
}

extern "C" int mx230_reserve(mx230_handle *h, size_t bytes) {
    MX_REQUIRE(h != nullptr, MX230_ERR_INVALID_ARG, "mx230_reserve: null handle");
    if (bytes <= h->ws_bytes) return MX230_OK;
    mx230_device_guard guard(h->device);
    MX_CHECK_CUDA(cudaDeviceSynchronize());
    if (h->ws) cudaFree(h->ws);
    h->ws = nullptr;
    h->ws_bytes = 0;
    h->staged.valid = 0;   // whatever was staged went with the old workspace
    MX_CHECK_CUDA(cudaMalloc(&h->ws, bytes));
    h->ws_bytes = bytes;
    return MX230_OK;
}

extern "C" int mx230_set_option(mx230_handle *h, int option, int value) {
    MX_REQUIRE(h != nullptr, MX230_ERR_INVALID_ARG, "mx230_set_option: null handle");
    switch (option) {
        case MX230_OPT_Q8_SCORE_MODE:
            MX_REQUIRE(value == MX230_Q8_SCORE_REF || value == MX230_Q8_SCORE_EXACT,
                       MX230_ERR_INVALID_ARG, "mx230_set_option: bad q8 score mode %d", value);
            h->q8_score_mode = value;
            return MX230_OK;
        case MX230_OPT_DECODE_CHUNK:
            MX_REQUIRE(value >= 0 && value <= 2048 && value % 128 == 0, MX230_ERR_INVALID_ARG,
                       "mx230_set_option: decode chunk must be 0 or a multiple of 128 up to 2048");
            h->decode_chunk = value;
            return MX230_OK;
        case MX230_OPT_DECODE_TENSOR:
            MX_REQUIRE(value == 0 || value == 1, MX230_ERR_INVALID_ARG,
                       "mx230_set_option: decode tensor switch must be 0 or 1");
            h->decode_tensor = value;
            return MX230_OK;
        case MX230_OPT_BWD_TWO_PASS:
            MX_REQUIRE(value == 0 || value == 1, MX230_ERR_INVALID_ARG,
                       "mx230_set_option: backward two-pass switch must be 0 or 1");
            h->bwd_two_pass = value;
            return MX230_OK;
        case MX230_OPT_BWD_REUSE_STAGED:
            MX_REQUIRE(value == 0 || value == 1, MX230_ERR_INVALID_ARG,
                       "mx230_set_option: backward staging-reuse switch must be 0 or 1");
            h->bwd_reuse_staged = value;
            return MX230_OK;
        case MX230_OPT_WAIT_LIMIT: {
            MX_REQUIRE(value >= 1, MX230_ERR_INVALID_ARG, "mx230_set_option: wait limit must be at least 1 (thousand cycles)");
            mx230_device_guard guard(h->device);
            MX_CHECK_CUDA(cudaDeviceSynchronize());
            const long long limit = 1000ll * value;
            MX_CHECK_CUDA(cudaMemcpy(h->status_dev + 4, &limit, sizeof(limit), cudaMemcpyHostToDevice));
            return MX230_OK;
        }
        case MX230_OPT_TEST_DROP_TILE:
            MX_REQUIRE(value >= -1, MX230_ERR_INVALID_ARG, "mx230_set_option: tile index %d", value);
            h->test_drop_tile = value;
            return MX230_OK;
        default:
            return mx230_fail(MX230_ERR_INVALID_ARG, "mx230_set_option: unknown option %d", option);
    }
}

extern "C" size_t mx230_flash_workspace_bytes(int batch_heads, int n, int with_backward) {
    if (batch_heads <= 0 || n <= 0) return 0;
    return mx230_flash_stage_bytes(batch_heads, n) * (with_backward ? 4 : 3) + mx230_flash_norm_bytes(batch_heads);
}

extern "C" size_t mx230_decode_workspace_bytes(int n_seq, int n_head, int max_splits) {
    if (n_seq <= 0 || n_head <= 0 || max_splits <= 0) return 0;
    return (size_t)n_seq * n_head * max_splits * 66 * sizeof(float);
}

extern "C" int mx230_check_status(mx230_handle *h, void *stream) {
    MX_REQUIRE(h != nullptr, MX230_ERR_INVALID_ARG, "mx230_check_status: null handle");
    mx230_device_guard guard(h->device);
    MX_CHECK_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
    int st[4] = {0, 0, 0, 0};
    MX_CHECK_CUDA(cudaMemcpy(st, h->status_dev, sizeof(st), cudaMemcpyDeviceToHost));
    if (st[0] != 0 || st[1] != 0) {
        cudaMemset(h->status_dev, 0, sizeof(st));
        return mx230_fail(MX230_ERR_DEVICE_STATUS,
                          "device status %d (1 = bounded wait timed out), detail %d", st[0], st[1]);
    }
    return MX230_OK;
}

// ---- seeded input generators (host code) ----
static inline uint64_t xorshift64star(uint64_t &s) {
    s ^= s >> 12;
    s ^= s << 25;
    s ^= s >> 27;
    return s * 0x2545F4914F6CDD1DULL;
}

extern "C" int mx230_pseudo_rand(float *out_host, size_t n, uint64_t seed) {
    MX_REQUIRE(out_host != nullptr || n == 0, MX230_ERR_INVALID_ARG, "pseudo_rand: null output");
    uint64_t s = seed;
    for (size_t i = 0; i < n; ++i) out_host[i] = (float)(xorshift64star(s) >> 40) / (float)(1ULL << 23) - 1.0f;
    return MX230_OK;
}

extern "C" int mx230_fill_normal(float *out_host, size_t n, uint64_t seed, uint64_t tensor_index) {
    MX_REQUIRE(out_host != nullptr || n == 0, MX230_ERR_INVALID_ARG, "fill_normal: null output");
    uint64_t s = seed * 16u + tensor_index;   // splitmix64 step: the generator's state must not be zero
    s += 0x9E3779B97F4A7C15ULL;
    s = (s ^ (s >> 30)) * 0xBF58476D1CE4E5B9ULL;
    s = (s ^ (s >> 27)) * 0x94D049BB133111EBULL;
    s ^= s >> 31;
    if (s == 0) s = 0x9E3779B97F4A7C15ULL;
    for (size_t i = 0; i < n; i += 2) {
        const double u1 = ((double)(xorshift64star(s) >> 11) + 1.0) / 9007199254740992.0;   // (0, 1]
        const double u2 = ((double)(xorshift64star(s) >> 11) + 1.0) / 9007199254740992.0;
        const double r = sqrt(-2.0 * log(u1)), a = 6.283185307179586476925 * u2;
        out_host[i] = (float)(r * cos(a));
        if (i + 1 < n) out_host[i + 1] = (float)(r * sin(a));
    }
    return MX230_OK;
}

int mx230_prof_begin(mx230_handle *h, cudaStream_t st, int kid) {
    if (h->prof_used >= MX230_PROF_CAP) return -1;
    if (h->prof_ev == nullptr) {
        h->prof_ev = new cudaEvent_t[2 * MX230_PROF_CAP];
        h->prof_kid = new int[MX230_PROF_CAP];
        for (int i = 0; i < 2 * MX230_PROF_CAP; ++i) h->prof_ev[i] = nullptr;
    }
    int slot = h->prof_used;
    for (int j = 0; j < 2; ++j)
        if (h->prof_ev[2 * slot + j] == nullptr && cudaEventCreate(&h->prof_ev[2 * slot + j]) != cudaSuccess)
            return -1;
    h->prof_used++;
    h->prof_kid[slot] = kid;
    cudaEventRecord(h->prof_ev[2 * slot], st);
    return slot;
}

void mx230_prof_end(mx230_handle *h, cudaStream_t st, int slot) {
    cudaEventRecord(h->prof_ev[2 * slot + 1], st);
}

// Folds the recorded event pairs into the per-kernel totals (synchronises on them).
static int prof_drain(mx230_handle *h) {
    for (int i = 0; i < h->prof_used; ++i) {
        MX_CHECK_CUDA(cudaEventSynchronize(h->prof_ev[2 * i + 1]));
        float ms = 0.0f;
        MX_CHECK_CUDA(cudaEventElapsedTime(&ms, h->prof_ev[2 * i], h->prof_ev[2 * i + 1]));
        h->prof_ms[h->prof_kid[i]] += ms;
        h->prof_count[h->prof_kid[i]]++;
    }
    h->prof_used = 0;
    return MX230_OK;
}

extern "C" int mx230_profile_enable(mx230_handle *h, int on) {
    MX_REQUIRE(h != nullptr, MX230_ERR_INVALID_ARG, "mx230_profile_enable: null handle");
    mx230_device_guard guard(h->device);
    if (!on && h->prof_on) {
        int rc = prof_drain(h);
        if (rc) return rc;
    }
    h->prof_on = on ? 1 : 0;
    return MX230_OK;
}

extern "C" int mx230_profile_reset(mx230_handle *h) {
    MX_REQUIRE(h != nullptr, MX230_ERR_INVALID_ARG, "mx230_profile_reset: null handle");
    mx230_device_guard guard(h->device);
    int rc = prof_drain(h);
    if (rc) return rc;
    for (int k = 0; k < MX230_K_COUNT; ++k) {
        h->prof_count[k] = 0;
        h->prof_ms[k] = 0.0;
    }
    return MX230_OK;
}

extern "C" int mx230_profile_read(mx230_handle *h, int kernel, long long *launches, double *total_ms) {
    MX_REQUIRE(h != nullptr && launches && total_ms, MX230_ERR_INVALID_ARG, "mx230_profile_read: null argument");
    MX_REQUIRE(kernel >= 0 && kernel < MX230_K_COUNT, MX230_ERR_INVALID_ARG,
               "mx230_profile_read: kernel id %d out of range", kernel);
    mx230_device_guard guard(h->device);
    int rc = prof_drain(h);
    if (rc) return rc;
    *launches = h->prof_count[kernel];
    *total_ms = h->prof_ms[kernel];
    return MX230_OK;
}

extern "C" const char *mx230_kernel_name(int kernel) {
    static const char *names[MX230_K_COUNT] = {
        "cast_bf16_kernel", "flash_fwd_kernel", "bwd_preprocess_kernel", "bwd_dq_kernel",
        "bwd_dkv_kernel", "rope_kernel", "copy_kv_kernel", "quantize_kv_kernel",
        "decode_f32_kernel", "decode_q8_kernel", "merge_partials_kernel", "prefill_stage_kernels",
        "gemv_heads_kernel", "bwd_fused_kernel"};
    return (kernel >= 0 && kernel < MX230_K_COUNT) ? names[kernel] : "?";
}

extern "C" long long mx230_launch_count(const mx230_handle *h) { return h ? h->launches : 0; }

int mx230_make_tmap_bf16(mx230_handle *h, CUtensorMap *out, const void *base, uint64_t rows,
                         uint64_t outer, uint64_t row_stride_bytes, uint64_t outer_stride_bytes,
                         uint32_t box_rows) {
    MX_REQUIRE(((uintptr_t)base & 15) == 0, MX230_ERR_INVALID_ARG,
               "tensor map base %p is not 16-byte aligned", base);
    MX_REQUIRE(row_stride_bytes % 16 == 0 && outer_stride_bytes % 16 == 0, MX230_ERR_INVALID_ARG,
               "tensor map strides must be multiples of 16 bytes");
    cuuint64_t dims[3] = {64, rows, outer};
    cuuint64_t strides[2] = {row_stride_bytes, outer_stride_bytes};
    cuuint32_t box[3] = {64, box_rows, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = h->encode_tiled(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void *>(base),
                                 dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                 CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                 CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return mx230_fail(MX230_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    return MX230_OK;
}

// 16-bit (bf16 or fp16) matrix [rows][inner], rows `row_stride_bytes` apart, as a three-dimensional map with an outer
// extent of 1 (the kernels' load helper is the 3-D form): boxes of box_inner x box_rows elements, 128-byte swizzle
// (box_inner * 2 <= 128), zero fill outside the matrix.
int mx230_make_tmap_2d_16bit(mx230_handle *h, CUtensorMap *out, const void *base, int fp16, uint64_t inner,
                             uint64_t rows, uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_rows) {
    MX_REQUIRE(((uintptr_t)base & 15) == 0, MX230_ERR_INVALID_ARG, "tensor map base %p is not 16-byte aligned", base);
    MX_REQUIRE(row_stride_bytes % 16 == 0 && box_inner * 2 <= 128 && box_rows <= 256, MX230_ERR_INVALID_ARG,
               "tensor map: row stride must be a multiple of 16 bytes and the box at most 128 bytes x 256 rows");
    cuuint64_t dims[3] = {inner, rows, 1};
    cuuint64_t strides[2] = {row_stride_bytes, row_stride_bytes * rows};
    cuuint32_t box[3] = {box_inner, box_rows, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = h->encode_tiled(out, fp16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3,
                                 const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                 CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                 CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return mx230_fail(MX230_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    return MX230_OK;
}

// fp32 [outer][rows][64] seen as 128-byte half rows: boxes of 32 rows x 32 floats, 128-byte swizzle
// (the staging layout of the fused backward's dQ reductions).
int mx230_make_tmap_f32_half_rows(mx230_handle *h, CUtensorMap *out, const void *base, uint64_t rows,
                                  uint64_t outer) {
    return mx230_make_tmap_f32_half_rows_strided(h, out, base, rows, outer, 64 * sizeof(float),
                                                 rows * 64 * sizeof(float));
}

// the same with the row and outer strides given in bytes (multiples of 16)
int mx230_make_tmap_f32_half_rows_strided(mx230_handle *h, CUtensorMap *out, const void *base, uint64_t rows,
                                          uint64_t outer, uint64_t row_stride_bytes, uint64_t outer_stride_bytes) {
    MX_REQUIRE(((uintptr_t)base & 15) == 0, MX230_ERR_INVALID_ARG,
               "tensor map base %p is not 16-byte aligned", base);
    MX_REQUIRE(row_stride_bytes % 16 == 0 && outer_stride_bytes % 16 == 0, MX230_ERR_INVALID_ARG,
               "tensor map strides must be multiples of 16 bytes");
    cuuint64_t dims[3] = {64, rows, outer};
    cuuint64_t strides[2] = {row_stride_bytes, outer_stride_bytes};
    cuuint32_t box[3] = {32, 32, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = h->encode_tiled(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<void *>(base),
                                 dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                 CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                 CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return mx230_fail(MX230_ERR_CUDA, "cuTensorMapEncodeTiled (fp32) failed with CUresult %d", (int)r);
    return MX230_OK;
}
