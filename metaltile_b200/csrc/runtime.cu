// Runtime behind include/mtcuda.h: context, device memory, the typed entry points and
// the name-keyed host-buffer dispatch that mirrors Context::dispatch_with_grid
// (crates/metaltile-runtime/src/context.rs:269-284).
#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <map>
#include <string>
#include <thread>
#include <vector>

#include "common.cuh"

using mtc::Ctx;
using mtc::fail;

struct mtc_ctx : public Ctx {};

namespace {

thread_local std::string g_no_ctx_error;

#define MTC_CUDA(ctx, expr, code)                                                              \
    do {                                                                                       \
        cudaError_t e__ = (expr);                                                              \
        if (e__ != cudaSuccess)                                                                \
            return fail(ctx, code, std::string(#expr) + ": " + cudaGetErrorString(e__));      \
    } while (0)

// Every entry runs with its context's device current: one host thread may drive contexts on several devices.
#define MTC_ENTER(ctx)                                                                                  \
    do {                                                                                                \
        int cur__ = -1;                                                                                 \
        if (cudaGetDevice(&cur__) != cudaSuccess || cur__ != (ctx)->device) {                           \
            cudaError_t e__ = cudaSetDevice((ctx)->device);                                             \
            if (e__ != cudaSuccess)                                                                     \
                return fail(ctx, MTC_ERR_NO_DEVICE, std::string("cudaSetDevice: ") + cudaGetErrorString(e__)); \
        }                                                                                               \
    } while (0)

bool dtype_ok(int dt) { return dt == MTC_F32 || dt == MTC_F16 || dt == MTC_BF16; }

// ---- kernel-name registry ------------------------------------------------------
// One row per reference kernel name the back end accepts.  `bits` < 0 means "not a
// dense kernel".  gs_const names the constexpr that carries the grouping:
// "gs_per_row" (hand-tuned int4/int8/mma kernels: group_size = k / gs_per_row) or
// "group_size" (generic _b* family).  has_n: whether an `n` constexpr is bound
// (mt_qmv / mt_qmv_int8_fast take N from the size of `out`).
enum Family { DENSE_QMV, DENSE_QMM, GATHER_CSR, GATHER_IDX, ROUTER_TOPK, MOE_PERMUTE, MOE_UNPERMUTE, SWIGLU, BATCHED_QKV, BATCHED_4, RMS_QMV, AFFINE_Q, AFFINE_DQ, DQ_GATHER, QVM, MOE_TAIL, EXPERT_QMV };
struct KernelRow {
    const char *name;
    Family family;
    int bits;
    const char *gs_const;
    bool has_n;
};
const KernelRow kKernels[] = {
    // crates/metaltile-std/src/mlx/quantized.rs:7,1475 (qmv), :343,650,1072,1602,1719,1870 (qmm bm1/2/4)
    {"mt_qmv", DENSE_QMV, 4, "gs_per_row", false},
    {"mt_qmv_int8_fast", DENSE_QMV, 8, "gs_per_row", false},
    {"mt_qmm", DENSE_QMV, 4, "gs_per_row", true},
    {"mt_qmm_bm2", DENSE_QMV, 4, "gs_per_row", true},
    {"mt_qmm_bm4", DENSE_QMV, 4, "gs_per_row", true},
    {"mt_qmm_int8_fast", DENSE_QMV, 8, "gs_per_row", true},
    {"mt_qmm_bm2_int8_fast", DENSE_QMV, 8, "gs_per_row", true},
    {"mt_qmm_bm4_int8_fast", DENSE_QMV, 8, "gs_per_row", true},
    // :2106,2408,2731,2990,3330 and the bit-stream MMA family :4720-5012
    {"mt_qmm_mma", DENSE_QMM, 4, "gs_per_row", true},
    {"mt_qmm_mma_m16", DENSE_QMM, 4, "gs_per_row", true},
    {"mt_qmm_mma_int8", DENSE_QMM, 8, "gs_per_row", true},
    {"mt_qmm_mma_m16_int8", DENSE_QMM, 8, "gs_per_row", true},
    {"mt_qmm_mma_int2", DENSE_QMM, 2, "gs_per_row", true},
    {"mt_qmm_mma_b3", DENSE_QMM, 3, "gs_per_row", true},
    {"mt_qmm_mma_b5", DENSE_QMM, 5, "gs_per_row", true},
    {"mt_qmm_mma_b6", DENSE_QMM, 6, "gs_per_row", true},
    // generic any-bits family :4273-4392, instantiated :4510-4523
    {"mt_qmv_b3", DENSE_QMV, 3, "group_size", true},
    {"mt_qmv_b4", DENSE_QMV, 4, "group_size", true},
    {"mt_qmv_b5", DENSE_QMV, 5, "group_size", true},
    {"mt_qmv_b6", DENSE_QMV, 6, "group_size", true},
    {"mt_qmv_b8", DENSE_QMV, 8, "group_size", true},
    {"mt_qmm_b3", DENSE_QMV, 3, "group_size", true},
    {"mt_qmm_b4", DENSE_QMV, 4, "group_size", true},
    {"mt_qmm_b5", DENSE_QMV, 5, "group_size", true},
    {"mt_qmm_b6", DENSE_QMV, 6, "group_size", true},
    {"mt_qmm_b8", DENSE_QMV, 8, "group_size", true},
    // decode projections that share x: crates/metaltile-std/src/ffai/batched_qkv_qgemv.rs:40-57,141-158 (one
    // concatenated out), crates/metaltile-std/src/ffai/batched_4_qgemv.rs:59-84 (four outputs)
    {"ffai_batched_qkv_qgemv", BATCHED_QKV, 4, "group_size", false},
    {"ffai_batched_qkv_qgemv_fast", BATCHED_QKV, 4, "group_size", false},
    {"ffai_batched_4_qgemv_fast", BATCHED_4, 4, "group_size", false},
    // RMSNorm fused into the decode projection: crates/metaltile-std/src/ffai/rms_norm_qgemv.rs:51-107,131-146
    {"ffai_rms_norm_qgemv", RMS_QMV, 4, "group_size", false},
    {"ffai_rms_norm_qgemv_fast", RMS_QMV, 4, "group_size", false},
    // the codec: crates/metaltile-std/src/mlx/quantized.rs:3575-4214
    {"mt_affine_quantize_int2", AFFINE_Q, 2, "group_size", false},
    {"mt_affine_quantize_int3", AFFINE_Q, 3, "group_size", false},
    {"mt_affine_quantize_int4", AFFINE_Q, 4, "group_size", false},
    {"mt_affine_quantize_int5", AFFINE_Q, 5, "group_size", false},
    {"mt_affine_quantize_int6", AFFINE_Q, 6, "group_size", false},
    {"mt_affine_quantize_int8", AFFINE_Q, 8, "group_size", false},
    {"mt_affine_dequantize_int2", AFFINE_DQ, 2, "group_size", false},
    {"mt_affine_dequantize_int3", AFFINE_DQ, 3, "group_size", false},
    {"mt_affine_dequantize_int4", AFFINE_DQ, 4, "group_size", false},
    {"mt_affine_dequantize_int5", AFFINE_DQ, 5, "group_size", false},
    {"mt_affine_dequantize_int6", AFFINE_DQ, 6, "group_size", false},
    {"mt_affine_dequantize_int8", AFFINE_DQ, 8, "group_size", false},
    // M = 1 MoE decode tail: crates/metaltile-std/src/ffai/moe_down_swiglu_accum.rs:158-318, ffai/dequant_gemv_expert_indexed.rs:56-103
    {"ffai_moe_down_swiglu_accum_int4_chain8", MOE_TAIL, 4, "group_size", false},
    {"dequant_gemv_int4_expert_indexed", EXPERT_QMV, 4, "group_size", false},
    // vecmat, transposed weights: crates/metaltile-std/src/mlx/quantized.rs:4397-4530,4582-4700
    {"mt_qvm_b3", QVM, 3, "group_size", true},
    {"mt_qvm_b4", QVM, 4, "group_size", true},
    {"mt_qvm_b5", QVM, 5, "group_size", true},
    {"mt_qvm_b6", QVM, 6, "group_size", true},
    {"mt_qvm_b8", QVM, 8, "group_size", true},
    {"mt_qvm_int4_fast", QVM, 4, "gs_per_col", true},
    // quantized embedding tables: crates/metaltile-std/src/ffai/dequant_gather.rs:44-101
    {"dequant_gather_int2", DQ_GATHER, 2, "group_size", false},
    {"dequant_gather_int3", DQ_GATHER, 3, "group_size", false},
    {"dequant_gather_int4", DQ_GATHER, 4, "group_size", false},
    {"dequant_gather_int5", DQ_GATHER, 5, "group_size", false},
    {"dequant_gather_int6", DQ_GATHER, 6, "group_size", false},
    {"dequant_gather_int8", DQ_GATHER, 8, "group_size", false},
    // MoE: crates/metaltile-std/src/ffai/moe.rs:65,222,283 (routing), :358,602-605,634,900,1363 (CSR gather),
    // :2256,2832-2835,2857,3231 (per-row-index gather); crates/metaltile-std/src/mlx/swiglu.rs:45
    {"mt_moe_router_topk", ROUTER_TOPK, -1, "", false},
    {"mt_moe_permute", MOE_PERMUTE, -1, "", false},
    {"mt_moe_unpermute", MOE_UNPERMUTE, -1, "", false},
    {"mt_swiglu", SWIGLU, -1, "", false},
    {"mt_moe_gather_qmm_int4", GATHER_CSR, 4, "group_size", false},
    {"mt_moe_gather_qmm_int4_m8", GATHER_CSR, 4, "group_size", false},
    {"mt_moe_gather_qmm_int4_m16", GATHER_CSR, 4, "group_size", false},
    {"mt_moe_gather_qmm_int4_m32", GATHER_CSR, 4, "group_size", false},
    {"mt_moe_gather_qmm_b3", GATHER_CSR, 3, "group_size", false},
    {"mt_moe_gather_qmm_b5", GATHER_CSR, 5, "group_size", false},
    {"mt_moe_gather_qmm_b6", GATHER_CSR, 6, "group_size", false},
    {"mt_moe_gather_qmm_b8", GATHER_CSR, 8, "group_size", false},
    {"mt_moe_gather_qmm_mma_int4", GATHER_IDX, 4, "group_size", false},
    {"mt_moe_gather_qmm_mma_int4_bm16", GATHER_IDX, 4, "group_size", false},
    {"mt_moe_gather_qmm_mma_int8", GATHER_IDX, 8, "group_size", false},
    {"mt_moe_gather_qmm_mma_b3", GATHER_IDX, 3, "group_size", false},
    {"mt_moe_gather_qmm_mma_b5", GATHER_IDX, 5, "group_size", false},
    {"mt_moe_gather_qmm_mma_b6", GATHER_IDX, 6, "group_size", false},
    {"mt_moe_gather_qmm_mma_b8", GATHER_IDX, 8, "group_size", false},
};
constexpr int kNumKernels = sizeof(kKernels) / sizeof(kKernels[0]);

const KernelRow *find_kernel(const char *name) {
    for (int i = 0; i < kNumKernels; ++i)
        if (std::strcmp(kKernels[i].name, name) == 0) return &kKernels[i];
    return nullptr;
}

mtc_named_buf *find_buf(mtc_named_buf *bufs, int n, const char *name) {
    for (int i = 0; i < n; ++i)
        if (bufs[i].name && std::strcmp(bufs[i].name, name) == 0) return &bufs[i];
    return nullptr;
}

bool read_const(mtc_named_buf *bufs, int n, const char *name, uint32_t *out) {
    mtc_named_buf *b = find_buf(bufs, n, name);
    if (!b || b->bytes < 4 || !b->data) return false;
    std::memcpy(out, b->data, 4);  // little-endian 4-byte uniform (run_kernel.rs:56-65)
    return true;
}

constexpr size_t kTcCounterBytes = 1u << 20;       // (tile, quarter) counters of the tcgen05 decode kernel: N up to 8 Mi rows

// Partial-sum planes of the tcgen05 decode kernel.  Grow-only; an outgrown block is kept until mtc_destroy, so a CUDA
// graph captured earlier never reads freed memory.  Growing allocates: not during stream capture.
// Option "qmv_stream": 1 (default) = the streaming decode kernel takes M = 1, where it is the fastest kernel of the
// library; 2 = every M <= 8 it supports (at 2 <= M <= 8 the register-ring kernel of qmv_mma.cu is faster: measured
// 13.3 against 21.7 us on 14336 x 4096 at M = 8); 0 = never.
inline bool stream_takes(const Ctx *ctx, int M) { return ctx->qmv_stream == 2 ? M <= 8 : (ctx->qmv_stream == 1 && M == 1); }
// A single projection on its own launch: below 8 Mi codes the CUDA-core kernel is the faster one (measured at M = 1:
// 1024 x 4096 3.4 against 3.9 us, 2048 x 2048 2.8 against 3.8, 4096 x 4096 5.5 = 5.4, 14336 x 4096 12.5 against 10.7).
constexpr long long kStreamMinCodes = 8ll << 20;
inline bool stream_takes_single(const Ctx *ctx, int M, int N, int K) {
    return stream_takes(ctx, M) && (ctx->qmv_stream == 2 || static_cast<long long>(N) * K >= kStreamMinCodes);
}

int ensure_tc_scratch(Ctx *ctx, size_t bytes, cudaStream_t st) {
    if (bytes <= ctx->tc_scratch_bytes) return MTC_OK;
    cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(st, &cs) == cudaSuccess && cs != cudaStreamCaptureStatusNone)
        return fail(ctx, MTC_ERR_BUFFER, "qmv: the partial-sum scratch has to grow, which cannot happen during stream capture; "
                                          "run the shape once before capturing");
    const size_t want = bytes + (bytes >> 1) + (1u << 20);
    void *p = nullptr;
    MTC_CUDA(ctx, cudaMalloc(&p, want), MTC_ERR_BUFFER);
    if (ctx->d_tc_scratch) ctx->retired.push_back(ctx->d_tc_scratch);
    ctx->d_tc_scratch = static_cast<float *>(p);
    ctx->tc_scratch_bytes = want;
    return MTC_OK;
}

int ensure_scratch(Ctx *ctx, size_t bytes) {
    if (bytes <= ctx->scratch_bytes) return MTC_OK;
    if (ctx->d_scratch) cudaFree(ctx->d_scratch);
    ctx->d_scratch = nullptr;
    ctx->scratch_bytes = 0;
    size_t want = bytes + (bytes >> 2) + (1u << 20);
    MTC_CUDA(ctx, cudaMalloc(&ctx->d_scratch, want), MTC_ERR_BUFFER);
    ctx->scratch_bytes = want;
    return MTC_OK;
}

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

int ensure_worklist(Ctx *ctx, size_t bytes, cudaStream_t st) {
    std::string why;
    cudaError_t e = mtc::grow_block(ctx, st, &ctx->d_worklist, &ctx->worklist_bytes, bytes, &why);
    if (e != cudaSuccess) return fail(ctx, MTC_ERR_BUFFER, "gather_qmm work list: " + (why.empty() ? std::string(cudaGetErrorString(e)) : why));
    return MTC_OK;
}

// One named host buffer staged in the context's scratch block for mtc_dispatch.
struct Staged {
    mtc_named_buf *buf;
    size_t need;       // bytes the kernel touches (checked against buf->bytes)
    size_t offset;     // offset in scratch
    char *dev;
};

}  // namespace

extern "C" {

int mtc_init(int device, mtc_ctx **out_ctx) {
    if (!out_ctx) return MTC_ERR_INVALID;
    *out_ctx = nullptr;
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || count == 0) {
        g_no_ctx_error = std::string("no CUDA device: ") + cudaGetErrorString(e);
        return MTC_ERR_NO_DEVICE;
    }
    if (device < 0 || device >= count) {
        g_no_ctx_error = "device index out of range";
        return MTC_ERR_NO_DEVICE;
    }
    if ((e = cudaSetDevice(device)) != cudaSuccess) {
        g_no_ctx_error = std::string("cudaSetDevice: ") + cudaGetErrorString(e);
        return MTC_ERR_NO_DEVICE;
    }
    cudaDeviceProp prop{};
    cudaGetDeviceProperties(&prop, device);
    if (prop.major != 10) {
        g_no_ctx_error = "this library is built for sm_100a (B200) only; found compute capability " +
                         std::to_string(prop.major) + "." + std::to_string(prop.minor);
        return MTC_ERR_NO_DEVICE;
    }
    mtc_ctx *ctx = new mtc_ctx();
    ctx->device = device;
    ctx->sm_count = prop.multiProcessorCount;
    ctx->l2_bytes = static_cast<size_t>(prop.l2CacheSize);
    if ((e = cudaMalloc(&ctx->d_status, sizeof(uint32_t))) != cudaSuccess ||
        (e = cudaMemset(ctx->d_status, 0, sizeof(uint32_t))) != cudaSuccess ||
        (e = mtc::qmv_init_device()) != cudaSuccess ||
        (e = mtc::qmv_stream_init_device()) != cudaSuccess ||
        (e = mtc::qmv_tc_init_device()) != cudaSuccess ||
        (e = cudaMalloc(&ctx->d_tc_counters, kTcCounterBytes)) != cudaSuccess ||
        (e = cudaMemset(ctx->d_tc_counters, 0, kTcCounterBytes)) != cudaSuccess ||
        (e = cudaMalloc(&ctx->d_worklist, 4u << 20)) != cudaSuccess) {
        g_no_ctx_error = std::string("context set-up: ") + cudaGetErrorString(e);
        delete ctx;
        return MTC_ERR_DISPATCH;
    }
    ctx->worklist_bytes = 4u << 20;
    *out_ctx = ctx;
    return MTC_OK;
}

int mtc_destroy(mtc_ctx *ctx) {
    if (!ctx) return MTC_ERR_INVALID;
    cudaSetDevice(ctx->device);
    if (ctx->d_status) cudaFree(ctx->d_status);
    if (ctx->d_scratch) cudaFree(ctx->d_scratch);
    if (ctx->d_worklist) cudaFree(ctx->d_worklist);
    if (ctx->d_xconv) cudaFree(ctx->d_xconv);
    if (ctx->d_gfrag) cudaFree(ctx->d_gfrag);
    if (ctx->d_moe) cudaFree(ctx->d_moe);
    if (ctx->d_norm) cudaFree(ctx->d_norm);
    if (ctx->d_qvm) cudaFree(ctx->d_qvm);
    if (ctx->d_tail) cudaFree(ctx->d_tail);
    if (ctx->d_flush) cudaFree(ctx->d_flush);
    if (ctx->d_ksplit) cudaFree(ctx->d_ksplit);
    if (ctx->d_tc_scratch) cudaFree(ctx->d_tc_scratch);
    if (ctx->d_tc_counters) cudaFree(ctx->d_tc_counters);
    for (void *p : ctx->retired) cudaFree(p);
    delete ctx;
    return MTC_OK;
}

const char *mtc_last_error(mtc_ctx *ctx) { return ctx ? ctx->last_error.c_str() : g_no_ctx_error.c_str(); }

int mtc_device_info(mtc_ctx *ctx, char *json, size_t cap) {
    if (!ctx || !json || cap == 0) return MTC_ERR_INVALID;
    MTC_ENTER(ctx);
    cudaDeviceProp prop{};
    MTC_CUDA(ctx, cudaGetDeviceProperties(&prop, ctx->device), MTC_ERR_NO_DEVICE);
    int drv = 0, rt = 0;
    cudaDriverGetVersion(&drv);
    cudaRuntimeGetVersion(&rt);
    int n = std::snprintf(json, cap,
                          "{\"device\": \"%s\", \"gpu_family\": \"sm_%d%d\", \"sm_count\": %d, \"cc\": \"%d.%d\", "
                          "\"hbm_bytes\": %zu, \"l2_bytes\": %d, \"smem_per_block_optin\": %zu, \"driver\": %d, "
                          "\"runtime\": %d}",
                          prop.name, prop.major, prop.minor, prop.multiProcessorCount, prop.major, prop.minor,
                          prop.totalGlobalMem, prop.l2CacheSize, prop.sharedMemPerBlockOptin, drv, rt);
    if (n < 0 || static_cast<size_t>(n) >= cap) return fail(ctx, MTC_ERR_BUFFER_SIZE, "device_info: buffer too small");
    return MTC_OK;
}

int mtc_alloc(mtc_ctx *ctx, size_t bytes, void **d_ptr) {
    if (!ctx || !d_ptr) return MTC_ERR_INVALID;
    MTC_ENTER(ctx);
    *d_ptr = nullptr;
    if (bytes == 0) return MTC_OK;
    MTC_CUDA(ctx, cudaMalloc(d_ptr, bytes), MTC_ERR_BUFFER);
    return MTC_OK;
}

int mtc_free(mtc_ctx *ctx, void *d_ptr) {
    if (!ctx) return MTC_ERR_INVALID;
    MTC_ENTER(ctx);
    if (d_ptr) MTC_CUDA(ctx, cudaFree(d_ptr), MTC_ERR_BUFFER);
    return MTC_OK;
}

int mtc_upload(mtc_ctx *ctx, void *stream, void *d_dst, const void *h_src, size_t bytes) {
    if (!ctx || (bytes && (!d_dst || !h_src))) return fail(ctx, MTC_ERR_INVALID, "upload: null pointer");
    MTC_ENTER(ctx);
    if (bytes)
        MTC_CUDA(ctx, cudaMemcpyAsync(d_dst, h_src, bytes, cudaMemcpyHostToDevice, static_cast<cudaStream_t>(stream)),
                 MTC_ERR_BUFFER);
    return MTC_OK;
}

int mtc_download(mtc_ctx *ctx, void *stream, void *h_dst, const void *d_src, size_t bytes) {
    if (!ctx || (bytes && (!h_dst || !d_src))) return fail(ctx, MTC_ERR_INVALID, "download: null pointer");
    MTC_ENTER(ctx);
    if (bytes)
        MTC_CUDA(ctx, cudaMemcpyAsync(h_dst, d_src, bytes, cudaMemcpyDeviceToHost, static_cast<cudaStream_t>(stream)),
                 MTC_ERR_BUFFER);
    return MTC_OK;
}

int mtc_memset(mtc_ctx *ctx, void *stream, void *d_ptr, int value, size_t bytes) {
    if (!ctx || (bytes && !d_ptr)) return fail(ctx, MTC_ERR_INVALID, "memset: null pointer");
    MTC_ENTER(ctx);
    if (bytes) MTC_CUDA(ctx, cudaMemsetAsync(d_ptr, value, bytes, static_cast<cudaStream_t>(stream)), MTC_ERR_BUFFER);
    return MTC_OK;
}

// A kernel that gave up on a bounded wait (or rejected an index) leaves a code in the status word and returns; the
// host learns of it at the next synchronising call.
static int check_status(mtc_ctx *ctx, const char *who) {
    uint32_t word = 0;
    MTC_CUDA(ctx, cudaMemcpy(&word, ctx->d_status, sizeof(uint32_t), cudaMemcpyDeviceToHost), MTC_ERR_DISPATCH);
    if (word != 0) {
        char buf[160];
        std::snprintf(buf, sizeof(buf), "%s: a kernel reported status 0x%x (a bounded device-side wait expired or an index was rejected); "
                      "results of that stream are not valid", who, word);
        return fail(ctx, MTC_ERR_TIMEOUT, buf);
    }
    return MTC_OK;
}

int mtc_sync(mtc_ctx *ctx, void *stream) {
    if (!ctx) return MTC_ERR_INVALID;
    MTC_ENTER(ctx);
    MTC_CUDA(ctx, cudaStreamSynchronize(static_cast<cudaStream_t>(stream)), MTC_ERR_DISPATCH);
    return check_status(ctx, "sync");
}

int mtc_sync_deadline(mtc_ctx *ctx, void *stream, int timeout_ms) {
    if (!ctx) return MTC_ERR_INVALID;
    MTC_ENTER(ctx);
    if (timeout_ms < 0) return mtc_sync(ctx, stream);
    cudaEvent_t ev = nullptr;
    MTC_CUDA(ctx, cudaEventCreateWithFlags(&ev, cudaEventDisableTiming), MTC_ERR_DISPATCH);
    cudaError_t e = cudaEventRecord(ev, static_cast<cudaStream_t>(stream));
    const auto t0 = std::chrono::steady_clock::now();
    while (e == cudaSuccess) {
        e = cudaEventQuery(ev);
        if (e == cudaSuccess) break;
        if (e != cudaErrorNotReady) break;
        e = cudaSuccess;
        const auto ms = std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now() - t0).count();
        if (ms >= timeout_ms) {
            cudaEventDestroy(ev);
            return fail(ctx, MTC_ERR_TIMEOUT, "sync: the stream did not finish within " + std::to_string(timeout_ms) + " ms (it keeps running)");
        }
        std::this_thread::sleep_for(std::chrono::microseconds(50));
    }
    cudaEventDestroy(ev);
    if (e != cudaSuccess) return fail(ctx, MTC_ERR_DISPATCH, std::string("sync: ") + cudaGetErrorString(e));
    return check_status(ctx, "sync");
}

int mtc_status_word(mtc_ctx *ctx, uint32_t *word) {
    if (!ctx || !word) return MTC_ERR_INVALID;
    MTC_ENTER(ctx);
    MTC_CUDA(ctx, cudaMemcpy(word, ctx->d_status, sizeof(uint32_t), cudaMemcpyDeviceToHost), MTC_ERR_DISPATCH);
    return MTC_OK;
}

int mtc_status_clear(mtc_ctx *ctx) {
    if (!ctx) return MTC_ERR_INVALID;
    MTC_ENTER(ctx);
    MTC_CUDA(ctx, cudaMemset(ctx->d_status, 0, sizeof(uint32_t)), MTC_ERR_DISPATCH);
    return MTC_OK;
}

// 2 <= M <= 16 on a shape only the CUDA-core kernel would take otherwise: the tensor-memory qmm kernel is preferred when
// option qmv_small_m_tc says so.
// Measured on B200 (2 / 3 / 6 / 8-bit and group 32, bf16, square matrices of 2048 - 8192): the CUDA-core kernel costs one
// FFMA per (code, token) in row tiles of 4, 8 or 16 tokens (4096 x 4096: 10-14 / 17-20 / 35-49 us; 8192 x 8192: 32-47 /
// 84-139 / 125-186 us), the tensor-memory kernel with K slices ~12 / 21 / 54 us whatever the token count.
static bool small_m_tc_rule(int mode, int M, int N, int K) {
    if (!mode || M < 2 || M > 16) return false;
    if (mode == 2) return true;
    const long long codes = static_cast<long long>(N) * K;
    if (M >= 9) return codes >= (2ll << 20);
    if (M >= 5) return codes >= (32ll << 20);
    return false;
}

static bool small_m_tc_preferred(mtc_ctx *ctx, int M, int N, int K, int bits, int group_size, int dtype, const void *w, const void *x,
                                 const void *out) {
    return small_m_tc_rule(ctx->qmv_small_m_tc, M, N, K) && mtc::qmm_tcgen05_supported(M, N, K, bits, group_size, dtype, w, x, out);
}

// The tcgen05 decode kernel, when it takes the shape: 0 = launched, 1 = not its shape, < 0 = error.
static int try_qmv_tc(mtc_ctx *ctx, void *stream, const void *w, const void *scales, const void *biases, const void *x,
                      void *const *outs, int n_outs, int M, int N, int K, int bits, int group_size, int dtype) {
    if (!ctx->qmv_tc || M < 1 || N < 1 || !mtc::qmv_tc_supported(M, N, K, bits, group_size, dtype, w, scales, biases, x)) return 1;
    if (mtc::qmv_tc_counter_bytes(N) > kTcCounterBytes) return 1;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int rc = ensure_tc_scratch(ctx, mtc::qmv_tc_scratch_bytes(M, N, K), st);
    if (rc != MTC_OK) return rc;
    cudaError_t e = mtc::launch_qmv_tc(ctx, st, w, scales, biases, x, outs, n_outs, M, N, K, group_size, dtype, ctx->d_tc_scratch,
                                       ctx->d_tc_counters);
    if (e != cudaSuccess) return fail(ctx, MTC_ERR_DISPATCH, std::string("qmv (tcgen05) launch: ") + cudaGetErrorString(e));
    return 0;
}

int mtc_qmv(mtc_ctx *ctx, void *stream, const void *w, const void *scales, const void *biases, const void *x,
            void *out, int M, int N, int K, int bits, int group_size, int dtype) {
    if (!ctx) return MTC_ERR_INVALID;
    MTC_ENTER(ctx);
    if (!dtype_ok(dtype)) return fail(ctx, MTC_ERR_UNSUPPORTED, "qmv: dtype must be f32, f16 or bf16");
    if (M > 0 && N > 0 && (!w || !scales || !biases || !x || !out)) return fail(ctx, MTC_ERR_INVALID, "qmv: null pointer");
    std::string why;
    {
        void *outs1[1] = {out};
        const int t = try_qmv_tc(ctx, stream, w, scales, biases, x, outs1, 1, M, N, K, bits, group_size, dtype);
        if (t <= 0) return t;
    }
    if (stream_takes_single(ctx, M, N, K) && mtc::qmv_stream_supported(M, N, K, bits, group_size, dtype, w, scales, biases, x)) {
        mtc_qmv_desc d{};
        d.w = w; d.scales = scales; d.biases = biases; d.x = x;
        d.outs[0] = out; d.n_outs = 1;
        d.M = M; d.N = N; d.K = K; d.bits = bits; d.group_size = group_size; d.dtype = dtype;
        cudaError_t e1 = mtc::launch_qmv_stream(ctx, static_cast<cudaStream_t>(stream), &d, 1);
        if (e1 != cudaSuccess) return fail(ctx, MTC_ERR_DISPATCH, std::string("qmv (stream) launch: ") + cudaGetErrorString(e1));
        return MTC_OK;
    }
    if (ctx->qmv_small_m_mma && (M >= 2 || ctx->qmv_small_m_mma == 2) &&
        mtc::qmv_mma_supported(M < 2 ? 2 : M, N, K, bits, group_size, dtype, w, x)) {
        cudaError_t e2 = mtc::launch_qmv_mma(ctx, static_cast<cudaStream_t>(stream), w, scales, biases, x, out, M, N, K,
                                             group_size, dtype);
        if (e2 != cudaSuccess) return fail(ctx, MTC_ERR_DISPATCH, std::string("qmv (mma) launch: ") + cudaGetErrorString(e2));
        return MTC_OK;
    }
    if (small_m_tc_preferred(ctx, M, N, K, bits, group_size, dtype, w, x, out)) {
        // a few token rows on a width or group the warp-level kernels do not take: one FFMA per (code, token) on CUDA
        // cores against the tensor-memory kernel with K cut into slices
        cudaError_t e3 = mtc::launch_qmm_tcgen05(ctx, static_cast<cudaStream_t>(stream), w, scales, biases, x, out, M, N, K, bits,
                                                 group_size, dtype, &why);
        if (e3 == cudaSuccess) return MTC_OK;
        // a scratch block would have to grow during stream capture: the CUDA-core kernel needs none
        if (e3 != cudaErrorStreamCaptureUnsupported)
            return fail(ctx, MTC_ERR_DISPATCH, "qmv (tcgen05 qmm) launch: " + (why.empty() ? std::string(cudaGetErrorString(e3)) : why));
        why.clear();
    }
    cudaError_t e = mtc::launch_qmv(ctx, static_cast<cudaStream_t>(stream), w, scales, biases, x, out, M, N, K, bits,
                                    group_size, dtype, &why);
    if (e == cudaErrorInvalidValue && !why.empty()) return fail(ctx, MTC_ERR_UNSUPPORTED, why);
    if (e != cudaSuccess) return fail(ctx, MTC_ERR_DISPATCH, std::string("qmv launch: ") + cudaGetErrorString(e));
    return MTC_OK;
}

int mtc_qmv_multi(mtc_ctx *ctx, void *stream, const void *w, const void *scales, const void *biases, const void *x,
                  void *const *outs, int n_outs, int M, int N, int K, int bits, int group_size, int dtype) {
    if (!ctx) return MTC_ERR_INVALID;
    MTC_ENTER(ctx);
    if (!dtype_ok(dtype)) return fail(ctx, MTC_ERR_UNSUPPORTED, "qmv_multi: dtype must be f32, f16 or bf16");
    if (!outs || n_outs < 1 || n_outs > 8) return fail(ctx, MTC_ERR_INVALID, "qmv_multi: 1 to 8 outputs");
    for (int i = 0; i < n_outs; ++i)
        if (!outs[i]) return fail(ctx, MTC_ERR_INVALID, "qmv_multi: null output");
    if (M > 0 && N > 0 && (!w || !scales || !biases || !x)) return fail(ctx, MTC_ERR_INVALID, "qmv_multi: null pointer");
    std::string why;
    {
        const int t = try_qmv_tc(ctx, stream, w, scales, biases, x, outs, n_outs, M, N, K, bits, group_size, dtype);
        if (t <= 0) return t;
    }
    if (stream_takes(ctx, M) && M > 0 && N > 0 && mtc::qmv_stream_supported(M, N, K, bits, group_size, dtype, w, scales, biases, x)) {
        mtc_qmv_desc d{};
        d.w = w; d.scales = scales; d.biases = biases; d.x = x;
        for (int i = 0; i < n_outs; ++i) d.outs[i] = outs[i];
        d.n_outs = n_outs;
        d.M = M; d.N = N; d.K = K; d.bits = bits; d.group_size = group_size; d.dtype = dtype;
        cudaError_t e1 = mtc::launch_qmv_stream(ctx, static_cast<cudaStream_t>(stream), &d, 1);
        if (e1 != cudaSuccess) return fail(ctx, MTC_ERR_DISPATCH, std::string("qmv_multi (stream) launch: ") + cudaGetErrorString(e1));
        return MTC_OK;
    }
    cudaError_t e = mtc::launch_qmv(ctx, static_cast<cudaStream_t>(stream), w, scales, biases, x, outs[0], M, N, K, bits,
                                    group_size, dtype, &why, outs + 1, n_outs - 1);
    if (e == cudaErrorInvalidValue && !why.empty()) return fail(ctx, MTC_ERR_UNSUPPORTED, why);
    if (e != cudaSuccess) return fail(ctx, MTC_ERR_DISPATCH, std::string("qmv_multi launch: ") + cudaGetErrorString(e));
    return MTC_OK;
}

static int check_desc(mtc_ctx *ctx, const mtc_qmv_desc &d, const char *who) {
    if (!dtype_ok(d.dtype)) return fail(ctx, MTC_ERR_UNSUPPORTED, std::string(who) + ": dtype must be f32, f16 or bf16");
    if (d.n_outs < 1 || d.n_outs > 8) return fail(ctx, MTC_ERR_INVALID, std::string(who) + ": 1 to 8 outputs per projection");
    for (int i = 0; i < d.n_outs; ++i)
        if (!d.outs[i]) return fail(ctx, MTC_ERR_INVALID, std::string(who) + ": null output");
    if (d.M < 0 || d.N < 0 || d.K <= 0) return fail(ctx, MTC_ERR_INVALID, std::string(who) + ": bad shape");
    if (d.M > 0 && d.N > 0 && (!d.w || !d.scales || !d.biases || !d.x)) return fail(ctx, MTC_ERR_INVALID, std::string(who) + ": null pointer");
    return MTC_OK;
}

int mtc_qmv_batched(mtc_ctx *ctx, void *stream, const mtc_qmv_desc *descs, int n) {
    if (!ctx) return MTC_ERR_INVALID;
    MTC_ENTER(ctx);
    if (!descs || n < 1 || n > 4) return fail(ctx, MTC_ERR_INVALID, "qmv_batched: 1 to 4 projections");
    bool fused = stream_takes(ctx, descs[0].M);
    for (int i = 0; i < n; ++i) {
        int rc = check_desc(ctx, descs[i], "qmv_batched");
        if (rc != MTC_OK) return rc;
        const mtc_qmv_desc &d = descs[i];
        if (d.x != descs[0].x || d.M != descs[0].M || d.K != descs[0].K || d.dtype != descs[0].dtype)
            return fail(ctx, MTC_ERR_INVALID, "qmv_batched: the projections must share x, M, K and dtype");
        fused = fused && d.group_size == descs[0].group_size;
        fused = fused && d.M > 0 && d.N > 0 &&
                mtc::qmv_stream_supported(d.M, d.N, d.K, d.bits, d.group_size, d.dtype, d.w, d.scales, d.biases, d.x);
    }
    if (fused) {
        cudaError_t e = mtc::launch_qmv_stream(ctx, static_cast<cudaStream_t>(stream), descs, n);
        if (e != cudaSuccess) return fail(ctx, MTC_ERR_DISPATCH, std::string("qmv_batched launch: ") + cudaGetErrorString(e));
        return MTC_OK;
    }
    for (int i = 0; i < n; ++i) {
        const mtc_qmv_desc &d = descs[i];
        int rc = d.n_outs == 1 ? mtc_qmv(ctx, stream, d.w, d.scales, d.biases, d.x, d.outs[0], d.M, d.N, d.K, d.bits, d.group_size, d.dtype)
                               : mtc_qmv_multi(ctx, stream, d.w, d.scales, d.biases, d.x, d.outs, d.n_outs, d.M, d.N, d.K, d.bits,
                                               d.group_size, d.dtype);
        if (rc != MTC_OK) return rc;
    }
    return MTC_OK;
}

int mtc_qmv_batched_sync(mtc_ctx *ctx, void *stream, const mtc_qmv_desc *descs, int n, const mtc_peer_sync *sync) {
    if (!ctx) return MTC_ERR_INVALID;
    MTC_ENTER(ctx);
    if (!sync) return mtc_qmv_batched(ctx, stream, descs, n);
    if (!descs || n < 1 || n > 4) return fail(ctx, MTC_ERR_INVALID, "qmv_batched_sync: 1 to 4 projections");
    for (int i = 0; i < n; ++i) {
        int rc = check_desc(ctx, descs[i], "qmv_batched_sync");
        if (rc != MTC_OK) return rc;
        const mtc_qmv_desc &d = descs[i];
        if (d.x != descs[0].x || d.M != descs[0].M || d.K != descs[0].K || d.dtype != descs[0].dtype || d.group_size != descs[0].group_size)
            return fail(ctx, MTC_ERR_INVALID, "qmv_batched_sync: the projections must share x, M, K, dtype and group size");
        if (ctx->qmv_stream == 0 || !mtc::qmv_stream_supported(d.M, d.N, d.K, d.bits, d.group_size, d.dtype, d.w, d.scales, d.biases, d.x))
            return fail(ctx, MTC_ERR_UNSUPPORTED, "qmv_batched_sync: only shapes of the streaming kernel (4-bit, f16 / bf16, M <= 8, "
                                                  "K % 512 == 0, group 64 or 128, 16-byte aligned pointers)");
    }
    cudaError_t e = mtc::launch_qmv_stream(ctx, static_cast<cudaStream_t>(stream), descs, n, sync);
    if (e == cudaErrorInvalidValue) return fail(ctx, MTC_ERR_INVALID, "qmv_batched_sync: 1 to 8 peers, rank < peers, no null pointer");
    if (e != cudaSuccess) return fail(ctx, MTC_ERR_DISPATCH, std::string("qmv_batched_sync launch: ") + cudaGetErrorString(e));
    return MTC_OK;
}

struct mtc_chain {
    mtc::StreamChain *fused = nullptr;        // the persistent-grid form, or
    std::vector<mtc_qmv_desc> descs;          // one launch per projection, in order
};

int mtc_chain_create(mtc_ctx *ctx, const mtc_qmv_desc *descs, int n, mtc_chain **out_chain) {
    if (!ctx) return MTC_ERR_INVALID;
    MTC_ENTER(ctx);
    if (!descs || n < 1 || !out_chain) return fail(ctx, MTC_ERR_INVALID, "chain_create: need at least one projection");
    *out_chain = nullptr;
    int phase_prev = 0;
    for (int i = 0; i < n; ++i) {
        int rc = check_desc(ctx, descs[i], "chain_create");
        if (rc != MTC_OK) return rc;
        if (descs[i].phase < phase_prev || descs[i].phase > phase_prev + 1 || (i == 0 && descs[i].phase != 0))
            return fail(ctx, MTC_ERR_INVALID, "chain_create: phases start at 0 and grow by at most one from one projection to the next");
        phase_prev = descs[i].phase;
    }
    MTC_CUDA(ctx, cudaSetDevice(ctx->device), MTC_ERR_NO_DEVICE);
    mtc_chain *c = new mtc_chain();
    c->descs.assign(descs, descs + n);
    if (ctx->qmv_stream) {
        std::string why;
        cudaError_t e = mtc::stream_chain_create(ctx, descs, n, &c->fused, &why);
        if (e != cudaSuccess && e != cudaErrorInvalidValue) {
            delete c;
            return fail(ctx, MTC_ERR_BUFFER, std::string("chain_create: ") + cudaGetErrorString(e));
        }
        if (e != cudaSuccess) {
            c->fused = nullptr;                // outside the streaming kernel's contract: one launch per projection
            cudaGetLastError();
        }
    }
    *out_chain = c;
    return MTC_OK;
}

int mtc_chain_is_fused(const mtc_chain *chain) { return chain && chain->fused ? 1 : 0; }

int mtc_chain_run(mtc_ctx *ctx, void *stream, mtc_chain *chain) {
    if (!ctx || !chain) return MTC_ERR_INVALID;
    MTC_ENTER(ctx);
    if (chain->fused) {
        cudaError_t e = mtc::stream_chain_run(ctx, static_cast<cudaStream_t>(stream), chain->fused);
        if (e != cudaSuccess) return fail(ctx, MTC_ERR_DISPATCH, std::string("chain_run launch: ") + cudaGetErrorString(e));
        return MTC_OK;
    }
    for (const mtc_qmv_desc &d : chain->descs) {
        int rc = d.n_outs == 1 ? mtc_qmv(ctx, stream, d.w, d.scales, d.biases, d.x, d.outs[0], d.M, d.N, d.K, d.bits, d.group_size, d.dtype)
                               : mtc_qmv_multi(ctx, stream, d.w, d.scales, d.biases, d.x, d.outs, d.n_outs, d.M, d.N, d.K, d.bits,
                                               d.group_size, d.dtype);
        if (rc != MTC_OK) return rc;
    }
    return MTC_OK;
}

int mtc_chain_destroy(mtc_ctx *ctx, mtc_chain *chain) {
    if (!ctx) return MTC_ERR_INVALID;
    MTC_ENTER(ctx);
    if (!chain) return MTC_OK;
    if (chain->fused) mtc::stream_chain_destroy(chain->fused);
    delete chain;
    return MTC_OK;
}

int mtc_ipc_export(mtc_ctx *ctx, void *d_ptr, void *handle64) {
    if (!ctx || !d_ptr || !handle64) return fail(ctx, MTC_ERR_INVALID, "ipc_export: null pointer");
    MTC_ENTER(ctx);
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
    MTC_CUDA(ctx, cudaIpcGetMemHandle(static_cast<cudaIpcMemHandle_t *>(handle64), d_ptr), MTC_ERR_BUFFER);
    return MTC_OK;
}

int mtc_ipc_open(mtc_ctx *ctx, const void *handle64, void **d_ptr) {
    if (!ctx || !handle64 || !d_ptr) return fail(ctx, MTC_ERR_INVALID, "ipc_open: null pointer");
    MTC_ENTER(ctx);
    cudaIpcMemHandle_t h;
    std::memcpy(&h, handle64, sizeof(h));
    MTC_CUDA(ctx, cudaIpcOpenMemHandle(d_ptr, h, cudaIpcMemLazyEnablePeerAccess), MTC_ERR_BUFFER);
    return MTC_OK;
}

int mtc_ipc_close(mtc_ctx *ctx, void *d_ptr) {
    if (!ctx || !d_ptr) return fail(ctx, MTC_ERR_INVALID, "ipc_close: null pointer");
    MTC_ENTER(ctx);
    MTC_CUDA(ctx, cudaIpcCloseMemHandle(d_ptr), MTC_ERR_BUFFER);
    return MTC_OK;
}

int mtc_peer_barrier(mtc_ctx *ctx, void *stream, void *const *peer_flags, int n_peers, int rank, void *local_flags,
                     void *epoch) {
    if (!ctx) return MTC_ERR_INVALID;
    MTC_ENTER(ctx);
    cudaError_t e = mtc::launch_peer_barrier(ctx, static_cast<cudaStream_t>(stream),
                                             reinterpret_cast<uint32_t *const *>(peer_flags), n_peers, rank,
                                             static_cast<uint32_t *>(local_flags), static_cast<uint32_t *>(epoch));
    if (e == cudaErrorInvalidValue) return fail(ctx, MTC_ERR_INVALID, "peer_barrier: 1 to 8 peers, rank < peers, no null pointer");
    if (e != cudaSuccess) return fail(ctx, MTC_ERR_DISPATCH, std::string("peer_barrier launch: ") + cudaGetErrorString(e));
    return MTC_OK;
}

// mt_qmm_for (crates/metaltile-std/src/mlx/quantized.rs:5040-5065) picks by M alone; here M <= 16 or
// f32 activations stay on the qmv kernels (CUDA cores, or warp-level MMAs for 2 <= M <= 16 with 4-bit codes), everything else goes to the tensor cores when the
// shape meets that kernel's contract (K % 64 == 0, power-of-two group >= 32).
// 17 <= M <= 64: the tcgen05 kernel needs (N / 128) x ceil(M / tile) work items to fill 148 SMs and paces at ~0.85 us
// per 64 of K whatever M is, so few token rows on a matrix of a few thousand rows leave most SMs idle (M = 32,
// 4096 x 4096: 54 us on 32 SMs).  The small-M tensor-core qmv in 16-row chunks streams the weights once per chunk
// on every SM instead (2 x 9.3 us for that case).  Taken for M <= 32 always, up to 64 while the tcgen05 grid would
// cover less than half of the SMs.
// With K slices (option "qmm_ksplit") the tcgen05 kernel fills the SMs on exactly those shapes, and wins from M = 33 on
// (4096 x 4096: 27 us against 30 / 34 / 42 us at M = 33 / 48 / 64), so the chunks keep 17 <= M <= 32 only.
static bool mma_chunks_preferred(int enabled, int ksplit, int sms, int M, int N, int K, int bits, int group_size, int dtype,
                                 const void *w, const void *x) {
    if (!enabled || M <= 16 || M > 64) return false;
    if (!mtc::qmv_mma_supported(16, N, K, bits, group_size, dtype, w, x)) return false;
    return M <= 32 || (!ksplit && ((N + 127) / 128) * 2 <= sms);
}

const char *mtc_qmm_route(int M, int N, int K, int bits, int group_size, int dtype) {
    if (M == 1 && static_cast<long long>(N) * K >= kStreamMinCodes &&
        mtc::qmv_stream_supported(M, N, K, bits, group_size, dtype, nullptr, nullptr, nullptr, nullptr))
        return "qmv_stream";      // option "qmv_stream" = 2 extends it to M <= 8 and to small matrices; fused launches take it at any size
    if (mma_chunks_preferred(1, 1, 148, M, N, K, bits, group_size, dtype, nullptr, nullptr)) return "qmv_mma_sync";
    if (M > 16 && mtc::qmm_tcgen05_supported(M, N, K, bits, group_size, dtype, nullptr, nullptr, nullptr))
        return "qmm_tcgen05";
    // alignment is a run-time property of the pointers; the route names the kernel an aligned call gets
    if (mtc::qmv_mma_supported(M, N, K, bits, group_size, dtype, nullptr, nullptr)) return "qmv_mma_sync";
    if (small_m_tc_rule(1, M, N, K) && mtc::qmm_tcgen05_supported(M, N, K, bits, group_size, dtype, nullptr, nullptr, nullptr))
        return "qmm_tcgen05";     // a few token rows on a width or group the warp-level kernels do not take (option "qmv_small_m_tc")
    return "qmv_cuda_core";
}

int mtc_qmm(mtc_ctx *ctx, void *stream, const void *w, const void *scales, const void *biases, const void *x,
            void *out, int M, int N, int K, int bits, int group_size, int dtype) {
    if (!ctx) return MTC_ERR_INVALID;
    MTC_ENTER(ctx);
    if (!dtype_ok(dtype)) return fail(ctx, MTC_ERR_UNSUPPORTED, "qmm: dtype must be f32, f16 or bf16");
    if (w && scales && biases && x && out &&
        mma_chunks_preferred(ctx->qmm_mma_chunks && ctx->qmv_small_m_mma, ctx->qmm_ksplit, ctx->sm_count, M, N, K, bits, group_size, dtype, w, x)) {
        const size_t esz = 2;      // f16 / bf16 only on this path
        for (int m0 = 0; m0 < M; m0 += 16) {
            const int mc = M - m0 < 16 ? M - m0 : 16;
            const char *xc = static_cast<const char *>(x) + static_cast<size_t>(m0) * K * esz;
            char *oc = static_cast<char *>(out) + static_cast<size_t>(m0) * N * esz;
            int rc = mtc_qmv(ctx, stream, w, scales, biases, xc, oc, mc, N, K, bits, group_size, dtype);
            if (rc != MTC_OK) return rc;
        }
        return MTC_OK;
    }
    if (M > 16 && mtc::qmm_tcgen05_supported(M, N, K, bits, group_size, dtype, w, x, out)) {
        if (!w || !scales || !biases || !x || !out) return fail(ctx, MTC_ERR_INVALID, "qmm: null pointer");
        std::string why;
        cudaError_t e = mtc::launch_qmm_tcgen05(ctx, static_cast<cudaStream_t>(stream), w, scales, biases, x, out, M,
                                                N, K, bits, group_size, dtype, &why);
        if (e != cudaSuccess)
            return fail(ctx, MTC_ERR_DISPATCH, "qmm launch: " + (why.empty() ? std::string(cudaGetErrorString(e)) : why));
        return MTC_OK;
    }
    return mtc_qmv(ctx, stream, w, scales, biases, x, out, M, N, K, bits, group_size, dtype);
}

static int affine_args_ok(mtc_ctx *ctx, const char *who, size_t n_elem, int bits, int group_size, int dtype) {
    if (!dtype_ok(dtype)) return fail(ctx, MTC_ERR_UNSUPPORTED, std::string(who) + ": dtype must be f32, f16 or bf16");
    const bool bits_ok = bits == 2 || bits == 3 || bits == 4 || bits == 5 || bits == 6 || bits == 8;
    if (!bits_ok || group_size <= 0 || (static_cast<long long>(group_size) * bits) % 32 != 0 || n_elem % static_cast<size_t>(group_size) != 0)
        return fail(ctx, MTC_ERR_UNSUPPORTED, std::string(who) + ": need bits in {2,3,4,5,6,8}, whole groups, group_size * bits % 32 == 0");
    return MTC_OK;
}

int mtc_affine_quantize(mtc_ctx *ctx, void *stream, const void *w, void *out, void *scales, void *biases, size_t n_elem, int bits,
                        int group_size, int dtype) {
    if (!ctx) return MTC_ERR_INVALID;
    MTC_ENTER(ctx);
    int rc = affine_args_ok(ctx, "affine_quantize", n_elem, bits, group_size, dtype);
    if (rc != MTC_OK) return rc;
    if (n_elem == 0) return MTC_OK;
    if (!w || !out || !scales || !biases) return fail(ctx, MTC_ERR_INVALID, "affine_quantize: null pointer");
    MTC_CUDA(ctx, mtc::launch_affine_quantize(ctx, static_cast<cudaStream_t>(stream), w, out, scales, biases, n_elem / group_size, bits,
                                              group_size, dtype), MTC_ERR_DISPATCH);
    return MTC_OK;
}

int mtc_affine_dequantize(mtc_ctx *ctx, void *stream, const void *w, const void *scales, const void *biases, void *out, size_t n_elem,
                          int bits, int group_size, int dtype) {
    if (!ctx) return MTC_ERR_INVALID;
    MTC_ENTER(ctx);
    int rc = affine_args_ok(ctx, "affine_dequantize", n_elem, bits, group_size, dtype);
    if (rc != MTC_OK) return rc;
    if (n_elem == 0) return MTC_OK;
    if (!w || !out || !scales || !biases) return fail(ctx, MTC_ERR_INVALID, "affine_dequantize: null pointer");
    MTC_CUDA(ctx, mtc::launch_affine_dequantize(ctx, static_cast<cudaStream_t>(stream), w, scales, biases, out, n_elem, bits, group_size,
                                                dtype), MTC_ERR_DISPATCH);
    return MTC_OK;
}

int mtc_dequant_gather(mtc_ctx *ctx, void *stream, const void *weight, const void *scales, const void *biases, const void *indices,
                       void *out, size_t n_tokens, int hidden, int vocab, int bits, int group_size, int dtype) {
    if (!ctx) return MTC_ERR_INVALID;
    MTC_ENTER(ctx);
    if (!dtype_ok(dtype)) return fail(ctx, MTC_ERR_UNSUPPORTED, "dequant_gather: dtype must be f32, f16 or bf16");
    const bool bits_ok = bits == 2 || bits == 3 || bits == 4 || bits == 5 || bits == 6 || bits == 8;
    if (!bits_ok || hidden <= 0 || vocab <= 0 || group_size <= 0 || hidden % group_size != 0 || (static_cast<long long>(hidden) * bits) % 32 != 0)
        return fail(ctx, MTC_ERR_UNSUPPORTED, "dequant_gather: need bits in {2,3,4,5,6,8}, group_size | hidden, hidden * bits % 32 == 0");
    if (n_tokens == 0) return MTC_OK;
    if (!weight || !scales || !biases || !indices || !out) return fail(ctx, MTC_ERR_INVALID, "dequant_gather: null pointer");
    MTC_CUDA(ctx, mtc::launch_dequant_gather(ctx, static_cast<cudaStream_t>(stream), weight, scales, biases, indices, out, n_tokens, hidden,
                                             vocab, bits, group_size, dtype), MTC_ERR_DISPATCH);
    return MTC_OK;
}

static int moe_decode_args_ok(mtc_ctx *ctx, const char *who, int n_slots, int in_dim, int out_dim, int n_experts, int group_size, int dtype) {
    if (!dtype_ok(dtype)) return fail(ctx, MTC_ERR_UNSUPPORTED, std::string(who) + ": dtype must be f32, f16 or bf16");
    if (n_slots < 1 || n_slots > 8 || in_dim <= 0 || out_dim < 0 || n_experts <= 0 || group_size <= 0 || in_dim % group_size != 0 ||
        group_size < 8 || (group_size & (group_size - 1)) != 0 || mtc::moe_decode_smem_bytes(n_slots, in_dim) > 200 * 1024)
        return fail(ctx, MTC_ERR_UNSUPPORTED, std::string(who) + ": need 1..8 slots, 4-bit weights, a power-of-two group_size >= 8 that divides in_dim, "
                                              "n_slots * in_dim * 4.5 bytes of shared memory <= 200 KB");
    return MTC_OK;
}

static int moe_decode_stage(mtc_ctx *ctx, cudaStream_t st, int n_slots, int in_dim) {
    std::string why;
    cudaError_t e = mtc::grow_block(ctx, st, &ctx->d_tail, &ctx->tail_bytes, mtc::moe_decode_smem_bytes(n_slots, in_dim), &why);
    if (e != cudaSuccess) return fail(ctx, MTC_ERR_BUFFER, "moe decode tail staging: " + (why.empty() ? std::string(cudaGetErrorString(e)) : why));
    return MTC_OK;
}

int mtc_moe_down_swiglu_accum(mtc_ctx *ctx, void *stream, const void *const *gates, const void *const *ups, int n_slots,
                              const void *expert_indices, const void *slot_weights, const void *w, const void *scales,
                              const void *biases, void *out, int in_dim, int out_dim, int n_experts, int group_size, int dtype) {
    if (!ctx) return MTC_ERR_INVALID;
    MTC_ENTER(ctx);
    int rc = moe_decode_args_ok(ctx, "moe_down_swiglu_accum", n_slots, in_dim, out_dim, n_experts, group_size, dtype);
    if (rc != MTC_OK) return rc;
    if (out_dim == 0) return MTC_OK;
    if (!gates || !ups || !expert_indices || !slot_weights || !w || !scales || !biases || !out) return fail(ctx, MTC_ERR_INVALID, "moe_down_swiglu_accum: null pointer");
    for (int k = 0; k < n_slots; ++k)
        if (!gates[k] || !ups[k]) return fail(ctx, MTC_ERR_INVALID, "moe_down_swiglu_accum: null gate / up");
    rc = moe_decode_stage(ctx, static_cast<cudaStream_t>(stream), n_slots, in_dim);
    if (rc != MTC_OK) return rc;
    MTC_CUDA(ctx, mtc::launch_moe_decode(ctx, static_cast<cudaStream_t>(stream), gates, ups, expert_indices, slot_weights, w, scales, biases, out,
                                         n_slots, in_dim, out_dim, n_experts, group_size, dtype, 1, static_cast<float *>(ctx->d_tail)), MTC_ERR_DISPATCH);
    return MTC_OK;
}

int mtc_qmv_expert_indexed(mtc_ctx *ctx, void *stream, const void *const *xs, int n_slots, const void *expert_indices, const void *w,
                           const void *scales, const void *biases, void *out, int in_dim, int out_dim, int n_experts, int group_size,
                           int dtype) {
    if (!ctx) return MTC_ERR_INVALID;
    MTC_ENTER(ctx);
    int rc = moe_decode_args_ok(ctx, "qmv_expert_indexed", n_slots, in_dim, out_dim, n_experts, group_size, dtype);
    if (rc != MTC_OK) return rc;
    if (out_dim == 0) return MTC_OK;
    if (!xs || !expert_indices || !w || !scales || !biases || !out) return fail(ctx, MTC_ERR_INVALID, "qmv_expert_indexed: null pointer");
    for (int k = 0; k < n_slots; ++k)
        if (!xs[k]) return fail(ctx, MTC_ERR_INVALID, "qmv_expert_indexed: null input");
    rc = moe_decode_stage(ctx, static_cast<cudaStream_t>(stream), n_slots, in_dim);
    if (rc != MTC_OK) return rc;
    MTC_CUDA(ctx, mtc::launch_moe_decode(ctx, static_cast<cudaStream_t>(stream), xs, nullptr, expert_indices, nullptr, w, scales, biases, out,
                                         n_slots, in_dim, out_dim, n_experts, group_size, dtype, 0, static_cast<float *>(ctx->d_tail)), MTC_ERR_DISPATCH);
    return MTC_OK;
}

int mtc_qvm(mtc_ctx *ctx, void *stream, const void *w, const void *scales, const void *biases, const void *x, void *out, int M, int N,
            int K, int bits, int group_size, int dtype) {
    if (!ctx) return MTC_ERR_INVALID;
    MTC_ENTER(ctx);
    if (!dtype_ok(dtype)) return fail(ctx, MTC_ERR_UNSUPPORTED, "qvm: dtype must be f32, f16 or bf16");
    const bool bits_ok = bits == 2 || bits == 3 || bits == 4 || bits == 5 || bits == 6 || bits == 8;
    if (!bits_ok || M < 0 || N < 0 || K <= 0 || group_size <= 0 || K % group_size != 0 || (static_cast<long long>(N) * bits) % 32 != 0)
        return fail(ctx, MTC_ERR_UNSUPPORTED, "qvm: need bits in {2,3,4,5,6,8}, group_size | K, N * bits % 32 == 0");
    if (M == 0 || N == 0) return MTC_OK;
    if (!w || !scales || !biases || !x || !out) return fail(ctx, MTC_ERR_INVALID, "qvm: null pointer");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int kc = 1;
    if (mtc::qvm_fast_supported(N, K, bits, group_size)) {
        kc = mtc::qvm_k_chunks(ctx->sm_count, N, K, bits, group_size);
        if (kc > 1) {
            std::string why;
            void *before = ctx->d_qvm;
            cudaError_t e = mtc::grow_block(ctx, st, &ctx->d_qvm, &ctx->qvm_bytes, mtc::qvm_scratch_bytes(M, N, kc), &why);
            if (e != cudaSuccess) return fail(ctx, MTC_ERR_BUFFER, "qvm partial sums: " + (why.empty() ? std::string(cudaGetErrorString(e)) : why));
            // a new block starts with its arrival counters at zero; every launch leaves them there
            if (ctx->d_qvm != before) MTC_CUDA(ctx, cudaMemsetAsync(ctx->d_qvm, 0, mtc::qvm_scratch_bytes(1, 0, 2), st), MTC_ERR_BUFFER);
        }
    }
    MTC_CUDA(ctx, mtc::launch_qvm(ctx, st, w, scales, biases, x, out, M, N, K, bits, group_size, dtype, ctx->d_qvm, kc),
             MTC_ERR_DISPATCH);
    return MTC_OK;
}

int mtc_rms_norm_qmv(mtc_ctx *ctx, void *stream, const void *x, const void *norm_weight, float eps, const void *w,
                     const void *scales, const void *biases, void *out, int N, int K, int bits, int group_size, int dtype) {
    if (!ctx) return MTC_ERR_INVALID;
    MTC_ENTER(ctx);
    if (!dtype_ok(dtype)) return fail(ctx, MTC_ERR_UNSUPPORTED, "rms_norm_qmv: dtype must be f32, f16 or bf16");
    if (N < 0 || K <= 0) return fail(ctx, MTC_ERR_INVALID, "rms_norm_qmv: sizes must be positive");
    if (N == 0) return MTC_OK;
    if (!x || !norm_weight || !w || !scales || !biases || !out) return fail(ctx, MTC_ERR_INVALID, "rms_norm_qmv: null pointer");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    std::string why;
    cudaError_t e = mtc::launch_qmv(ctx, st, w, scales, biases, x, out, 1, N, K, bits, group_size, dtype, &why, nullptr, 0, norm_weight, eps);
    if (e == cudaSuccess) return MTC_OK;
    if (e != cudaErrorNotSupported)
        return fail(ctx, e == cudaErrorInvalidValue ? MTC_ERR_UNSUPPORTED : MTC_ERR_DISPATCH,
                    "rms_norm_qmv launch: " + (why.empty() ? std::string(cudaGetErrorString(e)) : why));
    // shapes the fused kernel does not take (unaligned pointers, odd groups, K too long for one stage): normalise into a
    // row of the activation type, then the plain product
    e = mtc::grow_block(ctx, st, &ctx->d_norm, &ctx->norm_bytes, static_cast<size_t>(K) * mtc::dtype_size(dtype), &why);
    if (e != cudaSuccess) return fail(ctx, MTC_ERR_BUFFER, "rms_norm_qmv staging: " + (why.empty() ? std::string(cudaGetErrorString(e)) : why));
    MTC_CUDA(ctx, mtc::launch_rms_norm_row(st, x, norm_weight, ctx->d_norm, K, eps, dtype), MTC_ERR_DISPATCH);
    return mtc_qmv(ctx, stream, w, scales, biases, ctx->d_norm, out, 1, N, K, bits, group_size, dtype);
}

int mtc_qmm_multi(mtc_ctx *ctx, void *stream, const void *w, const void *scales, const void *biases, const void *x,
                  void *const *outs, int n_outs, long long ld, int M, int N, int K, int bits, int group_size, int dtype) {
    if (!ctx) return MTC_ERR_INVALID;
    MTC_ENTER(ctx);
    if (!outs || n_outs < 1 || n_outs > 8) return fail(ctx, MTC_ERR_INVALID, "qmm_multi: 1 to 8 destinations");
    if (ld < N) return fail(ctx, MTC_ERR_INVALID, "qmm_multi: the destination row stride must be at least N");
    if (M <= 0 || N <= 0) return MTC_OK;
    if (!w || !scales || !biases || !x) return fail(ctx, MTC_ERR_INVALID, "qmm_multi: null pointer");
    for (int i = 0; i < n_outs; ++i)
        if (!outs[i]) return fail(ctx, MTC_ERR_INVALID, "qmm_multi: null destination");
    if (M <= 16 || !mtc::qmm_tcgen05_supported(M, N, K, bits, group_size, dtype, w, x, outs[0]))
        return fail(ctx, MTC_ERR_UNSUPPORTED, "qmm_multi: only shapes of the tensor-core kernel (M > 16, f16 / bf16, K % 64 == 0, "
                                              "power-of-two group >= 32, 16-byte aligned w and x)");
    std::string why;
    cudaError_t e = mtc::launch_qmm_tcgen05(ctx, static_cast<cudaStream_t>(stream), w, scales, biases, x, outs[0], M, N, K, bits,
                                            group_size, dtype, &why, outs, n_outs, ld);
    if (e != cudaSuccess)
        return fail(ctx, MTC_ERR_DISPATCH, "qmm_multi launch: " + (why.empty() ? std::string(cudaGetErrorString(e)) : why));
    return MTC_OK;
}

int mtc_set_option(mtc_ctx *ctx, const char *name, int value) {
    if (!ctx || !name) return MTC_ERR_INVALID;
    if (std::strcmp(name, "qmm_tile_tokens") == 0) {
        if (value != 0 && (value < 16 || value > 256 || value % 16 != 0))
            return fail(ctx, MTC_ERR_UNSUPPORTED, "qmm_tile_tokens must be 0 or a multiple of 16 in [16, 256]");
        ctx->qmm_force_tn = value;
        return MTC_OK;
    }
    if (std::strcmp(name, "qmv_max_ctas_per_sm") == 0) {
        ctx->qmv_max_occ = value < 0 ? 0 : value;
        return MTC_OK;
    }
    if (std::strcmp(name, "qmv_small_m_mma") == 0) {
        ctx->qmv_small_m_mma = value < 0 ? 0 : (value > 2 ? 2 : value);
        return MTC_OK;
    }
    if (std::strcmp(name, "qmm_max_stages") == 0) {
        ctx->qmm_max_stages = value < 0 ? 0 : value;
        return MTC_OK;
    }
    if (std::strcmp(name, "qmm_wait_hint_ns") == 0) {
        ctx->qmm_wait_hint_ns = value < 0 ? 0 : value;
        return MTC_OK;
    }
    if (std::strcmp(name, "qmm_mma_chunks") == 0) {
        ctx->qmm_mma_chunks = value ? 1 : 0;
        return MTC_OK;
    }
    if (std::strcmp(name, "qmm_raw") == 0) {
        ctx->qmm_raw = value ? 1 : 0;
        return MTC_OK;
    }
    if (std::strcmp(name, "peer_poll_limit") == 0) {
        ctx->peer_poll_limit = value < 1 ? 1u : static_cast<uint32_t>(value);
        return MTC_OK;
    }
    if (std::strcmp(name, "qmv_tc") == 0) {
        ctx->qmv_tc = value ? 1 : 0;
        return MTC_OK;
    }
    if (std::strcmp(name, "qmv_stream") == 0) {
        ctx->qmv_stream = value < 0 ? 0 : (value > 2 ? 2 : value);
        return MTC_OK;
    }
    if (std::strcmp(name, "pdl_early_weights") == 0) {
        ctx->pdl_early_weights = value ? 1 : 0;
        return MTC_OK;
    }
    if (std::strcmp(name, "gather_stream") == 0) {
        ctx->gather_stream = value ? 1 : 0;
        return MTC_OK;
    }
    if (std::strcmp(name, "qmm_wide") == 0) {
        ctx->qmm_wide = value < 0 ? 0 : (value > 2 ? 2 : value);
        return MTC_OK;
    }
    if (std::strcmp(name, "qmm_ksplit") == 0) {
        ctx->qmm_ksplit = value ? 1 : 0;
        return MTC_OK;
    }
    if (std::strcmp(name, "qmv_small_m_tc") == 0) {
        ctx->qmv_small_m_tc = value < 0 ? 0 : (value > 2 ? 2 : value);
        return MTC_OK;
    }
    return fail(ctx, MTC_ERR_UNSUPPORTED, std::string("unknown option: ") + name);
}

int mtc_gather_qmm(mtc_ctx *ctx, void *stream, const void *x, const void *w, const void *scales, const void *biases,
                   const void *expert_offsets, const void *indices, void *out, int m_total, int n_out, int k_in,
                   int n_experts, int bits, int group_size, int dtype) {
    if (!ctx) return MTC_ERR_INVALID;
    MTC_ENTER(ctx);
    if (!dtype_ok(dtype)) return fail(ctx, MTC_ERR_UNSUPPORTED, "gather_qmm: dtype must be f32, f16 or bf16");
    if ((expert_offsets == nullptr) == (indices == nullptr))
        return fail(ctx, MTC_ERR_INVALID, "gather_qmm: give exactly one of expert_offsets and indices");
    const bool bits_ok = bits == 2 || bits == 3 || bits == 4 || bits == 5 || bits == 6 || bits == 8;
    if (!bits_ok || m_total < 0 || n_out < 0 || k_in <= 0 || n_experts <= 0 || group_size <= 0 || k_in % group_size != 0 ||
        (static_cast<long long>(k_in) * bits) % 32 != 0)
        return fail(ctx, MTC_ERR_UNSUPPORTED,
                    "gather_qmm: need bits in {2,3,4,5,6,8}, group_size | k_in, k_in*bits % 32 == 0, n_experts > 0");
    if (m_total == 0 || n_out == 0) return MTC_OK;
    if (!x || !w || !scales || !biases || !out) return fail(ctx, MTC_ERR_INVALID, "gather_qmm: null pointer");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // few rows per expert: the layer is bound by reading every expert's matrix once - the streaming kernel
    if (ctx->gather_stream && expert_offsets && static_cast<long long>(m_total) <= 64ll * n_experts &&
        mtc::gather_stream_supported(m_total, n_out, k_in, n_experts, bits, group_size, dtype, w, scales, biases, x)) {
        std::string why;
        cudaError_t e = mtc::grow_block(ctx, st, &ctx->d_gfrag, &ctx->gfrag_bytes, mtc::gather_stream_scratch_bytes(m_total, k_in), &why);
        if (e != cudaSuccess) return fail(ctx, MTC_ERR_BUFFER, "gather_qmm staging: " + (why.empty() ? std::string(cudaGetErrorString(e)) : why));
        const mtc::GatherMats one{w, scales, biases, out};
        e = mtc::launch_gather_stream(ctx, st, x, nullptr, nullptr, 0, &one, 1, static_cast<const uint32_t *>(expert_offsets), m_total,
                                      n_out, k_in, n_experts, group_size, dtype, ctx->d_gfrag);
        if (e != cudaSuccess) return fail(ctx, MTC_ERR_DISPATCH, std::string("gather_qmm (stream) launch: ") + cudaGetErrorString(e));
        return MTC_OK;
    }
    if (mtc::qmm_tcgen05_supported(m_total, n_out, k_in, bits, group_size, dtype, w, x, out) && n_experts <= 4096) {
        int rc = ensure_worklist(ctx, mtc::gather_items_bytes(m_total, n_experts, n_out, 16), st);
        if (rc != MTC_OK) return rc;
        std::string why;
        cudaError_t e = mtc::launch_gather_qmm_tcgen05(ctx, st, x, w, scales, biases,
                                                       static_cast<const uint32_t *>(expert_offsets),
                                                       static_cast<const uint32_t *>(indices), out, m_total, n_out, k_in,
                                                       n_experts, bits, group_size, dtype, ctx->d_worklist,
                                                       ctx->worklist_bytes, &why);
        if (e != cudaSuccess)
            return fail(ctx, MTC_ERR_DISPATCH, "gather_qmm launch: " + (why.empty() ? std::string(cudaGetErrorString(e)) : why));
        return MTC_OK;
    }
    MTC_CUDA(ctx, mtc::launch_gather_generic(st, x, w, scales, biases, static_cast<const uint32_t *>(expert_offsets),
                                             static_cast<const uint32_t *>(indices), out, m_total, k_in, n_out, n_experts,
                                             bits, group_size, dtype), MTC_ERR_DISPATCH);
    return MTC_OK;
}

int mtc_moe_experts(mtc_ctx *ctx, void *stream, const void *x, const void *sort_token_idx, int n_tokens, const mtc_qmat *gate,
                    const mtc_qmat *up, const mtc_qmat *down, const void *expert_offsets, void *y, int m_total, int hidden,
                    int inter, int n_experts, int bits, int group_size, int dtype) {
    if (!ctx) return MTC_ERR_INVALID;
    MTC_ENTER(ctx);
    if (!dtype_ok(dtype)) return fail(ctx, MTC_ERR_UNSUPPORTED, "moe_experts: dtype must be f32, f16 or bf16");
    if (m_total < 0 || hidden <= 0 || inter <= 0 || n_experts <= 0 || (sort_token_idx && n_tokens <= 0))
        return fail(ctx, MTC_ERR_INVALID, "moe_experts: sizes must be positive");
    if (m_total == 0) return MTC_OK;
    if (!x || !gate || !up || !down || !expert_offsets || !y || !gate->w || !gate->scales || !gate->biases || !up->w || !up->scales ||
        !up->biases || !down->w || !down->scales || !down->biases)
        return fail(ctx, MTC_ERR_INVALID, "moe_experts: null pointer");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const size_t esz = mtc::dtype_size(dtype);
    const size_t act_bytes = align_up(static_cast<size_t>(m_total) * inter * esz, 256), xp_bytes = align_up(static_cast<size_t>(m_total) * hidden * esz, 256);
    const bool streamed = ctx->gather_stream && static_cast<long long>(m_total) <= 64ll * n_experts &&
                          mtc::gather_stream_supported(m_total, inter, hidden, n_experts, bits, group_size, dtype, gate->w, gate->scales, gate->biases, x) &&
                          mtc::gather_stream_supported(m_total, inter, hidden, n_experts, bits, group_size, dtype, up->w, up->scales, up->biases, x) &&
                          mtc::gather_stream_supported(m_total, hidden, inter, n_experts, bits, group_size, dtype, down->w, down->scales, down->biases, nullptr);
    std::string why;
    cudaError_t e = mtc::grow_block(ctx, st, &ctx->d_moe, &ctx->moe_bytes, 2 * act_bytes + (streamed ? 0 : xp_bytes), &why);
    if (e != cudaSuccess) return fail(ctx, MTC_ERR_BUFFER, "moe_experts intermediates: " + (why.empty() ? std::string(cudaGetErrorString(e)) : why));
    char *g = static_cast<char *>(ctx->d_moe), *u = g + act_bytes, *xp = u + act_bytes;
    if (streamed) {
        // four launches: rows -> fragments (the permutation folded in), gate and up as one stream, SwiGLU -> fragments, down
        const size_t need = std::max(mtc::gather_stream_scratch_bytes(m_total, hidden), mtc::gather_stream_scratch_bytes(m_total, inter));
        e = mtc::grow_block(ctx, st, &ctx->d_gfrag, &ctx->gfrag_bytes, need, &why);
        if (e != cudaSuccess) return fail(ctx, MTC_ERR_BUFFER, "moe_experts staging: " + (why.empty() ? std::string(cudaGetErrorString(e)) : why));
        const mtc::GatherMats gu[2] = {{gate->w, gate->scales, gate->biases, g}, {up->w, up->scales, up->biases, u}};
        e = mtc::launch_gather_stream(ctx, st, x, nullptr, static_cast<const uint32_t *>(sort_token_idx), n_tokens, gu, 2,
                                      static_cast<const uint32_t *>(expert_offsets), m_total, inter, hidden, n_experts, group_size, dtype,
                                      ctx->d_gfrag);
        if (e != cudaSuccess) return fail(ctx, MTC_ERR_DISPATCH, std::string("moe_experts (gate, up) launch: ") + cudaGetErrorString(e));
        const mtc::GatherMats dn{down->w, down->scales, down->biases, y};
        e = mtc::launch_gather_stream(ctx, st, g, u, nullptr, 0, &dn, 1, static_cast<const uint32_t *>(expert_offsets), m_total, hidden, inter,
                                      n_experts, group_size, dtype, ctx->d_gfrag);
        if (e != cudaSuccess) return fail(ctx, MTC_ERR_DISPATCH, std::string("moe_experts (down) launch: ") + cudaGetErrorString(e));
        return MTC_OK;
    }
    // composed from the separate entries, same results
    const void *rows = x;
    int rc = MTC_OK;
    if (sort_token_idx) {
        rc = mtc_moe_permute(ctx, stream, x, sort_token_idx, xp, m_total, hidden, dtype);
        if (rc != MTC_OK) return rc;
        rows = xp;
    }
    rc = mtc_gather_qmm(ctx, stream, rows, gate->w, gate->scales, gate->biases, expert_offsets, nullptr, g, m_total, inter, hidden, n_experts, bits, group_size, dtype);
    if (rc != MTC_OK) return rc;
    rc = mtc_gather_qmm(ctx, stream, rows, up->w, up->scales, up->biases, expert_offsets, nullptr, u, m_total, inter, hidden, n_experts, bits, group_size, dtype);
    if (rc != MTC_OK) return rc;
    rc = mtc_swiglu(ctx, stream, g, u, g, static_cast<size_t>(m_total) * inter, dtype);
    if (rc != MTC_OK) return rc;
    return mtc_gather_qmm(ctx, stream, g, down->w, down->scales, down->biases, expert_offsets, nullptr, y, m_total, hidden, inter, n_experts, bits, group_size, dtype);
}

int mtc_gather_qmm_static(mtc_ctx *ctx, void *stream, const void *x, const void *w, const void *scales,
                          const void *biases, const void *expert_offsets, const void *indices, void *out, int m_total,
                          int n_out, int k_in, int n_experts, int bits, int group_size, int dtype) {
    if (!ctx) return MTC_ERR_INVALID;
    MTC_ENTER(ctx);
    if (dtype != MTC_F16 && dtype != MTC_BF16)
        return fail(ctx, MTC_ERR_UNSUPPORTED, "gather_qmm_static: dtype must be f16 or bf16 (the tensor-core path)");
    if ((expert_offsets == nullptr) == (indices == nullptr))
        return fail(ctx, MTC_ERR_INVALID, "gather_qmm_static: give exactly one of expert_offsets and indices");
    if (m_total < 0 || n_out < 0 || n_experts <= 0 || n_experts > 4096)
        return fail(ctx, MTC_ERR_UNSUPPORTED, "gather_qmm_static: need 0 < n_experts <= 4096 and non-negative sizes");
    if (m_total == 0 || n_out == 0) return MTC_OK;
    if (!x || !w || !scales || !biases || !out) return fail(ctx, MTC_ERR_INVALID, "gather_qmm_static: null pointer");
    if (!mtc::qmm_tcgen05_supported(m_total, n_out, k_in, bits, group_size, dtype, w, x, out))
        return fail(ctx, MTC_ERR_UNSUPPORTED,
                    "gather_qmm_static: needs bits in {2,3,4,5,6,8}, k_in % 64 == 0, a power-of-two group >= 32 and "
                    "16-byte aligned x and w");
    std::string why;
    cudaError_t e = mtc::launch_gather_qmm_static(ctx, static_cast<cudaStream_t>(stream), x, w, scales, biases,
                                                  static_cast<const uint32_t *>(expert_offsets),
                                                  static_cast<const uint32_t *>(indices), out, m_total, n_out, k_in,
                                                  n_experts, bits, group_size, dtype, &why);
    if (e == cudaErrorInvalidValue && !why.empty()) return fail(ctx, MTC_ERR_BUFFER_SIZE, why);
    if (e != cudaSuccess)
        return fail(ctx, MTC_ERR_DISPATCH, "gather_qmm_static launch: " + (why.empty() ? std::string(cudaGetErrorString(e)) : why));
    return MTC_OK;
}

const char *mtc_gather_qmm_route(int m_total, int n_out, int k_in, int n_experts, int bits, int group_size, int dtype) {
    if (n_experts > 0 && static_cast<long long>(m_total) <= 64ll * n_experts &&
        mtc::gather_stream_supported(m_total, n_out, k_in, n_experts, bits, group_size, dtype, nullptr, nullptr, nullptr, nullptr))
        return "gather_qmm_stream";        // the CSR form with option "gather_stream" at its default
    return mtc::qmm_tcgen05_supported(m_total, n_out, k_in, bits, group_size, dtype, nullptr, nullptr, nullptr)
               ? "gather_qmm_tcgen05" : "gather_qmm_cuda_core";
}

int mtc_moe_router_topk(mtc_ctx *ctx, void *stream, const void *router_logits, void *indices_out, void *weights_out,
                        int n_rows, int n_experts, int k, int norm_topk_prob, int dtype) {
    if (!ctx) return MTC_ERR_INVALID;
    MTC_ENTER(ctx);
    if (!dtype_ok(dtype)) return fail(ctx, MTC_ERR_UNSUPPORTED, "router_topk: dtype must be f32, f16 or bf16");
    // k <= 32 is the reference's hard cap (crates/metaltile-std/src/ffai/moe.rs:88-91); n_experts <= 32 * 32
    if (n_rows < 0 || n_experts <= 0 || n_experts > 1024 || k <= 0 || k > 32 || k > n_experts)
        return fail(ctx, MTC_ERR_UNSUPPORTED, "router_topk: need 0 < k <= min(32, n_experts), n_experts <= 1024");
    if (n_rows > 0 && (!router_logits || !indices_out || !weights_out)) return fail(ctx, MTC_ERR_INVALID, "router_topk: null pointer");
    MTC_CUDA(ctx, mtc::launch_router_topk(static_cast<cudaStream_t>(stream), router_logits, static_cast<uint32_t *>(indices_out),
                                          weights_out, n_rows, n_experts, k, norm_topk_prob, dtype), MTC_ERR_DISPATCH);
    return MTC_OK;
}

int mtc_moe_sort(mtc_ctx *ctx, void *stream, const void *topk_idx, int n_tokens, int k, int n_experts, void *sort_token_idx,
                 void *inv_perm, void *expert_offsets, void *row_expert) {
    if (!ctx) return MTC_ERR_INVALID;
    MTC_ENTER(ctx);
    if (n_tokens < 0 || k <= 0 || n_experts <= 0 || n_experts > 1024)
        return fail(ctx, MTC_ERR_UNSUPPORTED, "moe_sort: need k > 0 and 0 < n_experts <= 1024");
    if (!expert_offsets || (n_tokens > 0 && (!topk_idx || !sort_token_idx || !inv_perm)))
        return fail(ctx, MTC_ERR_INVALID, "moe_sort: null pointer");
    MTC_CUDA(ctx, mtc::launch_moe_sort(static_cast<cudaStream_t>(stream), static_cast<const uint32_t *>(topk_idx), n_tokens, k,
                                       n_experts, static_cast<uint32_t *>(sort_token_idx), static_cast<uint32_t *>(inv_perm),
                                       static_cast<uint32_t *>(expert_offsets), static_cast<uint32_t *>(row_expert),
                                       ctx->d_status), MTC_ERR_DISPATCH);
    return MTC_OK;
}

int mtc_moe_permute(mtc_ctx *ctx, void *stream, const void *tokens, const void *sort_token_idx, void *permuted, int n_rows,
                    int hidden, int dtype) {
    if (!ctx) return MTC_ERR_INVALID;
    MTC_ENTER(ctx);
    if (!dtype_ok(dtype) || n_rows < 0 || hidden <= 0) return fail(ctx, MTC_ERR_UNSUPPORTED, "moe_permute: bad dtype or shape");
    if (n_rows > 0 && (!tokens || !sort_token_idx || !permuted)) return fail(ctx, MTC_ERR_INVALID, "moe_permute: null pointer");
    MTC_CUDA(ctx, mtc::launch_permute(static_cast<cudaStream_t>(stream), tokens, static_cast<const uint32_t *>(sort_token_idx),
                                      permuted, n_rows, hidden, dtype), MTC_ERR_DISPATCH);
    return MTC_OK;
}

int mtc_moe_unpermute(mtc_ctx *ctx, void *stream, const void *expert_outputs, const void *inv_perm, const void *top_k_weights,
                      void *out, int n_tokens, int hidden, int k, int dtype) {
    if (!ctx) return MTC_ERR_INVALID;
    MTC_ENTER(ctx);
    if (!dtype_ok(dtype) || n_tokens < 0 || hidden <= 0 || k <= 0)
        return fail(ctx, MTC_ERR_UNSUPPORTED, "moe_unpermute: bad dtype or shape");
    if (n_tokens > 0 && (!expert_outputs || !inv_perm || !top_k_weights || !out))
        return fail(ctx, MTC_ERR_INVALID, "moe_unpermute: null pointer");
    MTC_CUDA(ctx, mtc::launch_unpermute(static_cast<cudaStream_t>(stream), expert_outputs, static_cast<const uint32_t *>(inv_perm),
                                        top_k_weights, out, n_tokens, hidden, k, dtype), MTC_ERR_DISPATCH);
    return MTC_OK;
}

int mtc_swiglu(mtc_ctx *ctx, void *stream, const void *gate, const void *up, void *out, size_t n, int dtype) {
    if (!ctx) return MTC_ERR_INVALID;
    MTC_ENTER(ctx);
    if (!dtype_ok(dtype)) return fail(ctx, MTC_ERR_UNSUPPORTED, "swiglu: dtype must be f32, f16 or bf16");
    if (n > 0 && (!gate || !up || !out)) return fail(ctx, MTC_ERR_INVALID, "swiglu: null pointer");
    MTC_CUDA(ctx, mtc::launch_swiglu(static_cast<cudaStream_t>(stream), gate, up, out, n, dtype), MTC_ERR_DISPATCH);
    return MTC_OK;
}

int mtc_unpack_codes(mtc_ctx *ctx, void *stream, const void *w, void *codes_u8, int N, int K, int bits) {
    if (!ctx) return MTC_ERR_INVALID;
    MTC_ENTER(ctx);
    if (bits < 1 || bits > 8 || (static_cast<long long>(K) * bits) % 32 != 0)
        return fail(ctx, MTC_ERR_UNSUPPORTED, "unpack_codes: need 1 <= bits <= 8 and K*bits % 32 == 0");
    MTC_CUDA(ctx, mtc::launch_unpack_codes(static_cast<cudaStream_t>(stream), w, codes_u8, N, K, bits), MTC_ERR_DISPATCH);
    return MTC_OK;
}

int mtc_kernel_count(void) { return kNumKernels; }
const char *mtc_kernel_name(int i) { return (i >= 0 && i < kNumKernels) ? kKernels[i].name : nullptr; }

}  // extern "C"

namespace {

// A chain of passes (mtc_dispatch_chain): what earlier passes produced, by buffer name, and where the next pass stages.
struct Produced {
    std::string name;
    char *dev;
    size_t bytes;
    mtc_named_buf *host;     // the output buffer of the producing pass; read back at the end unless a later pass consumes it
    bool consumed;
};
struct ChainCtx {
    bool measure = true;             // first walk: only the bytes every pass stages
    bool skip_upload = false;        // mtc_measure after its first launch: the inputs are already where this walk puts them
    size_t offset = 0;               // scratch bytes taken by the passes walked so far
    std::vector<Produced> produced;
};

// One pass.  Stand-alone (cc == nullptr): stage, launch, read the outputs back, synchronise.  In a chain: an input that an
// earlier pass produced under the same name is that pass's device buffer (no host copy), nothing is read back and nothing
// synchronises here.
int dispatch_pass(mtc_ctx *ctx, const char *kernel_name, int dtype, mtc_named_buf *bufs, int n_bufs, float *elapsed_us, ChainCtx *cc) {
    if (!ctx || !kernel_name || (!bufs && n_bufs > 0)) return MTC_ERR_INVALID;
    if (!dtype_ok(dtype)) return fail(ctx, MTC_ERR_UNSUPPORTED, "dispatch: dtype must be f32, f16 or bf16");
    const KernelRow *row = find_kernel(kernel_name);
    if (!row) return fail(ctx, MTC_ERR_FUNCTION_NOT_FOUND, std::string("unknown kernel: ") + kernel_name);
    const size_t esz = mtc::dtype_size(dtype);
    const std::string kn(kernel_name);

    // ---- bind buffers and constexprs by name, derive the shape, compute the bytes each buffer must hold
    std::vector<Staged> st_bufs;
    std::string err;
    auto need_buf = [&](const char *name, size_t need) -> Staged * {
        mtc_named_buf *b = find_buf(bufs, n_bufs, name);
        if (!b || !b->data) { if (err.empty()) err = kn + ": buffer '" + name + "' must be bound"; return nullptr; }
        st_bufs.push_back(Staged{b, need, 0, nullptr});
        return &st_bufs.back();
    };
    auto need_const = [&](const char *name, uint32_t *v) {
        if (!read_const(bufs, n_bufs, name, v) && err.empty()) err = kn + ": constexpr " + name + " missing";
    };
    st_bufs.reserve(32);
    float rms_eps = 0.0f;
    int nb = 0;                          // fused decode projections: count, rows of each, buffer names of each
    uint32_t b_out[4] = {0, 0, 0, 0};
    std::string b_names[4][4];
    uint32_t k = 0, n = 0, gsc = 0, k_in = 0, m_out = 0, n_exp = 0, gs = 0, hidden = 0, topk = 0, norm = 1, m_total = 0;
    size_t m = 0, rows = 0;
    switch (row->family) {
        case DENSE_QMV:
        case DENSE_QMM: {
            need_const("k", &k);
            need_const(row->gs_const, &gsc);
            if (row->has_n) need_const("n", &n);
            if (!err.empty()) break;
            mtc_named_buf *bx = find_buf(bufs, n_bufs, "x"), *bo = find_buf(bufs, n_bufs, "out");
            if (!bx || !bo) { err = kn + ": buffers w, scales, biases, x, out must be bound"; break; }
            if (k == 0 || gsc == 0) { err = kn + ": k and the group constexpr must be positive"; break; }
            gs = std::strcmp(row->gs_const, "gs_per_row") == 0 ? k / gsc : gsc;
            if (gs == 0 || k % gs != 0) return fail(ctx, MTC_ERR_UNSUPPORTED, kn + ": group size must divide k");
            if (!row->has_n) n = static_cast<uint32_t>(bo->bytes / esz);  // mt_qmv: M = 1, N = len(out)
            m = bx->bytes / (static_cast<size_t>(k) * esz);
            if (m == 0) return fail(ctx, MTC_ERR_BUFFER_SIZE, kn + ": x holds less than one row of k");
            if ((static_cast<unsigned long long>(k) * row->bits) % 32 != 0)
                return fail(ctx, MTC_ERR_UNSUPPORTED, kn + ": k*bits must be a multiple of 32");
            need_buf("w", static_cast<size_t>(n) * k * row->bits / 8);
            need_buf("scales", static_cast<size_t>(n) * (k / gs) * esz);
            need_buf("biases", static_cast<size_t>(n) * (k / gs) * esz);
            need_buf("x", m * k * esz);
            need_buf("out", m * n * esz);
            break;
        }
        case GATHER_CSR:
        case GATHER_IDX: {
            const bool csr = row->family == GATHER_CSR;
            need_const("k_in", &k_in);
            need_const("group_size", &gs);
            if (csr) { need_const("m_out", &m_out); need_const("n_experts", &n_exp); }
            else { need_const("n_out", &m_out); need_const("m_total", &m_total); }
            if (!err.empty()) break;
            mtc_named_buf *bx = find_buf(bufs, n_bufs, "x");
            mtc_named_buf *bw = find_buf(bufs, n_bufs, csr ? "weight_packed" : "w");
            if (!bx || !bw) { err = kn + ": buffers x and " + (csr ? "weight_packed" : "w") + " must be bound"; break; }
            if (k_in == 0 || gs == 0 || m_out == 0 || k_in % gs != 0 || (static_cast<unsigned long long>(k_in) * row->bits) % 32 != 0)
                return fail(ctx, MTC_ERR_UNSUPPORTED, kn + ": need k_in*bits % 32 == 0 and group_size | k_in");
            rows = csr ? bx->bytes / (static_cast<size_t>(k_in) * esz) : m_total;
            const size_t w_per_expert = static_cast<size_t>(m_out) * k_in * row->bits / 8;
            if (!csr) n_exp = static_cast<uint32_t>(bw->bytes / w_per_expert);   // stacked [E, n_out, k_in*bits/32]
            if (n_exp == 0) return fail(ctx, MTC_ERR_BUFFER_SIZE, kn + ": weights hold less than one expert");
            need_buf("x", rows * k_in * esz);
            need_buf(csr ? "weight_packed" : "w", static_cast<size_t>(n_exp) * w_per_expert);
            need_buf("scales", static_cast<size_t>(n_exp) * m_out * (k_in / gs) * esz);
            need_buf("biases", static_cast<size_t>(n_exp) * m_out * (k_in / gs) * esz);
            need_buf(csr ? "expert_offsets" : "indices", csr ? (static_cast<size_t>(n_exp) + 1) * 4 : rows * 4);
            need_buf("out", rows * m_out * esz);
            break;
        }
        case BATCHED_QKV:
        case BATCHED_4: {
            const bool qkv = row->family == BATCHED_QKV;
            nb = qkv ? 3 : 4;
            static const char *const sfx_qkv[3] = {"q", "k", "v"}, *const sfx_4[4] = {"a", "b", "c", "d"};
            for (int i = 0; i < nb; ++i) need_const((std::string("out_") + (qkv ? sfx_qkv[i] : sfx_4[i])).c_str(), &b_out[i]);
            need_const("in_dim", &k);
            need_const("group_size", &gs);
            if (!err.empty()) break;
            if (k == 0 || gs == 0 || k % gs != 0 || k % 8 != 0) return fail(ctx, MTC_ERR_UNSUPPORTED, kn + ": need group_size | in_dim and in_dim % 8 == 0");
            need_buf("x", static_cast<size_t>(k) * esz);
            size_t sum = 0;
            for (int i = 0; i < nb; ++i) {
                const std::string sf = qkv ? sfx_qkv[i] : sfx_4[i];
                b_names[i][0] = "w_" + sf;
                b_names[i][1] = "scales_" + sf;
                b_names[i][2] = "biases_" + sf;
                b_names[i][3] = sf + "_out";
                need_buf(b_names[i][0].c_str(), static_cast<size_t>(b_out[i]) * k / 2);
                need_buf(b_names[i][1].c_str(), static_cast<size_t>(b_out[i]) * (k / gs) * esz);
                need_buf(b_names[i][2].c_str(), static_cast<size_t>(b_out[i]) * (k / gs) * esz);
                if (!qkv) need_buf(b_names[i][3].c_str(), static_cast<size_t>(b_out[i]) * esz);
                sum += b_out[i];
            }
            if (qkv) need_buf("out", sum * esz);
            break;
        }
        case AFFINE_Q:
        case AFFINE_DQ: {
            need_const("group_size", &gs);
            if (!err.empty()) break;
            const bool quant = row->family == AFFINE_Q;
            mtc_named_buf *bw = find_buf(bufs, n_bufs, "w");
            if (!bw) { err = kn + ": buffers w, out, scales, biases must be bound"; break; }
            if (gs == 0 || (static_cast<unsigned long long>(gs) * row->bits) % 32 != 0)
                return fail(ctx, MTC_ERR_UNSUPPORTED, kn + ": group_size * bits must be a multiple of 32");
            rows = quant ? bw->bytes / esz : (bw->bytes / 4) * 32 / row->bits;      // elements
            rows -= rows % gs;
            need_buf("w", quant ? rows * esz : rows * row->bits / 8);
            need_buf("out", quant ? rows * row->bits / 8 : rows * esz);
            need_buf("scales", rows / gs * esz);
            need_buf("biases", rows / gs * esz);
            break;
        }
        case MOE_TAIL:
        case EXPERT_QMV: {
            need_const("in_dim", &k);
            need_const("out_dim", &n);
            need_const("group_size", &gs);
            if (!err.empty()) break;
            mtc_named_buf *bw = find_buf(bufs, n_bufs, "weights_stacked");
            if (!bw) { err = kn + ": buffer 'weights_stacked' must be bound"; break; }
            if (k == 0 || n == 0 || gs == 0 || k % gs != 0 || k % 8 != 0) return fail(ctx, MTC_ERR_UNSUPPORTED, kn + ": need group_size | in_dim and in_dim % 8 == 0");
            n_exp = static_cast<uint32_t>(bw->bytes / (static_cast<size_t>(n) * k / 2));
            if (n_exp == 0) return fail(ctx, MTC_ERR_BUFFER_SIZE, kn + ": weights hold less than one expert");
            need_buf("weights_stacked", static_cast<size_t>(n_exp) * n * k / 2);
            need_buf("scales_stacked", static_cast<size_t>(n_exp) * n * (k / gs) * esz);
            need_buf("biases_stacked", static_cast<size_t>(n_exp) * n * (k / gs) * esz);
            need_buf("output", static_cast<size_t>(n) * esz);
            if (row->family == MOE_TAIL) {
                for (int i = 0; i < 8; ++i) {
                    b_names[i / 4][i % 4] = "gate_" + std::to_string(i);      // 16 names in the two name tables
                    b_names[2 + i / 4][i % 4] = "up_" + std::to_string(i);
                    need_buf(b_names[i / 4][i % 4].c_str(), static_cast<size_t>(k) * esz);
                    need_buf(b_names[2 + i / 4][i % 4].c_str(), static_cast<size_t>(k) * esz);
                }
                need_buf("expert_indices", 8 * 4);
                need_buf("slot_weights", 8 * esz);
            } else {
                need_buf("input", static_cast<size_t>(k) * esz);
                need_buf("expert_index", 4);
            }
            break;
        }
        case QVM: {
            need_const("k", &k);
            need_const("n", &n);
            need_const(row->gs_const, &gsc);
            if (!err.empty()) break;
            mtc_named_buf *bx = find_buf(bufs, n_bufs, "x");
            if (!bx) { err = kn + ": buffers w, scales, biases, x, out must be bound"; break; }
            if (k == 0 || n == 0 || gsc == 0) { err = kn + ": k, n and the group constexpr must be positive"; break; }
            gs = std::strcmp(row->gs_const, "gs_per_col") == 0 ? k / gsc : gsc;
            if (gs == 0 || k % gs != 0 || (static_cast<unsigned long long>(n) * row->bits) % 32 != 0)
                return fail(ctx, MTC_ERR_UNSUPPORTED, kn + ": group size must divide k and n * bits must be a multiple of 32");
            m = bx->bytes / (static_cast<size_t>(k) * esz);
            if (m == 0) return fail(ctx, MTC_ERR_BUFFER_SIZE, kn + ": x holds less than one row of k");
            need_buf("w", static_cast<size_t>(k) * n * row->bits / 8);
            need_buf("scales", static_cast<size_t>(k / gs) * n * esz);
            need_buf("biases", static_cast<size_t>(k / gs) * n * esz);
            need_buf("x", m * k * esz);
            need_buf("out", m * n * esz);
            break;
        }
        case DQ_GATHER: {
            need_const("hidden", &hidden);
            need_const("group_size", &gs);
            if (!err.empty()) break;
            mtc_named_buf *bw = find_buf(bufs, n_bufs, "weight"), *bi = find_buf(bufs, n_bufs, "indices");
            if (!bw || !bi) { err = kn + ": buffers weight, scales, biases, indices, out must be bound"; break; }
            if (hidden == 0 || gs == 0 || hidden % gs != 0 || (static_cast<unsigned long long>(hidden) * row->bits) % 32 != 0)
                return fail(ctx, MTC_ERR_UNSUPPORTED, kn + ": need group_size | hidden and hidden * bits % 32 == 0");
            rows = bi->bytes / 4;                                                  // tokens
            n_exp = static_cast<uint32_t>(bw->bytes / (static_cast<size_t>(hidden) * row->bits / 8));    // vocab
            if (n_exp == 0) return fail(ctx, MTC_ERR_BUFFER_SIZE, kn + ": weight holds less than one row");
            need_buf("weight", static_cast<size_t>(n_exp) * hidden * row->bits / 8);
            need_buf("scales", static_cast<size_t>(n_exp) * (hidden / gs) * esz);
            need_buf("biases", static_cast<size_t>(n_exp) * (hidden / gs) * esz);
            need_buf("indices", rows * 4);
            need_buf("out", rows * hidden * esz);
            break;
        }
        case RMS_QMV: {
            need_const("in_dim", &k);
            need_const("group_size", &gs);
            if (!err.empty()) break;
            mtc_named_buf *bo = find_buf(bufs, n_bufs, "output"), *be = find_buf(bufs, n_bufs, "eps_buf");
            if (!bo || !be || !be->data || be->bytes < 4) { err = kn + ": buffers x, norm_weight, weight, scales, biases, output, eps_buf must be bound"; break; }
            if (k == 0 || gs == 0 || k % gs != 0 || k % 8 != 0) return fail(ctx, MTC_ERR_UNSUPPORTED, kn + ": need group_size | in_dim and in_dim % 8 == 0");
            n = static_cast<uint32_t>(bo->bytes / esz);
            std::memcpy(&rms_eps, be->data, 4);
            need_buf("x", static_cast<size_t>(k) * esz);
            need_buf("norm_weight", static_cast<size_t>(k) * esz);
            need_buf("weight", static_cast<size_t>(n) * k / 2);
            need_buf("scales", static_cast<size_t>(n) * (k / gs) * esz);
            need_buf("biases", static_cast<size_t>(n) * (k / gs) * esz);
            need_buf("output", static_cast<size_t>(n) * esz);
            break;
        }
        case ROUTER_TOPK: {
            need_const("n_experts", &n_exp);
            need_const("k", &topk);
            if (!read_const(bufs, n_bufs, "norm_topk_prob", &norm)) norm = 1;
            if (!err.empty()) break;
            mtc_named_buf *bl = find_buf(bufs, n_bufs, "router_logits");
            if (!bl) { err = kn + ": buffer 'router_logits' must be bound"; break; }
            if (n_exp == 0) { err = kn + ": n_experts must be positive"; break; }
            rows = bl->bytes / (static_cast<size_t>(n_exp) * esz);
            need_buf("router_logits", rows * n_exp * esz);
            need_buf("indices_out", rows * topk * 4);
            need_buf("weights_out", rows * topk * esz);
            break;
        }
        case MOE_PERMUTE: {
            need_const("hidden", &hidden);
            if (!err.empty()) break;
            mtc_named_buf *bi = find_buf(bufs, n_bufs, "sort_token_idx"), *bt = find_buf(bufs, n_bufs, "tokens");
            if (!bi || !bt) { err = kn + ": buffers tokens, sort_token_idx, permuted must be bound"; break; }
            rows = bi->bytes / 4;
            need_buf("tokens", bt->bytes);   // row indices are data: the kernel reads the rows they name
            need_buf("sort_token_idx", rows * 4);
            need_buf("permuted", rows * hidden * esz);
            break;
        }
        case MOE_UNPERMUTE: {
            need_const("hidden", &hidden);
            need_const("k", &topk);
            if (!err.empty()) break;
            mtc_named_buf *bi = find_buf(bufs, n_bufs, "inv_perm");
            if (!bi || topk == 0) { err = kn + ": buffer 'inv_perm' must be bound and k positive"; break; }
            rows = bi->bytes / (4 * static_cast<size_t>(topk));
            need_buf("expert_outputs", rows * topk * hidden * esz);
            need_buf("inv_perm", rows * topk * 4);
            need_buf("top_k_weights", rows * topk * esz);
            need_buf("out", rows * hidden * esz);
            break;
        }
        case SWIGLU: {
            mtc_named_buf *bg = find_buf(bufs, n_bufs, "gate");
            if (!bg) { err = kn + ": buffer 'gate' must be bound"; break; }
            rows = bg->bytes / esz;
            need_buf("gate", rows * esz);
            need_buf("up", rows * esz);
            need_buf("out", rows * esz);
            break;
        }
    }
    if (!err.empty()) return fail(ctx, MTC_ERR_BUFFER, err);
    // An undersized buffer is an error (crates/metaltile-runtime/src/dispatch/buffer_plan.rs:68-76).
    size_t total = 0;
    for (Staged &sb : st_bufs) {
        if (sb.buf->bytes < sb.need)
            return fail(ctx, MTC_ERR_BUFFER_SIZE, kn + ": buffer '" + sb.buf->name + "' holds " + std::to_string(sb.buf->bytes) +
                                                     " bytes, the kernel needs " + std::to_string(sb.need));
        sb.offset = total;
        total += align_up(sb.need ? sb.need : 1, 256);
    }
    MTC_CUDA(ctx, cudaSetDevice(ctx->device), MTC_ERR_NO_DEVICE);
    int rc = MTC_OK;
    if (cc && cc->measure) {
        cc->offset += total;
        return MTC_OK;
    }
    if (!cc) {
        rc = ensure_scratch(ctx, total);
        if (rc != MTC_OK) return rc;
    }
    const size_t base_off = cc ? cc->offset : 0;
    if (cc) cc->offset += total;
    cudaStream_t st = nullptr;
    for (Staged &sb : st_bufs) {
        sb.dev = static_cast<char *>(ctx->d_scratch) + base_off + sb.offset;
        Produced *from = nullptr;
        if (cc && !sb.buf->is_output)
            for (Produced &pr : cc->produced)
                if (pr.name == sb.buf->name) from = &pr;          // the latest producer of that name
        if (from) {
            if (from->bytes < sb.need)
                return fail(ctx, MTC_ERR_BUFFER_SIZE, kn + ": buffer '" + sb.buf->name + "' was produced with " + std::to_string(from->bytes) +
                                                         " bytes by an earlier pass, this pass needs " + std::to_string(sb.need));
            sb.dev = from->dev;
            from->consumed = true;
        } else if (sb.need && !(cc && cc->skip_upload)) {
            MTC_CUDA(ctx, cudaMemcpyAsync(sb.dev, sb.buf->data, sb.need, cudaMemcpyHostToDevice, st), MTC_ERR_BUFFER);
        }
    }
    auto dev = [&](const char *name) -> char * {
        for (Staged &sb : st_bufs)
            if (std::strcmp(sb.buf->name, name) == 0) return sb.dev;
        return nullptr;
    };
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    if (elapsed_us) {
        MTC_CUDA(ctx, cudaEventCreate(&e0), MTC_ERR_DISPATCH);
        MTC_CUDA(ctx, cudaEventCreate(&e1), MTC_ERR_DISPATCH);
        cudaEventRecord(e0, st);
    }
    switch (row->family) {
        case DENSE_QMM:
            rc = mtc_qmm(ctx, st, dev("w"), dev("scales"), dev("biases"), dev("x"), dev("out"), static_cast<int>(m),
                         static_cast<int>(n), static_cast<int>(k), row->bits, static_cast<int>(gs), dtype);
            break;
        case DENSE_QMV:
            rc = mtc_qmv(ctx, st, dev("w"), dev("scales"), dev("biases"), dev("x"), dev("out"), static_cast<int>(m),
                         static_cast<int>(n), static_cast<int>(k), row->bits, static_cast<int>(gs), dtype);
            break;
        case GATHER_CSR:
            rc = mtc_gather_qmm(ctx, st, dev("x"), dev("weight_packed"), dev("scales"), dev("biases"), dev("expert_offsets"),
                                nullptr, dev("out"), static_cast<int>(rows), static_cast<int>(m_out), static_cast<int>(k_in),
                                static_cast<int>(n_exp), row->bits, static_cast<int>(gs), dtype);
            break;
        case GATHER_IDX:
            rc = mtc_gather_qmm(ctx, st, dev("x"), dev("w"), dev("scales"), dev("biases"), nullptr, dev("indices"), dev("out"),
                                static_cast<int>(rows), static_cast<int>(m_out), static_cast<int>(k_in), static_cast<int>(n_exp),
                                row->bits, static_cast<int>(gs), dtype);
            break;
        case BATCHED_QKV:
        case BATCHED_4: {
            // one launch for all projections (mtc_qmv_batched); y of the q / k / v form is one concatenated vector
            mtc_qmv_desc ds[4] = {};
            size_t off = 0;
            for (int i = 0; i < nb; ++i) {
                ds[i].w = dev(b_names[i][0].c_str());
                ds[i].scales = dev(b_names[i][1].c_str());
                ds[i].biases = dev(b_names[i][2].c_str());
                ds[i].x = dev("x");
                ds[i].outs[0] = row->family == BATCHED_QKV ? dev("out") + off * esz : dev(b_names[i][3].c_str());
                ds[i].n_outs = 1;
                ds[i].M = 1;
                ds[i].N = static_cast<int>(b_out[i]);
                ds[i].K = static_cast<int>(k);
                ds[i].bits = 4;
                ds[i].group_size = static_cast<int>(gs);
                ds[i].dtype = dtype;
                off += b_out[i];
            }
            rc = mtc_qmv_batched(ctx, st, ds, nb);
            break;
        }
        case AFFINE_Q:
            rc = mtc_affine_quantize(ctx, st, dev("w"), dev("out"), dev("scales"), dev("biases"), rows, row->bits, static_cast<int>(gs), dtype);
            break;
        case AFFINE_DQ:
            rc = mtc_affine_dequantize(ctx, st, dev("w"), dev("scales"), dev("biases"), dev("out"), rows, row->bits, static_cast<int>(gs), dtype);
            break;
        case MOE_TAIL: {
            const void *gs8[8], *us8[8];
            for (int i = 0; i < 8; ++i) {
                gs8[i] = dev(b_names[i / 4][i % 4].c_str());
                us8[i] = dev(b_names[2 + i / 4][i % 4].c_str());
            }
            rc = mtc_moe_down_swiglu_accum(ctx, st, gs8, us8, 8, dev("expert_indices"), dev("slot_weights"), dev("weights_stacked"),
                                           dev("scales_stacked"), dev("biases_stacked"), dev("output"), static_cast<int>(k), static_cast<int>(n),
                                           static_cast<int>(n_exp), static_cast<int>(gs), dtype);
            break;
        }
        case EXPERT_QMV: {
            const void *xs1[1] = {dev("input")};
            rc = mtc_qmv_expert_indexed(ctx, st, xs1, 1, dev("expert_index"), dev("weights_stacked"), dev("scales_stacked"), dev("biases_stacked"),
                                        dev("output"), static_cast<int>(k), static_cast<int>(n), static_cast<int>(n_exp), static_cast<int>(gs), dtype);
            break;
        }
        case QVM:
            rc = mtc_qvm(ctx, st, dev("w"), dev("scales"), dev("biases"), dev("x"), dev("out"), static_cast<int>(m), static_cast<int>(n),
                         static_cast<int>(k), row->bits, static_cast<int>(gs), dtype);
            break;
        case DQ_GATHER:
            rc = mtc_dequant_gather(ctx, st, dev("weight"), dev("scales"), dev("biases"), dev("indices"), dev("out"), rows,
                                    static_cast<int>(hidden), static_cast<int>(n_exp), row->bits, static_cast<int>(gs), dtype);
            break;
        case RMS_QMV:
            rc = mtc_rms_norm_qmv(ctx, st, dev("x"), dev("norm_weight"), rms_eps, dev("weight"), dev("scales"), dev("biases"), dev("output"),
                                  static_cast<int>(n), static_cast<int>(k), 4, static_cast<int>(gs), dtype);
            break;
        case ROUTER_TOPK:
            rc = mtc_moe_router_topk(ctx, st, dev("router_logits"), dev("indices_out"), dev("weights_out"), static_cast<int>(rows),
                                     static_cast<int>(n_exp), static_cast<int>(topk), static_cast<int>(norm), dtype);
            break;
        case MOE_PERMUTE:
            rc = mtc_moe_permute(ctx, st, dev("tokens"), dev("sort_token_idx"), dev("permuted"), static_cast<int>(rows),
                                 static_cast<int>(hidden), dtype);
            break;
        case MOE_UNPERMUTE:
            rc = mtc_moe_unpermute(ctx, st, dev("expert_outputs"), dev("inv_perm"), dev("top_k_weights"), dev("out"),
                                   static_cast<int>(rows), static_cast<int>(hidden), static_cast<int>(topk), dtype);
            break;
        case SWIGLU:
            rc = mtc_swiglu(ctx, st, dev("gate"), dev("up"), dev("out"), rows, dtype);
            break;
    }
    if (elapsed_us) cudaEventRecord(e1, st);
    if (cc) {
        if (rc == MTC_OK)
            for (Staged &sb : st_bufs)
                if (sb.buf->is_output) cc->produced.push_back(Produced{sb.buf->name, sb.dev, sb.need, sb.buf, false});
        if (elapsed_us) {
            cudaEventDestroy(e0);
            cudaEventDestroy(e1);
        }
        return rc;
    }
    if (rc == MTC_OK) {
        // every is_output parameter is read back (crates/metaltile-runtime/src/dispatch/single_dispatch.rs:100-117)
        for (Staged &sb : st_bufs)
            if (sb.buf->is_output && sb.need) cudaMemcpyAsync(sb.buf->data, sb.dev, sb.need, cudaMemcpyDeviceToHost, st);
        cudaError_t e = cudaStreamSynchronize(st);
        if (e != cudaSuccess) rc = fail(ctx, MTC_ERR_DISPATCH, std::string("dispatch: ") + cudaGetErrorString(e));
        else rc = check_status(ctx, "dispatch");
    }
    if (elapsed_us) {
        float ms = 0.f;
        if (rc == MTC_OK && cudaEventElapsedTime(&ms, e0, e1) == cudaSuccess) *elapsed_us = ms * 1000.0f;
        cudaEventDestroy(e0);
        cudaEventDestroy(e1);
    }
    return rc;
}

}  // namespace

extern "C" {

int mtc_dispatch(mtc_ctx *ctx, const char *kernel_name, int dtype, mtc_named_buf *bufs, int n_bufs,
                 const uint32_t grid[3], const uint32_t tpg[3], float *elapsed_us) {
    (void)grid; (void)tpg;  // launch geometry belongs to the back end
    if (!ctx) return MTC_ERR_INVALID;
    MTC_ENTER(ctx);
    return dispatch_pass(ctx, kernel_name, dtype, bufs, n_bufs, elapsed_us, nullptr);
}

int mtc_dispatch_chain(mtc_ctx *ctx, const mtc_dispatch_spec *specs, int n_specs, float *elapsed_us) {
    if (!ctx || (!specs && n_specs > 0) || n_specs < 0) return MTC_ERR_INVALID;
    MTC_ENTER(ctx);
    if (n_specs == 0) return MTC_OK;
    ChainCtx cc;
    for (int i = 0; i < n_specs; ++i) {              // every pass is checked and sized before anything is enqueued
        int rc = dispatch_pass(ctx, specs[i].kernel_name, specs[i].dtype, specs[i].bufs, specs[i].n_bufs, nullptr, &cc);
        if (rc != MTC_OK) return rc;
    }
    int rc = ensure_scratch(ctx, cc.offset);
    if (rc != MTC_OK) return rc;
    cc.measure = false;
    cc.offset = 0;
    cudaStream_t st = nullptr;
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    if (elapsed_us) {
        MTC_CUDA(ctx, cudaEventCreate(&e0), MTC_ERR_DISPATCH);
        MTC_CUDA(ctx, cudaEventCreate(&e1), MTC_ERR_DISPATCH);
        cudaEventRecord(e0, st);
    }
    for (int i = 0; i < n_specs && rc == MTC_OK; ++i)
        rc = dispatch_pass(ctx, specs[i].kernel_name, specs[i].dtype, specs[i].bufs, specs[i].n_bufs, nullptr, &cc);
    if (elapsed_us) cudaEventRecord(e1, st);
    if (rc == MTC_OK) {
        // only buffers that no later pass consumed go back to the host (context.rs:347-353); one synchronisation for the chain
        for (Produced &pr : cc.produced)
            if (!pr.consumed && pr.bytes) cudaMemcpyAsync(pr.host->data, pr.dev, pr.bytes, cudaMemcpyDeviceToHost, st);
    }
    cudaError_t e = cudaStreamSynchronize(st);       // also on failure: nothing of the chain is in flight when this returns
    if (rc == MTC_OK) {
        if (e != cudaSuccess) rc = fail(ctx, MTC_ERR_DISPATCH, std::string("dispatch_chain: ") + cudaGetErrorString(e));
        else rc = check_status(ctx, "dispatch_chain");
    }
    if (elapsed_us) {
        float ms = 0.f;
        if (rc == MTC_OK && cudaEventElapsedTime(&ms, e0, e1) == cudaSuccess) *elapsed_us = ms * 1000.0f;
        cudaEventDestroy(e0);
        cudaEventDestroy(e1);
    }
    return rc;
}

int mtc_measure(mtc_ctx *ctx, const char *kernel_name, int dtype, mtc_named_buf *bufs, int n_bufs, int warmup, int iters,
                int cold_l2, double *samples_us, mtc_bench_stats *stats) {
    if (!ctx || !kernel_name || (!bufs && n_bufs > 0)) return MTC_ERR_INVALID;
    MTC_ENTER(ctx);
    if (warmup < 0 || iters < 1 || iters > (1 << 20)) return fail(ctx, MTC_ERR_INVALID, "measure: need warmup >= 0 and 1 <= iters <= 2^20");
    ChainCtx cc;
    int rc = dispatch_pass(ctx, kernel_name, dtype, bufs, n_bufs, nullptr, &cc);       // checks and sizes, enqueues nothing
    if (rc != MTC_OK) return rc;
    rc = ensure_scratch(ctx, cc.offset);
    if (rc != MTC_OK) return rc;
    cudaStream_t st = nullptr;
    constexpr size_t kFlushBytes = 256u << 20;                                         // twice the 126 MB L2
    if (cold_l2) {
        std::string why;
        cudaError_t e = mtc::grow_block(ctx, st, &ctx->d_flush, &ctx->flush_bytes, kFlushBytes, &why);
        if (e != cudaSuccess) return fail(ctx, MTC_ERR_BUFFER, std::string("measure: flush block: ") + cudaGetErrorString(e));
    }
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    MTC_CUDA(ctx, cudaEventCreate(&e0), MTC_ERR_DISPATCH);
    MTC_CUDA(ctx, cudaEventCreate(&e1), MTC_ERR_DISPATCH);
    cc.measure = false;
    cc.offset = 0;
    std::vector<double> samples;
    samples.reserve(iters);
    // One untimed launch stages the inputs (the only host-to-device copies of the call); every later walk finds them in place.
    rc = dispatch_pass(ctx, kernel_name, dtype, bufs, n_bufs, nullptr, &cc);
    cc.skip_upload = true;
    if (rc == MTC_OK && cudaStreamSynchronize(st) != cudaSuccess) rc = fail(ctx, MTC_ERR_DISPATCH, "measure: the first launch failed");
    for (int pass = 0; pass < warmup + iters && rc == MTC_OK; ++pass) {
        cc.offset = 0;
        cc.produced.clear();
        if (cold_l2) cudaMemsetAsync(ctx->d_flush, pass & 0xff, kFlushBytes, st);        // outside the timed pair of events
        cudaEventRecord(e0, st);
        rc = dispatch_pass(ctx, kernel_name, dtype, bufs, n_bufs, nullptr, &cc);
        cudaEventRecord(e1, st);
        if (rc != MTC_OK) break;
        cudaError_t e = cudaEventSynchronize(e1);
        float ms = 0.f;
        if (e != cudaSuccess || cudaEventElapsedTime(&ms, e0, e1) != cudaSuccess) {
            rc = fail(ctx, MTC_ERR_DISPATCH, std::string("measure: ") + cudaGetErrorString(e));
            break;
        }
        if (pass >= warmup) samples.push_back(static_cast<double>(ms) * 1000.0);
    }
    if (rc == MTC_OK) {
        for (Produced &pr : cc.produced)                                               // the last launch's outputs go back once
            if (pr.bytes) cudaMemcpyAsync(pr.host->data, pr.dev, pr.bytes, cudaMemcpyDeviceToHost, st);
    }
    cudaError_t e = cudaStreamSynchronize(st);
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    if (rc != MTC_OK) return rc;
    if (e != cudaSuccess) return fail(ctx, MTC_ERR_DISPATCH, std::string("measure: ") + cudaGetErrorString(e));
    rc = check_status(ctx, "measure");
    if (rc != MTC_OK) return rc;
    if (samples_us) std::copy(samples.begin(), samples.end(), samples_us);
    if (stats) {
        // the summary the reference prints (crates/metaltile-std/src/stats.rs:24-47): sorted samples, n/2, n*95/100, n*99/100
        std::vector<double> s(samples);
        std::sort(s.begin(), s.end());
        const size_t n = s.size();
        double mean = 0.0, var = 0.0;
        for (double v : s) mean += v;
        mean /= static_cast<double>(n);
        for (double v : s) var += (v - mean) * (v - mean);
        var /= static_cast<double>(n);
        stats->min_us = s[0];
        stats->mean_us = mean;
        stats->median_us = s[n / 2];
        stats->p95_us = s[std::min(n * 95 / 100, n - 1)];
        stats->p99_us = s[std::min(n * 99 / 100, n - 1)];
        stats->stddev_us = std::sqrt(var);
        stats->cv_pct = mean > 0.0 ? stats->stddev_us / mean * 100.0 : 0.0;
        stats->iters = static_cast<int>(n);
    }
    return MTC_OK;
}

}  // extern "C"
