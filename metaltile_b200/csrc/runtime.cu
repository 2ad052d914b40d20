// Runtime behind include/mtcuda.h: context, device memory, the typed entry points and
// the name-keyed host-buffer dispatch that mirrors Context::dispatch_with_grid
// (crates/metaltile-runtime/src/context.rs:269-284).
#include <cstdio>
#include <cstring>
#include <map>
#include <string>
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

bool dtype_ok(int dt) { return dt == MTC_F32 || dt == MTC_F16 || dt == MTC_BF16; }

// ---- kernel-name registry ------------------------------------------------------
// One row per reference kernel name the back end accepts.  `bits` < 0 means "not a
// dense kernel".  gs_const names the constexpr that carries the grouping:
// "gs_per_row" (hand-tuned int4/int8/mma kernels: group_size = k / gs_per_row) or
// "group_size" (generic _b* family).  has_n: whether an `n` constexpr is bound
// (mt_qmv / mt_qmv_int8_fast take N from the size of `out`).
enum Family { DENSE_QMV, DENSE_QMM };
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
        (e = mtc::qmv_init_device()) != cudaSuccess) {
        g_no_ctx_error = std::string("context set-up: ") + cudaGetErrorString(e);
        delete ctx;
        return MTC_ERR_DISPATCH;
    }
    *out_ctx = ctx;
    return MTC_OK;
}

int mtc_destroy(mtc_ctx *ctx) {
    if (!ctx) return MTC_ERR_INVALID;
    cudaSetDevice(ctx->device);
    if (ctx->d_status) cudaFree(ctx->d_status);
    if (ctx->d_scratch) cudaFree(ctx->d_scratch);
    delete ctx;
    return MTC_OK;
}

const char *mtc_last_error(mtc_ctx *ctx) { return ctx ? ctx->last_error.c_str() : g_no_ctx_error.c_str(); }

int mtc_device_info(mtc_ctx *ctx, char *json, size_t cap) {
    if (!ctx || !json || cap == 0) return MTC_ERR_INVALID;
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
    *d_ptr = nullptr;
    if (bytes == 0) return MTC_OK;
    MTC_CUDA(ctx, cudaMalloc(d_ptr, bytes), MTC_ERR_BUFFER);
    return MTC_OK;
}

int mtc_free(mtc_ctx *ctx, void *d_ptr) {
    if (!ctx) return MTC_ERR_INVALID;
    if (d_ptr) MTC_CUDA(ctx, cudaFree(d_ptr), MTC_ERR_BUFFER);
    return MTC_OK;
}

int mtc_upload(mtc_ctx *ctx, void *stream, void *d_dst, const void *h_src, size_t bytes) {
    if (!ctx || (bytes && (!d_dst || !h_src))) return fail(ctx, MTC_ERR_INVALID, "upload: null pointer");
    if (bytes)
        MTC_CUDA(ctx, cudaMemcpyAsync(d_dst, h_src, bytes, cudaMemcpyHostToDevice, static_cast<cudaStream_t>(stream)),
                 MTC_ERR_BUFFER);
    return MTC_OK;
}

int mtc_download(mtc_ctx *ctx, void *stream, void *h_dst, const void *d_src, size_t bytes) {
    if (!ctx || (bytes && (!h_dst || !d_src))) return fail(ctx, MTC_ERR_INVALID, "download: null pointer");
    if (bytes)
        MTC_CUDA(ctx, cudaMemcpyAsync(h_dst, d_src, bytes, cudaMemcpyDeviceToHost, static_cast<cudaStream_t>(stream)),
                 MTC_ERR_BUFFER);
    return MTC_OK;
}

int mtc_memset(mtc_ctx *ctx, void *stream, void *d_ptr, int value, size_t bytes) {
    if (!ctx || (bytes && !d_ptr)) return fail(ctx, MTC_ERR_INVALID, "memset: null pointer");
    if (bytes) MTC_CUDA(ctx, cudaMemsetAsync(d_ptr, value, bytes, static_cast<cudaStream_t>(stream)), MTC_ERR_BUFFER);
    return MTC_OK;
}

int mtc_sync(mtc_ctx *ctx, void *stream) {
    if (!ctx) return MTC_ERR_INVALID;
    MTC_CUDA(ctx, cudaStreamSynchronize(static_cast<cudaStream_t>(stream)), MTC_ERR_DISPATCH);
    return MTC_OK;
}

int mtc_status_word(mtc_ctx *ctx, uint32_t *word) {
    if (!ctx || !word) return MTC_ERR_INVALID;
    MTC_CUDA(ctx, cudaMemcpy(word, ctx->d_status, sizeof(uint32_t), cudaMemcpyDeviceToHost), MTC_ERR_DISPATCH);
    return MTC_OK;
}

int mtc_qmv(mtc_ctx *ctx, void *stream, const void *w, const void *scales, const void *biases, const void *x,
            void *out, int M, int N, int K, int bits, int group_size, int dtype) {
    if (!ctx) return MTC_ERR_INVALID;
    if (!dtype_ok(dtype)) return fail(ctx, MTC_ERR_UNSUPPORTED, "qmv: dtype must be f32, f16 or bf16");
    if (M > 0 && N > 0 && (!w || !scales || !biases || !x || !out)) return fail(ctx, MTC_ERR_INVALID, "qmv: null pointer");
    std::string why;
    cudaError_t e = mtc::launch_qmv(ctx, static_cast<cudaStream_t>(stream), w, scales, biases, x, out, M, N, K, bits,
                                    group_size, dtype, &why);
    if (e == cudaErrorInvalidValue && !why.empty()) return fail(ctx, MTC_ERR_UNSUPPORTED, why);
    if (e != cudaSuccess) return fail(ctx, MTC_ERR_DISPATCH, std::string("qmv launch: ") + cudaGetErrorString(e));
    return MTC_OK;
}

const char *mtc_qmm_route(int M, int N, int K, int bits, int group_size, int dtype) {
    (void)N; (void)K; (void)bits; (void)group_size;
    if (M <= 16 || dtype == MTC_F32) return "qmv_cuda_core";
    return "qmv_cuda_core";
}

int mtc_qmm(mtc_ctx *ctx, void *stream, const void *w, const void *scales, const void *biases, const void *x,
            void *out, int M, int N, int K, int bits, int group_size, int dtype) {
    return mtc_qmv(ctx, stream, w, scales, biases, x, out, M, N, K, bits, group_size, dtype);
}

int mtc_unpack_codes(mtc_ctx *ctx, void *stream, const void *w, void *codes_u8, int N, int K, int bits) {
    if (!ctx) return MTC_ERR_INVALID;
    if (bits < 1 || bits > 8 || (static_cast<long long>(K) * bits) % 32 != 0)
        return fail(ctx, MTC_ERR_UNSUPPORTED, "unpack_codes: need 1 <= bits <= 8 and K*bits % 32 == 0");
    MTC_CUDA(ctx, mtc::launch_unpack_codes(static_cast<cudaStream_t>(stream), w, codes_u8, N, K, bits), MTC_ERR_DISPATCH);
    return MTC_OK;
}

int mtc_kernel_count(void) { return kNumKernels; }
const char *mtc_kernel_name(int i) { return (i >= 0 && i < kNumKernels) ? kKernels[i].name : nullptr; }

int mtc_dispatch(mtc_ctx *ctx, const char *kernel_name, int dtype, mtc_named_buf *bufs, int n_bufs,
                 const uint32_t grid[3], const uint32_t tpg[3], float *elapsed_us) {
    (void)grid; (void)tpg;  // launch geometry belongs to the back end
    if (!ctx || !kernel_name || (!bufs && n_bufs > 0)) return MTC_ERR_INVALID;
    if (!dtype_ok(dtype)) return fail(ctx, MTC_ERR_UNSUPPORTED, "dispatch: dtype must be f32, f16 or bf16");
    const KernelRow *row = find_kernel(kernel_name);
    if (!row) return fail(ctx, MTC_ERR_FUNCTION_NOT_FOUND, std::string("unknown kernel: ") + kernel_name);
    const size_t esz = mtc::dtype_size(dtype);

    mtc_named_buf *bw = find_buf(bufs, n_bufs, "w"), *bs = find_buf(bufs, n_bufs, "scales"),
                  *bb = find_buf(bufs, n_bufs, "biases"), *bx = find_buf(bufs, n_bufs, "x"),
                  *bo = find_buf(bufs, n_bufs, "out");
    if (!bw || !bs || !bb || !bx || !bo)
        return fail(ctx, MTC_ERR_BUFFER, std::string(kernel_name) + ": buffers w, scales, biases, x, out must be bound");
    uint32_t k = 0, n = 0, gsc = 0;
    if (!read_const(bufs, n_bufs, "k", &k) || k == 0)
        return fail(ctx, MTC_ERR_BUFFER, std::string(kernel_name) + ": constexpr k missing");
    if (!read_const(bufs, n_bufs, row->gs_const, &gsc) || gsc == 0)
        return fail(ctx, MTC_ERR_BUFFER, std::string(kernel_name) + ": constexpr " + row->gs_const + " missing");
    const uint32_t group_size = std::strcmp(row->gs_const, "gs_per_row") == 0 ? k / gsc : gsc;
    if (group_size == 0 || k % group_size != 0)
        return fail(ctx, MTC_ERR_UNSUPPORTED, std::string(kernel_name) + ": group size must divide k");
    if (row->has_n) {
        if (!read_const(bufs, n_bufs, "n", &n) || n == 0)
            return fail(ctx, MTC_ERR_BUFFER, std::string(kernel_name) + ": constexpr n missing");
    } else {
        n = static_cast<uint32_t>(bo->bytes / esz);  // mt_qmv: M = 1, N = len(out)
    }
    const size_t m = bx->bytes / (static_cast<size_t>(k) * esz);
    if (m == 0) return fail(ctx, MTC_ERR_BUFFER_SIZE, std::string(kernel_name) + ": x holds less than one row of k");
    if ((static_cast<unsigned long long>(k) * row->bits) % 32 != 0)
        return fail(ctx, MTC_ERR_UNSUPPORTED, std::string(kernel_name) + ": k*bits must be a multiple of 32");
    const size_t need_w = static_cast<size_t>(n) * k * row->bits / 8;
    const size_t need_sb = static_cast<size_t>(n) * (k / group_size) * esz;
    const size_t need_x = m * k * esz, need_o = m * n * esz;
    // An undersized buffer is an error (crates/metaltile-runtime/src/dispatch/buffer_plan.rs:68-76).
    if (bw->bytes < need_w) return fail(ctx, MTC_ERR_BUFFER_SIZE, "buffer 'w' smaller than n*k*bits/8 bytes");
    if (bs->bytes < need_sb) return fail(ctx, MTC_ERR_BUFFER_SIZE, "buffer 'scales' smaller than n*(k/group) elements");
    if (bb->bytes < need_sb) return fail(ctx, MTC_ERR_BUFFER_SIZE, "buffer 'biases' smaller than n*(k/group) elements");
    if (bo->bytes < need_o) return fail(ctx, MTC_ERR_BUFFER_SIZE, "buffer 'out' smaller than m*n elements");

    MTC_CUDA(ctx, cudaSetDevice(ctx->device), MTC_ERR_NO_DEVICE);
    const size_t o_w = 0, o_s = align_up(need_w, 256), o_b = o_s + align_up(need_sb, 256),
                 o_x = o_b + align_up(need_sb, 256), o_o = o_x + align_up(need_x, 256);
    int rc = ensure_scratch(ctx, o_o + align_up(need_o, 256));
    if (rc != MTC_OK) return rc;
    char *base = static_cast<char *>(ctx->d_scratch);
    cudaStream_t st = nullptr;
    MTC_CUDA(ctx, cudaMemcpyAsync(base + o_w, bw->data, need_w, cudaMemcpyHostToDevice, st), MTC_ERR_BUFFER);
    MTC_CUDA(ctx, cudaMemcpyAsync(base + o_s, bs->data, need_sb, cudaMemcpyHostToDevice, st), MTC_ERR_BUFFER);
    MTC_CUDA(ctx, cudaMemcpyAsync(base + o_b, bb->data, need_sb, cudaMemcpyHostToDevice, st), MTC_ERR_BUFFER);
    MTC_CUDA(ctx, cudaMemcpyAsync(base + o_x, bx->data, need_x, cudaMemcpyHostToDevice, st), MTC_ERR_BUFFER);
    MTC_CUDA(ctx, cudaMemcpyAsync(base + o_o, bo->data, need_o, cudaMemcpyHostToDevice, st), MTC_ERR_BUFFER);
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    if (elapsed_us) {
        MTC_CUDA(ctx, cudaEventCreate(&e0), MTC_ERR_DISPATCH);
        MTC_CUDA(ctx, cudaEventCreate(&e1), MTC_ERR_DISPATCH);
        cudaEventRecord(e0, st);
    }
    if (row->family == DENSE_QMM)
        rc = mtc_qmm(ctx, st, base + o_w, base + o_s, base + o_b, base + o_x, base + o_o, static_cast<int>(m),
                     static_cast<int>(n), static_cast<int>(k), row->bits, static_cast<int>(group_size), dtype);
    else
        rc = mtc_qmv(ctx, st, base + o_w, base + o_s, base + o_b, base + o_x, base + o_o, static_cast<int>(m),
                     static_cast<int>(n), static_cast<int>(k), row->bits, static_cast<int>(group_size), dtype);
    if (elapsed_us) cudaEventRecord(e1, st);
    if (rc == MTC_OK) {
        for (int i = 0; i < n_bufs; ++i)
            if (bufs[i].is_output && &bufs[i] == bo)
                cudaMemcpyAsync(bo->data, base + o_o, need_o, cudaMemcpyDeviceToHost, st);
        cudaError_t e = cudaStreamSynchronize(st);
        if (e != cudaSuccess) rc = fail(ctx, MTC_ERR_DISPATCH, std::string("dispatch: ") + cudaGetErrorString(e));
    }
    if (elapsed_us) {
        float ms = 0.f;
        if (rc == MTC_OK && cudaEventElapsedTime(&ms, e0, e1) == cudaSuccess) *elapsed_us = ms * 1000.0f;
        cudaEventDestroy(e0);
        cudaEventDestroy(e1);
    }
    return rc;
}

}  // extern "C"
