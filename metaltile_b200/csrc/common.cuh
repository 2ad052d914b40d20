// Shared device/host helpers for the sm_100a kernels behind include/mtcuda.h.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>

#include "../../include/mtcuda.h"

namespace mtc {

constexpr int kNumSMsB200 = 148;

struct Ctx {
    int device = 0;
    int sm_count = kNumSMsB200;
    size_t l2_bytes = 0;
    std::string last_error;
    uint32_t *d_status = nullptr;  // device status word (bounded waits / rejected indices)
    void *d_scratch = nullptr;     // grow-only scratch owned by the context
    size_t scratch_bytes = 0;
};

inline int fail(Ctx *ctx, int code, const std::string &msg) {
    if (ctx) ctx->last_error = msg;
    return code;
}

inline size_t dtype_size(int dt) { return dt == MTC_F32 ? 4 : 2; }

// ---- dtype-generic element access (dtype is a launch-time constant) ----------
__device__ __forceinline__ float ld_as_f32(const void *p, size_t i, int dt) {
    if (dt == MTC_F32) return __ldg(reinterpret_cast<const float *>(p) + i);
    unsigned short h = __ldg(reinterpret_cast<const unsigned short *>(p) + i);
    if (dt == MTC_BF16) return __uint_as_float(static_cast<uint32_t>(h) << 16);
    return __half2float(__ushort_as_half(h));
}

__device__ __forceinline__ void st_from_f32(void *p, size_t i, float v, int dt) {
    if (dt == MTC_F32) {
        reinterpret_cast<float *>(p)[i] = v;
    } else if (dt == MTC_BF16) {
        reinterpret_cast<__nv_bfloat16 *>(p)[i] = __float2bfloat16_rn(v);
    } else {
        reinterpret_cast<__half *>(p)[i] = __float2half_rn(v);
    }
}

__device__ __forceinline__ float bf16_bits_to_f32(uint32_t h) { return __uint_as_float(h << 16); }

// Code k of a row stored as an LSB-first bit-stream of u32 words; a code may
// straddle two words (odd widths).  Same extraction as the reference's generic
// kernels (crates/metaltile-std/src/mlx/quantized.rs:4366-4379).
__device__ __forceinline__ uint32_t code_at(const uint32_t *row, uint32_t k, int bits) {
    uint32_t bit_off = k * static_cast<uint32_t>(bits);
    uint32_t word = bit_off >> 5, sh = bit_off & 31u;
    uint32_t lo = __ldg(row + word) >> sh;
    if (32u - sh < static_cast<uint32_t>(bits)) lo |= __ldg(row + word + 1) << (32u - sh);
    return lo & ((1u << bits) - 1u);
}

// Launchers implemented per .cu file; all return cudaError_t from the launch.
cudaError_t launch_qmv(Ctx *ctx, cudaStream_t st, const void *w, const void *scales, const void *biases,
                       const void *x, void *out, int M, int N, int K, int bits, int group_size, int dt,
                       std::string *why);
cudaError_t qmv_init_device();
cudaError_t launch_unpack_codes(cudaStream_t st, const void *w, void *codes, int N, int K, int bits);

}  // namespace mtc
