// affine — the codec either side of the quantized matmuls: float tensor -> packed codes + per-group scale / bias, and back.
//
//   quantize   per group of G values:  scale = (max - min) / (2^b - 1)  (1 when below 1e-7),  bias = min,
//              q = trunc(clamp((v - bias) * (1 / scale) + 0.5, 0, 2^b - 1));  codes packed LSB-first, one bit-stream per
//              group; scale and bias stored in the activation type
//   dequantize out[i] = scale[i / G] * q_i + bias[i / G], rounded to the activation type
//
// Stands in for mt_affine_quantize_int{2,3,4,5,6,8} and mt_affine_dequantize_int{2,3,4,5,6,8}
// (crates/metaltile-std/src/mlx/quantized.rs:3575-4214; one template there too).  Every float operation is a separately
// rounded f32 operation (no fused multiply-add), so codes and values are those of the scalar CPU formula bit for bit.
// Both kernels are HBM-bound element-wise passes over data that is touched once (weights are quantized at load time):
// a thread owns 32 codes = b whole words, so packed words are read and written as whole words and 16-bit values as
// 16-byte vectors.
#include "common.cuh"

namespace mtc {
namespace {

template <int BITS>
__device__ __forceinline__ uint32_t code_of(const uint32_t (&w)[BITS], int k) {      // k: compile-time after unrolling
    const int bit = k * BITS, word = bit >> 5, sh = bit & 31;
    uint32_t q = w[word] >> sh;
    if (sh + BITS > 32) q |= w[word + 1] << (32 - sh);
    return q & ((1u << BITS) - 1u);
}

// One thread per 32 consecutive codes (BITS words); group_size % 32 == 0 so that the 32 values share one scale / bias.
template <int BITS>
__global__ void __launch_bounds__(256) affine_dequantize_kernel(const uint32_t *w, const void *scales, const void *biases, void *out,
                                                                size_t n_chunks, int group_size, int dt, int vec_ok) {
    for (size_t c = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; c < n_chunks;
         c += static_cast<size_t>(gridDim.x) * blockDim.x) {
        uint32_t words[BITS];
#pragma unroll
        for (int i = 0; i < BITS; ++i) words[i] = __ldg(w + c * BITS + i);
        const size_t g = (c * 32) / group_size;
        const float s = ld_as_f32(scales, g, dt), b = ld_as_f32(biases, g, dt);
        float v[32];
#pragma unroll
        for (int k = 0; k < 32; ++k) v[k] = __fadd_rn(__fmul_rn(s, static_cast<float>(code_of<BITS>(words, k))), b);
        const size_t o = c * 32;
        if (dt == MTC_F32) {
            if (vec_ok) {
                float4 *p = reinterpret_cast<float4 *>(static_cast<float *>(out) + o);
#pragma unroll
                for (int q = 0; q < 8; ++q) p[q] = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
            } else {
#pragma unroll
                for (int k = 0; k < 32; ++k) static_cast<float *>(out)[o + k] = v[k];
            }
        } else {
            uint32_t h[16];
#pragma unroll
            for (int q = 0; q < 16; ++q) {
                if (dt == MTC_BF16) {
                    const __nv_bfloat162 p2 = __floats2bfloat162_rn(v[2 * q], v[2 * q + 1]);
                    h[q] = *reinterpret_cast<const uint32_t *>(&p2);
                } else {
                    const __half2 p2 = __floats2half2_rn(v[2 * q], v[2 * q + 1]);
                    h[q] = *reinterpret_cast<const uint32_t *>(&p2);
                }
            }
            if (vec_ok) {
                uint4 *p = reinterpret_cast<uint4 *>(static_cast<uint16_t *>(out) + o);
#pragma unroll
                for (int q = 0; q < 4; ++q) p[q] = make_uint4(h[4 * q], h[4 * q + 1], h[4 * q + 2], h[4 * q + 3]);
            } else {
                uint16_t *p = static_cast<uint16_t *>(out) + o;
#pragma unroll
                for (int q = 0; q < 16; ++q) {
                    p[2 * q] = static_cast<uint16_t>(h[q] & 0xFFFFu);
                    p[2 * q + 1] = static_cast<uint16_t>(h[q] >> 16);
                }
            }
        }
    }
}

// One warp per group (group_size % 32 == 0): min / max by shuffles, then 32 codes at a time - lane L owns code L of the
// chunk, the chunk's BITS words are OR-reduced over the warp and written by lanes 0 .. BITS-1.
template <int BITS>
__global__ void __launch_bounds__(256) affine_quantize_kernel(const void *w, uint32_t *out, void *scales, void *biases, size_t n_groups,
                                                              int group_size, int dt) {
    const int lane = threadIdx.x & 31;
    const size_t warp0 = (blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x) >> 5;
    const size_t nwarps = (static_cast<size_t>(gridDim.x) * blockDim.x) >> 5;
    const float n_bins = static_cast<float>((1u << BITS) - 1u);
    const int chunks = group_size >> 5;
    for (size_t g = warp0; g < n_groups; g += nwarps) {
        const size_t base = g * group_size;
        float mn = INFINITY, mx = -INFINITY;
        for (int c = 0; c < chunks; ++c) {
            const float v = ld_as_f32(w, base + c * 32 + lane, dt);
            mn = fminf(mn, v);
            mx = fmaxf(mx, v);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        }
        const float raw = __fdiv_rn(__fsub_rn(mx, mn), n_bins);
        const float scale = raw < 1.0e-7f ? 1.0f : raw;
        const float inv = __fdiv_rn(1.0f, scale);
        if (lane == 0) {
            st_from_f32(scales, g, scale, dt);
            st_from_f32(biases, g, mn, dt);
        }
        uint32_t *og = out + g * (static_cast<size_t>(group_size) * BITS / 32);
        const int bit = lane * BITS, word = bit >> 5, sh = bit & 31;
        for (int c = 0; c < chunks; ++c) {
            const float v = ld_as_f32(w, base + c * 32 + lane, dt);
            float qf = __fadd_rn(__fmul_rn(__fsub_rn(v, mn), inv), 0.5f);
            qf = qf > n_bins ? n_bins : (qf < 0.0f ? 0.0f : qf);
            const uint32_t q = static_cast<uint32_t>(qf);
            uint32_t mine = 0u;
#pragma unroll
            for (int j = 0; j < BITS; ++j) {
                uint32_t part = 0u;
                if (word == j) part = q << sh;
                if (word + 1 == j && sh + BITS > 32) part = q >> (32 - sh);
                const uint32_t all = __reduce_or_sync(0xffffffffu, part);
                if (lane == j) mine = all;
            }
            if (lane < BITS) og[c * BITS + lane] = mine;
        }
    }
}

// One thread per 32 consecutive values = BITS whole output words; the group_size / 32 threads of a group (a power of two,
// adjacent lanes) share min and max through xor-shuffles.  One pass: the values stay in registers between the reduction
// and the packing.  `w` 16-byte aligned.
template <int BITS>
__global__ void __launch_bounds__(256) affine_quantize32_kernel(const void *w, uint32_t *out, void *scales, void *biases, size_t n_chunks,
                                                                int tpg /* threads per group */, int dt) {
    const float n_bins = static_cast<float>((1u << BITS) - 1u);
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    // whole warps stay in the loop (the shuffles need every lane); lanes past the end work on chunk 0 and store nothing
    for (size_t c0 = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x - (threadIdx.x & 31); c0 < n_chunks; c0 += stride) {
        const size_t c = c0 + (threadIdx.x & 31);
        const bool on = c < n_chunks;
        const size_t cc = on ? c : 0;
        float v[32];
        if (dt == MTC_F32) {
            const float4 *p = reinterpret_cast<const float4 *>(static_cast<const float *>(w) + cc * 32);
#pragma unroll
            for (int q = 0; q < 8; ++q) {
                const float4 t = __ldg(p + q);
                v[4 * q] = t.x; v[4 * q + 1] = t.y; v[4 * q + 2] = t.z; v[4 * q + 3] = t.w;
            }
        } else {
            const uint4 *p = reinterpret_cast<const uint4 *>(static_cast<const uint16_t *>(w) + cc * 32);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const uint4 t = __ldg(p + q);
                const uint32_t u[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
                for (int h = 0; h < 4; ++h) {
                    if (dt == MTC_BF16) {
                        v[8 * q + 2 * h] = __uint_as_float(u[h] << 16);
                        v[8 * q + 2 * h + 1] = __uint_as_float(u[h] & 0xFFFF0000u);
                    } else {
                        const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&u[h]));
                        v[8 * q + 2 * h] = f.x;
                        v[8 * q + 2 * h + 1] = f.y;
                    }
                }
            }
        }
        float mn = v[0], mx = v[0];
#pragma unroll
        for (int k = 1; k < 32; ++k) {
            mn = fminf(mn, v[k]);
            mx = fmaxf(mx, v[k]);
        }
        for (int o = 1; o < tpg; o <<= 1) {
            mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        }
        const float raw = __fdiv_rn(__fsub_rn(mx, mn), n_bins);
        const float scale = raw < 1.0e-7f ? 1.0f : raw;
        const float inv = __fdiv_rn(1.0f, scale);
        uint32_t words[BITS];
#pragma unroll
        for (int j = 0; j < BITS; ++j) words[j] = 0u;
#pragma unroll
        for (int k = 0; k < 32; ++k) {
            float qf = __fadd_rn(__fmul_rn(__fsub_rn(v[k], mn), inv), 0.5f);
            qf = qf > n_bins ? n_bins : (qf < 0.0f ? 0.0f : qf);
            const uint32_t q = static_cast<uint32_t>(qf);
            const int bit = k * BITS, word = bit >> 5, sh = bit & 31;       // compile-time after unrolling
            words[word] |= q << sh;
            if (sh + BITS > 32) words[word + 1] |= q >> (32 - sh);
        }
        if (on) {
#pragma unroll
            for (int j = 0; j < BITS; ++j) out[c * BITS + j] = words[j];
            if ((c & (tpg - 1)) == 0) {
                st_from_f32(scales, c / tpg, scale, dt);
                st_from_f32(biases, c / tpg, mn, dt);
            }
        }
    }
}

// dequant_gather_int* (crates/metaltile-std/src/ffai/dequant_gather.rs:44-94): rows indices[t] of a quantized table
// [vocab, hidden], dequantized into out [n_tokens, hidden].  One thread per 32 values of an output row (hidden and the
// group size are multiples of 32); an index outside the table reads row 0 and is reported (status 0x904).
template <int BITS>
__global__ void __launch_bounds__(256) dequant_gather_kernel(const uint32_t *w, const void *scales, const void *biases,
                                                             const uint32_t *indices, void *out, size_t n_tokens, int hidden,
                                                             int group_size, int vocab, int dt, int vec_ok, uint32_t *status) {
    const int cpr = hidden >> 5;                                   // chunks per row
    const size_t n_chunks = n_tokens * cpr;
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n_chunks;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const size_t tok = i / cpr;
        const int c = static_cast<int>(i - tok * cpr);
        uint32_t row = __ldg(indices + tok);
        if (row >= static_cast<uint32_t>(vocab)) {
            atomicCAS(status, 0u, 0x904u);
            row = 0;
        }
        const uint32_t *rw = w + (static_cast<size_t>(row) * cpr + c) * BITS;
        uint32_t words[BITS];
#pragma unroll
        for (int j = 0; j < BITS; ++j) words[j] = __ldg(rw + j);
        const size_t g = static_cast<size_t>(row) * (hidden / group_size) + (c * 32) / group_size;
        const float s = ld_as_f32(scales, g, dt), b = ld_as_f32(biases, g, dt);
        float v[32];
#pragma unroll
        for (int k = 0; k < 32; ++k) v[k] = __fadd_rn(__fmul_rn(static_cast<float>(code_of<BITS>(words, k)), s), b);
        const size_t o = tok * hidden + c * 32;
        if (dt == MTC_F32) {
#pragma unroll
            for (int k = 0; k < 32; ++k) static_cast<float *>(out)[o + k] = v[k];
        } else {
            uint32_t h[16];
#pragma unroll
            for (int q = 0; q < 16; ++q) {
                if (dt == MTC_BF16) {
                    const __nv_bfloat162 p2 = __floats2bfloat162_rn(v[2 * q], v[2 * q + 1]);
                    h[q] = *reinterpret_cast<const uint32_t *>(&p2);
                } else {
                    const __half2 p2 = __floats2half2_rn(v[2 * q], v[2 * q + 1]);
                    h[q] = *reinterpret_cast<const uint32_t *>(&p2);
                }
            }
            if (vec_ok) {
                uint4 *p = reinterpret_cast<uint4 *>(static_cast<uint16_t *>(out) + o);
#pragma unroll
                for (int q = 0; q < 4; ++q) p[q] = make_uint4(h[4 * q], h[4 * q + 1], h[4 * q + 2], h[4 * q + 3]);
            } else {
                uint16_t *p = static_cast<uint16_t *>(out) + o;
#pragma unroll
                for (int q = 0; q < 16; ++q) {
                    p[2 * q] = static_cast<uint16_t>(h[q] & 0xFFFFu);
                    p[2 * q + 1] = static_cast<uint16_t>(h[q] >> 16);
                }
            }
        }
    }
}

// any hidden / group size: one thread per output element
__global__ void __launch_bounds__(256) dequant_gather_generic(const uint32_t *w, const void *scales, const void *biases,
                                                              const uint32_t *indices, void *out, size_t n_tokens, int hidden,
                                                              int group_size, int vocab, int bits, int dt, uint32_t *status) {
    const size_t n = n_tokens * hidden;
    const size_t wpr = static_cast<size_t>(hidden) * bits / 32;
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n; i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const size_t tok = i / hidden;
        const uint32_t d = static_cast<uint32_t>(i - tok * hidden);
        uint32_t row = __ldg(indices + tok);
        if (row >= static_cast<uint32_t>(vocab)) {
            atomicCAS(status, 0u, 0x904u);
            row = 0;
        }
        const float q = static_cast<float>(code_at(w + row * wpr, d, bits));
        const size_t g = static_cast<size_t>(row) * (hidden / group_size) + d / group_size;
        st_from_f32(out, i, __fadd_rn(__fmul_rn(q, ld_as_f32(scales, g, dt)), ld_as_f32(biases, g, dt)), dt);
    }
}

// any group size, any alignment: one thread per element (dequantize) / one thread per group (quantize)
__global__ void __launch_bounds__(256) affine_dequantize_generic(const uint32_t *w, const void *scales, const void *biases, void *out,
                                                                 size_t n_elem, int group_size, int bits, int dt) {
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n_elem;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const size_t g = i / group_size;
        // the stream restarts at every group: group_size * bits is a multiple of 32
        const uint32_t *gw = w + g * (static_cast<size_t>(group_size) * bits / 32);
        const float q = static_cast<float>(code_at(gw, static_cast<uint32_t>(i - g * group_size), bits));
        st_from_f32(out, i, __fadd_rn(__fmul_rn(ld_as_f32(scales, g, dt), q), ld_as_f32(biases, g, dt)), dt);
    }
}

__global__ void __launch_bounds__(128) affine_quantize_generic(const void *w, uint32_t *out, void *scales, void *biases, size_t n_groups,
                                                               int group_size, int bits, int dt) {
    const float n_bins = static_cast<float>((1u << bits) - 1u);
    for (size_t g = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; g < n_groups;
         g += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const size_t base = g * group_size;
        float mn = INFINITY, mx = -INFINITY;
        for (int i = 0; i < group_size; ++i) {
            const float v = ld_as_f32(w, base + i, dt);
            mn = fminf(mn, v);
            mx = fmaxf(mx, v);
        }
        const float raw = __fdiv_rn(__fsub_rn(mx, mn), n_bins);
        const float scale = raw < 1.0e-7f ? 1.0f : raw;
        const float inv = __fdiv_rn(1.0f, scale);
        st_from_f32(scales, g, scale, dt);
        st_from_f32(biases, g, mn, dt);
        const size_t wpg = static_cast<size_t>(group_size) * bits / 32;
        uint32_t *og = out + g * wpg;
        uint32_t cur = 0u;
        for (int i = 0; i < group_size; ++i) {
            float qf = __fadd_rn(__fmul_rn(__fsub_rn(ld_as_f32(w, base + i, dt), mn), inv), 0.5f);
            qf = qf > n_bins ? n_bins : (qf < 0.0f ? 0.0f : qf);
            const uint32_t q = static_cast<uint32_t>(qf);
            const int bit = i * bits, sh = bit & 31;
            cur |= q << sh;
            if (sh + bits >= 32) {
                og[bit >> 5] = cur;
                cur = sh + bits > 32 ? q >> (32 - sh) : 0u;
            }
        }
    }
}

int grid_for(size_t work, int per_block, int sms) {
    size_t g = (work + per_block - 1) / per_block;
    const size_t cap = static_cast<size_t>(sms) * 16;
    if (g > cap) g = cap;
    return g < 1 ? 1 : static_cast<int>(g);
}

}  // namespace

cudaError_t launch_affine_dequantize(Ctx *ctx, cudaStream_t st, const void *w, const void *scales, const void *biases, void *out,
                                     size_t n_elem, int bits, int group_size, int dt) {
    if (n_elem == 0) return cudaSuccess;
    const uint32_t *ww = static_cast<const uint32_t *>(w);
    if (group_size % 32 != 0 || n_elem % 32 != 0) {
        affine_dequantize_generic<<<grid_for(n_elem, 256, ctx->sm_count), 256, 0, st>>>(ww, scales, biases, out, n_elem, group_size, bits, dt);
        return cudaGetLastError();
    }
    const size_t chunks = n_elem / 32;
    const int vec_ok = reinterpret_cast<uintptr_t>(out) % 16 == 0 ? 1 : 0;
    const int grid = grid_for(chunks, 256, ctx->sm_count);
    switch (bits) {
        case 2: affine_dequantize_kernel<2><<<grid, 256, 0, st>>>(ww, scales, biases, out, chunks, group_size, dt, vec_ok); break;
        case 3: affine_dequantize_kernel<3><<<grid, 256, 0, st>>>(ww, scales, biases, out, chunks, group_size, dt, vec_ok); break;
        case 4: affine_dequantize_kernel<4><<<grid, 256, 0, st>>>(ww, scales, biases, out, chunks, group_size, dt, vec_ok); break;
        case 5: affine_dequantize_kernel<5><<<grid, 256, 0, st>>>(ww, scales, biases, out, chunks, group_size, dt, vec_ok); break;
        case 6: affine_dequantize_kernel<6><<<grid, 256, 0, st>>>(ww, scales, biases, out, chunks, group_size, dt, vec_ok); break;
        default: affine_dequantize_kernel<8><<<grid, 256, 0, st>>>(ww, scales, biases, out, chunks, group_size, dt, vec_ok); break;
    }
    return cudaGetLastError();
}

cudaError_t launch_dequant_gather(Ctx *ctx, cudaStream_t st, const void *w, const void *scales, const void *biases, const void *indices,
                                  void *out, size_t n_tokens, int hidden, int vocab, int bits, int group_size, int dt) {
    if (n_tokens == 0 || hidden == 0) return cudaSuccess;
    const uint32_t *ww = static_cast<const uint32_t *>(w), *ix = static_cast<const uint32_t *>(indices);
    if (hidden % 32 != 0 || group_size % 32 != 0) {
        dequant_gather_generic<<<grid_for(n_tokens * hidden, 256, ctx->sm_count), 256, 0, st>>>(ww, scales, biases, ix, out, n_tokens, hidden,
                                                                                              group_size, vocab, bits, dt, ctx->d_status);
        return cudaGetLastError();
    }
    const int vec_ok = reinterpret_cast<uintptr_t>(out) % 16 == 0 ? 1 : 0;
    const int grid = grid_for(n_tokens * (hidden / 32), 256, ctx->sm_count);
#define MTC_DG(B) dequant_gather_kernel<B><<<grid, 256, 0, st>>>(ww, scales, biases, ix, out, n_tokens, hidden, group_size, vocab, dt, vec_ok, ctx->d_status)
    switch (bits) {
        case 2: MTC_DG(2); break;
        case 3: MTC_DG(3); break;
        case 4: MTC_DG(4); break;
        case 5: MTC_DG(5); break;
        case 6: MTC_DG(6); break;
        default: MTC_DG(8); break;
    }
#undef MTC_DG
    return cudaGetLastError();
}

cudaError_t launch_affine_quantize(Ctx *ctx, cudaStream_t st, const void *w, void *out, void *scales, void *biases, size_t n_groups,
                                   int bits, int group_size, int dt) {
    if (n_groups == 0) return cudaSuccess;
    uint32_t *oo = static_cast<uint32_t *>(out);
    if (group_size % 32 != 0) {
        affine_quantize_generic<<<grid_for(n_groups, 128, ctx->sm_count), 128, 0, st>>>(w, oo, scales, biases, n_groups, group_size, bits, dt);
        return cudaGetLastError();
    }
    const int tpg = group_size / 32;
    if ((tpg & (tpg - 1)) == 0 && tpg <= 32 && reinterpret_cast<uintptr_t>(w) % 16 == 0) {
        const size_t chunks = n_groups * tpg;
        const int g32 = grid_for(chunks, 256, ctx->sm_count);
        switch (bits) {
            case 2: affine_quantize32_kernel<2><<<g32, 256, 0, st>>>(w, oo, scales, biases, chunks, tpg, dt); break;
            case 3: affine_quantize32_kernel<3><<<g32, 256, 0, st>>>(w, oo, scales, biases, chunks, tpg, dt); break;
            case 4: affine_quantize32_kernel<4><<<g32, 256, 0, st>>>(w, oo, scales, biases, chunks, tpg, dt); break;
            case 5: affine_quantize32_kernel<5><<<g32, 256, 0, st>>>(w, oo, scales, biases, chunks, tpg, dt); break;
            case 6: affine_quantize32_kernel<6><<<g32, 256, 0, st>>>(w, oo, scales, biases, chunks, tpg, dt); break;
            default: affine_quantize32_kernel<8><<<g32, 256, 0, st>>>(w, oo, scales, biases, chunks, tpg, dt); break;
        }
        return cudaGetLastError();
    }
    const int grid = grid_for(n_groups, 8, ctx->sm_count);
    switch (bits) {
        case 2: affine_quantize_kernel<2><<<grid, 256, 0, st>>>(w, oo, scales, biases, n_groups, group_size, dt); break;
        case 3: affine_quantize_kernel<3><<<grid, 256, 0, st>>>(w, oo, scales, biases, n_groups, group_size, dt); break;
        case 4: affine_quantize_kernel<4><<<grid, 256, 0, st>>>(w, oo, scales, biases, n_groups, group_size, dt); break;
        case 5: affine_quantize_kernel<5><<<grid, 256, 0, st>>>(w, oo, scales, biases, n_groups, group_size, dt); break;
        case 6: affine_quantize_kernel<6><<<grid, 256, 0, st>>>(w, oo, scales, biases, n_groups, group_size, dt); break;
        default: affine_quantize_kernel<8><<<grid, 256, 0, st>>>(w, oo, scales, biases, n_groups, group_size, dt); break;
    }
    return cudaGetLastError();
}

}  // namespace mtc
