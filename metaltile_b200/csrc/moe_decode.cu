// moe_decode — the M = 1 tail of a mixture-of-experts layer, expert ids read on the device:
//
//   fused     out[row] = sum_k sw[k] * sum_d w(e_k, row, d) * inner_k[d],   inner_k[d] = silu(gate_k[d]) * up_k[d]
//             (ffai_moe_down_swiglu_accum_int4_chain8, crates/metaltile-std/src/ffai/moe_down_swiglu_accum.rs:158-318:
//              mt_swiglu x n_slots, the expert-indexed down projection x n_slots and mt_scalar_fma_chain8 in one launch)
//   indexed   out[k][row] = sum_d w(e_k, row, d) * x_k[d]
//             (dequant_gemv_int4_expert_indexed, crates/metaltile-std/src/ffai/dequant_gemv_expert_indexed.rs:56-103)
//
// w(e, row, d) = q * scale + bias of the stacked 4-bit matrices [E, out_dim, in_dim / 8] (scales / biases
// [E, out_dim, in_dim / G]).  HBM-bound: n_slots x out_dim x in_dim / 2 bytes read once.  A CTA stages the inner
// activations of all slots once in shared memory, in f32 (never rounded to the activation type, as the reference keeps
// them), pre-multiplied by the slot weight and by 2^(64 - p) for the nibble position p they meet, so that a code is used
// where it sits in its word (read as an f32 subnormal: no shift, no conversion; one LOP3 and one FFMA per code).  A warp
// owns an output row: every slot's 4-bit row is in_dim / 2 contiguous bytes, read as whole lines; per word
// acc_s += scale * sum(q x), acc_b += bias * sum(x); one shuffle reduction per row.
#include "common.cuh"

namespace mtc {
namespace {

constexpr int kMdWarps = 8;
constexpr int kMdMaxSlots = 8;

struct MdArgs {
    const uint32_t *w;
    const void *scales, *biases;
    const void *gate[kMdMaxSlots], *up[kMdMaxSlots];     // fused: per-slot gate / up; indexed: gate[k] = x_k, up unused
    const uint32_t *experts;                             // [n_slots]
    const void *slot_w;                                  // fused: [n_slots] routing weights
    void *out;                                           // fused: [out_dim]; indexed: [n_slots, out_dim]
    uint32_t *status;
    int n_slots, in_dim, out_dim, gs, n_experts, dt, fused;
    const float *staged;                                  // xp then xw, written by moe_decode_prep_kernel
    int gpr, wpg_shift;                                   // groups per row; log2(group_size / 8): the group size is a power of two
};

// 8 consecutive elements of a T array as f32: one 16-byte load for 16-bit types when the pointer allows it
__device__ __forceinline__ void md_load8(const void *p, size_t i0, int dt, float (&v)[8]) {
    if (dt != MTC_F32 && (reinterpret_cast<uintptr_t>(p) & 15) == 0) {
        const uint4 t = __ldg(reinterpret_cast<const uint4 *>(static_cast<const uint16_t *>(p) + i0));
        const uint32_t u[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
        for (int h = 0; h < 4; ++h) {
            if (dt == MTC_BF16) {
                v[2 * h] = __uint_as_float(u[h] << 16);
                v[2 * h + 1] = __uint_as_float(u[h] & 0xFFFF0000u);
            } else {
                const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&u[h]));
                v[2 * h] = f.x;
                v[2 * h + 1] = f.y;
            }
        }
    } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = ld_as_f32(p, i0 + j, dt);
    }
}

// position of the lowest bit of nibble i where the kernel reads it: nibbles 6 and 7 come from the word shifted down by 16
__device__ __forceinline__ constexpr int md_pos(int i) { return i < 6 ? 4 * i : 4 * i - 16; }

// The inner activations of every slot, once per call: xp[k][d] = v * 2^(64 - p(d % 8)) and xw[k][d / 8] = sum of the word's
// eight v, with v = silu(gate_k[d]) * up_k[d] * slot_weight[k] (fused) or x_k[d] (indexed), all f32.
__global__ void __launch_bounds__(256) moe_decode_prep_kernel(const MdArgs a, float *staged) {
    const int words = a.in_dim >> 3;
    float *xp = staged, *xw = staged + static_cast<size_t>(a.n_slots) * a.in_dim;
    const int k = blockIdx.y;
    const float sw = a.fused ? ld_as_f32(a.slot_w, k, a.dt) : 1.0f;
    for (int wd = blockIdx.x * blockDim.x + threadIdx.x; wd < words; wd += gridDim.x * blockDim.x) {
        float gv[8], uv[8];
        md_load8(a.gate[k], static_cast<size_t>(wd) * 8, a.dt, gv);
        if (a.fused) md_load8(a.up[k], static_cast<size_t>(wd) * 8, a.dt, uv);
        float sum = 0.0f;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            float v = gv[j];
            if (a.fused) v = (v / (1.0f + expf(-v))) * uv[j] * sw;
            sum += v;
            xp[static_cast<size_t>(k) * a.in_dim + wd * 8 + j] = v * __uint_as_float(static_cast<uint32_t>(127 + 64 - md_pos(j)) << 23);
        }
        xw[k * words + wd] = sum;
    }
}

// WPL: packed words of a weight row per lane (in_dim <= 256 * WPL); 0 = any in_dim (a plain loop).  With WPL > 0 the
// slot and word loops are fully unrolled, so that the loads of a row - up to 8 slots x WPL words, their scales and
// biases - are all in flight before the first is used: a warp has one short row per slot and nothing else to hide
// the latency of its loads behind.
template <int WPL>
__global__ void __launch_bounds__(kMdWarps * 32) moe_decode_kernel(const MdArgs a) {
    extern __shared__ __align__(16) float md_sm[];
    const int words = a.in_dim >> 3;
    float *xp = md_sm;                                    // [n_slots][in_dim]   inner * sw * 2^(64 - p)
    float *xw = xp + static_cast<size_t>(a.n_slots) * a.in_dim;       // [n_slots][words]    sum of the word's 8 inner * sw
    __shared__ uint32_t s_exp[kMdMaxSlots];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (threadIdx.x < a.n_slots) {
        uint32_t e = a.experts[threadIdx.x];
        if (e >= static_cast<uint32_t>(a.n_experts)) {
            atomicCAS(a.status, 0u, 0x905u);              // not an expert of the stack: expert 0 is read instead
            e = 0;
        }
        s_exp[threadIdx.x] = e;
    }
    // the staged activations were prepared once by moe_decode_prep_kernel: a plain copy (xp and xw are contiguous)
    {
        const int n4 = (a.n_slots * a.in_dim + a.n_slots * words) >> 2;       // in_dim % 8 == 0: both parts are whole float4s
        const float4 *src = reinterpret_cast<const float4 *>(a.staged);
        float4 *dst = reinterpret_cast<float4 *>(md_sm);
        for (int i = threadIdx.x; i < n4; i += blockDim.x) dst[i] = __ldg(src + i);
    }
    __syncthreads();
    const int gpr = a.gpr, wsh = a.wpg_shift;             // groups per row, log2(words per group)
    for (int row = blockIdx.x * kMdWarps + warp; row < a.out_dim; row += gridDim.x * kMdWarps) {
        float acc_s = 0.0f, acc_b = 0.0f;
        float per_slot = 0.0f;
        if (WPL > 0) {
            uint32_t wreg[kMdMaxSlots][WPL > 0 ? WPL : 1];
            float sreg[kMdMaxSlots][WPL > 0 ? WPL : 1], breg[kMdMaxSlots][WPL > 0 ? WPL : 1];
#pragma unroll
            for (int k = 0; k < kMdMaxSlots; ++k) {
                const size_t r = static_cast<size_t>(s_exp[k < a.n_slots ? k : 0]) * a.out_dim + row;
#pragma unroll
                for (int i = 0; i < WPL; ++i) {
                    const int wd = lane + 32 * i;
                    const bool in = k < a.n_slots && wd < words;
                    wreg[k][i] = in ? __ldg(a.w + r * words + wd) : 0u;
                    sreg[k][i] = in ? ld_as_f32(a.scales, r * gpr + (wd >> wsh), a.dt) : 0.0f;
                    breg[k][i] = in ? ld_as_f32(a.biases, r * gpr + (wd >> wsh), a.dt) : 0.0f;
                }
            }
#pragma unroll
            for (int k = 0; k < kMdMaxSlots; ++k) {
                if (k < a.n_slots) {
                    const float *xk = xp + static_cast<size_t>(k) * a.in_dim, *xwk = xw + static_cast<size_t>(k) * words;
#pragma unroll
                    for (int i = 0; i < WPL; ++i) {
                        const int wd = lane + 32 * i;
                        if (wd < words) {
                            const uint32_t word = wreg[k][i], hi = word >> 16;
                            const float4 x0 = *reinterpret_cast<const float4 *>(xk + wd * 8), x1 = *reinterpret_cast<const float4 *>(xk + wd * 8 + 4);
                            float raw = x0.x * __uint_as_float(word & 0x0000000Fu);
                            raw = fmaf(x0.y, __uint_as_float(word & 0x000000F0u), raw);
                            raw = fmaf(x0.z, __uint_as_float(word & 0x00000F00u), raw);
                            raw = fmaf(x0.w, __uint_as_float(word & 0x0000F000u), raw);
                            raw = fmaf(x1.x, __uint_as_float(word & 0x000F0000u), raw);
                            raw = fmaf(x1.y, __uint_as_float(word & 0x00F00000u), raw);
                            raw = fmaf(x1.z, __uint_as_float(hi & 0x00000F00u), raw);
                            raw = fmaf(x1.w, __uint_as_float(hi & 0x0000F000u), raw);
                            acc_s = fmaf(sreg[k][i], raw, acc_s);
                            acc_b = fmaf(breg[k][i], xwk[wd], acc_b);
                        }
                    }
                    if (!a.fused) {                        // one output per slot
                        float v = fmaf(acc_s, 3.8685626227668134e25f /* 2^85 */, acc_b);
#pragma unroll
                        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
                        if (lane == 0) st_from_f32(a.out, static_cast<size_t>(k) * a.out_dim + row, v, a.dt);
                        acc_s = acc_b = 0.0f;
                    }
                }
            }
        } else
        for (int k = 0; k < a.n_slots; ++k) {
            const size_t r = static_cast<size_t>(s_exp[k]) * a.out_dim + row;
            const uint32_t *rw = a.w + r * words;
            const float *xk = xp + static_cast<size_t>(k) * a.in_dim, *xwk = xw + static_cast<size_t>(k) * words;
            for (int wd = lane; wd < words; wd += 32) {
                const uint32_t word = __ldg(rw + wd), hi = word >> 16;
                const float4 x0 = *reinterpret_cast<const float4 *>(xk + wd * 8), x1 = *reinterpret_cast<const float4 *>(xk + wd * 8 + 4);
                float raw = x0.x * __uint_as_float(word & 0x0000000Fu);
                raw = fmaf(x0.y, __uint_as_float(word & 0x000000F0u), raw);
                raw = fmaf(x0.z, __uint_as_float(word & 0x00000F00u), raw);
                raw = fmaf(x0.w, __uint_as_float(word & 0x0000F000u), raw);
                raw = fmaf(x1.x, __uint_as_float(word & 0x000F0000u), raw);
                raw = fmaf(x1.y, __uint_as_float(word & 0x00F00000u), raw);
                raw = fmaf(x1.z, __uint_as_float(hi & 0x00000F00u), raw);
                raw = fmaf(x1.w, __uint_as_float(hi & 0x0000F000u), raw);
                const size_t g = r * gpr + (wd >> wsh);
                acc_s = fmaf(ld_as_f32(a.scales, g, a.dt), raw, acc_s);
                acc_b = fmaf(ld_as_f32(a.biases, g, a.dt), xwk[wd], acc_b);
            }
            if (!a.fused) {                                // one output per slot
                float v = fmaf(acc_s, 3.8685626227668134e25f /* 2^85 */, acc_b);
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
                if (lane == 0) st_from_f32(a.out, static_cast<size_t>(k) * a.out_dim + row, v, a.dt);
                acc_s = acc_b = 0.0f;
            }
        }
        if (a.fused) {
            per_slot = fmaf(acc_s, 3.8685626227668134e25f /* 2^85 */, acc_b);
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) per_slot += __shfl_xor_sync(0xffffffffu, per_slot, o);
            if (lane == 0) st_from_f32(a.out, static_cast<size_t>(row), per_slot, a.dt);
        }
    }
}

}  // namespace

size_t moe_decode_smem_bytes(int n_slots, int in_dim) {
    return static_cast<size_t>(n_slots) * in_dim * 4 + static_cast<size_t>(n_slots) * (in_dim / 8) * 4;
}

// fused = 1: gate / up per slot, slot weights, out [out_dim];  fused = 0: xs[k] per slot, out [n_slots, out_dim]
cudaError_t launch_moe_decode(Ctx *ctx, cudaStream_t st, const void *const *gate, const void *const *up, const void *experts,
                              const void *slot_w, const void *w, const void *scales, const void *biases, void *out, int n_slots, int in_dim,
                              int out_dim, int n_experts, int group_size, int dt, int fused, float *staged) {
    MdArgs a{};
    a.w = static_cast<const uint32_t *>(w);
    a.scales = scales;
    a.biases = biases;
    for (int k = 0; k < n_slots; ++k) {
        a.gate[k] = gate[k];
        a.up[k] = up ? up[k] : nullptr;
    }
    a.experts = static_cast<const uint32_t *>(experts);
    a.slot_w = slot_w;
    a.out = out;
    a.status = ctx->d_status;
    a.n_slots = n_slots;
    a.in_dim = in_dim;
    a.out_dim = out_dim;
    a.gs = group_size;
    a.n_experts = n_experts;
    a.dt = dt;
    a.fused = fused;
    a.gpr = in_dim / group_size;
    a.wpg_shift = 0;
    while ((8 << a.wpg_shift) < group_size) ++a.wpg_shift;
    const size_t smem = moe_decode_smem_bytes(n_slots, in_dim);
    a.staged = staged;
    moe_decode_prep_kernel<<<dim3((in_dim / 8 + 255) / 256, n_slots), 256, 0, st>>>(a, staged);
    cudaError_t pe = cudaGetLastError();
    if (pe != cudaSuccess) return pe;
    int grid = (out_dim + kMdWarps - 1) / kMdWarps;
    if (grid > ctx->sm_count * 4) grid = ctx->sm_count * 4;
    const int wpl = (in_dim / 8 + 31) / 32;
    static PerDeviceAttr attr[5];
    cudaError_t e;
#define MTC_MD(W)                                                                   \
    e = attr[W].set(moe_decode_kernel<W>, 200 * 1024);                               \
    if (e != cudaSuccess) return e;                                                  \
    moe_decode_kernel<W><<<grid, kMdWarps * 32, smem, st>>>(a)
    if (wpl == 1) { MTC_MD(1); }
    else if (wpl == 2) { MTC_MD(2); }
    else if (wpl == 3) { MTC_MD(3); }
    else if (wpl == 4) { MTC_MD(4); }
    else { MTC_MD(0); }
#undef MTC_MD
    return cudaGetLastError();
}

}  // namespace mtc
