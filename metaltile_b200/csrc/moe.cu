// MoE routing kernels around gather_qmm: router top-k, the expert sort, permute, unpermute, SwiGLU,
// and the any-shape CUDA-core gather_qmm used when the tensor-core kernel's contract is not met.
// Reference: crates/metaltile-std/src/ffai/moe.rs:65-302,358-433 and crates/metaltile-std/src/mlx/swiglu.rs:45-57.
#include "common.cuh"

namespace mtc {
namespace {

// ---- mt_moe_router_topk (moe.rs:65-192) -----------------------------------------------------------
// One warp per token row.  k passes of arg-max over the experts not chosen yet: each lane scans its
// experts j = lane, lane+32, ... in ascending order with a strict '>' (so NaN never wins and a lane keeps
// its lowest index among equals), then the warp takes the maximum value and, among the lanes holding
// it, the minimum index: ties go to the lower expert index.  Weights: exp(z - max_all) divided by the
// sum over the chosen k (norm_topk_prob = 1) or over all experts (= 0).
constexpr int kMaxPerLane = 32;   // n_experts <= 1024

__global__ void __launch_bounds__(128) router_topk_kernel(const void *logits, uint32_t *indices_out, void *weights_out,
                                                          int n_rows, int n_experts, int k, int norm_topk_prob, int dt) {
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= n_rows) return;
    const size_t base = static_cast<size_t>(row) * n_experts;
    const int per_lane = (n_experts + 31) / 32;
    float z[kMaxPerLane];
    float row_max = -INFINITY;
#pragma unroll
    for (int r = 0; r < kMaxPerLane; ++r) {
        z[r] = -INFINITY;
        if (r < per_lane) {
            const int j = r * 32 + lane;
            if (j < n_experts) {
                z[r] = ld_as_f32(logits, base + j, dt);
                if (z[r] > row_max) row_max = z[r];
            }
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) row_max = fmaxf(row_max, __shfl_xor_sync(0xffffffffu, row_max, o));
    float row_sum = 0.0f;
#pragma unroll
    for (int r = 0; r < kMaxPerLane; ++r)
        if (r < per_lane && r * 32 + lane < n_experts) row_sum += expf(z[r] - row_max);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) row_sum += __shfl_xor_sync(0xffffffffu, row_sum, o);

    uint32_t taken = 0;            // bit r: this lane's expert r*32+lane was chosen in an earlier pass
    float my_val = -INFINITY;      // lane i < k keeps the value of pass i
    uint32_t my_idx = 0;
    for (int it = 0; it < k; ++it) {
        float best = -INFINITY;
        uint32_t best_idx = 0;
#pragma unroll
        for (int r = 0; r < kMaxPerLane; ++r) {
            if (r < per_lane) {
                const int j = r * 32 + lane;
                if (j < n_experts) {
                    const float cand = ((taken >> r) & 1u) ? -INFINITY : z[r];
                    if (cand > best) { best = cand; best_idx = static_cast<uint32_t>(j); }
                }
            }
        }
        float gbest = best;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) gbest = fmaxf(gbest, __shfl_xor_sync(0xffffffffu, gbest, o));
        uint32_t cand_idx = (best == gbest) ? best_idx : 0xFFFFFFFFu;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) cand_idx = min(cand_idx, __shfl_xor_sync(0xffffffffu, cand_idx, o));
        if ((cand_idx & 31u) == static_cast<uint32_t>(lane) && cand_idx != 0xFFFFFFFFu) taken |= 1u << (cand_idx >> 5);
        if (lane == it) { my_val = gbest; my_idx = cand_idx; }
    }
    const float e = lane < k ? expf(my_val - row_max) : 0.0f;
    float sum_chosen = e;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum_chosen += __shfl_xor_sync(0xffffffffu, sum_chosen, o);
    const float wgt = e / (norm_topk_prob == 1 ? sum_chosen : row_sum);
    if (lane < k) {
        indices_out[static_cast<size_t>(row) * k + lane] = my_idx;
        st_from_f32(weights_out, static_cast<size_t>(row) * k + lane, wgt, dt);
    }
}

// ---- MoE sort ------------------------------------------------------------------------------------
// The reference leaves the sort to its caller (moe.rs:253-271 states the contract only).  Definition
// used here: stable sort of the flat slots f = token*k + slot by (expert[f], f).  One CTA of 1024
// threads; warp w owns the contiguous slots [w * per, (w + 1) * per) and walks them 32 at a time:
// (1) per-warp, per-expert counts (lanes of a sub-chunk are grouped per expert with __match_any_sync; no
// atomics: a warp only writes its own row), (2) per expert a prefix over the 32 warps and the expert
// totals, scanned into expert_offsets, (3) the same walk again, now placing: position = first row of the
// expert + slots of earlier warps + slots of earlier sub-chunks of this warp + rank inside the sub-chunk.
constexpr int kSortThreads = 1024;

__global__ void __launch_bounds__(kSortThreads) moe_sort_kernel(const uint32_t *topk_idx, int total, int k, int n_experts,
                                                                uint32_t *sort_token_idx, uint32_t *inv_perm,
                                                                uint32_t *expert_offsets, uint32_t *row_expert,
                                                                uint32_t *status) {
    extern __shared__ uint32_t sm[];
    uint32_t *cursor = sm;                         // [n_experts + 1] first row of every expert
    uint32_t *wcnt = sm + n_experts + 1;           // [32][n_experts] per-warp counts, then running positions
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int per = ((total + 32 * 32 - 1) / (32 * 32)) * 32;          // slots per warp, whole sub-chunks
    const int f0 = warp * per, f1 = min(f0 + per, total);
    for (int i = tid; i < 32 * n_experts; i += kSortThreads) wcnt[i] = 0;
    __syncthreads();
    uint32_t *mine = wcnt + warp * n_experts;
    for (int c = f0; c < f1; c += 32) {
        const int f = c + lane;
        const bool have = f < f1;
        const uint32_t e = have ? topk_idx[f] : 0xFFFFFFFFu;
        const bool ok = have && e < static_cast<uint32_t>(n_experts);
        if (have && !ok) atomicCAS(status, 0u, 0x501u);        // expert id out of range: recorded, slot skipped
        const uint32_t peers = __match_any_sync(0xffffffffu, ok ? e : 0xFFFFFFFFu);
        if (ok && __popc(peers & ((1u << lane) - 1u)) == 0) mine[e] += __popc(peers);
        __syncwarp();
    }
    __syncthreads();
    for (int ee = tid; ee < n_experts; ee += kSortThreads) {   // per expert: exclusive prefix over the warps, total
        uint32_t run = 0;
        for (int w = 0; w < 32; ++w) {
            const uint32_t c = wcnt[w * n_experts + ee];
            wcnt[w * n_experts + ee] = run;
            run += c;
        }
        cursor[ee + 1] = run;
    }
    if (tid == 0) cursor[0] = 0;
    __syncthreads();
    if (warp == 0) {                               // inclusive scan of cursor[1..E] by one warp
        uint32_t carry = 0;
        for (int b = 0; b < n_experts; b += 32) {
            const int e = b + lane;
            uint32_t v = e < n_experts ? cursor[e + 1] : 0u;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const uint32_t t = __shfl_up_sync(0xffffffffu, v, o);
                if (lane >= o) v += t;
            }
            if (e < n_experts) cursor[e + 1] = v + carry;
            carry += __shfl_sync(0xffffffffu, v, 31);
        }
    }
    __syncthreads();
    for (int e = tid; e <= n_experts; e += kSortThreads) expert_offsets[e] = cursor[e];
    for (int c = f0; c < f1; c += 32) {
        const int f = c + lane;
        const bool have = f < f1;
        const uint32_t e = have ? topk_idx[f] : 0xFFFFFFFFu;
        const bool ok = have && e < static_cast<uint32_t>(n_experts);
        const uint32_t peers = __match_any_sync(0xffffffffu, ok ? e : 0xFFFFFFFFu);
        const uint32_t rank = __popc(peers & ((1u << lane) - 1u));
        uint32_t before = 0;
        if (ok) before = mine[e];                  // slots of this expert in earlier warps and earlier sub-chunks
        __syncwarp();
        if (ok && rank == 0) mine[e] = before + __popc(peers);
        __syncwarp();
        if (ok) {
            const uint32_t pos = cursor[e] + before + rank;
            sort_token_idx[pos] = static_cast<uint32_t>(f / k);
            inv_perm[f] = pos;
            if (row_expert) row_expert[pos] = e;
        }
    }
}

// ---- mt_moe_permute (moe.rs:283-302): permuted[p, :] = tokens[sort_token_idx[p], :] ----------------
__global__ void __launch_bounds__(256) permute_kernel(const uint8_t *tokens, const uint32_t *sort_token_idx, uint8_t *permuted,
                                                      int n_rows, size_t row_bytes, int vec16) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int p = blockIdx.x * (blockDim.x >> 5) + warp; p < n_rows; p += gridDim.x * (blockDim.x >> 5)) {
        const uint8_t *src = tokens + static_cast<size_t>(sort_token_idx[p]) * row_bytes;
        uint8_t *dst = permuted + static_cast<size_t>(p) * row_bytes;
        if (vec16) {
            for (size_t i = lane; i < row_bytes / 16; i += 32)
                reinterpret_cast<uint4 *>(dst)[i] = __ldg(reinterpret_cast<const uint4 *>(src) + i);
        } else {
            for (size_t i = lane; i < row_bytes; i += 32) dst[i] = src[i];
        }
    }
}

// ---- mt_moe_unpermute (moe.rs:222-249): out[t,h] = sum_j w[t,j] * eo[inv_perm[t,j], h], f32, j ascending ----
__global__ void __launch_bounds__(256) unpermute_kernel(const void *expert_out, const uint32_t *inv_perm, const void *weights,
                                                        void *out, int n_tokens, int hidden, int k, int dt) {
    const int t = blockIdx.x;
    if (t >= n_tokens) return;
    for (int h = threadIdx.x; h < hidden; h += blockDim.x) {
        float acc = 0.0f;
        for (int j = 0; j < k; ++j) {
            const uint32_t pos = __ldg(inv_perm + static_cast<size_t>(t) * k + j);
            const float v = ld_as_f32(expert_out, static_cast<size_t>(pos) * hidden + h, dt);
            const float w = ld_as_f32(weights, static_cast<size_t>(t) * k + j, dt);
            acc = acc + w * v;
        }
        st_from_f32(out, static_cast<size_t>(t) * hidden + h, acc, dt);
    }
}

// 16-bit activations, hidden % 8 == 0, 16-byte aligned rows: 8 columns per thread, one 128-bit load per expert row
__global__ void __launch_bounds__(256) unpermute16_kernel(const uint4 *expert_out, const uint32_t *inv_perm, const void *weights,
                                                          uint4 *out, int n_tokens, int hidden8, int k, int dt) {
    const int t = blockIdx.x;
    if (t >= n_tokens) return;
    for (int h8 = threadIdx.x; h8 < hidden8; h8 += blockDim.x) {
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int j = 0; j < k; ++j) {
            const uint32_t pos = __ldg(inv_perm + static_cast<size_t>(t) * k + j);
            const float w = ld_as_f32(weights, static_cast<size_t>(t) * k + j, dt);
            const uint4 v = __ldg(expert_out + static_cast<size_t>(pos) * hidden8 + h8);
            const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                float lo, hi;
                if (dt == MTC_BF16) {
                    lo = __uint_as_float(u[q] << 16);
                    hi = __uint_as_float(u[q] & 0xFFFF0000u);
                } else {
                    const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&u[q]));
                    lo = f.x; hi = f.y;
                }
                acc[2 * q] = acc[2 * q] + w * lo;
                acc[2 * q + 1] = acc[2 * q + 1] + w * hi;
            }
        }
        uint32_t o[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            if (dt == MTC_BF16) {
                const __nv_bfloat162 p2 = __floats2bfloat162_rn(acc[2 * q], acc[2 * q + 1]);
                o[q] = *reinterpret_cast<const uint32_t *>(&p2);
            } else {
                const __half2 p2 = __floats2half2_rn(acc[2 * q], acc[2 * q + 1]);
                o[q] = *reinterpret_cast<const uint32_t *>(&p2);
            }
        }
        out[static_cast<size_t>(t) * hidden8 + h8] = make_uint4(o[0], o[1], o[2], o[3]);
    }
}

// ---- mt_swiglu (swiglu.rs:45-57): silu(g) * u in f32 ------------------------------------------------
__global__ void __launch_bounds__(256) swiglu_kernel(const void *gate, const void *up, void *out, size_t n, int dt) {
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const float g = ld_as_f32(gate, i, dt), u = ld_as_f32(up, i, dt);
        const float s = g / (1.0f + expf(-g));
        st_from_f32(out, i, s * u, dt);
    }
}

// 16-bit activations, n % 8 == 0, 16-byte aligned: 8 elements per thread
__global__ void __launch_bounds__(256) swiglu16_kernel(const uint4 *gate, const uint4 *up, uint4 *out, size_t n8, int dt) {
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n8;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const uint4 gv = __ldg(gate + i), uv = __ldg(up + i);
        const uint32_t g4[4] = {gv.x, gv.y, gv.z, gv.w}, u4[4] = {uv.x, uv.y, uv.z, uv.w};
        uint32_t o[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            float g0, g1, u0, u1;
            if (dt == MTC_BF16) {
                g0 = __uint_as_float(g4[q] << 16); g1 = __uint_as_float(g4[q] & 0xFFFF0000u);
                u0 = __uint_as_float(u4[q] << 16); u1 = __uint_as_float(u4[q] & 0xFFFF0000u);
            } else {
                const float2 gf = __half22float2(*reinterpret_cast<const __half2 *>(&g4[q]));
                const float2 uf = __half22float2(*reinterpret_cast<const __half2 *>(&u4[q]));
                g0 = gf.x; g1 = gf.y; u0 = uf.x; u1 = uf.y;
            }
            const float r0 = (g0 / (1.0f + expf(-g0))) * u0, r1 = (g1 / (1.0f + expf(-g1))) * u1;
            if (dt == MTC_BF16) {
                const __nv_bfloat162 p2 = __floats2bfloat162_rn(r0, r1);
                o[q] = *reinterpret_cast<const uint32_t *>(&p2);
            } else {
                const __half2 p2 = __floats2half2_rn(r0, r1);
                o[q] = *reinterpret_cast<const uint32_t *>(&p2);
            }
        }
        out[i] = make_uint4(o[0], o[1], o[2], o[3]);
    }
}

// ---- any-shape gather_qmm on CUDA cores (moe.rs:358-433 and the b{3,5,6,8} macro :461-599) ----------
// One warp per output element (row t, column n); lanes stride over k; the expert of row t is the
// first e with t < expert_offsets[e+1], or indices[t] when given.
__global__ void __launch_bounds__(256)
gather_generic_kernel(const void *x, const uint32_t *w, const void *scales, const void *biases,
                      const uint32_t *expert_offsets, const uint32_t *indices, void *out, int t_rows, int k_in,
                      int n_out, int n_experts, int bits, int gs, int dt) {
    const int lane = threadIdx.x & 31;
    const long long gw = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (gw >= static_cast<long long>(t_rows) * n_out) return;
    const int row = static_cast<int>(gw / n_out), n = static_cast<int>(gw % n_out);
    int expert = -1;                      // a row that no expert's range covers is left untouched, as on the tensor-core paths
    if (indices) {
        expert = static_cast<int>(indices[row]);
    } else {
        for (int e = 0; e < n_experts; ++e)
            if (static_cast<uint32_t>(row) >= expert_offsets[e] && static_cast<uint32_t>(row) < expert_offsets[e + 1]) { expert = e; break; }
    }
    if (expert < 0 || expert >= n_experts) return;
    const size_t wpr = static_cast<size_t>(k_in) * bits / 32, gpr = k_in / gs;
    const size_t grow = static_cast<size_t>(expert) * n_out + n;
    const uint32_t *wr = w + grow * wpr;
    float acc = 0.0f;
    for (int k = lane; k < k_in; k += 32) {
        const float s = ld_as_f32(scales, grow * gpr + k / gs, dt);
        const float b = ld_as_f32(biases, grow * gpr + k / gs, dt);
        const float q = static_cast<float>(code_at(wr, k, bits));
        acc = fmaf(fmaf(q, s, b), ld_as_f32(x, static_cast<size_t>(row) * k_in + k, dt), acc);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) st_from_f32(out, static_cast<size_t>(row) * n_out + n, acc, dt);
}

}  // namespace

cudaError_t launch_router_topk(cudaStream_t st, const void *logits, uint32_t *idx, void *wts, int n_rows, int n_experts,
                               int k, int norm, int dt) {
    if (n_rows <= 0) return cudaSuccess;
    router_topk_kernel<<<(n_rows + 3) / 4, 128, 0, st>>>(logits, idx, wts, n_rows, n_experts, k, norm, dt);
    return cudaGetLastError();
}

cudaError_t launch_moe_sort(cudaStream_t st, const uint32_t *topk_idx, int n_tokens, int k, int n_experts, uint32_t *sti,
                            uint32_t *inv, uint32_t *offsets, uint32_t *row_expert, uint32_t *status) {
    const size_t smem = (static_cast<size_t>(n_experts) + 1 + 32 * static_cast<size_t>(n_experts)) * sizeof(uint32_t);
    static PerDeviceAttr attr;
    cudaError_t e = attr.set(moe_sort_kernel, 200 * 1024);
    if (e != cudaSuccess) return e;
    moe_sort_kernel<<<1, kSortThreads, smem, st>>>(topk_idx, n_tokens * k, k, n_experts, sti, inv, offsets, row_expert, status);
    return cudaGetLastError();
}

cudaError_t launch_permute(cudaStream_t st, const void *tokens, const uint32_t *sti, void *permuted, int n_rows, int hidden,
                           int dt) {
    if (n_rows <= 0) return cudaSuccess;
    const size_t row_bytes = static_cast<size_t>(hidden) * dtype_size(dt);
    const int vec = row_bytes % 16 == 0 && reinterpret_cast<uintptr_t>(tokens) % 16 == 0 &&
                    reinterpret_cast<uintptr_t>(permuted) % 16 == 0;
    int grid = (n_rows + 7) / 8;
    if (grid > kNumSMsB200 * 8) grid = kNumSMsB200 * 8;
    permute_kernel<<<grid, 256, 0, st>>>(static_cast<const uint8_t *>(tokens), sti, static_cast<uint8_t *>(permuted), n_rows,
                                         row_bytes, vec);
    return cudaGetLastError();
}

cudaError_t launch_unpermute(cudaStream_t st, const void *eo, const uint32_t *inv, const void *wts, void *out, int n_tokens,
                             int hidden, int k, int dt) {
    if (n_tokens <= 0) return cudaSuccess;
    const auto al16 = [](const void *p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; };
    if (dt != MTC_F32 && hidden % 8 == 0 && al16(eo) && al16(out))
        unpermute16_kernel<<<n_tokens, 256, 0, st>>>(static_cast<const uint4 *>(eo), inv, wts, static_cast<uint4 *>(out), n_tokens,
                                                     hidden / 8, k, dt);
    else
        unpermute_kernel<<<n_tokens, 256, 0, st>>>(eo, inv, wts, out, n_tokens, hidden, k, dt);
    return cudaGetLastError();
}

cudaError_t launch_swiglu(cudaStream_t st, const void *gate, const void *up, void *out, size_t n, int dt) {
    if (n == 0) return cudaSuccess;
    const auto al16 = [](const void *p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; };
    const bool vec = dt != MTC_F32 && n % 8 == 0 && al16(gate) && al16(up) && al16(out);
    const size_t work = vec ? n / 8 : n;
    size_t grid = (work + 255) / 256;
    if (grid > static_cast<size_t>(kNumSMsB200) * 16) grid = static_cast<size_t>(kNumSMsB200) * 16;
    if (vec)
        swiglu16_kernel<<<static_cast<int>(grid), 256, 0, st>>>(static_cast<const uint4 *>(gate), static_cast<const uint4 *>(up),
                                                               static_cast<uint4 *>(out), n / 8, dt);
    else
        swiglu_kernel<<<static_cast<int>(grid), 256, 0, st>>>(gate, up, out, n, dt);
    return cudaGetLastError();
}

cudaError_t launch_gather_generic(cudaStream_t st, const void *x, const void *w, const void *scales, const void *biases,
                                  const uint32_t *offsets, const uint32_t *indices, void *out, int t_rows, int k_in, int n_out,
                                  int n_experts, int bits, int gs, int dt) {
    const long long warps = static_cast<long long>(t_rows) * n_out;
    if (warps <= 0) return cudaSuccess;
    const long long grid = (warps + 7) / 8;
    gather_generic_kernel<<<static_cast<unsigned>(grid), 256, 0, st>>>(x, static_cast<const uint32_t *>(w), scales, biases,
                                                                       offsets, indices, out, t_rows, k_in, n_out, n_experts,
                                                                       bits, gs, dt);
    return cudaGetLastError();
}

}  // namespace mtc
