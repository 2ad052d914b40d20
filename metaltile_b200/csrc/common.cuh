// Shared device/host helpers for the sm_100a kernels behind include/mtcuda.h.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>
#include <vector>

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
    int qmm_force_tn = 0;          // option "qmm_tile_tokens": 0 = choose per shape
    int qmv_max_occ = 0;           // option "qmv_max_ctas_per_sm": > 0 caps the CTAs per SM of the qmv kernel's grid
    int qmv_small_m_mma = 1;       // option "qmv_small_m_mma": 0 keeps 2 <= M <= 16 on the CUDA-core kernel
    int qmm_max_stages = 0;        // option "qmm_max_stages": > 0 caps the ring depth (diagnostic: how much the ring hides)
    int qmm_wait_hint_ns = 5000;      // option "qmm_wait_hint_ns": base suspend-time hint of the kernel's mbarrier waits
    int qmm_mma_chunks = 1;        // option "qmm_mma_chunks": 0 = 17 <= M <= 64 always on the tcgen05 kernel
    int qmm_raw = 1;               // option "qmm_raw": 0 = dequant warps load their packed words straight from global memory
    int qmm_wide = 1;              // option "qmm_wide": 0 = a dense work item never covers two token chunks (one W stage, two X chunks)
    uint32_t peer_poll_limit = 1u << 22;   // option "peer_poll_limit": polls of mtc_peer_barrier before it gives up on a peer
    int qmv_tc = 0;                // option "qmv_tc": 1 = M <= 8 decode shapes run on the tcgen05 decode kernel (qmv_tc.cu; slower than the stream kernel today)
    float *d_tc_scratch = nullptr; // partial sums of the tcgen05 decode kernel's K chunks (grow-only; outgrown blocks stay alive)
    size_t tc_scratch_bytes = 0;
    uint32_t *d_tc_counters = nullptr;   // its arrival counters, zero between launches
    std::vector<void *> retired;   // outgrown scratch blocks: freed by mtc_destroy, so that captured graphs never see freed memory
    int qmv_stream = 1;            // option "qmv_stream": 0 = never use the streaming decode kernel (qmv_stream.cu)
    int pdl_early_weights = 1;     // option "pdl_early_weights": 0 = no load of w / scales / biases before the previous kernel of the stream is complete
    void *d_worklist = nullptr;    // gather_qmm work list (grow-only, owned by the context)
    size_t worklist_bytes = 0;
    void *d_xconv = nullptr;       // scaled-f16 copy of bf16 activations for the tensor-core kernels (grow-only)
    size_t xconv_bytes = 0;
    void *d_gfrag = nullptr;       // streaming gather: activations in fragment order, their sums, the table of passes (grow-only)
    size_t gfrag_bytes = 0;
    int gather_stream = 1;         // option "gather_stream": 0 = grouped products never take the streaming kernel (gather_stream.cu)
    void *d_tail = nullptr;        // MoE decode tail: the staged inner activations of a call (grow-only)
    size_t tail_bytes = 0;
    void *d_qvm = nullptr;         // mtc_qvm: arrival counters (zero between launches), then the partial sums of the K chunks (grow-only)
    size_t qvm_bytes = 0;
    void *d_norm = nullptr;        // mtc_rms_norm_qmv on shapes the fused kernel does not take: the normalised row (grow-only)
    size_t norm_bytes = 0;
    void *d_ksplit = nullptr;      // tcgen05 qmm with K slices: the f32 partial sums of a launch (grow-only)
    size_t ksplit_bytes = 0;
    int qmm_ksplit = 1;            // option "qmm_ksplit": 0 = a dense launch with few weight-row tiles never cuts K into slices
    int qmv_small_m_tc = 1;        // option "qmv_small_m_tc": 0 = M <= 16 never takes the tcgen05 kernel; 2 = whenever it supports the shape (M >= 2)
    void *d_flush = nullptr;       // mtc_measure with cold_l2: a block larger than L2 that a memset rewrites between timed launches
    size_t flush_bytes = 0;
    void *d_moe = nullptr;         // mtc_moe_experts: gate and up outputs (and permuted rows on the composed path) (grow-only)
    size_t moe_bytes = 0;
};

// Grow-only device block of a context.  The block only ever moves outside stream capture (a captured graph holds its
// address), and an outgrown block stays allocated until mtc_destroy: work already enqueued, or a graph captured
// earlier, may still name it.  Kernels that use such a block run on the caller's stream in call order; two streams
// that use one context at the same time must not both use entries that need the same block.
inline cudaError_t grow_block(Ctx *ctx, cudaStream_t st, void **block, size_t *have, size_t need, std::string *why) {
    if (need <= *have) return cudaSuccess;
    cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(st, &cs) == cudaSuccess && cs != cudaStreamCaptureStatusNone) {
        if (why) *why = "a scratch block of the context must grow, which cannot happen during stream capture: run this shape once before capturing";
        return cudaErrorStreamCaptureUnsupported;
    }
    const size_t want = need + (need >> 1) + (1u << 20);
    void *p = nullptr;
    cudaError_t e = cudaMalloc(&p, want);
    if (e != cudaSuccess) return e;
    if (*block) ctx->retired.push_back(*block);
    *block = p;
    *have = want;
    return cudaSuccess;
}

inline int fail(Ctx *ctx, int code, const std::string &msg) {
    if (ctx) ctx->last_error = msg;
    return code;
}

inline size_t dtype_size(int dt) { return dt == MTC_F32 ? 4 : 2; }

// cudaFuncAttributeMaxDynamicSharedMemorySize belongs to (kernel, device): one flag per device, not per process.
// set(fn) applies `bytes` to the kernel on the current device the first time that device launches it.
struct PerDeviceAttr {
    bool done[64] = {};
    template <typename Fn>
    cudaError_t set(Fn fn, size_t bytes) {
        int dev = 0;
        cudaError_t e = cudaGetDevice(&dev);
        if (e != cudaSuccess) return e;
        if (dev >= 0 && dev < 64 && done[dev]) return cudaSuccess;
        e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes));
        if (e == cudaSuccess && dev >= 0 && dev < 64) done[dev] = true;
        return e;
    }
};

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
                       std::string *why, void *const *extra_outs = nullptr, int n_extra = 0, const void *norm_w = nullptr,
                       float eps = 0.0f);
cudaError_t launch_rms_norm_row(cudaStream_t st, const void *x, const void *norm_w, void *out, int K, float eps, int dt);
// all ranks have stored: one flag per peer, written with system-scope release, awaited with a bounded poll
cudaError_t launch_peer_barrier(Ctx *ctx, cudaStream_t st, uint32_t *const *peer_flags, int n_peers, int rank,
                                uint32_t *local_flags, uint32_t *epoch);
cudaError_t qmv_init_device();
// streaming decode kernel (qmv_stream.cu): 1-4 projections that share x in one launch, and prepared chains
bool qmv_stream_supported(int M, int N, int K, int bits, int group_size, int dt, const void *w, const void *scales,
                          const void *biases, const void *x);
cudaError_t qmv_stream_init_device();
cudaError_t launch_qmv_stream(Ctx *ctx, cudaStream_t st, const mtc_qmv_desc *descs, int n, const mtc_peer_sync *sync = nullptr);
bool qmv_tc_supported(int M, int N, int K, int bits, int group_size, int dt, const void *w, const void *scales,
                      const void *biases, const void *x);
cudaError_t qmv_tc_init_device();
size_t qmv_tc_scratch_bytes(int M, int N, int K);
size_t qmv_tc_counter_bytes(int N);
cudaError_t launch_qmv_tc(Ctx *ctx, cudaStream_t st, const void *w, const void *scales, const void *biases, const void *x,
                          void *const *outs, int n_out, int M, int N, int K, int group_size, int dt, float *scratch,
                          uint32_t *counters);
struct StreamChain;
cudaError_t stream_chain_create(Ctx *ctx, const mtc_qmv_desc *descs, int n, StreamChain **out, std::string *why);
cudaError_t stream_chain_run(Ctx *ctx, cudaStream_t st, StreamChain *c);
void stream_chain_destroy(StreamChain *c);
bool qmv_mma_supported(int M, int N, int K, int bits, int group_size, int dt, const void *w, const void *x);
cudaError_t launch_qmv_mma(Ctx *ctx, cudaStream_t st, const void *w, const void *scales, const void *biases, const void *x,
                           void *out, int M, int N, int K, int group_size, int dt);
bool qmm_tcgen05_supported(int M, int N, int K, int bits, int group_size, int dt, const void *w, const void *x,
                           const void *out);
cudaError_t launch_qmm_tcgen05(Ctx *ctx, cudaStream_t st, const void *w, const void *scales, const void *biases,
                               const void *x, void *out, int M, int N, int K, int bits, int group_size, int dt,
                               std::string *why, void *const *outs = nullptr, int n_outs = 1, long long out_ld = 0);
size_t gather_items_bytes(int total_rows, int n_experts, int N, int TN_hint);
cudaError_t launch_gather_qmm_tcgen05(Ctx *ctx, cudaStream_t st, const void *x, const void *w, const void *scales,
                                      const void *biases, const uint32_t *expert_offsets, const uint32_t *indices,
                                      void *out, int total_rows, int N, int K, int n_experts, int bits, int group_size,
                                      int dt, void *scratch, size_t scratch_bytes, std::string *why);
cudaError_t launch_gather_qmm_static(Ctx *ctx, cudaStream_t st, const void *x, const void *w, const void *scales,
                                     const void *biases, const uint32_t *expert_offsets, const uint32_t *indices,
                                     void *out, int total_rows, int N, int K, int n_experts, int bits, int group_size,
                                     int dt, std::string *why);
cudaError_t launch_router_topk(cudaStream_t st, const void *logits, uint32_t *idx, void *wts, int n_rows, int n_experts,
                               int k, int norm, int dt);
cudaError_t launch_moe_sort(cudaStream_t st, const uint32_t *topk_idx, int n_tokens, int k, int n_experts, uint32_t *sti,
                            uint32_t *inv, uint32_t *offsets, uint32_t *row_expert, uint32_t *status);
cudaError_t launch_permute(cudaStream_t st, const void *tokens, const uint32_t *sti, void *permuted, int n_rows, int hidden,
                           int dt);
cudaError_t launch_unpermute(cudaStream_t st, const void *eo, const uint32_t *inv, const void *wts, void *out, int n_tokens,
                             int hidden, int k, int dt);
cudaError_t launch_swiglu(cudaStream_t st, const void *gate, const void *up, void *out, size_t n, int dt);
bool gather_stream_supported(int m_total, int n_out, int K, int n_experts, int bits, int group_size, int dtype, const void *w,
                             const void *scales, const void *biases, const void *x);
size_t gather_stream_scratch_bytes(int m_total, int K);
struct GatherMats {
    const void *w, *scales, *biases;
    void *out;
};
cudaError_t launch_gather_stream(Ctx *ctx, cudaStream_t st, const void *x, const void *x2, const uint32_t *row_src, int n_src_rows,
                                 const GatherMats *mats, int n_mats, const uint32_t *expert_offsets, int m_total, int n_out, int K,
                                 int n_experts, int group_size, int dtype, void *scratch);
cudaError_t launch_affine_dequantize(Ctx *ctx, cudaStream_t st, const void *w, const void *scales, const void *biases, void *out,
                                     size_t n_elem, int bits, int group_size, int dt);
size_t moe_decode_smem_bytes(int n_slots, int in_dim);
cudaError_t launch_moe_decode(Ctx *ctx, cudaStream_t st, const void *const *gate, const void *const *up, const void *experts,
                              const void *slot_w, const void *w, const void *scales, const void *biases, void *out, int n_slots, int in_dim,
                              int out_dim, int n_experts, int group_size, int dt, int fused, float *staged);
int qvm_k_chunks(int sms, int N, int K, int bits, int group_size);
bool qvm_fast_supported(int N, int K, int bits, int group_size);
cudaError_t launch_qvm(Ctx *ctx, cudaStream_t st, const void *w, const void *scales, const void *biases, const void *x, void *out,
                       int M, int N, int K, int bits, int group_size, int dt, void *scratch, int KC);
size_t qvm_scratch_bytes(int M, int N, int KC);
cudaError_t launch_dequant_gather(Ctx *ctx, cudaStream_t st, const void *w, const void *scales, const void *biases, const void *indices,
                                  void *out, size_t n_tokens, int hidden, int vocab, int bits, int group_size, int dt);
cudaError_t launch_affine_quantize(Ctx *ctx, cudaStream_t st, const void *w, void *out, void *scales, void *biases, size_t n_groups,
                                   int bits, int group_size, int dt);
cudaError_t launch_gather_generic(cudaStream_t st, const void *x, const void *w, const void *scales, const void *biases,
                                  const uint32_t *offsets, const uint32_t *indices, void *out, int t_rows, int k_in, int n_out,
                                  int n_experts, int bits, int gs, int dt);
cudaError_t launch_unpack_codes(cudaStream_t st, const void *w, void *codes, int N, int K, int bits);

}  // namespace mtc
