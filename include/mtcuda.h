/*
 * mtcuda.h — C ABI of the B200 (sm_100a) back end for metaltile's affine
 * group-quantized matmul family: qmv (decode), qmm (prefill), the MoE
 * gather_qmm and the routing kernels around it.
 *
 * This is the boundary a `metaltile-runtime` CUDA backend binds through FFI.
 * Each entry names the reference interface it stands in for (paths relative to
 * the metaltile repository).  Conventions:
 *   - every call returns an `mtc_status` (0 = ok, negative = error); the
 *     message of the last error of a context is read with mtc_last_error();
 *   - one mtc_ctx per device, not thread-safe (the reference's Context is
 *     !Send and its tests serialise GPU access: crates/metaltile-std/tests/common/mod.rs:11-27);
 *   - pointers named d_* / w / scales / biases / x / out of the typed ops are
 *     DEVICE pointers (16-byte aligned); `stream` is a cudaStream_t passed as
 *     void* (NULL = default stream); typed ops are asynchronous and never block;
 *   - layouts are exactly the reference's: w u32[N, K*bits/32] (row = LSB-first
 *     bit-stream, low field first along K), scales/biases T[N, K/group_size],
 *     x T[M, K], out T[M, N] row-major; T in {f32, f16, bf16};
 *   - there is no CPU fallback: without a CUDA device mtc_init fails with
 *     MTC_ERR_NO_DEVICE and nothing else can be called.
 */
#ifndef MTCUDA_H
#define MTCUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct mtc_ctx mtc_ctx;

/* Activation dtype T (metaltile-core DType::{F32,F16,BF16},
 * crates/metaltile-core/src/dsl/dtype.rs:11-33). */
typedef enum { MTC_F32 = 0, MTC_F16 = 1, MTC_BF16 = 2 } mtc_dtype;

/* Mirrors the variants of MetalTileError (crates/metaltile-runtime/src/error.rs:7-56). */
typedef enum {
    MTC_OK = 0,
    MTC_ERR_NO_DEVICE = -1,          /* NoDevice */
    MTC_ERR_BUFFER = -2,             /* Buffer: allocation / copy failed, bad pointer or alignment */
    MTC_ERR_BUFFER_SIZE = -3,        /* BufferSize: a named buffer is smaller than the kernel needs */
    MTC_ERR_DISPATCH = -4,           /* Dispatch: launch or execution error */
    MTC_ERR_FUNCTION_NOT_FOUND = -5, /* FunctionNotFound: unknown kernel name */
    MTC_ERR_UNSUPPORTED = -6,        /* Unsupported: shape / bits / dtype outside the kernel's contract */
    MTC_ERR_TIMEOUT = -7,            /* a bounded device-side wait expired (see mtc_status_word) */
    MTC_ERR_INVALID = -8             /* null / inconsistent argument */
} mtc_status;

/* ---- lifecycle: Context::new (crates/metaltile-runtime/src/context.rs:160-240) ---- */
int mtc_init(int device, mtc_ctx **out_ctx);
int mtc_destroy(mtc_ctx *ctx);
const char *mtc_last_error(mtc_ctx *ctx); /* valid until the next call on ctx; ctx may be NULL */
/* `tile device --json` keys (crates/metaltile-cli/src/cmd/device.rs:55-66) plus
 * sm_count, cc, hbm_bytes, l2_bytes, driver, runtime. */
int mtc_device_info(mtc_ctx *ctx, char *json, size_t cap);

/* ---- memory: Context::upload_resident / ResidentBuffer (context.rs:330-350,104-117),
 *      GpuRunner::buffer_bytes / buffer_zeros / read_bytes
 *      (crates/metaltile-std/src/runner.rs:317-360) ---- */
int mtc_alloc(mtc_ctx *ctx, size_t bytes, void **d_ptr);
int mtc_free(mtc_ctx *ctx, void *d_ptr);
int mtc_upload(mtc_ctx *ctx, void *stream, void *d_dst, const void *h_src, size_t bytes);
int mtc_download(mtc_ctx *ctx, void *stream, void *h_dst, const void *d_src, size_t bytes);
int mtc_memset(mtc_ctx *ctx, void *stream, void *d_ptr, int value, size_t bytes);
/* commit + waitUntilCompleted (single_dispatch.rs:95-98).  Returns MTC_ERR_TIMEOUT when a kernel of this context has
 * given up on a bounded device-side wait since the status word was last cleared (the kernel has returned, the GPU
 * is usable, the results are not); mtc_sync_deadline also returns MTC_ERR_TIMEOUT when the stream has not finished
 * after timeout_ms milliseconds of host time (timeout_ms < 0: wait without a deadline). */
int mtc_sync(mtc_ctx *ctx, void *stream);
int mtc_sync_deadline(mtc_ctx *ctx, void *stream, int timeout_ms);
/* 0 when no kernel has reported a bounded-wait expiry or a rejected index since the context was created or the
 * word was cleared; otherwise the code of the first report: 0x101-0x402 roles of the tensor-core kernel, 0x601 + r
 * rank r never arrived at a peer barrier, 0x701 / 0x702 phase counter / partial-sum slot of a chained launch. */
int mtc_status_word(mtc_ctx *ctx, uint32_t *word);
int mtc_status_clear(mtc_ctx *ctx);

/* ---- typed ops (device pointers, asynchronous on `stream`) ---- */

/* mt_qmv and the generic mt_qmv_b{3,4,5,6,8} / mt_qmm_b* / mt_qmm{,_bm2,_bm4} and
 * dequant_gemv_int2 family: out[m,n] = sum_k (q*scale + bias) * x[m,k], f32
 * accumulate (crates/metaltile-std/src/mlx/quantized.rs:7-308,343-1441,4273-4392;
 * crates/metaltile-std/src/ffai/dequant_gemv.rs:52-105).  Any M (tuned for M <= 16), bits in
 * {2,3,4,5,6,8}, K*bits % 32 == 0, group_size | K.  M = 1 and every general case run on CUDA cores;
 * 2 <= M <= 16 with 4-bit codes, f16/bf16 activations, K % 64 == 0 and a power-of-two group >= 64 use
 * warp-level tensor-core MMAs on the integer codes (f32 accumulate, affine part applied per group). */
int mtc_qmv(mtc_ctx *ctx, void *stream, const void *w, const void *scales, const void *biases,
            const void *x, void *out, int M, int N, int K, int bits, int group_size, int dtype);

/* mt_qmm_for + mt_qmm_mma* (quantized.rs:5040-5065,2106-2362): picks the kernel
 * from M like the reference's selector: M <= 16 -> the qmv path above; larger M
 * with f16/bf16 activations -> the tensor-core (tcgen05) prefill kernel, which
 * like mt_qmm_mma dequantises the weight tile to T before the MMA
 * (quantized.rs:2245-2252); f32 activations always take the CUDA-core path.
 * Ragged M needs no padding (the reference pads to 32: quantized_mma_dynamic_m.rs:46-112). */
int mtc_qmm(mtc_ctx *ctx, void *stream, const void *w, const void *scales, const void *biases,
            const void *x, void *out, int M, int N, int K, int bits, int group_size, int dtype);
/* Name of the kernel family mtc_qmm would run for these arguments with aligned pointers and default options
 * ("qmv_stream", "qmv_cuda_core", "qmv_mma_sync", "qmm_tcgen05"); the analogue of asserting on
 * mt_qmm_for's routing (quantized.rs:5127-5199). */
const char *mtc_qmm_route(int M, int N, int K, int bits, int group_size, int dtype);

/* ---- fused and chained decode projections ----
 * mtc_qmv_desc: one projection, the arguments of mtc_qmv plus up to 8 destinations of the [M, N] result (each gets
 * the same bytes: local buffer, peer GPUs' buffers) and, in a chain, the phase it belongs to.
 *
 * mtc_qmv_batched: 1 to 4 projections that read the SAME activations (same x, M, K, dtype) in one launch, each
 * writing its own output.  With the outputs laid out one after the other this is ffai_batched_qkv_qgemv(_fast)
 * (crates/metaltile-std/src/ffai/batched_qkv_qgemv.rs:1-35: q, k, v in one dispatch, one concatenated result) and
 * ffai_batched_4_qgemv (crates/metaltile-std/src/ffai/batched_4_qgemv.rs:1-45).  Shapes outside the streaming
 * kernel's contract (4-bit, f16 / bf16, M <= 8, K % 256 == 0, group 64 or 128) run as separate mtc_qmv launches.
 *
 * mtc_chain_*: a prepared list of projections walked by ONE persistent grid, the counterpart of
 * Context::dispatch_chain (crates/metaltile-runtime/src/context.rs:363-395: several passes, one commit, ordering
 * between passes, no host round trip).  Projections of one phase are independent; a projection of phase p may read
 * (as x) what phases < p wrote: the grid passes a device-side counter between phases (bounded wait: status word
 * 0x701 on expiry) instead of a launch boundary, and keeps requesting the weights of later phases meanwhile.
 * Phases start at 0 and grow by at most one from one projection to the next.  mtc_chain_create copies the
 * descriptors (the buffers they name must stay valid and in place until mtc_chain_destroy); mtc_chain_run is
 * asynchronous on `stream` and may be captured in a CUDA graph; runs of one chain must not overlap on the GPU.
 * Chains outside the streaming kernel's contract run as one mtc_qmv launch per projection, in order. */
typedef struct {
    const void *w, *scales, *biases, *x;
    void *outs[8];
    int n_outs;
    int M, N, K, bits, group_size, dtype;
    int phase;
} mtc_qmv_desc;
typedef struct mtc_chain mtc_chain;
int mtc_qmv_batched(mtc_ctx *ctx, void *stream, const mtc_qmv_desc *descs, int n);
/* mtc_qmv_batched for the sharded decode path with the hand-off between the GPUs inside the kernel (no counterpart in the
 * reference, which is a single-device library).  Every rank enqueues the same sequence of launches; a launch stores its
 * results into every rank's buffers (descs[i].outs), waits - before it reads x - until every peer has finished the launch
 * that matches this rank's previous one (bounded poll: status word 0x601 + peer on expiry), and when its last CTA is done
 * publishes the next epoch into word `rank` of every peer's flag array.  peer_flags[q] = rank q's flag array (8 x uint32,
 * shared with mtc_ipc_*), local_flags = this rank's own; epoch and ticket = one uint32 each of this rank's memory; all
 * zeroed once.  Only shapes the streaming kernel takes (else MTC_ERR_UNSUPPORTED).  A buffer region may be rewritten only
 * by a launch that comes after every rank's readers of it, i.e. at least one launch of this kind later. */
typedef struct {
    void *peer_flags[8];
    void *local_flags, *epoch, *ticket;
    int n_peers, rank;
} mtc_peer_sync;
int mtc_qmv_batched_sync(mtc_ctx *ctx, void *stream, const mtc_qmv_desc *descs, int n, const mtc_peer_sync *sync);
int mtc_chain_create(mtc_ctx *ctx, const mtc_qmv_desc *descs, int n, mtc_chain **out_chain);
int mtc_chain_run(mtc_ctx *ctx, void *stream, mtc_chain *chain);
int mtc_chain_destroy(mtc_ctx *ctx, mtc_chain *chain);
/* 1 when the chain runs on the persistent streaming kernel, 0 when it falls back to one launch per projection. */
int mtc_chain_is_fused(const mtc_chain *chain);

/* ---- sharded decode: the output all-gather done by the kernel's own stores (one process per GPU) ----
 * None of these has a counterpart in the reference, which is a single-device library; they serve the N-split
 * (column-parallel) sharding of a projection over the GPUs of one node.
 *
 * mtc_qmv_multi: mtc_qmv that writes its [M, N] output tile to outs[0..n_outs) (1 to 8 destinations, same layout
 * and dtype each).  With outs[i] = rank i's copy of the gathered buffer, offset to this rank's slot, the all-gather
 * is the store.  M = 1 on the vectorised CUDA-core path (power-of-two group, aligned pointers, K staged whole);
 * one destination works for every shape mtc_qmv takes on that path.
 * mtc_ipc_export / mtc_ipc_open / mtc_ipc_close: share a buffer from mtc_alloc with the other rank processes
 * (cudaIpc handle, 64 bytes; opening enables peer access; plain peer mappings, no multicast object).
 * mtc_peer_barrier: enqueue a one-warp kernel that tells every peer "my stores so far are done" and waits until
 * every peer has said the same.  peer_flags[p] = rank p's flag array (8 x uint32, zeroed once, shared with
 * mtc_ipc_*), local_flags = this rank's own array, epoch = one uint32 of this rank's memory, zeroed once; every rank
 * must enqueue the same sequence of barriers.  The wait is bounded (a few seconds): on expiry the status word becomes
 * 0x601 + the rank that never arrived and the kernel returns. */
int mtc_qmv_multi(mtc_ctx *ctx, void *stream, const void *w, const void *scales, const void *biases, const void *x,
                  void *const *outs, int n_outs, int M, int N, int K, int bits, int group_size, int dtype);
/* mt_affine_quantize_int{2,3,4,5,6,8} / mt_affine_dequantize_int{2,3,4,5,6,8} (crates/metaltile-std/src/mlx/quantized.rs:
 * 3575-4214): the producer and the inverse of the packed format the matmuls read.
 *   quantize:   w T[n_elem] -> out u32[n_elem * bits / 32] (LSB-first bit-stream, one per group), scales / biases T[n_elem / G]:
 *               scale = (max - min) / (2^bits - 1) (1 when below 1e-7), bias = min,
 *               q = trunc(clamp((v - bias) * (1 / scale) + 0.5, 0, 2^bits - 1))
 *   dequantize: out T[n_elem] = scale * q + bias
 * Every float operation is rounded to f32 on its own (no fused multiply-add): codes and values equal the scalar CPU
 * formula bit for bit.  Whole groups only, group_size * bits % 32 == 0. */
int mtc_affine_quantize(mtc_ctx *ctx, void *stream, const void *w, void *out, void *scales, void *biases, size_t n_elem, int bits,
                        int group_size, int dtype);
int mtc_affine_dequantize(mtc_ctx *ctx, void *stream, const void *w, const void *scales, const void *biases, void *out,
                          size_t n_elem, int bits, int group_size, int dtype);
/* The M = 1 tail of a mixture-of-experts layer with the expert ids read on the device (4-bit stacked weights
 * w u32[E, out_dim, in_dim/8], scales / biases T[E, out_dim, in_dim/G], expert_indices u32[n_slots], 1 <= n_slots <= 8):
 *   mtc_moe_down_swiglu_accum - ffai_moe_down_swiglu_accum_int4_chain8 (crates/metaltile-std/src/ffai/moe_down_swiglu_accum.rs:
 *       158-318): out[row] = sum_k slot_weights[k] * sum_d w(e_k, row, d) * silu(gates[k][d]) * ups[k][d]; gates[k], ups[k] T[in_dim];
 *       the inner activations stay in f32 (shared memory), as in the reference;
 *   mtc_qmv_expert_indexed    - dequant_gemv_int4_expert_indexed (ffai/dequant_gemv_expert_indexed.rs:56-103), for n_slots
 *       inputs at once: out[k][row] = sum_d w(e_k, row, d) * xs[k][d]; out T[n_slots, out_dim].
 * An expert id outside the stack reads expert 0 and is reported through the status word (0x905). */
int mtc_moe_down_swiglu_accum(mtc_ctx *ctx, void *stream, const void *const *gates, const void *const *ups, int n_slots,
                              const void *expert_indices, const void *slot_weights, const void *w, const void *scales,
                              const void *biases, void *out, int in_dim, int out_dim, int n_experts, int group_size, int dtype);
int mtc_qmv_expert_indexed(mtc_ctx *ctx, void *stream, const void *const *xs, int n_slots, const void *expert_indices, const void *w,
                           const void *scales, const void *biases, void *out, int in_dim, int out_dim, int n_experts, int group_size,
                           int dtype);
/* mt_qvm_b{3,4,5,6,8} / mt_qvm_int4_fast (crates/metaltile-std/src/mlx/quantized.rs:4397-4530,4582-4700): the quantized
 * vector-matrix product, y = x W with W stored transposed: w u32[K, N*bits/32] (row d = LSB-first bit-stream of N codes),
 * scales / biases T[K/G, N] (groups along K), x T[M, K], out T[M, N]:
 *     out[m, c] = sum_d (q(d, c) * scale[d/G, c] + bias[d/G, c]) * x[m, d]        (f32 accumulation).
 * K is split over CTAs; the partial sums live in a grow-only block of the context and are added in a fixed order. */
int mtc_qvm(mtc_ctx *ctx, void *stream, const void *w, const void *scales, const void *biases, const void *x, void *out, int M, int N,
            int K, int bits, int group_size, int dtype);
/* dequant_gather_int{2,3,4,5,6,8} (crates/metaltile-std/src/ffai/dequant_gather.rs:44-101): rows indices[t] (u32) of a
 * quantized table weight u32[vocab, hidden*bits/32], scales / biases T[vocab, hidden/G], dequantized into
 * out T[n_tokens, hidden] = q * scale + bias (separately rounded f32 operations).  An index outside the table reads
 * row 0 and is reported through the status word (0x904). */
int mtc_dequant_gather(mtc_ctx *ctx, void *stream, const void *weight, const void *scales, const void *biases, const void *indices,
                       void *out, size_t n_tokens, int hidden, int vocab, int bits, int group_size, int dtype);
/* ffai_rms_norm_qgemv / _fast (crates/metaltile-std/src/ffai/rms_norm_qgemv.rs:51-107,131-146): the decode projection
 * of the RMS-normalised activation in one launch,
 *     out[n] = sum_k w(n, k) * (x[k] * norm_weight[k] * inv_rms),   inv_rms = 1 / sqrt(mean(x^2) + eps),
 * x, norm_weight T[K]; the normalised activation stays in f32 (it is staged in shared memory, never rounded to T and
 * never written to global memory), as in the reference.  Shapes the fused kernel does not take (unaligned pointers,
 * groups that are not a power of two, K too long for one shared-memory stage) are normalised into a row of type T
 * first and then run through mtc_qmv. */
int mtc_rms_norm_qmv(mtc_ctx *ctx, void *stream, const void *x, const void *norm_weight, float eps, const void *w,
                     const void *scales, const void *biases, void *out, int N, int K, int bits, int group_size, int dtype);
/* mtc_qmm whose [M, N] result is a column block of wider row-major matrices, written to 1 to 8 destinations (no
 * counterpart in the reference): outs[i] points at row 0 of the block inside destination i, ld = elements between
 * consecutive rows of a destination (>= N).  With the peers' mappings of one [M, N_total] buffer per rank (mtc_ipc_*) as
 * destinations, an N-split prefill matmul gathers itself: every rank's epilogue stores its column block into every
 * rank's copy while the next tiles are computed; mtc_peer_barrier afterwards makes the blocks visible everywhere.
 * Plain stores through peer mappings only.  Shapes of the tensor-core kernel only (else MTC_ERR_UNSUPPORTED). */
int mtc_qmm_multi(mtc_ctx *ctx, void *stream, const void *w, const void *scales, const void *biases, const void *x,
                  void *const *outs, int n_outs, long long ld, int M, int N, int K, int bits, int group_size, int dtype);
int mtc_ipc_export(mtc_ctx *ctx, void *d_ptr, void *handle64);
int mtc_ipc_open(mtc_ctx *ctx, const void *handle64, void **d_ptr);
int mtc_ipc_close(mtc_ctx *ctx, void *d_ptr);
int mtc_peer_barrier(mtc_ctx *ctx, void *stream, void *const *peer_flags, int n_peers, int rank, void *local_flags,
                     void *epoch);

/* Tuning knobs of the back end, the counterpart of the reference's per-kernel MslConfig /
 * TileConfig switches (crates/metaltile-codegen/src/msl/config.rs:27-96,
 * crates/metaltile-core/src/toolchain/config.rs:11-96).  Options:
 *   "qmm_tile_tokens"  token rows per tensor-core work item (0 = chosen per shape; else a multiple
 *                      of 16 in [16, 256])
 *   "qmm_wait_hint_ns" suspend-time hint (ns) of the tensor-core kernel's waits that have slack: the TMA producer and the
 *                      epilogue warps (default 5000; 0 = plain polling)
 *   "qmv_small_m_mma"  0: keep 2 <= M <= 16 on the CUDA-core kernel (default 1: 4-bit codes with f16/bf16
 *                      activations and a group that is a multiple of 64 use the warp-level tensor cores);
 *                      2: M = 1 takes that path too (same results within round-off; not faster on B200)
 *   "qmm_mma_chunks"   0: 17 <= M <= 64 always runs on the tcgen05 kernel (default 1: 4-bit, f16/bf16, group >= 64
 *                      shapes run as 16-row chunks of the small-M tensor-core qmv when that fills the GPU better)
 *   "qmm_raw"          0: the dequant warps of the tensor-core kernel load packed words straight from global
 *                      memory instead of through the shared-memory staging buffers (default 1)
 *   "qmm_wide"         a dense work item of the tensor-core kernel covers two 256-row token chunks (one dequantised
 *                      weight stage meets two activation chunks; same results): 0 never, 1 (default) when that saves
 *                      rounds of the grid (M > 256), 2 whenever M > 256
 *   "qmm_ksplit"       0: a dense launch of the tensor-core kernel never cuts K into slices (default 1: with one token
 *                      chunk (M <= 256) and weight-row tiles for less than half of the SMs, K is cut into up to 16
 *                      slices that run as work items of their own; f32 partial sums in a context scratch block are
 *                      added in slice order by a second kernel - deterministic, same products)
 *   "qmv_small_m_tc"   2 <= M <= 16 on shapes the warp-level kernels do not take (other widths than 4-bit, group 32):
 *                      1 (default) 9 <= M <= 16, and 5 <= M <= 8 on matrices of 32 Mi codes or more, run on the
 *                      tensor-core kernel (f16 / bf16, K % 64 == 0, power-of-two group >= 32) instead of one FFMA per
 *                      (code, token) on CUDA cores; 0 never; 2 whenever that kernel takes the shape
 *   "qmv_stream"       the streaming decode kernel (4-bit, f16 / bf16, K % 512 == 0, group 64 or 128, 16-byte aligned
 *                      pointers): 1 (default) takes M = 1 - a single projection from 8 Mi codes on (below that the
 *                      CUDA-core kernel is faster), fused projections at any size; 2 takes every M <= 8 at any size
 *                      (slower than the register-ring kernel at M >= 2); 0 never.  mtc_qmv_batched fuses its projections into one launch where this kernel
 *                      takes them and launches them one by one otherwise
 *   "qmv_tc"           1: those shapes run on the tensor-memory decode kernel instead (slower today; default 0)
 *   "gather_stream"    0: grouped products never take the weight-streaming kernel (default 1: the CSR form with
 *                      4-bit codes, f16 / bf16, k_in % 256 == 0, group 64 or 128 and m_total <= 64 n_experts does)
 *   "pdl_early_weights" 0: no decode kernel reads w, scales or biases before the previous kernel of its stream is
 *                      complete.  Default 1: the decode kernels are launched with programmatic dependent launch and
 *                      start copying WEIGHTS while the previous kernel drains - weights are constants of the model;
 *                      a caller whose previous kernel on the stream WRITES them (an on-stream repack, dequant or
 *                      copy of the shard) must set this to 0 or synchronise first.  x and every store always wait.
 *   "peer_poll_limit"  polls of a wait on another GPU (mtc_peer_barrier, mtc_qmv_batched_sync) before it gives up
 *                      and records 0x601 + rank in the status word (default 4194304)
 * Scratch blocks.  bf16 mtc_qmm, mtc_gather_qmm, mtc_moe_experts and the tensor-memory decode kernel keep work lists
 * and staged activations in grow-only blocks of the context.  A block moves only outside stream capture (a call that
 * would have to grow one during capture fails with MTC_ERR_BUFFER: run the shape once before capturing), and an outgrown
 * block stays allocated until mtc_destroy, so graphs captured earlier and work already enqueued never see freed memory.
 * The blocks are per context, not per stream: calls of these entries from two streams that may overlap on the GPU race
 * on them - keep them on one stream, or order the streams with events, or use one context per stream. */
int mtc_set_option(mtc_ctx *ctx, const char *name, int value);

/* mt_moe_gather_qmm_int4 / _b{3,5,6,8} / _m8 / _m16 / _m32 (CSR form: expert_offsets u32[E+1],
 * crates/metaltile-std/src/ffai/moe.rs:358-433,461-605,634,900,1363) and mt_moe_gather_qmm_mma_*
 * (per-row form: indices u32[m_total], moe.rs:2256-2533,2552-2835): out[t, n] = sum_k x[t,k] * w(E(t), n, k).
 * x rows are sorted by expert; w is stacked u32[E, n_out, k_in*bits/32], scales/biases T[E, n_out, k_in/group].
 * Exactly one of expert_offsets / indices is non-NULL.  f16/bf16 activations with k_in % 64 == 0 and a
 * power-of-two group >= 32 run on the tensor cores (few rows per expert - see "gather_stream" - on the
 * weight-streaming kernel, else on the tensor-memory kernel), everything else on CUDA cores.  Offsets that reach
 * past m_total or run backwards are clamped (rows that do not exist are neither read nor written) and reported
 * through the status word (0x901). */
int mtc_gather_qmm(mtc_ctx *ctx, void *stream, const void *x, const void *w, const void *scales,
                   const void *biases, const void *expert_offsets, const void *indices, void *out,
                   int m_total, int n_out, int k_in, int n_experts, int bits, int group_size, int dtype);
/* mtc_gather_qmm without any allocation (no counterpart in the reference; added for hosts that may
 * not allocate device memory where they run a MoE layer: processes whose device memory is handed out
 * in full by their own allocator at start-up, and latency-critical loops that must not take the
 * allocator's lock or risk an out-of-memory error mid-step).  Same arguments and results as
 * mtc_gather_qmm on its tensor-core path; the work list and the f16 copy of bf16 activations live in one
 * fixed array inside the library image (about 17 MiB per GPU that loads the library, kept until exit).
 * Limits: at most 16384 work items (n_out/128 x (m_total/chunk + n_experts)); with bf16 activations
 * m_total * k_in <= 8 Mi elements and m_total <= 65536; f16 or bf16 only, k_in % 64 == 0, power-of-two
 * group >= 32.  Larger sizes return MTC_ERR_BUFFER_SIZE, other shapes MTC_ERR_UNSUPPORTED.  The first call on
 * a device looks up the array's device address (make it before any stream capture).  All calls share the
 * array: two calls that overlap on the GPU (different streams) race; calls on one stream are safe. */
int mtc_gather_qmm_static(mtc_ctx *ctx, void *stream, const void *x, const void *w, const void *scales,
                          const void *biases, const void *expert_offsets, const void *indices, void *out,
                          int m_total, int n_out, int k_in, int n_experts, int bits, int group_size, int dtype);
/* The expert MLP of a mixture-of-experts layer, rows sorted by expert - the stages the reference draws between
 * mt_moe_permute and mt_moe_unpermute (crates/metaltile-std/src/ffai/moe.rs:11-35) with mt_swiglu
 * (crates/metaltile-std/src/mlx/swiglu.rs:45-57) in the middle; the reference fuses the tail of it in
 * crates/metaltile-std/src/ffai/moe_down_swiglu_accum.rs:1-110:
 *     y[r, :] = down_e( silu(gate_e(x_r)) * up_e(x_r) ),   e = the expert that owns sorted row r (expert_offsets),
 *     x_r = x[sort_token_idx[r]] when sort_token_idx is given (x then has n_tokens rows), else x[r].
 * gate, up: [n_experts, inter, hidden*bits/32]; down: [n_experts, hidden, inter*bits/32]; y: [m_total, hidden].
 * The gate and up products and the SwiGLU are rounded to the activation type exactly as the separate entries
 * (mtc_moe_permute, mtc_gather_qmm twice, mtc_swiglu, mtc_gather_qmm) round them: same results bit for bit.
 * Few rows per expert (m_total <= 64 n_experts; 4-bit, f16 / bf16, group 64 / 128, hidden and inter multiples of 256):
 * four launches on the weight-streaming kernel - rows to MMA fragments with the permutation folded in, gate and up as
 * one stream over both matrices, SwiGLU to fragments, down.  Other shapes: composed from the separate entries.
 * The intermediates live in grow-only blocks of the context (they move only outside stream capture). */
typedef struct {
    const void *w, *scales, *biases;
} mtc_qmat;
int mtc_moe_experts(mtc_ctx *ctx, void *stream, const void *x, const void *sort_token_idx, int n_tokens, const mtc_qmat *gate,
                    const mtc_qmat *up, const mtc_qmat *down, const void *expert_offsets, void *y, int m_total, int hidden,
                    int inter, int n_experts, int bits, int group_size, int dtype);
const char *mtc_gather_qmm_route(int m_total, int n_out, int k_in, int n_experts, int bits, int group_size, int dtype);

/* mt_moe_router_topk (moe.rs:65-192): indices_out u32[n_rows, k], weights_out T[n_rows, k]; ties go to
 * the lower expert index, NaN never wins; norm_topk_prob 1 = softmax over the chosen k, 0 = chosen
 * probabilities of the softmax over all experts. */
int mtc_moe_router_topk(mtc_ctx *ctx, void *stream, const void *router_logits, void *indices_out,
                        void *weights_out, int n_rows, int n_experts, int k, int norm_topk_prob, int dtype);

/* The expert sort the reference leaves to its caller (contract: moe.rs:253-271,200-207,311-314).
 * Stable sort of flat slots f = token*k + slot by (expert[f], f): sort_token_idx u32[n_tokens*k]
 * (source token of permuted row p), inv_perm u32[n_tokens, k] (row of (token, slot)), expert_offsets
 * u32[n_experts+1] (CSR), row_expert u32[n_tokens*k] (expert of permuted row p; may be NULL). */
int mtc_moe_sort(mtc_ctx *ctx, void *stream, const void *topk_idx, int n_tokens, int k, int n_experts,
                 void *sort_token_idx, void *inv_perm, void *expert_offsets, void *row_expert);

/* mt_moe_permute (moe.rs:283-302): permuted[p, :] = tokens[sort_token_idx[p], :], bit-exact copy. */
int mtc_moe_permute(mtc_ctx *ctx, void *stream, const void *tokens, const void *sort_token_idx,
                    void *permuted, int n_rows, int hidden, int dtype);

/* mt_moe_unpermute (moe.rs:222-249): out[t, h] = sum_j top_k_weights[t, j] * expert_outputs[inv_perm[t, j], h],
 * f32 accumulate, j ascending. */
int mtc_moe_unpermute(mtc_ctx *ctx, void *stream, const void *expert_outputs, const void *inv_perm,
                      const void *top_k_weights, void *out, int n_tokens, int hidden, int k, int dtype);

/* mt_swiglu (crates/metaltile-std/src/mlx/swiglu.rs:45-57): out = silu(gate) * up, computed in f32. */
int mtc_swiglu(mtc_ctx *ctx, void *stream, const void *gate, const void *up, void *out, size_t n, int dtype);

/* Integer codes of a packed matrix, one byte per code, for bit-exact checks of
 * the unpacker against the oracle (no reference counterpart as a kernel; the
 * layout is quantized.rs:4296-4314 and :4354-4379). */
int mtc_unpack_codes(mtc_ctx *ctx, void *stream, const void *w, void *codes_u8, int N, int K,
                     int bits);

/* ---- name-keyed dispatch with HOST buffers: Context::dispatch_with_grid
 *      (crates/metaltile-runtime/src/context.rs:269-284) ----
 * `bufs` binds host byte buffers and 4-byte little-endian constexprs BY NAME
 * (run_kernel.rs:56-65,100-107).  Inputs are uploaded, the kernel selected by the
 * reference's kernel name (e.g. "mt_qmv", "mt_qmm_mma", "mt_qmv_b3",
 * "mt_moe_gather_qmm_int4") runs, and every buffer flagged is_output is copied back
 * into its host storage before the call returns (single_dispatch.rs:100-117).
 * grid / tpg are accepted for signature parity and ignored: launch geometry
 * belongs to the back end.  elapsed_us (may be NULL) receives the device time
 * of the kernel alone, like DispatchResult::elapsed_us (single_dispatch.rs:119). */
typedef struct {
    const char *name;
    void *data;      /* host pointer */
    size_t bytes;
    int is_output;   /* 1: copied back after the kernel */
} mtc_named_buf;

int mtc_dispatch(mtc_ctx *ctx, const char *kernel_name, int dtype, mtc_named_buf *bufs, int n_bufs,
                 const uint32_t grid[3], const uint32_t tpg[3], float *elapsed_us);
/* Several passes committed together - Context::dispatch_chain (crates/metaltile-runtime/src/context.rs:347-395):
 * the passes run in order on the device with no host round trip between them.  A buffer that pass i marks is_output
 * and that a later pass binds under the same name as an input stays on the device (the later pass's host bytes for it
 * are ignored); only outputs that no later pass consumed are copied back, after the last pass, with one
 * synchronisation.  Every pass is checked (names, constexprs, sizes) before anything is enqueued.  elapsed_us (may be
 * NULL): device time of the whole chain.  Errors as mtc_dispatch. */
typedef struct {
    const char *kernel_name;
    int dtype;
    mtc_named_buf *bufs;
    int n_bufs;
} mtc_dispatch_spec;
int mtc_dispatch_chain(mtc_ctx *ctx, const mtc_dispatch_spec *specs, int n_specs, float *elapsed_us);

/* Timed repetitions of one kernel - GpuRunner::measure / GpuRunner::bench / bench_gbps
 * (crates/metaltile-std/src/runner.rs:413-442,638-650) with the summary of BenchStats::from_samples
 * (crates/metaltile-std/src/stats.rs:5-47).  The buffers are bound by name as for mtc_dispatch and staged on the
 * device ONCE by an untimed first launch; then `warmup` untimed and `iters` timed launches run, each timed launch
 * between its own pair of events (device time of the kernel alone, no copies).  cold_l2 != 0 rewrites a 256 MiB block
 * (twice the L2) before every launch, outside the timed pair - the counterpart of GpuRunner::flush_slc
 * (runner.rs:444-458).  samples_us (may be NULL) receives the `iters` samples in launch order; stats (may be NULL) the
 * summary: sorted samples, median = s[n/2], p95 = s[n*95/100], p99 = s[n*99/100], population standard deviation,
 * cv_pct = stddev / mean * 100.  Buffers flagged is_output hold the last launch's result when the call returns. */
typedef struct {
    double min_us, mean_us, median_us, p95_us, p99_us, stddev_us, cv_pct;
    int iters;
} mtc_bench_stats;
int mtc_measure(mtc_ctx *ctx, const char *kernel_name, int dtype, mtc_named_buf *bufs, int n_bufs, int warmup, int iters,
                int cold_l2, double *samples_us, mtc_bench_stats *stats);
/* Number of kernel names mtc_dispatch knows, and the i-th name (registry walk:
 * all_kernels(), crates/metaltile-core/src/toolchain/registry.rs:56-78). */
int mtc_kernel_count(void);
const char *mtc_kernel_name(int i);

#ifdef __cplusplus
}
#endif
#endif /* MTCUDA_H */
