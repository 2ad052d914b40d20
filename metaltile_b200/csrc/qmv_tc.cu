// qmv_tc — decode-time quantized matrix-vector products (M <= 8 token rows, 4-bit codes, 16-bit activations) on the
// sm_100a tensor cores with the packed codes themselves as the A operand in tensor memory.
//
//   out[m, n] = sum_k (q(n,k) * scale[n, k/G] + bias[n, k/G]) * x[m, k]                 (f32 accumulate)
//
// Stands in for mt_qmv / mt_qmm{,_bm2,_bm4} / mt_qmv_b4 (crates/metaltile-std/src/mlx/quantized.rs:7-308,343-1441,
// 4273-4392).
//
// Why.  A decode projection is a weight stream: what limits it on B200 is not HBM but the instructions spent per
// byte.  With warp-level MMAs every lane has to build operand fragments and apply the group's scale and bias
// (about 80 issued instructions per 1024 codes, measured); here a thread only masks nibbles:
//   * a 16-bit float whose exponent field is 0 or 1 is linear in its low 8 bits (the subnormals and the first
//     binade form one ramp): value = bits * 2^-24 (f16) or bits * 2^-133 (bf16).  `w & 0x000F000F` is therefore two
//     ready operands (q0, q4) * c, `w & 0x00F000F0` two operands 16 * (q1, q5) * c, and one shift by 8 gives the other
//     four nibbles: 5 integer instructions per 8 codes, no conversion;
//   * thread r of a 128-row tile owns weight row r: it reads its packed words from a swizzled shared-memory copy,
//     masks them and writes the 16-bit pairs straight into its own lane of tensor memory (tcgen05.st) - 32 columns
//     per 64 codes;
//   * one thread issues tcgen05.mma (M = 128 rows, N = 16 token columns, K = 16) with A from tensor memory and the
//     activations (staged once per K chunk in the matching k order, 128-byte swizzle) from shared memory; every
//     quantization group gets its own 16 accumulator columns, so the group's scale is applied once per (row, group)
//     when an epilogue warp reads them back:  acc += scale * D_g + bias * sum_g(x);
//   * the nibbles at bits 4-7 carry a factor 16 which their activations are staged without; bf16 activations are
//     staged times 2^64 so that products stay normal f32 numbers (exact; |x| < 2^59 required).
// The row tiles are few (N / 128), so K is split over CTAs as well: a work item is (row tile, K chunk of 256 codes),
// items are tile-major and dealt in contiguous ranges to one persistent CTA per SM, so the chunks of a tile are
// consecutive items whose sums stay in the epilogue warp's registers; only the tiles at the ends of a CTA's range are
// shared with a neighbour: those sums go to a scratch plane and the last CTA to arrive adds the planes of the tile in
// chunk order (deterministic).
//
// Roles in a CTA of 28 warps: 16 mask warps (two slices that take alternate items and own four tensor-memory stages
// each - every barrier is visited by the same warps in every phase, which a parity wait needs; per slice 4 lane
// quarters x 2 halves of every 64-code block; the two halves share a cp.async ring of packed words, up to three
// items ahead); 4 epilogue warps (one per lane quarter; scales and biases requested three items ahead); 4 MMA issuers
// (two per slice, two blocks each, issued interleaved because an MMA that adds to the accumulator of the one before it
// waits out the whole pipeline, ~120 cycles at N = 16); 4 warps that copy an item's activations, converted once per
// CTA, into the swizzled operand buffers.  Every wait is bounded: on expiry the status word gets 0x8xx, all roles
// leave their loops, tensor memory is released and the kernel returns.
//
// State (B200, 4-bit g64 bf16, graph replay): M = 1, 14336 x 4096: 20 us against 12.6 us of the warp-level MMA stream
// kernel (qmv_stream.cu); the masking warps need ~4000 cycles per item and pair of warps where ~800 would keep up with
// HBM.  It is therefore off by default (option "qmv_tc").
#include "common.cuh"

namespace mtc {
namespace {

constexpr int kMaskWarps = 16;
constexpr int kEpiWarp0 = 16, kMmaWarp0 = 20, kAuxWarp = 24;    // MMA issuers: warps 20..23; activation stagers: warps 24..27
constexpr int kTcThreads = 28 * 32;
constexpr int kStages = 8;                    // A-operand stages in tensor memory, 32 columns (64 codes) each
constexpr int kACol0 = 256;                   // A ring: columns 256..511; accumulators: 4 x 64 columns from 0
constexpr int kDBufs = 4;                     // accumulator buffers (items the MMAs may run ahead of the epilogue)
constexpr int kDBuf = 64;                     // accumulator columns per buffer: 4 groups x 16 token columns
constexpr int kSbBytes = 32 * 128;            // a super-block of one lane quarter: 32 rows x 128 bytes (256 codes)
constexpr int kMaxAhead = 3;                  // packed words: up to three super-blocks ahead (ring depth = ahead + 2: one in use, one the partner warp may still read)
constexpr uint32_t kTcSpin = 1u << 22;
constexpr int kMaxKbPerChunk = 4;             // K chunk = 256 codes: one super-block per item
constexpr int kBBufs = 4;                     // staged activation chunks in flight (one per item when K is split)

struct TcArgs {
    const uint32_t *w;
    const void *scales, *biases, *x;
    void *out[8];
    int n_out;
    int M, N, K;
    int gsh;                 // log2(group / 64): 0 or 1
    int rowbytes, gpr;       // K / 2, K / group
    int kb_per_chunk;        // 64-code blocks per K chunk: 4 or 8
    int chunks, tiles;       // K / chunk, ceil(N / 128)
    int items;               // chunks * tiles, chunk-major: id = chunk * tiles + tile
    float *scratch;          // [chunks][M][N] partial sums (chunks > 1)
    uint32_t *counters;      // [tiles * 4] arrivals per (tile, lane quarter), zero between launches
    uint32_t *status;
    uint32_t idesc;
    int early_weights;
    int bf16;
    uint32_t off_p, off_ring;    // shared-memory layout after the sums
    int ahead;                   // super-blocks of packed words requested ahead per pair of mask warps: 1..3
};

struct __align__(8) TcCtl {
    uint64_t full_a[kStages], empty_a[kStages];
    uint64_t acc_full[kDBufs], acc_empty[kDBufs];
    uint64_t b_full[kBBufs], b_empty[kBBufs];
    uint32_t tmem_base;
    volatile uint32_t abort;
};

constexpr uint32_t kOffB = 1024;                                   // activations: kBBufs buffers x 8 blocks x 2 KB
constexpr uint32_t kOffXs = kOffB + kBBufs * kMaxKbPerChunk * 2048;      // sums of x per (64-code block, token): K / 64 x 8 floats
constexpr size_t kTcSmemMax = 226 * 1024;
// then: the activations of the whole K extent in operand order (off_p: M x K x 2 bytes), then the rings (off_ring)

__device__ __forceinline__ uint32_t su32(const void *p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void mb_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(su32(bar)), "r"(count));
}
__device__ __forceinline__ void mb_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(su32(bar)) : "memory");
}
__device__ __forceinline__ bool mb_try(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(su32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait; false (with the CTA's abort flag and the status word raised) when it expires or another role gave up.
// `sleep_ns` > 0: the thread sleeps between polls.  A spinning try_wait is a shared-memory-pipe instruction: a dozen
// roles polling at full rate delay the loads, tensor-memory stores and arrivals of the warps that do the work.
__device__ __forceinline__ bool mb_wait(uint64_t *bar, uint32_t parity, TcCtl *ctl, uint32_t *status, uint32_t code,
                                        uint32_t sleep_ns = 0) {
    for (uint32_t i = 0; i < kTcSpin; ++i) {
        if (mb_try(bar, parity)) {
            return true;
        }
        if (sleep_ns) __nanosleep(sleep_ns);
        if ((i & 63u) == 63u && ctl->abort) return false;
    }
    ctl->abort = 1u;
    atomicCAS(status, 0u, code);
    return false;
}
__device__ __forceinline__ bool mb_wait_warp(uint64_t *bar, uint32_t parity, TcCtl *ctl, uint32_t *status, uint32_t code,
                                             uint32_t sleep_ns = 0) {
    uint32_t ok = 1;
    if ((threadIdx.x & 31) == 0) ok = mb_wait(bar, parity, ctl, status, code, sleep_ns) ? 1u : 0u;
    return __shfl_sync(0xffffffffu, ok, 0) != 0;
}
__device__ __forceinline__ bool elect_one_tc() {
    uint32_t pred;
    asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
    return pred != 0;
}
__device__ __forceinline__ void tc_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(su32(bar)) : "memory");
}
// A operand from tensor memory (8 columns per K = 16), B operand from shared memory
__device__ __forceinline__ void umma_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tm_st16(uint32_t taddr, const uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
          "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]) : "memory");
}
__device__ __forceinline__ void tm_ld8(uint32_t taddr, uint32_t (&v)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]) : "r"(taddr));
}
__device__ __forceinline__ void tm_ld1(uint32_t taddr, uint32_t &v) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x1.b32 {%0}, [%1];" : "=r"(v) : "r"(taddr));
}
__device__ __forceinline__ void tm_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tm_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor: K-major operand, 128-byte swizzle, 8-row atoms 1024 bytes apart.
__device__ __forceinline__ uint64_t desc_sw128(uint32_t saddr) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4);
    d |= static_cast<uint64_t>(1) << 16;
    d |= static_cast<uint64_t>(1024 >> 4) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(2) << 61;
    return d;
}
__device__ __forceinline__ void cpa16(uint32_t dst, const void *src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}

template <bool BF16>
__device__ __forceinline__ float half_to_f32(uint32_t bits16) {
    if (BF16) return __uint_as_float(bits16 << 16);
    return __half2float(__ushort_as_half(static_cast<unsigned short>(bits16)));
}

// item id -> (tile, chunk): items are tile-major, so the chunks of a row tile are consecutive items of (mostly) one CTA
// and their partial sums stay in the epilogue warp's registers
__device__ __forceinline__ void item_of(const TcArgs &a, int id, int &chunk, int &tile) {
    tile = id / a.chunks;
    chunk = id - tile * a.chunks;
}

template <bool BF16, bool M1>
__global__ void __launch_bounds__(kTcThreads, 1) qmv_tc_kernel(const __grid_constant__ TcArgs a) {
    extern __shared__ __align__(1024) unsigned char sm[];
    TcCtl *ctl = reinterpret_cast<TcCtl *>(sm);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int KB = a.kb_per_chunk;                 // 64-code blocks per item
    const int SBI = KB >> 2;                       // super-blocks per item: 1 or 2
    const int id0 = static_cast<int>(static_cast<long long>(a.items) * blockIdx.x / gridDim.x);
    const int id1 = static_cast<int>(static_cast<long long>(a.items) * (blockIdx.x + 1) / gridDim.x);
    const int n_items = id1 - id0;

    asm volatile("griddepcontrol.launch_dependents;");
    if (threadIdx.x == 0) {
        for (int s = 0; s < 2; ++s) {              // one pair of barriers per slice: its four stages are handed over together
            mb_init(&ctl->full_a[s], 8);           // four lane quarters x two 32-code halves
            mb_init(&ctl->empty_a[s], 2);          // one tcgen05.commit per MMA issuer of the slice
        }
        for (int b = 0; b < kDBufs; ++b) {
            mb_init(&ctl->acc_full[b], 2);         // one tcgen05.commit per MMA issuer of the item's slice
            mb_init(&ctl->acc_empty[b], 4);        // the four epilogue warps
        }
        for (int b = 0; b < kBBufs; ++b) {
            mb_init(&ctl->b_full[b], 1);
            mb_init(&ctl->b_empty[b], 2);          // one tcgen05.commit per MMA issuer of the item's slice
        }
        ctl->abort = 0u;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == kAuxWarp) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(su32(&ctl->tmem_base)), "r"(512));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
    }
    tc_before();
    __syncthreads();
    tc_after();
    const uint32_t tmem_base = ctl->tmem_base;

    if (warp >= kMaskWarps) {
        // ---------------- once per CTA: the activations in operand order (the mask warps are already copying weights) ----
        // 16 codes -> 16 k slots [0, 4, 1, 5, 2, 6, 3, 7] then the same + 8, slots 2, 3, 6, 7 of each 8 holding x / 16
        // (their codes arrive as 16 q); bf16 values times 2^64.  P[m][k]: 2 bytes per slot; xs[block][m]: the plain sum
        // of the block's 64 activations (f32).
        asm volatile("griddepcontrol.wait;" ::: "memory");
        const int tid = threadIdx.x - kMaskWarps * 32, nthr = kTcThreads - kMaskWarps * 32;
        for (uint32_t i = tid; i < kBBufs * kMaxKbPerChunk * 2048 / 16; i += nthr)        // token rows >= M stay zero
            reinterpret_cast<uint4 *>(sm + kOffB)[i] = make_uint4(0u, 0u, 0u, 0u);
        float *xs = reinterpret_cast<float *>(sm + kOffXs);
        unsigned char *P = sm + a.off_p;
        const int upr = a.K >> 4;                       // 16-code units per token row
        const int units = a.M * upr;
        for (int u0 = 0; u0 < units; u0 += nthr) {      // whole warps stay in the loop: the sums use shuffles
            const int u = u0 + tid;
            const bool on = u < units;
            const int m = on ? u / upr : 0, ur = on ? u - m * upr : 0;      // token, unit within the row (block ur >> 2, sub-block ur & 3)
            uint4 v0 = make_uint4(0u, 0u, 0u, 0u), v1 = v0;
            if (on) {
                const uint4 *src = reinterpret_cast<const uint4 *>(static_cast<const uint16_t *>(a.x) + static_cast<size_t>(m) * a.K + ur * 16);
                v0 = __ldg(src);
                v1 = __ldg(src + 1);
            }
            const uint32_t uw[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};   // word i: codes 2i, 2i+1
            uint32_t e[8], o[8];
            float sum = 0.0f;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                if (BF16) {
                    const float lo = __uint_as_float(uw[i] << 16), hi = __uint_as_float(uw[i] & 0xFFFF0000u);
                    sum += lo + hi;
                    e[i] = (__float_as_uint(lo * 18446744073709551616.0f) >> 16) | (__float_as_uint(hi * 18446744073709551616.0f) & 0xFFFF0000u);
                    o[i] = (__float_as_uint(lo * 1152921504606846976.0f) >> 16) | (__float_as_uint(hi * 1152921504606846976.0f) & 0xFFFF0000u);
                } else {
                    const __half2 h2 = *reinterpret_cast<const __half2 *>(&uw[i]);
                    const float2 f = __half22float2(h2);
                    sum += f.x + f.y;
                    e[i] = uw[i];
                    const __half2 sc = __hmul2(h2, __float2half2_rn(0.0625f));
                    o[i] = *reinterpret_cast<const uint32_t *>(&sc);
                }
            }
            // the four sub-blocks of a 64-code block sit in four neighbouring lanes (K / 16 is a multiple of 4)
            sum += __shfl_xor_sync(0xffffffffu, sum, 1);
            sum += __shfl_xor_sync(0xffffffffu, sum, 2);
            if (on) {
                // slots (0,4) (1,5)/16 (2,6) (3,7)/16 of codes 0..7: code c is the (c & 1) half of word c >> 1
                uint4 *dst = reinterpret_cast<uint4 *>(P + (static_cast<size_t>(m) * a.K + ur * 16) * 2);
                dst[0] = make_uint4(__byte_perm(e[0], e[2], 0x5410), __byte_perm(o[0], o[2], 0x7632),
                                    __byte_perm(e[1], e[3], 0x5410), __byte_perm(o[1], o[3], 0x7632));
                dst[1] = make_uint4(__byte_perm(e[4], e[6], 0x5410), __byte_perm(o[4], o[6], 0x7632),
                                    __byte_perm(e[5], e[7], 0x5410), __byte_perm(o[5], o[7], 0x7632));
                if ((ur & 3) == 0) xs[(ur >> 2) * 8 + m] = sum;
            }
        }
        asm volatile("bar.sync 9, %0;" ::"n"(kTcThreads - kMaskWarps * 32) : "memory");
    }

    if (warp < kMaskWarps) {
        // ---------------- mask warps: packed words -> A operand in tensor memory ----------------
        // warp = 8 sl + 4 hh + q: slice sl takes the super-blocks n = sl, sl + 2, ... of this CTA and owns the stages
        // 4 sl .. 4 sl + 3 (one per 64-code block of a super-block), so every barrier of a stage is visited by the same
        // warps in every phase; q is the lane quarter (32 weight rows), hh the 32-code half of each block.
        const int q = warp & 3, hh = (warp >> 2) & 1, sl = warp >> 3;
        const int pair = sl * 4 + q;                  // the two warps (hh = 0, 1) of a pair share one ring of packed words
        const int ahead = a.ahead, depth = ahead + 2;
        unsigned char *ring_p = sm + a.off_ring + static_cast<size_t>(pair) * depth * kSbBytes;
        const uint32_t ring = su32(ring_p);
        const int total_sb = n_items * SBI;        // super-blocks of this CTA, in item order
        // copy side: each warp of the pair copies 16 of the 32 rows: lane -> row 16 hh + 4 i + (lane >> 3), 16-byte
        // chunk lane & 7 (stored at chunk ^ (row & 7))
        auto issue = [&](int n, int slot) {
            const int it = SBI == 2 ? (n >> 1) : n, sbi = n - it * SBI;
            int chunk, tile;
            item_of(a, id0 + it, chunk, tile);
            const int crow = 16 * hh + (lane >> 3), cch = lane & 7;
            const char *src = reinterpret_cast<const char *>(a.w) + static_cast<size_t>(chunk * KB + sbi * 4) * 32 + cch * 16;
            const uint32_t dst = ring + slot * kSbBytes;
            const int row0 = tile * 128 + q * 32;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int r = 4 * i + crow;
                const int grow = min(row0 + r, a.N - 1);                 // rows past N re-read the last row
                cpa16(dst + r * 128 + ((cch ^ (r & 7)) << 4), src + static_cast<size_t>(grow) * a.rowbytes);
            }
        };
        if (!a.early_weights) asm volatile("griddepcontrol.wait;" ::: "memory");
        int n_issue = sl;
#pragma unroll 1
        for (int p = 0; p < ahead; ++p) {
            if (n_issue < total_sb) issue(n_issue, p);
            asm volatile("cp.async.commit_group;" ::: "memory");
            n_issue += 2;
        }
        int slot = 0;
        constexpr uint32_t m0 = 0x000F000Fu, m1 = 0x00F000F0u;
        const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + kACol0 + sl * 128 + hh * 16;
        bool ok = true;
        uint32_t use = 0;                             // uses of this slice's stages so far
        for (int n = sl; n < total_sb; n += 2, ++use) {       // a warp that gave up keeps meeting its partner at the barrier
            // the slot about to be refilled was read two super-blocks ago, before the pair's last barrier
            int islot = slot + ahead >= depth ? slot + ahead - depth : slot + ahead;
            if (n_issue < total_sb) issue(n_issue, islot);
            asm volatile("cp.async.commit_group;" ::: "memory");
            n_issue += 2;
            if (ahead == 3) asm volatile("cp.async.wait_group 3;" ::: "memory");
            else if (ahead == 2) asm volatile("cp.async.wait_group 2;" ::: "memory");
            else asm volatile("cp.async.wait_group 1;" ::: "memory");
            asm volatile("bar.sync %0, 64;" ::"r"(1 + pair) : "memory");   // both halves of the rows have landed
            const unsigned char *raw = ring_p + slot * kSbBytes + lane * 128;
            // the slice's four stages are free once the MMAs of its previous super-block have completed
            if (ok && use > 0) ok = mb_wait_warp(&ctl->empty_a[sl], (use & 1) ^ 1, ctl, a.status, 0x801);
            if (ok) {
                tc_after();
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const uint4 wv = *reinterpret_cast<const uint4 *>(raw + (((2 * j + hh) ^ (lane & 7)) << 4));
                    const uint32_t wd[4] = {wv.x, wv.y, wv.z, wv.w};
                    uint32_t v[16];
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const uint32_t s8 = wd[i] >> 8;
                        v[4 * i + 0] = wd[i] & m0;         // codes 0, 4 of the word
                        v[4 * i + 1] = wd[i] & m1;         // 16 x codes 1, 5
                        v[4 * i + 2] = s8 & m0;            // codes 2, 6
                        v[4 * i + 3] = s8 & m1;            // 16 x codes 3, 7
                    }
                    tm_st16(lane_addr + j * 32, v);
                }
                tm_wait_st();                              // one wait and one hand-over for the four blocks
                tc_before();
                __syncwarp();
                if (lane == 0) mb_arrive(&ctl->full_a[sl]);
            }
            slot = slot + 1 == depth ? 0 : slot + 1;
        }
        asm volatile("cp.async.wait_group 0;" ::: "memory");
    } else if (warp >= kMmaWarp0 && warp < kMmaWarp0 + 4) {
        // ---------------- MMA issuers ----------------
        // Two issuers per slice, each with two of the four 64-code blocks of the slice's super-blocks.  A block is 4
        // MMAs (K = 16 each) into its own 16 accumulator columns, and an MMA that adds to the accumulator of the one
        // before it waits out the whole pipeline (~120 cycles at N = 16, measured): so the two blocks are issued
        // interleaved, and four issuers keep eight independent chains in flight.  Every barrier an issuer waits on is
        // one it visits in every phase (its slice's stages, the accumulator buffers of its slice's items).  The whole
        // warp runs the loop (addresses stay warp-uniform); one elected lane issues.
        const int sl = (warp - kMmaWarp0) >> 1, j0 = ((warp - kMmaWarp0) & 1) * 2;
        const bool split = a.chunks > 1;           // K is split: every item has its own activation buffer
        bool ok = true;
        for (int it = sl; it < n_items && ok; it += 2) {
            const int bsel = split ? (it & (kBBufs - 1)) : 0;
            if ((split || it < 2) && !(ok = mb_wait_warp(&ctl->b_full[bsel], split ? (it / kBBufs) & 1 : 0, ctl, a.status, 0x811, 100))) break;
            const int buf = it & (kDBufs - 1);
            if (it >= kDBufs && !(ok = mb_wait_warp(&ctl->acc_empty[buf], ((it / kDBufs) & 1) ^ 1, ctl, a.status, 0x812, 100))) break;
            const int st = sl * 4 + j0;             // this slice's use it >> 1 of its stages
            if (!(ok = mb_wait_warp(&ctl->full_a[sl], (it >> 1) & 1, ctl, a.status, 0x813, 40))) break;
            tc_after();
            const uint32_t ta = tmem_base + kACol0 + st * 32;
            const uint64_t bd = desc_sw128(su32(sm + kOffB + (bsel * kMaxKbPerChunk + j0) * 2048));
            const uint32_t dg = tmem_base + buf * kDBuf + j0 * 16;
            if (elect_one_tc()) {
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    umma_ts(dg, ta + 8 * k, bd + 2 * k, a.idesc, k ? 1u : 0u);
                    umma_ts(dg + 16, ta + 32 + 8 * k, bd + 128 + 2 * k, a.idesc, k ? 1u : 0u);   // the next block: 2048 bytes on
                }
                tc_commit(&ctl->empty_a[sl]);
                if (split) tc_commit(&ctl->b_empty[bsel]);      // the activation buffer may be refilled once these MMAs are done
                tc_commit(&ctl->acc_full[buf]);
            }
            __syncwarp();
        }
    } else if (warp >= kAuxWarp) {
        // ---------------- activations of an item -> B operand buffer ----------------
        // The activations were converted once (prestage_x); an item needs 4 blocks x 128 bytes per token copied
        // into rows 0..M-1 of the buffer's 128-byte-swizzled blocks.  Stager k owns buffer k and the items k, k + 4, ...;
        // when K is not split, stager 0 fills buffer 0 once.
        const int k = warp - kAuxWarp;
        const bool split = a.chunks > 1;
        unsigned char *bb = sm + kOffB + k * kMaxKbPerChunk * 2048;
        const unsigned char *P = sm + a.off_p;
        const int c16 = lane & 7, kb = lane >> 3;          // 16-byte chunk of a block row, block
        bool ok = true;
        const int last = split ? n_items : (k == 0 && n_items > 0 ? 1 : 0);
        for (int it = k, use = 0; it < last && ok; it += 4, ++use) {
            const int chunk = (id0 + it) % a.chunks;
            if (use > 0 && !(ok = mb_wait_warp(&ctl->b_empty[k], (use & 1) ^ 1, ctl, a.status, 0x821, 400))) break;
            for (int m = 0; m < a.M; ++m) {
                const uint4 v = *reinterpret_cast<const uint4 *>(P + (static_cast<size_t>(m) * a.K + (chunk * 4 + kb) * 64) * 2 + c16 * 16);
                *reinterpret_cast<uint4 *>(bb + kb * 2048 + m * 128 + ((c16 ^ (m & 7)) << 4)) = v;
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy stores -> async proxy (MMA)
            __syncwarp();
            if (lane == 0) mb_arrive(&ctl->b_full[k]);
        }
    } else if (warp >= kEpiWarp0 && warp < kEpiWarp0 + 4) {
        // ---------------- epilogue: accumulators of every group -> scale, bias, partial sums ----------------
        const int q = warp - kEpiWarp0;
        asm volatile("griddepcontrol.wait;" ::: "memory");
        bool ok = true;
        const int ngrp = KB >> a.gsh;                     // groups per item
        constexpr int MT = M1 ? 1 : 8;
        float acc[MT];
#pragma unroll
        for (int m = 0; m < MT; ++m) acc[m] = 0.0f;
        int run_c0 = 0;
        // scales and biases (4 or 2 groups x 2 bytes per row and item): loaded three items ahead of their use
        auto load_sb = [&](int it, uint2 &sv, uint2 &bv) {
            sv = make_uint2(0u, 0u);
            bv = sv;
            if (it >= n_items) return;
            int chunk, tile;
            item_of(a, id0 + it, chunk, tile);
            const int nr = min(tile * 128 + q * 32 + lane, a.N - 1);
            const uint16_t *sp = static_cast<const uint16_t *>(a.scales) + static_cast<size_t>(nr) * a.gpr + chunk * ngrp;
            const uint16_t *bp = static_cast<const uint16_t *>(a.biases) + static_cast<size_t>(nr) * a.gpr + chunk * ngrp;
            if (ngrp == 4) {
                sv = __ldg(reinterpret_cast<const uint2 *>(sp));
                bv = __ldg(reinterpret_cast<const uint2 *>(bp));
            } else {
                sv.x = __ldg(reinterpret_cast<const uint32_t *>(sp));
                bv.x = __ldg(reinterpret_cast<const uint32_t *>(bp));
            }
        };
        uint2 pf_s[3], pf_b[3];
        load_sb(0, pf_s[0], pf_b[0]);
        load_sb(1, pf_s[1], pf_b[1]);
        load_sb(2, pf_s[2], pf_b[2]);
        for (int it = 0; it < n_items && ok; ++it) {
            int chunk, tile;
            item_of(a, id0 + it, chunk, tile);
            const int buf = it & (kDBufs - 1);
            const int n = tile * 128 + q * 32 + lane;     // weight row == output column of this thread
            // scales and biases of this row for the groups of this item were requested three items ago
            const uint2 sw2 = pf_s[0], bw2 = pf_b[0];
            pf_s[0] = pf_s[1]; pf_b[0] = pf_b[1];
            pf_s[1] = pf_s[2]; pf_b[1] = pf_b[2];
            load_sb(it + 3, pf_s[2], pf_b[2]);
            const uint32_t sw[2] = {sw2.x, sw2.y}, bw[2] = {bw2.x, bw2.y};
            if (!(ok = mb_wait_warp(&ctl->acc_full[buf], (it / kDBufs) & 1, ctl, a.status, 0x831, 100))) break;
            tc_after();
            const float *xs = reinterpret_cast<const float *>(sm + kOffXs) + chunk * 4 * 8;      // sums of x of this item's 4 blocks
            const uint32_t t0 = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * kDBuf;
            // a run = the consecutive chunks of one row tile that this CTA owns: its sums stay in registers
            if (it == 0 || chunk == 0) {
                run_c0 = chunk;
#pragma unroll
                for (int m = 0; m < MT; ++m) acc[m] = 0.0f;
            }
            uint32_t d[4][MT];                        // one accumulator per 64-code block
#pragma unroll
            for (int kb = 0; kb < 4; ++kb) {
                if constexpr (M1) tm_ld1(t0 + kb * 16, d[kb][0]);
                else tm_ld8(t0 + kb * 16, d[kb]);
            }
            tm_wait_ld();
            tc_before();
            __syncwarp();
            if (lane == 0) mb_arrive(&ctl->acc_empty[buf]);   // the accumulators are in registers: the buffer may be rewritten
#pragma unroll
            for (int kb = 0; kb < 4; ++kb) {
                const int g = kb >> a.gsh;               // the block's group within the item
                const uint32_t s16 = (g & 1) ? (sw[g >> 1] >> 16) : (sw[g >> 1] & 0xFFFFu);
                const uint32_t b16 = (g & 1) ? (bw[g >> 1] >> 16) : (bw[g >> 1] & 0xFFFFu);
                const float sc = half_to_f32<BF16>(s16), bi = half_to_f32<BF16>(b16);
                // c * 2^(pre-scale) leaves here: f16 codes are q * 2^-24; bf16 codes q * 2^-133 against x * 2^64
                const float scp = sc * (BF16 ? 5.9029581035870565e20f /* 2^69 */ : 16777216.0f /* 2^24 */);
#pragma unroll
                for (int m = 0; m < MT; ++m) acc[m] = fmaf(scp, __uint_as_float(d[kb][m]), fmaf(bi, xs[kb * 8 + m], acc[m]));
            }
            if (chunk != a.chunks - 1 && it != n_items - 1) continue;          // the run goes on
            const int dt = BF16 ? MTC_BF16 : MTC_F16;
            if (run_c0 == 0 && chunk == a.chunks - 1) {
                // the whole K extent of this tile was this CTA's: store
                if (n < a.N) {
#pragma unroll
                    for (int m = 0; m < MT; ++m)
                        if (m < a.M)
                            for (int o = 0; o < a.n_out; ++o) st_from_f32(a.out[o], static_cast<size_t>(m) * a.N + n, acc[m], dt);
                }
            } else {
                // the tile is shared with neighbouring CTAs: this run's sums go to the plane of its first chunk; the last
                // run to arrive adds the runs of the tile in chunk order and stores
                if (n < a.N) {
#pragma unroll
                    for (int m = 0; m < MT; ++m)
                        if (m < a.M) a.scratch[(static_cast<size_t>(run_c0) * a.M + m) * a.N + n] = acc[m];
                }
                // CTA b owns the items [items * b / grid, items * (b + 1) / grid): the owner of item id is
                // floor(((id + 1) * grid - 1) / items)
                const long long G = gridDim.x, I = a.items;
                const long long first_id = static_cast<long long>(tile) * a.chunks;
                const int b_first = static_cast<int>(((first_id + 1) * G - 1) / I);
                const int b_last = static_cast<int>(((first_id + a.chunks) * G - 1) / I);
                __syncwarp();
                uint32_t old = 0;
                if (lane == 0) {
                    __threadfence();
                    old = atomicAdd(a.counters + tile * 4 + q, 1u);
                }
                old = __shfl_sync(0xffffffffu, old, 0);
                if (old == static_cast<uint32_t>(b_last - b_first)) {
                    __threadfence();
                    if (n < a.N) {
                        float v[MT];
#pragma unroll
                        for (int m = 0; m < MT; ++m) v[m] = 0.0f;
                        for (int b = b_first; b <= b_last; ++b) {
                            const long long s0 = I * b / G;
                            const int c0 = static_cast<int>(s0 > first_id ? s0 - first_id : 0);    // first chunk of b's run
#pragma unroll
                            for (int m = 0; m < MT; ++m)
                                if (m < a.M) v[m] += __ldcg(a.scratch + (static_cast<size_t>(c0) * a.M + m) * a.N + n);
                        }
#pragma unroll
                        for (int m = 0; m < MT; ++m)
                            if (m < a.M)
                                for (int o = 0; o < a.n_out; ++o) st_from_f32(a.out[o], static_cast<size_t>(m) * a.N + n, v[m], dt);
                    }
                    if (lane == 0) a.counters[tile * 4 + q] = 0u;      // ready for the next launch
                }
            }
        }
    }

    tc_before();
    __syncthreads();
    if (warp == kAuxWarp) {
        tc_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512));
    }
}

// Shared memory after the operand buffers: sums (K / 64 x 8 floats), activations in operand order (M x K x 2 bytes),
// then the rings of the 8 mask-warp pairs, as deep as fits (1 to 3 super-blocks ahead).  false: the activations do not fit.
bool tc_layout(int M, int K, uint32_t &off_p, uint32_t &off_ring, int &ahead, size_t &smem) {
    const size_t xs = (static_cast<size_t>(K / 64) * 8 * 4 + 127) / 128 * 128;
    const size_t pb = (static_cast<size_t>(M) * K * 2 + 127) / 128 * 128;
    off_p = static_cast<uint32_t>(kOffXs + xs);
    off_ring = static_cast<uint32_t>(off_p + pb);
    for (ahead = kMaxAhead; ahead >= 1; --ahead) {
        smem = off_ring + static_cast<size_t>(kMaskWarps / 2) * (ahead + 2) * kSbBytes;
        if (smem <= kTcSmemMax) return true;
    }
    return false;
}

}  // namespace

bool qmv_tc_supported(int M, int N, int K, int bits, int group_size, int dt, const void *w, const void *scales,
                      const void *biases, const void *x) {
    const auto al = [](const void *p, size_t a) { return reinterpret_cast<uintptr_t>(p) % a == 0; };
    if (bits != 4 || M < 1 || M > 8 || N < 1 || (dt != MTC_BF16 && dt != MTC_F16)) return false;
    if (K % 512 != 0 || (group_size != 64 && group_size != 128)) return false;
    if (static_cast<long long>(N) * (K / 2) >= (1ll << 31)) return false;
    uint32_t op = 0, orr = 0;
    int ahead = 0;
    size_t smem = 0;
    if (!tc_layout(M, K, op, orr, ahead, smem)) return false;
    return al(w, 16) && al(x, 16) && al(scales, 16) && al(biases, 16);
}

cudaError_t qmv_tc_init_device() {
    cudaError_t e;
    if ((e = cudaFuncSetAttribute(qmv_tc_kernel<true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kTcSmemMax))) != cudaSuccess) return e;
    if ((e = cudaFuncSetAttribute(qmv_tc_kernel<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kTcSmemMax))) != cudaSuccess) return e;
    if ((e = cudaFuncSetAttribute(qmv_tc_kernel<false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kTcSmemMax))) != cudaSuccess) return e;
    return cudaFuncSetAttribute(qmv_tc_kernel<false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kTcSmemMax));
}

size_t qmv_tc_scratch_bytes(int M, int N, int K) { return static_cast<size_t>(K / 256) * M * N * sizeof(float); }
size_t qmv_tc_counter_bytes(int N) { return static_cast<size_t>((N + 127) / 128) * 4 * sizeof(uint32_t); }

// scratch: qmv_tc_scratch_bytes; counters: qmv_tc_counter_bytes, zero before the first launch (the kernel leaves them zero)
cudaError_t launch_qmv_tc(Ctx *ctx, cudaStream_t st, const void *w, const void *scales, const void *biases, const void *x,
                          void *const *outs, int n_out, int M, int N, int K, int group_size, int dt, float *scratch,
                          uint32_t *counters) {
    TcArgs a{};
    a.w = static_cast<const uint32_t *>(w);
    a.scales = scales;
    a.biases = biases;
    a.x = x;
    for (int i = 0; i < n_out && i < 8; ++i) a.out[i] = outs[i];
    a.n_out = n_out;
    a.M = M;
    a.N = N;
    a.K = K;
    a.gsh = group_size == 64 ? 0 : 1;
    a.rowbytes = K / 2;
    a.gpr = K / group_size;
    a.tiles = (N + 127) / 128;
    const int sms = ctx->sm_count;
    const int kc = 256;
    a.kb_per_chunk = kc / 64;
    a.chunks = K / kc;
    a.items = a.chunks * a.tiles;
    a.scratch = scratch;
    a.counters = counters;
    a.status = ctx->d_status;
    const uint32_t fmt = dt == MTC_BF16 ? 1u : 0u;
    a.idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | (static_cast<uint32_t>(16 >> 3) << 17) | (static_cast<uint32_t>(128 >> 4) << 24);
    a.early_weights = ctx->pdl_early_weights;
    a.bf16 = dt == MTC_BF16;
    size_t smem = 0;
    if (!tc_layout(M, K, a.off_p, a.off_ring, a.ahead, smem)) return cudaErrorInvalidValue;
    int grid = a.items < sms ? a.items : sms;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kTcThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t le;
    if (dt == MTC_BF16) le = M == 1 ? cudaLaunchKernelEx(&cfg, qmv_tc_kernel<true, true>, a) : cudaLaunchKernelEx(&cfg, qmv_tc_kernel<true, false>, a);
    else le = M == 1 ? cudaLaunchKernelEx(&cfg, qmv_tc_kernel<false, true>, a) : cudaLaunchKernelEx(&cfg, qmv_tc_kernel<false, false>, a);
    return le;
}

}  // namespace mtc
