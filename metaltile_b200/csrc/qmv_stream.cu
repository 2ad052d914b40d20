// qmv_stream — decode-time quantized matrix-vector products (M <= 8 token rows, 4-bit codes, 16-bit activations)
// as a weight STREAM: every warp copies its own slice of the packed matrix into a private shared-memory ring with
// 16-byte asynchronous copies that run several slices ahead - across row tiles, across projections and across the
// phases of a chain - and multiplies what has landed on the warp-level tensor cores.
//
//   out[m, n] = sum_k (q(n,k) * scale[n, k/G] + bias[n, k/G]) * x[m, k]                 (f32 accumulate)
//
// Stands in for mt_qmv / mt_qmm{,_bm2,_bm4} / mt_qmv_b4 (crates/metaltile-std/src/mlx/quantized.rs:7-308,343-1441,
// 4273-4392) and, as a chain of projections walked by one persistent grid, for several passes committed together
// through Context::dispatch_chain (crates/metaltile-runtime/src/context.rs:363-395) and for the fused decode
// projections that share one activation vector (crates/metaltile-std/src/ffai/batched_qkv_qgemv.rs:1-35,
// crates/metaltile-std/src/ffai/batched_4_qgemv.rs:1-45).
//
// Why this shape.  A decode projection is 2-60 MB of weights read once: the only thing that matters is that
// HBM requests never stop.  Measured on B200 with no arithmetic at all: one bulk-copy (TMA) producer per SM tops out
// at 16 bytes per cycle (4.6 TB/s over 148 SMs) whatever the copy size, per-row bulk copies below 2 KB are slower
// still, while sixteen warps per SM each keeping 2-4 KB of 16-byte cp.async copies in flight reach the full
// 6.6 TB/s.  So the copies are issued by the consuming warps themselves (5 instructions per 2 KB), need no
// cross-warp hand-off, and the ring of a warp is the only thing it ever waits for.
//
// Arithmetic.  The integer codes are the A operand of mma.sync.m16n8k16 without any conversion: a 16-bit float whose
// exponent field is zero (or one) is linear in its low 8 bits, value = bits * 2^-24 (f16) or bits * 2^-133 (bf16) -
// the subnormals and the first binade form one linear ramp, and the tensor cores multiply them exactly (checked on
// B200).  `word & 0x000F000F` is therefore two ready operands q * c, `word & 0x00F000F0` two operands 16 q * c,
// and one shift by 8 gives the other four nibbles: 5 integer instructions per 8 codes.  The nibbles at bits 4-7 go
// through their own accumulator chain, which is folded in with a factor 1/16 per group.  bf16 activations are
// staged multiplied by 2^64 (exact) so that products stay normal f32 numbers; the factor c * 2^64 is removed once
// per output.  Per 64-code segment and group:  acc_s += scale * sum(q x),  acc_b += bias * sum(x).
//
// Mapping.  A row tile is 16 weight rows; the warps of a CTA split its K extent in runs of 256 codes (128 bytes per
// row: one line).  Lane 4g+t holds tile rows pi(g) and 8+pi(g) and words 2t, 2t+1 of each 64-code segment; MMA j of a
// segment uses nibbles j and j+4 of those words, and the activations are staged in shared memory in exactly that
// order (a pure 16-bit permutation).  Rows sit 144 bytes apart in a ring slot and pi(g) = 2(g&3) + (g>>2), so every
// 8-byte fragment load of a half-warp touches 32 distinct banks.  Partial sums of the warps that share a tile are
// added in shared memory in a fixed order (deterministic results) by whichever warp arrives last.
//
// Domain notes: |x| < 2^63 for bf16 (the staged value overflows beyond that); group size 64 or 128; K % 256 == 0.
#include <vector>

#include "common.cuh"

namespace mtc {
namespace {

constexpr int kNW = 8;                         // warps per CTA; two CTAs share an SM
constexpr int kThreads = kNW * 32;
constexpr int kRunSegs = 8;                    // 64-code segments per run: 512 codes, 256 bytes per weight row
constexpr int kRowPitch = 272;                 // 256 bytes of a run + 16: rows two apart land 8 banks apart
constexpr int kSlotW = 16 * kRowPitch;         // packed words of a run: 16 rows
constexpr int kSlotBytes = kSlotW + 512;       // + scales [16 rows x 16 B], biases [16 rows x 16 B]
constexpr int kRedSlots = 4;                   // row tiles whose partial sums may be pending at once
constexpr uint32_t kSpin = 1u << 22;           // bounded waits: then the status word says which one gave up

enum : int { F_STAGE = 1, F_WAIT = 2, F_SIGNAL = 4 };

struct SProj {
    const uint32_t *w;
    const void *scales, *biases, *x;
    void *out[8];
    int n_out, M, N, K;
    int rowbytes, gpr2;  // bytes per weight row (K / 2), bytes per row of scales (2 K / group)
    int rpt;             // runs of 512 codes per row
    int ksh;             // log2 of the warps that share a row tile (<= rpt)
    int phase;           // chain: x may be read once every projection of the earlier phases is complete
    int inv_mp;          // ceil(65536 / Mp), Mp = M rounded up to even: idx / Mp = (idx * inv_mp) >> 16 for idx < 128
};

constexpr int kMaxInline = 4;

struct SArgs {
    SProj inl[kMaxInline];   // a launch of 1-4 projections that share their activations carries them here
    int n_inl;
    int rows_q, rows_r;      // inline launch: total units = rows_q * gridDim.x + rows_r, a unit being 1 << unit_sh rows
    int unit_sh;             // 4 when a CTA has more than one row tile: shares end on tile boundaries, so no CTA pays a pass for a sliver
    const SProj *projs;      // chain: device array, nullptr for an inline launch
    const int4 *pieces;      // chain: [gridDim.x][max_pieces] {projection, row0, row1, flags}; projection < 0 ends a list
    int max_pieces;
    uint32_t *sync;          // chain: one counter per phase, then the exit counter
    int n_phases;
    uint32_t *status;
    int early_weights;       // 1: weight copies start before griddepcontrol.wait (weights are constants of the model)
    uint32_t off_xsum, off_red, off_ring;    // shared-memory layout (the activation fragments start at kOffX)
    uint32_t red_slot_floats;
    // sharded decode (n_peers > 0): the hand-off between the GPUs of a node rides in the kernels.  Before it reads its
    // activations a launch waits until every peer has published the epoch this rank's previous launch ended with
    // (bounded poll, status 0x601 + peer on expiry); when its last CTA is done it publishes the next epoch to every peer.
    uint32_t *peer_flags[8];   // peer q's flag words, mapped here; word `rank` is written by this rank
    uint32_t *local_flags;     // this rank's flag words: word q is written by rank q
    uint32_t *epoch;           // this rank's epoch counter (device memory, zeroed once)
    uint32_t *ticket;          // CTAs of the current launch that are done (zero between launches)
    int n_peers, rank;
    uint32_t poll_limit;
};

struct __align__(16) Ctl {
    uint32_t cnt[kRedSlots];             // warps that have written their partial sums of the tile in this slot
    volatile uint32_t gen[kRedSlots];    // completed reductions per slot
    volatile uint32_t abort;
    uint32_t pad[7];
};
constexpr uint32_t kOffX = 128;

__device__ __forceinline__ uint32_t s_u32(const void *p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void cp16(uint32_t dst, const void *src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp8(uint32_t dst, const void *src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int DEPTH>
__device__ __forceinline__ void cp_wait_oldest() {      // all but the newest DEPTH-1 groups have landed
    if (DEPTH == 2) asm volatile("cp.async.wait_group 1;" ::: "memory");
    else if (DEPTH == 3) asm volatile("cp.async.wait_group 2;" ::: "memory");
    else asm volatile("cp.async.wait_group 3;" ::: "memory");
}

template <bool BF16, bool kZero>
__device__ __forceinline__ void hmma(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    if (kZero) {
        if (BF16)
            asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.0f));
        else
            asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.0f));
    } else {
        if (BF16)
            asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
        else
            asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    }
}

// 16-bit field H (0 or 1) of a word as f32
template <bool BF16, int H>
__device__ __forceinline__ float f32_of_half(uint32_t word) {
    if (BF16) return __uint_as_float(H ? (word & 0xFFFF0000u) : (word << 16));
    const __half2 v = *reinterpret_cast<const __half2 *>(&word);
    return H ? __high2float(v) : __low2float(v);
}
__device__ __forceinline__ uint32_t word_of(const uint4 &v, int i) { return i == 0 ? v.x : i == 1 ? v.y : i == 2 ? v.z : v.w; }

// Stage the activations of a projection: B fragments in MMA order plus the per-segment sums.
//   fragment unit (16 bytes) of (segment s, token m, quad-lane t, half h): ((s*M + m)*4 + t)*2 + (h ^ (m & 1));
//   half h holds fragments j = 2h, 2h+1:  .x/.z = (x[16t + j], x[16t + j + 4]),  .y/.w = the same 8 further on;
//   the odd fragments (j = 1, 3) hold x / 16: their codes arrive as 16 q (exact for bf16, whose staged values carry
//   2^64; for f16 exact unless |x| < 2^-10, where the quotient is a subnormal f16: absolute error below 2^-25);
//   xsum: sum of the 64 activations of (segment s, token m), unscaled, f32 - M = 1: xsum[s]; else xsum[s*8 + m], 0 for m >= M.
// The 16 activations x[16t .. 16t + 15] of a segment as this lane's two fragment units, and their sum.
template <bool BF16>
__device__ __forceinline__ void stage_item(const uint4 &v0, const uint4 &v1, uint4 &f01, uint4 &f23, float &sum) {
    const uint32_t u[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};   // word q holds (h[2q], h[2q+1])
    uint32_t e[8], o[8];              // as staged for the even fragments; / 16 for the odd ones
    sum = 0.0f;
#pragma unroll
    for (int q = 0; q < 8; ++q) {
        if (BF16) {
            const float lo = __uint_as_float(u[q] << 16), hi = __uint_as_float(u[q] & 0xFFFF0000u);
            sum += lo + hi;
            // times 2^64 (2^60) on both halves at once: an exact change of exponent, subnormals included (inf beyond 2^63)
            asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(e[q]) : "r"(u[q]), "r"(0x5F805F80u));
            asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(o[q]) : "r"(u[q]), "r"(0x5D805D80u));
        } else {
            const __half2 h2 = *reinterpret_cast<const __half2 *>(&u[q]);
            const float2 f = __half22float2(h2);
            sum += f.x + f.y;
            e[q] = u[q];
            const __half2 sc = __hmul2(h2, __float2half2_rn(0.0625f));
            o[q] = *reinterpret_cast<const uint32_t *>(&sc);
        }
    }
    // fragment j: .x = (h[j], h[j+4]) of the first 8 values, .y = the same of the second 8
    f01 = make_uint4(__byte_perm(e[0], e[2], 0x5410), __byte_perm(e[4], e[6], 0x5410), __byte_perm(o[0], o[2], 0x7632),
                     __byte_perm(o[4], o[6], 0x7632));
    f23 = make_uint4(__byte_perm(e[1], e[3], 0x5410), __byte_perm(e[5], e[7], 0x5410), __byte_perm(o[1], o[3], 0x7632),
                     __byte_perm(o[5], o[7], 0x7632));
}

template <bool BF16, bool M1>
__device__ __forceinline__ void stage_x(const void *x, int K, int M, unsigned char *sm, uint32_t off_xsum) {
    const int nseg = K >> 6;
    float *xsum = reinterpret_cast<float *>(sm + off_xsum);
    if (!M1 && M < 8) {
        for (int i = threadIdx.x; i < nseg * 8; i += kThreads) xsum[i] = 0.0f;
        __syncthreads();
    }
    uint4 *xb = reinterpret_cast<uint4 *>(sm + kOffX);
    const int t = threadIdx.x & 3;
    for (int s0 = (threadIdx.x >> 5) * 8; s0 < nseg; s0 += kThreads / 4) {   // a warp takes 8 segments; the four lanes of a quad share (s, m)
        const int s = s0 + ((threadIdx.x & 31) >> 2);
        const bool on = s < nseg;                                            // whole warps stay in the loop: the sums use shuffles
        for (int m = 0; m < M; ++m) {
            uint4 v0 = make_uint4(0u, 0u, 0u, 0u), v1 = v0;
            if (on) {
                const uint4 *p = reinterpret_cast<const uint4 *>(static_cast<const uint16_t *>(x) + static_cast<size_t>(m) * K +
                                                                 static_cast<size_t>(s) * 64 + 16 * t);
                v0 = __ldg(p);        // x[16t + 0..7]
                v1 = __ldg(p + 1);    // x[16t + 8..15]
            }
            uint4 f01, f23;
            float sum;
            stage_item<BF16>(v0, v1, f01, f23, sum);
            sum += __shfl_xor_sync(0xffffffffu, sum, 1);
            sum += __shfl_xor_sync(0xffffffffu, sum, 2);
            if (on) {
                const int unit = ((s * M + m) * 4 + t) * 2;
                xb[unit + (m & 1)] = f01;
                xb[unit + ((m & 1) ^ 1)] = f23;
                if (t == 0) xsum[M1 ? s : s * 8 + m] = sum;
            }
        }
    }
}

// One token, a warp stages only the segments [seg0, seg1) that its own runs read: no warp waits for another.  All of a
// round's loads are issued before the first is converted.
template <bool BF16>
__device__ __forceinline__ void stage_x_warp(const void *x, int seg0, int seg1, unsigned char *sm, uint32_t off_xsum, int lane) {
    float *xsum = reinterpret_cast<float *>(sm + off_xsum);
    uint4 *xb = reinterpret_cast<uint4 *>(sm + kOffX);
    const int t = lane & 3, nitems = (seg1 - seg0) * 4;
    constexpr int U = 4;
    for (int base = 0; base < nitems; base += 32 * U) {
        uint4 v0[U], v1[U];
#pragma unroll
        for (int i = 0; i < U; ++i) {
            const int it = base + 32 * i + lane;
            v0[i] = v1[i] = make_uint4(0u, 0u, 0u, 0u);
            if (it < nitems) {
                const uint4 *p = reinterpret_cast<const uint4 *>(static_cast<const uint16_t *>(x) + static_cast<size_t>(seg0 + (it >> 2)) * 64 + 16 * t);
                v0[i] = __ldg(p);
                v1[i] = __ldg(p + 1);
            }
        }
#pragma unroll
        for (int i = 0; i < U; ++i) {
            const int it = base + 32 * i + lane;
            if (base + 32 * i >= nitems) break;                              // warp-uniform
            uint4 f01, f23;
            float sum;
            stage_item<BF16>(v0[i], v1[i], f01, f23, sum);
            sum += __shfl_xor_sync(0xffffffffu, sum, 1);
            sum += __shfl_xor_sync(0xffffffffu, sum, 2);
            if (it < nitems) {
                const int s = seg0 + (it >> 2);
                xb[(s * 4 + t) * 2] = f01;
                xb[(s * 4 + t) * 2 + 1] = f23;
                if (t == 0) xsum[s] = sum;
            }
        }
    }
}

// The position of a warp in its sequence of runs, on the copy side (which is DEPTH - 1 runs ahead of the arithmetic).
struct CopyIt {
    const char *w, *sb;       // packed words; scales (lanes 0-15) or biases (lanes 16-31)
    int rowbytes, gpr2;       // bytes per weight row, bytes per scale row
    int row0, row1;           // rows of the piece
    int tile, tiles, slots;   // this warp's current tile, tiles of the piece, tiles in progress at once
    int run, rb, re;          // current run, this warp's run range within a tile
    int j;                    // piece index
    bool valid;
};

// One run: 16 rows x 256 bytes of packed words (8 copies of 16 bytes per lane: lane -> row 2q + (lane >> 4),
// chunk lane & 15) and 16 rows x 16 (8) bytes of scales and of biases (one copy per lane).  Rows past the end of the
// piece re-read its last row, so every byte of the slot is defined.
template <int GSH>
__device__ __forceinline__ void issue_run(const CopyIt &c, uint32_t slot, int lane) {
    const int r0 = c.row0 + c.tile * 16;
    const int last = c.row1 - 1;
    const int crow = lane >> 4, cch = lane & 15;
    const char *src = c.w + static_cast<size_t>(c.run) * 256 + cch * 16;
    const uint32_t dst = slot + crow * kRowPitch + cch * 16;
    if (r0 + 15 <= last) {                       // a whole tile (the usual case): one pointer walks the rows
        const char *p = src + static_cast<size_t>(r0 + crow) * c.rowbytes;
        const size_t step = static_cast<size_t>(2 * c.rowbytes);
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            cp16(dst + q * 2 * kRowPitch, p);
            p += step;
        }
    } else {
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            const int row = min(r0 + crow + 2 * q, last);
            cp16(dst + q * 2 * kRowPitch, src + static_cast<size_t>(row) * c.rowbytes);
        }
    }
    const int srow = min(r0 + (lane & 15), last);
    const uint32_t sdst = slot + kSlotW + (lane >> 4) * 256 + (lane & 15) * 16;
    if (GSH == 0) cp16(sdst, c.sb + static_cast<size_t>(srow) * c.gpr2 + static_cast<size_t>(c.run) * 16);
    else cp8(sdst, c.sb + static_cast<size_t>(srow) * c.gpr2 + static_cast<size_t>(c.run) * 8);
}

// One 64-code segment for the two rows and (up to) two tokens of this lane; P (0..7) is its place in the run.
//   as[i] += scale * c * sum(q x),  ab[i] += bias * sum(x);  i = 0,1: row ra, tokens 2t, 2t+1;  i = 2,3: row rb.
// The nibbles at bits 4-7 carry a factor 16, which their activations were staged without (x / 16), so all four MMAs of
// a segment add into one accumulator.
template <bool BF16, int GSH, bool M1, int P>
__device__ __forceinline__ void consume_segment(const unsigned char *slot_lo, const unsigned char *slot_hi, const uint4 &sl,
                                                const uint4 &sh, const uint4 &bl, const uint4 &bh, const unsigned char *xa,
                                                const unsigned char *xb, uint32_t xstride, const float *xs, float (&as)[4],
                                                float (&ab)[4]) {
    constexpr uint32_t m0 = 0x000F000Fu, m1 = 0x00F000F0u;
    const uint2 cl = *reinterpret_cast<const uint2 *>(slot_lo + P * 32);
    const uint2 ch = *reinterpret_cast<const uint2 *>(slot_hi + P * 32);
    const uint4 f01 = *reinterpret_cast<const uint4 *>(xa + (M1 ? P * 128 : P * xstride));
    const uint4 f23 = *reinterpret_cast<const uint4 *>(xb + (M1 ? P * 128 : P * xstride));
    float d[4];
    hmma<BF16, true>(d, cl.x & m0, ch.x & m0, cl.y & m0, ch.y & m0, f01.x, f01.y);            // nibbles 0, 4
    hmma<BF16, false>(d, cl.x & m1, ch.x & m1, cl.y & m1, ch.y & m1, f01.z, f01.w);           // nibbles 1, 5 (x 16)
    const uint32_t c0 = cl.x >> 8, c1 = ch.x >> 8, c2 = cl.y >> 8, c3 = ch.y >> 8;
    hmma<BF16, false>(d, c0 & m0, c1 & m0, c2 & m0, c3 & m0, f23.x, f23.y);                   // nibbles 2, 6
    hmma<BF16, false>(d, c0 & m1, c1 & m1, c2 & m1, c3 & m1, f23.z, f23.w);                   // nibbles 3, 7 (x 16)
    constexpr int gi = P >> GSH;                 // group of this segment within the run
    constexpr int hf = gi & 1;
    const float s_lo = f32_of_half<BF16, hf>(word_of(sl, gi >> 1)), s_hi = f32_of_half<BF16, hf>(word_of(sh, gi >> 1));
    if (M1) {
        as[0] = fmaf(s_lo, d[0], as[0]);         // the bias term of a one-token run is added per run (consume_run)
        as[2] = fmaf(s_hi, d[2], as[2]);
    } else {
        const float b_lo = f32_of_half<BF16, hf>(word_of(bl, gi >> 1)), b_hi = f32_of_half<BF16, hf>(word_of(bh, gi >> 1));
        const float2 x_sum = *reinterpret_cast<const float2 *>(xs + P * 8);
        as[0] = fmaf(s_lo, d[0], as[0]);
        as[1] = fmaf(s_lo, d[1], as[1]);
        as[2] = fmaf(s_hi, d[2], as[2]);
        as[3] = fmaf(s_hi, d[3], as[3]);
        ab[0] = fmaf(b_lo, x_sum.x, ab[0]);
        ab[1] = fmaf(b_lo, x_sum.y, ab[1]);
        ab[2] = fmaf(b_hi, x_sum.x, ab[2]);
        ab[3] = fmaf(b_hi, x_sum.y, ab[3]);
    }
}

// The eight segments of a run.  slot_lo / slot_hi: this lane's 8 bytes of the first segment in tile rows ra and rb;
// xa / xb: its two fragment halves of the run's first segment (xstride bytes per segment); xs: the activation sums.
template <bool BF16, int GSH, bool M1>
__device__ __forceinline__ void consume_run(const unsigned char *slot, uint32_t a_lo, uint32_t ra16, const unsigned char *xa,
                                            const unsigned char *xb, uint32_t xstride, const float *xs, float (&as)[4],
                                            float (&ab)[4]) {
    const unsigned char *slot_lo = slot + a_lo, *slot_hi = slot_lo + 8 * kRowPitch;
    const uint4 sl = *reinterpret_cast<const uint4 *>(slot + kSlotW + ra16), sh = *reinterpret_cast<const uint4 *>(slot + kSlotW + ra16 + 128);
    uint4 bl = make_uint4(0u, 0u, 0u, 0u), bh = bl;
    if (M1) {
        // One token: the four lanes of a quad hold the same sums, so each adds the bias term of two of the run's eight
        // segments (2t, 2t + 1) and the quad's parts meet once per row tile (tile_bias_sum).
        const int t = (threadIdx.x & 3);
        const float2 x_sum = *reinterpret_cast<const float2 *>(xs + 2 * t);
        if (GSH == 0) {                          // a group per segment: the pair of biases is one word
            const uint32_t wl = *reinterpret_cast<const uint32_t *>(slot + kSlotW + 256 + ra16 + 4 * t);
            const uint32_t wh = *reinterpret_cast<const uint32_t *>(slot + kSlotW + 256 + ra16 + 128 + 4 * t);
            ab[0] = fmaf(f32_of_half<BF16, 0>(wl), x_sum.x, ab[0]);
            ab[0] = fmaf(f32_of_half<BF16, 1>(wl), x_sum.y, ab[0]);
            ab[2] = fmaf(f32_of_half<BF16, 0>(wh), x_sum.x, ab[2]);
            ab[2] = fmaf(f32_of_half<BF16, 1>(wh), x_sum.y, ab[2]);
        } else {                                 // a group per two segments: one bias for both
            const uint32_t wl = *reinterpret_cast<const uint16_t *>(slot + kSlotW + 256 + ra16 + 2 * t);
            const uint32_t wh = *reinterpret_cast<const uint16_t *>(slot + kSlotW + 256 + ra16 + 128 + 2 * t);
            ab[0] = fmaf(f32_of_half<BF16, 0>(wl), x_sum.x + x_sum.y, ab[0]);
            ab[2] = fmaf(f32_of_half<BF16, 0>(wh), x_sum.x + x_sum.y, ab[2]);
        }
    } else {
        bl = *reinterpret_cast<const uint4 *>(slot + kSlotW + 256 + ra16);
        bh = *reinterpret_cast<const uint4 *>(slot + kSlotW + 256 + ra16 + 128);
    }
    consume_segment<BF16, GSH, M1, 0>(slot_lo, slot_hi, sl, sh, bl, bh, xa, xb, xstride, xs, as, ab);
    consume_segment<BF16, GSH, M1, 1>(slot_lo, slot_hi, sl, sh, bl, bh, xa, xb, xstride, xs, as, ab);
    consume_segment<BF16, GSH, M1, 2>(slot_lo, slot_hi, sl, sh, bl, bh, xa, xb, xstride, xs, as, ab);
    consume_segment<BF16, GSH, M1, 3>(slot_lo, slot_hi, sl, sh, bl, bh, xa, xb, xstride, xs, as, ab);
    consume_segment<BF16, GSH, M1, 4>(slot_lo, slot_hi, sl, sh, bl, bh, xa, xb, xstride, xs, as, ab);
    consume_segment<BF16, GSH, M1, 5>(slot_lo, slot_hi, sl, sh, bl, bh, xa, xb, xstride, xs, as, ab);
    consume_segment<BF16, GSH, M1, 6>(slot_lo, slot_hi, sl, sh, bl, bh, xa, xb, xstride, xs, as, ab);
    consume_segment<BF16, GSH, M1, 7>(slot_lo, slot_hi, sl, sh, bl, bh, xa, xb, xstride, xs, as, ab);
}

// What the arithmetic side needs of a piece, read once when the piece starts.
struct PieceInfo {
    const void *x;
    void *out0;
    int M, N, K, n_out, rpt, ksh, phase, inv_mp;
};

template <bool BF16, int GSH, bool M1, int DEPTH>
__global__ void __launch_bounds__(kThreads, 2) qmv_stream_kernel(const __grid_constant__ SArgs a) {
    extern __shared__ __align__(128) unsigned char sm[];
    Ctl *ctl = reinterpret_cast<Ctl *>(sm);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const bool chain = a.projs != nullptr;

    asm volatile("griddepcontrol.launch_dependents;");
    if (threadIdx.x < kRedSlots) {
        ctl->cnt[threadIdx.x] = 0u;
        ctl->gen[threadIdx.x] = 0u;
    }
    if (threadIdx.x == 0) ctl->abort = 0u;
    __syncthreads();

    auto get_piece = [&](int j, int4 &pc) -> bool {
        if (chain) {
            if (j >= a.max_pieces) return false;
            pc = __ldg(a.pieces + static_cast<size_t>(blockIdx.x) * a.max_pieces + j);
            return pc.x >= 0;
        }
        // inline launch: the rows of all projections form one range that is dealt evenly (CTA b takes q rows, the
        // first r CTAs one more); piece j is this CTA's part of projection j (possibly empty)
        if (j >= a.n_inl) return false;
        const int b = blockIdx.x;
        const int lo_u = b * a.rows_q + min(b, a.rows_r);
        const int lo_all = lo_u << a.unit_sh, hi_all = (lo_u + a.rows_q + (b < a.rows_r ? 1 : 0)) << a.unit_sh;
        int before = 0;
        for (int q = 0; q < j; ++q) before += a.inl[q].N;
        const int n = a.inl[j].N;
        const int r0 = min(max(lo_all - before, 0), n), r1 = min(max(hi_all - before, 0), n);
        pc = make_int4(j, r0, r1, j == 0 ? F_STAGE : 0);
        return true;
    };
    auto proj = [&](int idx) -> const SProj & { return chain ? a.projs[idx] : a.inl[idx]; };

    // ---- copy side --------------------------------------------------------------------------------------------
    unsigned char *ring_p = sm + a.off_ring + static_cast<size_t>(warp) * DEPTH * kSlotBytes;
    const uint32_t ring = s_u32(ring_p);
    CopyIt cit;
    cit.j = 0;
    cit.valid = false;
    auto copy_enter = [&]() {       // position on the first run of piece cit.j or a later one that has work for this warp
        for (;;) {
            int4 pc;
            if (!get_piece(cit.j, pc)) {
                cit.valid = false;
                return;
            }
            const SProj &P = proj(pc.x);
            const int ksh = P.ksh, KS = 1 << ksh, rpt = P.rpt;
            cit.slots = kNW >> ksh;
            const int ks = warp & (KS - 1);
            cit.rb = (ks * rpt) >> ksh;
            cit.re = ((ks + 1) * rpt) >> ksh;
            cit.row0 = pc.y;
            cit.row1 = pc.z;
            cit.tiles = (pc.z - pc.y + 15) >> 4;
            cit.tile = warp >> ksh;
            if (cit.tile < cit.tiles && cit.rb < cit.re) {
                cit.w = reinterpret_cast<const char *>(P.w);
                cit.sb = static_cast<const char *>(lane < 16 ? P.scales : P.biases);
                cit.rowbytes = P.rowbytes;
                cit.gpr2 = P.gpr2;
                cit.run = cit.rb;
                cit.valid = true;
                return;
            }
            ++cit.j;
        }
    };
    auto copy_next = [&](uint32_t slot) {      // issue the current run (if any) and move on
        if (cit.valid) {
            issue_run<GSH>(cit, slot, lane);
            if (++cit.run == cit.re) {
                cit.run = cit.rb;
                cit.tile += cit.slots;
                if (cit.tile >= cit.tiles) {
                    ++cit.j;
                    copy_enter();
                }
            }
        }
        cp_commit();
    };

    if (!a.early_weights) asm volatile("griddepcontrol.wait;" ::: "memory");
    copy_enter();
    // the whole ring is requested before anything waits: the copies run while the previous kernel of the stream drains
    // and while this CTA stages its activations
#pragma unroll 1
    for (int p = 0; p < DEPTH; ++p) copy_next(ring + p * kSlotBytes);
    int cslot = 0;
    // the weights do not depend on the previous kernel of the stream; the activations and every store do
    if (a.early_weights) asm volatile("griddepcontrol.wait;" ::: "memory");
    if (a.n_peers > 0) {
        // every peer has finished the launch that matches this rank's previous one: its stores into this rank's
        // buffers (possibly this launch's activations) have landed
        if (threadIdx.x < a.n_peers) {
            const uint32_t want = *reinterpret_cast<volatile uint32_t *>(a.epoch);
            bool seen = false;
            for (uint32_t i = 0; i < a.poll_limit; ++i) {
                uint32_t v;
                asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(a.local_flags + threadIdx.x) : "memory");
                if (static_cast<int32_t>(v - want) >= 0) {
                    seen = true;
                    break;
                }
                __nanosleep(20);
            }
            if (!seen) atomicCAS(a.status, 0u, 0x601u + threadIdx.x);      // that rank never arrived; carry on, the host is told
        }
        __syncthreads();
    }

    // ---- arithmetic side ----------------------------------------------------------------------------------------
    const int pi = 2 * (g & 3) + (g >> 2);                      // tile row of MMA row g (and 8 + pi of MMA row g + 8)
    const uint32_t a_lo = pi * kRowPitch + t * 8;
    const uint32_t ra16 = pi * 16;
    float *red_all = reinterpret_cast<float *>(sm + a.off_red);
    int tile_base = 0;                                          // row tiles of the earlier pieces of this CTA
    bool ok = true;

#pragma unroll 1
    for (int j = 0;; ++j) {
        int4 pc;
        if (!get_piece(j, pc)) break;
        PieceInfo I;
        {
            const SProj &P = proj(pc.x);
            I.x = P.x; I.out0 = P.out[0]; I.M = P.M; I.N = P.N; I.K = P.K; I.n_out = P.n_out; I.rpt = P.rpt; I.ksh = P.ksh;
            I.phase = P.phase; I.inv_mp = P.inv_mp;
        }
        if (pc.w & F_WAIT) {
            // every CTA has finished the earlier phases: their outputs may be this projection's activations
            if (threadIdx.x == 0) {
                const uint32_t want = gridDim.x;
                bool seen = false;
                for (uint32_t i = 0; i < kSpin; ++i) {
                    uint32_t v;
                    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(a.sync + (I.phase - 1)) : "memory");
                    if (v >= want) {
                        seen = true;
                        break;
                    }
                    __nanosleep(32);
                }
                if (!seen) {
                    ctl->abort = 1u;
                    atomicCAS(a.status, 0u, 0x701u);
                }
            }
            __syncthreads();
            if (ctl->abort) break;                               // uniform: every thread reads the flag after the barrier
        }
        if (pc.w & F_STAGE) {
            if (j > 0) __syncthreads();                          // every warp is done with the previous activations
            if (M1 && (1 << I.ksh) == kNW) {
                // the warps of a CTA split K eight ways: each stages what its own runs read and goes on alone
                stage_x_warp<BF16>(I.x, ((warp * I.rpt) >> I.ksh) * kRunSegs, (((warp + 1) * I.rpt) >> I.ksh) * kRunSegs, sm, a.off_xsum, lane);
                __syncwarp();
            } else {
                stage_x<BF16, M1>(I.x, I.K, I.M, sm, a.off_xsum);
                __syncthreads();
            }
        }
        const int M = M1 ? 1 : I.M, Mp = (M + 1) & ~1;
        const int ksh = I.ksh, KS = 1 << ksh, slots = kNW >> ksh, ks = warp & (KS - 1);
        const int rb = (ks * I.rpt) >> ksh, re = ((ks + 1) * I.rpt) >> ksh;
        const int tiles = (pc.z - pc.y + 15) >> 4;
        const int meff = g < M ? g : 0;                          // lanes without a token read token 0; their columns are dropped
        const uint32_t xstride = M * 128;
        const unsigned char *x0 = sm + kOffX + ((meff * 4 + t) * 2 + (meff & 1)) * 16;
        const unsigned char *x1 = sm + kOffX + (((meff * 4 + t) * 2 + (meff & 1)) ^ 1) * 16;
        const float *xs0 = reinterpret_cast<const float *>(sm + a.off_xsum) + (M1 ? 0 : 2 * t);

#pragma unroll 1
        for (int tile = warp >> ksh; tile < tiles && ok; tile += slots) {
            float as[4] = {0.f, 0.f, 0.f, 0.f}, ab[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 1
            for (int run = rb; run < re; ++run) {
                cp_wait_oldest<DEPTH>();                         // this run has landed (this lane's copies)
                __syncwarp();                                    // ... and every other lane's
                const unsigned char *slot = ring_p + cslot * kSlotBytes;
                const uint32_t so = run * kRunSegs;              // first segment of the run
                consume_run<BF16, GSH, M1>(slot, a_lo, ra16, x0 + so * xstride, x1 + so * xstride, xstride,
                                           xs0 + (M1 ? so : so * 8), as, ab);
                __syncwarp();                                    // every lane is done with the slot: refill it
                copy_next(ring + cslot * kSlotBytes);
                if (++cslot == DEPTH) cslot = 0;
            }

            // ---- add up the warps that share this tile; the last one to arrive stores ----
            const uint32_t tseq = static_cast<uint32_t>(tile_base + tile);
            const int rs = tseq & (kRedSlots - 1);
            const uint32_t want_gen = tseq / kRedSlots;
            if (ctl->gen[rs] != want_gen) {                      // rare: the slot's previous tile is still being added up
                if (lane == 0) {
                    bool free_slot = false;
                    for (uint32_t i = 0; i < kSpin; ++i) {
                        if (ctl->gen[rs] == want_gen) {
                            free_slot = true;
                            break;
                        }
                        if (ctl->abort) break;
                    }
                    if (!free_slot) {
                        ctl->abort = 1u;
                        atomicCAS(a.status, 0u, 0x702u);
                    }
                }
                __syncwarp();
                ok = ctl->abort == 0u;
                if (!ok) break;                                  // this warp stops computing but still meets the CTA's barriers
            }
            if (M1) {                                            // the quad's parts of the bias term (consume_run)
                ab[0] += __shfl_xor_sync(0xffffffffu, ab[0], 1);
                ab[2] += __shfl_xor_sync(0xffffffffu, ab[2], 1);
                ab[0] += __shfl_xor_sync(0xffffffffu, ab[0], 2);
                ab[2] += __shfl_xor_sync(0xffffffffu, ab[2], 2);
            }
            // c * 2^(pre-scale) leaves once per output: f16 codes are q * 2^-24; bf16 codes q * 2^-133 against x * 2^64
            const float post = BF16 ? 5.9029581035870565e20f /* 2^69 */ : 16777216.0f /* 2^24 */;
            float *mine = red_all + rs * a.red_slot_floats + warp * (16 * Mp);
            if (2 * t < Mp) {
                *reinterpret_cast<float2 *>(mine + pi * Mp + 2 * t) = make_float2(fmaf(as[0], post, ab[0]), fmaf(as[1], post, ab[1]));
                *reinterpret_cast<float2 *>(mine + (pi + 8) * Mp + 2 * t) = make_float2(fmaf(as[2], post, ab[2]), fmaf(as[3], post, ab[3]));
            }
            __syncwarp();
            uint32_t old = 0;
            if (lane == 0) {
                __threadfence_block();
                old = atomicAdd(&ctl->cnt[rs], 1u);
            }
            old = __shfl_sync(0xffffffffu, old, 0);
            if (old == static_cast<uint32_t>(KS - 1)) {
                __threadfence_block();
                const float *first = red_all + rs * a.red_slot_floats + (warp & ~(KS - 1)) * (16 * Mp);
                const int r0 = pc.y + tile * 16;
                const int dt = BF16 ? MTC_BF16 : MTC_F16;
                for (int idx = lane; idx < 16 * Mp; idx += 32) {
                    float pv[kNW];                               // all partial sums in flight, then added in warp order
#pragma unroll
                    for (int q = 0; q < kNW; ++q) pv[q] = q < KS ? first[q * 16 * Mp + idx] : 0.0f;
                    float v = pv[0];
#pragma unroll
                    for (int q = 1; q < kNW; ++q) v += pv[q];
                    const int row = (idx * I.inv_mp) >> 16, tok = idx - row * Mp;      // idx / Mp for idx < 128
                    const int n = r0 + row;
                    if (tok < M && n < pc.z) {
                        const size_t o = static_cast<size_t>(tok) * I.N + n;
                        st_from_f32(I.out0, o, v, dt);
                        if (I.n_out > 1) {
                            const SProj &P = proj(pc.x);
                            for (int d = 1; d < I.n_out; ++d) st_from_f32(P.out[d], o, v, dt);
                        }
                    }
                }
                __syncwarp();
                if (lane == 0) {
                    ctl->cnt[rs] = 0u;
                    __threadfence_block();
                    ctl->gen[rs] = want_gen + 1u;
                }
            }
        }
        tile_base += tiles;
        if (pc.w & F_SIGNAL) {
            __syncthreads();                                     // every store of this CTA for the phase has been issued
            if (threadIdx.x == 0) {
                __threadfence();
                asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(a.sync + I.phase) : "memory");
            }
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    if (a.n_peers > 0) {
        __syncthreads();                                         // every store of this CTA has been issued
        if (threadIdx.x == 0) {
            __threadfence();
            if (atomicAdd(a.ticket, 1u) == gridDim.x - 1) {      // the last CTA of the launch
                *a.ticket = 0u;
                const uint32_t e = *reinterpret_cast<volatile uint32_t *>(a.epoch) + 1u;
                __threadfence_system();
                for (int q = 0; q < a.n_peers; ++q)
                    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(a.peer_flags[q] + a.rank), "r"(e) : "memory");
                *reinterpret_cast<volatile uint32_t *>(a.epoch) = e;
            }
        }
    }
    if (chain) {
        // the last CTA to leave clears the counters for the next run of the chain
        __syncthreads();
        if (threadIdx.x == 0) {
            __threadfence();
            const uint32_t n = atomicAdd(a.sync + a.n_phases, 1u);
            if (n == gridDim.x - 1) {
                for (int p = 0; p <= a.n_phases; ++p) a.sync[p] = 0u;
                __threadfence();
            }
        }
    }
}

// ---- host side -------------------------------------------------------------------------------------------------

struct Plan {
    int depth = 0, per_sm = 0;
    size_t smem = 0;
    uint32_t off_xsum = 0, off_red = 0, off_ring = 0, red_slot_floats = 0;
};

inline size_t up128(size_t v) { return (v + 127) / 128 * 128; }

constexpr size_t kSmemTwoPerSm = 113 * 1024;     // two CTAs per SM
constexpr size_t kSmemOnePerSm = 226 * 1024;

// Shared-memory layout for the largest projection of a launch: two CTAs per SM when a ring of two slots per warp fits
// beside the activations, else one; depth 0 = the activations do not fit at all.
Plan make_plan(int max_mk /* max M*K */, int max_k, int max_m) {
    Plan p;
    const int mp = (max_m + 1) & ~1;
    const size_t xfrag = up128(static_cast<size_t>(max_mk) * 2);
    const size_t xsum = up128(static_cast<size_t>(max_k / 64) * (max_m == 1 ? 4 : 32));
    p.red_slot_floats = static_cast<uint32_t>(kNW * 16 * mp);
    const size_t red = up128(static_cast<size_t>(kRedSlots) * p.red_slot_floats * 4);
    p.off_xsum = static_cast<uint32_t>(kOffX + xfrag);
    p.off_red = static_cast<uint32_t>(p.off_xsum + xsum);
    p.off_ring = static_cast<uint32_t>(p.off_red + red);
    const size_t per_depth = static_cast<size_t>(kNW) * kSlotBytes;
    for (int per_sm = 2; per_sm >= 1; --per_sm) {
        const size_t cap = per_sm == 2 ? kSmemTwoPerSm : kSmemOnePerSm;
        if (cap < p.off_ring + 2 * per_depth) continue;
        int depth = static_cast<int>((cap - p.off_ring) / per_depth);
        if (depth > 3) depth = 3;
        p.depth = depth;
        p.per_sm = per_sm;
        p.smem = p.off_ring + depth * per_depth;
        return p;
    }
    return p;
}

void fill_proj(SProj &p, const void *w, const void *scales, const void *biases, const void *x, void *const *outs, int n_out,
               int M, int N, int K, int group_size, int phase) {
    p = SProj{};
    p.w = static_cast<const uint32_t *>(w);
    p.scales = scales;
    p.biases = biases;
    p.x = x;
    for (int i = 0; i < n_out && i < 8; ++i) p.out[i] = outs[i];
    p.n_out = n_out;
    p.M = M;
    p.N = N;
    p.K = K;
    p.rowbytes = K / 2;
    p.gpr2 = 2 * (K / group_size);
    p.rpt = K / (64 * kRunSegs);
    int ksh = 0;
    while ((2 << ksh) <= kNW && (2 << ksh) <= p.rpt) ++ksh;
    p.ksh = ksh;
    p.phase = phase;
    const int mp = (M + 1) & ~1;
    p.inv_mp = (65536 + mp - 1) / mp;
}

using KernelFn = void (*)(const SArgs);

// kernel variant by (activation type, group 64 / 128, one token / several, ring depth 2 / 3)
KernelFn pick_kernel(bool bf16, int gsh, bool m1, int depth) {
#define MTC_PICK(B, G, M_)  (depth == 2 ? static_cast<KernelFn>(qmv_stream_kernel<B, G, M_, 2>) : static_cast<KernelFn>(qmv_stream_kernel<B, G, M_, 3>))
    if (bf16) {
        if (gsh == 0) return m1 ? MTC_PICK(true, 0, true) : MTC_PICK(true, 0, false);
        return m1 ? MTC_PICK(true, 1, true) : MTC_PICK(true, 1, false);
    }
    if (gsh == 0) return m1 ? MTC_PICK(false, 0, true) : MTC_PICK(false, 0, false);
    return m1 ? MTC_PICK(false, 1, true) : MTC_PICK(false, 1, false);
#undef MTC_PICK
}

}  // namespace

bool qmv_stream_supported(int M, int N, int K, int bits, int group_size, int dt, const void *w, const void *scales,
                          const void *biases, const void *x) {
    const auto al = [](const void *p, size_t a) { return reinterpret_cast<uintptr_t>(p) % a == 0; };
    if (bits != 4 || M < 1 || M > 8 || N < 1 || (dt != MTC_BF16 && dt != MTC_F16)) return false;
    if (K % (64 * kRunSegs) != 0 || (group_size != 64 && group_size != 128)) return false;
    if (static_cast<long long>(N) * (K / 2) >= (1ll << 31)) return false;
    if (!al(w, 16) || !al(x, 16) || !al(scales, 16) || !al(biases, 16)) return false;
    return make_plan(M * K, K, M).depth >= 2;
}

// Opt every variant into its dynamic shared memory (per device: called from mtc_init with that device current).
cudaError_t qmv_stream_init_device() {
    for (int v = 0; v < 16; ++v) {
        cudaError_t e = cudaFuncSetAttribute(pick_kernel(v & 1, (v >> 1) & 1, (v >> 2) & 1, 2 + ((v >> 3) & 1)),
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kSmemOnePerSm));
        if (e != cudaSuccess) return e;
    }
    return cudaSuccess;
}

static cudaError_t launch_stream_kernel(cudaStream_t st, const SArgs &a, KernelFn fn, int grid, size_t smem) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, fn, a);
}

static void fill_layout(SArgs &a, Ctx *ctx, const Plan &plan) {
    a.status = ctx->d_status;
    a.early_weights = ctx->pdl_early_weights;
    a.off_xsum = plan.off_xsum;
    a.off_red = plan.off_red;
    a.off_ring = plan.off_ring;
    a.red_slot_floats = plan.red_slot_floats;
}

// 1 to 4 projections that read the same activations (one launch; each writes its own outputs).
cudaError_t launch_qmv_stream(Ctx *ctx, cudaStream_t st, const mtc_qmv_desc *d, int n, const mtc_peer_sync *sync) {
    if (n < 1 || n > kMaxInline) return cudaErrorInvalidValue;
    SArgs a{};
    if (sync) {
        if (sync->n_peers < 1 || sync->n_peers > 8 || sync->rank < 0 || sync->rank >= sync->n_peers || !sync->local_flags ||
            !sync->epoch || !sync->ticket)
            return cudaErrorInvalidValue;
        for (int q = 0; q < sync->n_peers; ++q) {
            if (!sync->peer_flags[q]) return cudaErrorInvalidValue;
            a.peer_flags[q] = static_cast<uint32_t *>(sync->peer_flags[q]);
        }
        a.local_flags = static_cast<uint32_t *>(sync->local_flags);
        a.epoch = static_cast<uint32_t *>(sync->epoch);
        a.ticket = static_cast<uint32_t *>(sync->ticket);
        a.n_peers = sync->n_peers;
        a.rank = sync->rank;
        a.poll_limit = ctx->peer_poll_limit;
    }
    long long rows = 0;
    for (int i = 0; i < n; ++i) {
        if (d[i].x != d[0].x || d[i].M != d[0].M || d[i].K != d[0].K || d[i].dtype != d[0].dtype || d[i].group_size != d[0].group_size)
            return cudaErrorInvalidValue;
        fill_proj(a.inl[i], d[i].w, d[i].scales, d[i].biases, d[i].x, d[i].outs, d[i].n_outs, d[i].M, d[i].N, d[i].K,
                  d[i].group_size, 0);
        rows += d[i].N;
    }
    a.n_inl = n;
    const int M = d[0].M, K = d[0].K;
    const Plan plan = make_plan(M * K, K, M);
    if (plan.depth < 2) return cudaErrorInvalidValue;
    fill_layout(a, ctx, plan);
    // one CTA per resident slot of the machine, at least 8 rows each
    long long grid = static_cast<long long>(ctx->sm_count) * plan.per_sm;
    if (grid > (rows + 7) / 8) grid = (rows + 7) / 8;
    if (grid < 1) grid = 1;
    // Shares in whole row tiles once a CTA has more than one: 14336 + 14336 rows over 296 CTAs are 96.9 rows each, which
    // dealt by rows is seven passes (the last for one row) on 255 CTAs and dealt by tiles is six on 280 and seven on 16.
    a.unit_sh = rows / grid >= 16 ? 4 : 0;
    const long long units = (rows + (1 << a.unit_sh) - 1) >> a.unit_sh;
    a.rows_q = static_cast<int>(units / grid);
    a.rows_r = static_cast<int>(units % grid);
    return launch_stream_kernel(st, a, pick_kernel(d[0].dtype == MTC_BF16, d[0].group_size == 64 ? 0 : 1, M == 1, plan.depth),
                                static_cast<int>(grid), plan.smem);
}

// ---- chains: several projections, one persistent grid ------------------------------------------------------------

struct StreamChain {
    std::vector<SProj> projs;
    SProj *d_projs = nullptr;
    int4 *d_pieces = nullptr;
    uint32_t *d_sync = nullptr;
    int max_pieces = 0, n_phases = 0, grid = 0;
    KernelFn fn = nullptr;
    Plan plan;
};

void stream_chain_destroy(StreamChain *c) {
    if (!c) return;
    if (c->d_projs) cudaFree(c->d_projs);
    if (c->d_pieces) cudaFree(c->d_pieces);
    if (c->d_sync) cudaFree(c->d_sync);
    delete c;
}

// descs: n projections; phases must be non-decreasing.  Within a phase the rows of all projections are dealt to the
// CTAs in contiguous byte-balanced shares, so a CTA's list is a few (projection, row range) pieces per phase.
cudaError_t stream_chain_create(Ctx *ctx, const mtc_qmv_desc *descs, int n, StreamChain **out, std::string *why) {
    *out = nullptr;
    if (n < 1) {
        if (why) *why = "chain: no projections";
        return cudaErrorInvalidValue;
    }
    StreamChain *c = new StreamChain();
    int max_mk = 0, max_k = 0, max_m = 1;
    const int dt = descs[0].dtype, gs = descs[0].group_size;
    const bool m1 = descs[0].M == 1;
    int phase_prev = 0, n_phases = 1;
    for (int i = 0; i < n; ++i) {
        const mtc_qmv_desc &d = descs[i];
        if (d.dtype != dt || d.group_size != gs || (d.M == 1) != m1 || d.bits != 4 || d.n_outs < 1 || d.n_outs > 8 ||
            !qmv_stream_supported(d.M, d.N, d.K, d.bits, d.group_size, d.dtype, d.w, d.scales, d.biases, d.x)) {
            if (why) *why = "chain: projection " + std::to_string(i) + " is outside the streaming kernel's contract (4-bit, one of f16 / bf16 and "
                            "one group size (64 or 128) for the whole chain, M = 1 throughout or 2 <= M <= 8 throughout, K % 512 == 0, "
                            "16-byte aligned pointers)";
            delete c;
            return cudaErrorInvalidValue;
        }
        if (d.phase < phase_prev || d.phase > phase_prev + 1 || (i == 0 && d.phase != 0)) {
            if (why) *why = "chain: phases must start at 0 and grow by at most one from one projection to the next";
            delete c;
            return cudaErrorInvalidValue;
        }
        phase_prev = d.phase;
        n_phases = d.phase + 1;
        SProj p;
        fill_proj(p, d.w, d.scales, d.biases, d.x, d.outs, d.n_outs, d.M, d.N, d.K, d.group_size, d.phase);
        c->projs.push_back(p);
        if (d.M * d.K > max_mk) max_mk = d.M * d.K;
        if (d.K > max_k) max_k = d.K;
        if (d.M > max_m) max_m = d.M;
    }
    c->plan = make_plan(max_mk, max_k, max_m);
    if (c->plan.depth < 2) {
        if (why) *why = "chain: activations do not fit in shared memory";
        delete c;
        return cudaErrorInvalidValue;
    }
    c->grid = ctx->sm_count * c->plan.per_sm;
    c->n_phases = n_phases;
    c->fn = pick_kernel(dt == MTC_BF16, gs == 64 ? 0 : 1, m1, c->plan.depth);
    const int G = c->grid;
    // pieces per CTA
    std::vector<std::vector<int4>> lists(G);
    int i0 = 0;
    while (i0 < n) {
        int i1 = i0;
        while (i1 < n && descs[i1].phase == descs[i0].phase) ++i1;
        // cost of a row = its packed bytes (+ scales and biases)
        std::vector<double> row_cost(i1 - i0);
        double total = 0.0;
        for (int i = i0; i < i1; ++i) {
            row_cost[i - i0] = c->projs[i].rowbytes + 2.0 * c->projs[i].gpr2;
            total += row_cost[i - i0] * c->projs[i].N;
        }
        // CTA b takes cost range [b, b+1) * total / G; walk the projections
        double acc = 0.0;
        std::vector<size_t> first_len(G);
        for (int b = 0; b < G; ++b) first_len[b] = lists[b].size();
        for (int i = i0; i < i1; ++i) {
            const SProj &p = c->projs[i];
            const double rc = row_cost[i - i0];
            int row = 0;
            while (row < p.N) {
                int b = static_cast<int>((acc + 1e-9) * G / total);
                if (b >= G) b = G - 1;
                const double end_cost = (b + 1) * total / G;
                int rows = static_cast<int>((end_cost - acc) / rc + 0.5);
                if (rows < 1) rows = 1;
                if (row + rows > p.N) rows = p.N - row;
                lists[b].push_back(make_int4(i, row, row + rows, 0));
                acc += rows * rc;
                row += rows;
            }
        }
        for (int b = 0; b < G; ++b) {
            if (lists[b].size() == first_len[b]) lists[b].push_back(make_int4(i0, 0, 0, 0));     // nothing to do: still takes part in the phase
            if (descs[i0].phase > 0) lists[b][first_len[b]].w |= F_WAIT;
            lists[b].back().w |= F_SIGNAL;
        }
        i0 = i1;
    }
    // activations are staged when they differ from the ones in shared memory (or may have been rewritten: a new phase)
    size_t max_pieces = 0;
    for (int b = 0; b < G; ++b) {
        const void *cur_x = nullptr;
        int cur_m = -1, cur_k = -1;
        for (int4 &pc : lists[b]) {
            const SProj &p = c->projs[pc.x];
            if ((pc.w & F_WAIT) || p.x != cur_x || p.M != cur_m || p.K != cur_k) pc.w |= F_STAGE;
            cur_x = p.x;
            cur_m = p.M;
            cur_k = p.K;
        }
        if (lists[b].size() > max_pieces) max_pieces = lists[b].size();
    }
    c->max_pieces = static_cast<int>(max_pieces) + 1;
    std::vector<int4> flat(static_cast<size_t>(G) * c->max_pieces, make_int4(-1, 0, 0, 0));
    for (int b = 0; b < G; ++b)
        for (size_t q = 0; q < lists[b].size(); ++q) flat[static_cast<size_t>(b) * c->max_pieces + q] = lists[b][q];
    cudaError_t e;
    if ((e = cudaMalloc(&c->d_projs, c->projs.size() * sizeof(SProj))) != cudaSuccess ||
        (e = cudaMalloc(&c->d_pieces, flat.size() * sizeof(int4))) != cudaSuccess ||
        (e = cudaMalloc(&c->d_sync, (n_phases + 1) * sizeof(uint32_t))) != cudaSuccess ||
        (e = cudaMemcpy(c->d_projs, c->projs.data(), c->projs.size() * sizeof(SProj), cudaMemcpyHostToDevice)) != cudaSuccess ||
        (e = cudaMemcpy(c->d_pieces, flat.data(), flat.size() * sizeof(int4), cudaMemcpyHostToDevice)) != cudaSuccess ||
        (e = cudaMemset(c->d_sync, 0, (n_phases + 1) * sizeof(uint32_t))) != cudaSuccess) {
        stream_chain_destroy(c);
        return e;
    }
    *out = c;
    return cudaSuccess;
}

cudaError_t stream_chain_run(Ctx *ctx, cudaStream_t st, StreamChain *c) {
    SArgs a{};
    a.projs = c->d_projs;
    a.pieces = c->d_pieces;
    a.max_pieces = c->max_pieces;
    a.sync = c->d_sync;
    a.n_phases = c->n_phases;
    fill_layout(a, ctx, c->plan);
    if (c->n_phases > 1) {
        // CTAs wait for one another at phase boundaries: all of them must be resident, which a cooperative launch
        // guarantees (or refuses)
        void *args[] = {&a};
        return cudaLaunchCooperativeKernel(reinterpret_cast<const void *>(c->fn), dim3(c->grid), dim3(kThreads), args, c->plan.smem, st);
    }
    return launch_stream_kernel(st, a, c->fn, c->grid, c->plan.smem);
}

}  // namespace mtc
