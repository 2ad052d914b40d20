// qmv for 2 <= M <= 16 token rows with 4-bit codes and 16-bit activations, on the warp-level tensor
// cores (mma.sync m16n8k16, f32 accumulate).  Same contract as the CUDA-core kernel of qmv.cu:
//   out[m, n] = sum_k (q(n,k) * scale[n, k/G] + bias[n, k/G]) * x[m, k]
// (mt_qmm, mt_qmm_bm2, mt_qmm_bm4, mt_qmm_b4: crates/metaltile-std/src/mlx/quantized.rs:343-1441,4519-4523).
//
// Why: on CUDA cores every (code, token) pair costs one FFMA, so M = 8..16 is FFMA-bound at 5-10 % of
// the HBM roofline.  Here a code costs ~0.9 integer ops regardless of M: the integer codes themselves are
// the A operand (a code q < 16 is exact in bf16 and f16), the activations are the B operand, and the
// affine part is applied per group on the f32 accumulators,
//   acc += scale * (sum_k (OFF + q) x  -  OFF * sum_k x) + bias * sum_k x,
// where OFF (128 for bf16, 1024 for f16) is the exponent trick that turns `(word >> 4j) & 0x000F000F | magic`
// into two ready-made 16-bit floats OFF + q without any conversion instruction (qmv_mma_kernel).  The ring kernel
// (qmv_mma_ring_kernel) goes one step further, as the streaming decode kernel does: the codes are the A operand as they
// sit in the words - a 16-bit float with exponent field 0 is linear in its low bits - so a segment needs 16 LOP3 and
// 4 shifts instead of 16 + 12, no OFF correction, and the activations are staged pre-scaled (stage_x_ring).
//
// Mapping.  A warp owns 16 weight rows; lane = 4*g + t holds rows g and g+8.  Per 64-code segment a lane
// loads 8 bytes of each of its two rows (words 2t, 2t+1 of the segment), i.e. every byte of the packed
// matrix is loaded exactly once.  MMA j (j = 0..3) of a segment uses nibbles j and j+4 of those words, so
// its 16 k-slots are the k values {16t + j, 16t + j + 4, 16t + 8 + j, 16t + 8 + j + 4 : t = 0..3} of the
// segment; the contraction index may be permuted freely as long as the B operand follows, and B (the
// activations) is staged in shared memory in exactly that order.  No cross-lane reduction is needed.
// Group sizes that are multiples of 64 only (one scale/bias pair per segment and row).
#include "common.cuh"

namespace mtc {
namespace {

constexpr int kMmaWarps = 8;
constexpr int kStageBytes = 64 * 1024;   // activations staged at a time: 64 segments (4096 k) for M <= 8, 32 for M <= 16
constexpr int kMmaPF = 8;                // 64-code segments of packed words in flight per lane

struct MmaArgs {
    const uint32_t *w;
    const void *scales, *biases, *x;
    void *out;
    int M, N, K, gs_shift, dt;
    int wpr, gpr, nseg;      // words / groups per weight row, 64-code segments per row
    int tiles, ksplit_shift, iters;
    int block_segs;          // ring kernel: segments of x staged at a time (a multiple of 8 << ksplit_shift)
};

// d = a * b + (kZero ? 0 : d): m16n8k16, 16-bit operands, f32 accumulators
template <bool BF16, bool kZero>
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    if (kZero) {
        if (BF16)
            asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                         : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3])
                         : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(0.0f));
        else
            asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                         : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3])
                         : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(0.0f));
    } else {
        if (BF16)
            asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                         : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
        else
            asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                         : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
}

// Two codes of a packed word as two 16-bit floats OFF + q: nibbles j and j+4, one shift and one LOP3.
template <int J>
__device__ __forceinline__ uint32_t code_pair(uint32_t word, uint32_t magic) {
    uint32_t r;
    const uint32_t sh = J == 0 ? word : word >> (4 * J);
    asm("lop3.b32 %0, %1, 0x000F000F, %2, 0xEA;" : "=r"(r) : "r"(sh), "r"(magic));   // (sh & mask) | magic
    return r;
}

// All MMAs of one 64-code segment for the rows and tokens of this lane: d = sum (OFF + q) x, xs = sum x.
template <int NT, bool BF16, bool kSum = true>
__device__ __forceinline__ void segment_mmas(float (&d)[NT][4], float (&xs)[NT][4], const uint2 cl, const uint2 ch,
                                             const uint4 *frag /* this lane's chunk 0 of the segment */, int lane) {
    constexpr uint32_t magic = BF16 ? 0x43004300u : 0x64006400u;
    constexpr uint32_t one2 = BF16 ? 0x3F803F80u : 0x3C003C00u;
    const uint32_t ones[4] = {one2, one2, one2, one2};
    const int sw = (lane >> 2) & 1;                      // the XOR of frag_chunk
    uint4 bf[2][NT];
#pragma unroll
    for (int jp = 0; jp < 2; ++jp)
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) bf[jp][nt] = frag[nt * 64 + (jp ^ sw)];
#define MTC_STEP(J, ZERO)                                                                                 \
    {                                                                                                     \
        const uint32_t af[4] = {code_pair<J>(cl.x, magic), code_pair<J>(ch.x, magic), code_pair<J>(cl.y, magic), \
                                code_pair<J>(ch.y, magic)};                                               \
        _Pragma("unroll") for (int nt = 0; nt < NT; ++nt) {                                               \
            const uint4 f = bf[(J) >> 1][nt];                                                             \
            const uint32_t b0 = ((J) & 1) ? f.z : f.x, b1 = ((J) & 1) ? f.w : f.y;                        \
            mma16816<BF16, ZERO>(d[nt], af, b0, b1);                                                      \
            if (kSum) mma16816<BF16, ZERO>(xs[nt], ones, b0, b1);                                         \
        }                                                                                                 \
    }
    MTC_STEP(0, true)
    MTC_STEP(1, false)
    MTC_STEP(2, false)
    MTC_STEP(3, false)
#undef MTC_STEP
}

// Shared-memory address (in 16-byte chunks) of the B fragments of (segment s, token tile nt, lane, j pair jp):
// a lane's four uint2 fragments (j = 0..3) are 32 contiguous bytes, read as two 16-byte loads; the XOR keeps
// each quarter-warp of such a load on 32 distinct banks.
template <int NT>
__device__ __forceinline__ int frag_chunk(int s, int nt, int lane, int jp) {
    return ((s * NT + nt) * 32 + lane) * 2 + (jp ^ ((lane >> 2) & 1));
}

// Stage segments [seg0, seg0 + nseg) of x as B fragments in MMA order: a pure 16-bit permutation.
//   fragment j of lane 4*m' + t, token m = nt*8 + m':
//     .x = (x[m][64s+16t+j], x[m][64s+16t+j+4]) low half first, .y = the same 8 further on
template <int NT>
__device__ __forceinline__ void stage_x_mma(const MmaArgs &a, uint4 *xb, int seg0, int nseg) {
    const int total = nseg * NT * 32;                          // (segment, token, t) triples
    constexpr int U = 4;                                       // loads of U triples in flight per thread
    for (int base = threadIdx.x; base < total; base += blockDim.x * U) {
        uint4 v0[U], v1[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int i = base + u * blockDim.x;
            const int t = i & 3, m = (i >> 2) % (NT * 8), s = i / (NT * 32);
            v0[u] = v1[u] = make_uint4(0u, 0u, 0u, 0u);
            if (i < total && m < a.M) {
                const uint4 *p = reinterpret_cast<const uint4 *>(static_cast<const uint16_t *>(a.x) + static_cast<size_t>(m) * a.K +
                                                                 static_cast<size_t>(seg0 + s) * 64 + 16 * t);
                v0[u] = __ldg(p);       // x[16t + 0..7]  as halves h0..h7:  word q holds (h[2q], h[2q+1])
                v1[u] = __ldg(p + 1);   // x[16t + 8..15]
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int i = base + u * blockDim.x;
            if (i >= total) break;
            const int t = i & 3, m = (i >> 2) % (NT * 8), s = i / (NT * 32);
            // fragment j: .x = (h[j], h[j+4]) of v0, .y = the same of v1
            const uint4 f01 = make_uint4(__byte_perm(v0[u].x, v0[u].z, 0x5410), __byte_perm(v1[u].x, v1[u].z, 0x5410),      // j = 0
                                         __byte_perm(v0[u].x, v0[u].z, 0x7632), __byte_perm(v1[u].x, v1[u].z, 0x7632));     // j = 1
            const uint4 f23 = make_uint4(__byte_perm(v0[u].y, v0[u].w, 0x5410), __byte_perm(v1[u].y, v1[u].w, 0x5410),      // j = 2
                                         __byte_perm(v0[u].y, v0[u].w, 0x7632), __byte_perm(v1[u].y, v1[u].w, 0x7632));     // j = 3
            const int nt = m >> 3, lane = (m & 7) * 4 + t;
            xb[frag_chunk<NT>(s, nt, lane, 0)] = f01;
            xb[frag_chunk<NT>(s, nt, lane, 1)] = f23;
        }
    }
}

__device__ __forceinline__ float f32_of16(uint32_t h, bool bf16) {
    return bf16 ? __uint_as_float(h << 16) : __half2float(__ushort_as_half(static_cast<unsigned short>(h)));
}

template <int NT, bool BF16>
__global__ void __launch_bounds__(kMmaWarps * 32, 2) qmv_mma_kernel(const MmaArgs a) {
    extern __shared__ __align__(16) unsigned char smem_mma[];
    constexpr int kBlockSegs = kStageBytes / (NT * 1024);
    constexpr float off = BF16 ? 128.0f : 1024.0f;
    uint4 *xb = reinterpret_cast<uint4 *>(smem_mma);                               // kStageBytes of B fragments
    float *red = reinterpret_cast<float *>(smem_mma + kStageBytes);                // [warps][32][NT*4]

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int ksh = a.ksplit_shift, KS = 1 << ksh, slots = kMmaWarps >> ksh, slot = warp >> ksh, ks = warp & (KS - 1);
    // balanced contiguous partition of the 16-row tiles over the CTAs
    const int tile_begin = static_cast<int>((static_cast<long long>(blockIdx.x) * a.tiles) / gridDim.x);
    const int tile_end = static_cast<int>((static_cast<long long>(blockIdx.x + 1) * a.tiles) / gridDim.x);
    const int seg_step = KS;                            // this warp's segments: ks, ks + KS, ...
    const int per_block = kBlockSegs >> ksh;            // of which this many per staged block (a multiple of kMmaPF)
    const int nblocks = (a.nseg + kBlockSegs - 1) / kBlockSegs;
    const int grp_shift = a.gs_shift - 6;               // segment -> group

    asm volatile("griddepcontrol.launch_dependents;");
    bool waited = false;

    for (int it = 0; it < a.iters; ++it) {
        const int tile = tile_begin + it * slots + slot;
        const bool active = tile < tile_end;
        const int n_lo = tile * 16 + g, n_hi = n_lo + 8;
        const int r_lo = max(0, min(n_lo, a.N - 1)), r_hi = max(0, min(n_hi, a.N - 1));   // rows past N re-read the last row
        const uint2 *w_lo = reinterpret_cast<const uint2 *>(a.w + static_cast<size_t>(r_lo) * a.wpr) + t;   // + 4 uint2 per segment
        const uint2 *w_hi = reinterpret_cast<const uint2 *>(a.w + static_cast<size_t>(r_hi) * a.wpr) + t;
        const uint16_t *sc_lo = static_cast<const uint16_t *>(a.scales) + static_cast<size_t>(r_lo) * a.gpr;
        const uint16_t *sc_hi = static_cast<const uint16_t *>(a.scales) + static_cast<size_t>(r_hi) * a.gpr;
        const uint16_t *bi_lo = static_cast<const uint16_t *>(a.biases) + static_cast<size_t>(r_lo) * a.gpr;
        const uint16_t *bi_hi = static_cast<const uint16_t *>(a.biases) + static_cast<size_t>(r_hi) * a.gpr;
        float acc[NT][4];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int q = 0; q < 4; ++q) acc[nt][q] = 0.0f;

        // packed words of kMmaPF segments in flight per lane, requested before the activations are staged:
        // the weights do not depend on the previous kernel of the stream
        uint2 wl[kMmaPF], wh[kMmaPF];
        int s_req = ks;                                  // next segment to request
#pragma unroll
        for (int p = 0; p < kMmaPF; ++p) {
            if (active && s_req < a.nseg) {
                wl[p] = __ldg(w_lo + s_req * 4);
                wh[p] = __ldg(w_hi + s_req * 4);
            }
            s_req += seg_step;
        }
        if (!waited) {
            asm volatile("griddepcontrol.wait;" ::: "memory");
            waited = true;
        }

        for (int kb = 0; kb < nblocks; ++kb) {
            const int seg0 = kb * kBlockSegs;
            if (it == 0 || nblocks > 1) {                // one block holding all of K is kept across tiles
                __syncthreads();
                stage_x_mma<NT>(a, xb, seg0, min(kBlockSegs, a.nseg - seg0));
                __syncthreads();
            }
            if (!active) continue;
            int s = seg0 + ks;                           // this warp's next segment
            for (int r = 0; r < per_block; r += kMmaPF) {
                if (s >= a.nseg) break;
#pragma unroll
                for (int p = 0; p < kMmaPF; ++p) {
                    if (s < a.nseg) {
                        // scale and bias of this group for rows g and g+8, used after the MMAs
                        const int grp = s >> grp_shift;
                        const uint32_t rs_lo = __ldg(sc_lo + grp), rs_hi = __ldg(sc_hi + grp);
                        const uint32_t rb_lo = __ldg(bi_lo + grp), rb_hi = __ldg(bi_hi + grp);
                        const int sl = s & (kBlockSegs - 1);
                        float d[NT][4], xs[NT][4];
                        segment_mmas<NT, BF16>(d, xs, wl[p], wh[p], xb + (sl * NT * 32 + lane) * 2, lane);
                        // the slot is free: request the segment kMmaPF rounds ahead
                        if (s_req < a.nseg) {
                            wl[p] = __ldg(w_lo + s_req * 4);
                            wh[p] = __ldg(w_hi + s_req * 4);
                        }
                        // affine part on the accumulators this lane holds: rows g / g+8, tokens 2t, 2t+1
                        const float s_lo = f32_of16(rs_lo, BF16), s_hi = f32_of16(rs_hi, BF16);
                        const float b_lo = fmaf(-off, s_lo, f32_of16(rb_lo, BF16)), b_hi = fmaf(-off, s_hi, f32_of16(rb_hi, BF16));
#pragma unroll
                        for (int nt = 0; nt < NT; ++nt) {
                            acc[nt][0] = fmaf(s_lo, d[nt][0], fmaf(b_lo, xs[nt][0], acc[nt][0]));
                            acc[nt][1] = fmaf(s_lo, d[nt][1], fmaf(b_lo, xs[nt][1], acc[nt][1]));
                            acc[nt][2] = fmaf(s_hi, d[nt][2], fmaf(b_hi, xs[nt][0], acc[nt][2]));
                            acc[nt][3] = fmaf(s_hi, d[nt][3], fmaf(b_hi, xs[nt][1], acc[nt][3]));
                        }
                    }
                    s += seg_step;
                    s_req += seg_step;
                }
            }
        }

        if (KS > 1) {   // split-K: the warps of a slot add up in shared memory
            float *mine = red + (warp * 32 + lane) * (NT * 4);
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int q = 0; q < 4; ++q) mine[nt * 4 + q] = acc[nt][q];
            __syncthreads();
            if (ks == 0) {
                for (int o = 1; o < KS; ++o) {
                    const float *other = red + ((warp + o) * 32 + lane) * (NT * 4);
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                        for (int q = 0; q < 4; ++q) acc[nt][q] += other[nt * 4 + q];
                }
            }
            __syncthreads();   // the partial sums are rewritten by the next tile
        }
        if (active && ks == 0) {
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const int m0 = nt * 8 + 2 * t;
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const int m = m0 + (q & 1), n = (q & 2) ? n_hi : n_lo;
                    if (m < a.M && n < a.N) st_from_f32(a.out, static_cast<size_t>(m) * a.N + n, acc[nt][q], BF16 ? MTC_BF16 : MTC_F16);
                }
            }
        }
    }
    if (!waited) asm volatile("griddepcontrol.wait;" ::: "memory");
}

// ---- group size 64, 128 or 256, K a multiple of 512: packed words through a shared-memory ring ----
// Loading the A fragments straight from global memory costs one 32-byte sector per row and instruction, eight
// cache lines per warp-load, and the L1 tag stage becomes the limit.  Here a warp copies a run of 8 consecutive
// segments of its 16 rows (16 x 256 bytes of packed words, plus the 16, 8 or 4 bytes of scales and of biases that
// 8, 4 or 2 groups per row take) with
// 16-byte asynchronous copies that cover whole lines and bypass L1, into a private two-deep ring, and reads the
// fragments back with conflict-free 8-byte shared loads.  No register holds data in flight.
constexpr int kRingWarps = 16;
constexpr int kRunWBytes = 16 * 256;                 // packed words of a run: 16 rows x 8 segments x 32 bytes
constexpr int kRunBytes = kRunWBytes + 2 * 256;      // + scales and biases: 16 rows x 8 groups x 2 bytes each

template <int BYTES>
__device__ __forceinline__ void cp_async_small(uint32_t dst, const void *src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], %2;" ::"r"(dst), "l"(src), "n"(BYTES) : "memory");
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
// Activations of the ring kernel: only the M real tokens are staged, so M = 1 keeps 32768 k values resident and
// every practical K is staged once per CTA.  16-byte unit of (segment s, token m, quad-lane t, half h):
//   ((s*M + m)*4 + t)*2 + (h ^ (m & 1));  half h holds the fragments j = 2h, 2h+1 of stage_x_mma's order.
// The fragments of the odd MMAs of a segment (j = 1, 3: the nibbles at bits 4-7, which enter the product as 16 q) hold
// x / 16; bf16 activations are staged times 2^64 (2^60) so that products with the codes - read in place as bf16
// subnormals q * 2^-133 - stay normal numbers; both changes of exponent are exact (f16: unless |x| < 2^-10, where the
// quotient is a subnormal f16: absolute error below 2^-25).  xsum[s * Mp + m] = sum of the 64 unscaled activations of
// (segment s, token m) in f32; tokens M .. Mp - 1 (padding) get 0.
template <bool BF16>
__device__ __forceinline__ void stage_x_ring(const MmaArgs &a, uint4 *xb, float *xsum, int Mp, int seg0, int nseg) {
    // thread -> quad-lane t (2 bits), token m (mb bits), segment = pass * s_step + (thread >> (2 + mb)): no division
    const int mb = a.M <= 1 ? 0 : a.M <= 2 ? 1 : a.M <= 4 ? 2 : a.M <= 8 ? 3 : 4;
    const int t = threadIdx.x & 3, m = (threadIdx.x >> 2) & ((1 << mb) - 1), s_first = threadIdx.x >> (2 + mb),
              s_step = blockDim.x >> (2 + mb);
    if (m >= Mp) return;
    const bool real = m < a.M;                                   // a padding token only zeroes its sums
    const unsigned quad = 0xFu << (threadIdx.x & 28);            // the four lanes of a quad share (m, s) and stay together
    constexpr int U = 4;
    const uint16_t *xrow = static_cast<const uint16_t *>(a.x) + static_cast<size_t>(real ? m : 0) * a.K + static_cast<size_t>(seg0) * 64 + 16 * t;
    for (int s0 = s_first; s0 < nseg; s0 += s_step * U) {
        uint4 v0[U], v1[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int s = s0 + u * s_step;
            v0[u] = v1[u] = make_uint4(0u, 0u, 0u, 0u);
            if (s < nseg && real) {
                const uint4 *p = reinterpret_cast<const uint4 *>(xrow + static_cast<size_t>(s) * 64);
                v0[u] = __ldg(p);
                v1[u] = __ldg(p + 1);
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int s = s0 + u * s_step;
            if (s >= nseg) break;
            const uint32_t raw[8] = {v0[u].x, v0[u].y, v0[u].z, v0[u].w, v1[u].x, v1[u].y, v1[u].z, v1[u].w};
            float sum = 0.0f;
#pragma unroll
            for (int q = 0; q < 8; ++q) {
                if (BF16) {
                    sum += __uint_as_float(raw[q] << 16) + __uint_as_float(raw[q] & 0xFFFF0000u);
                } else {
                    const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&raw[q]));
                    sum += f.x + f.y;
                }
            }
            sum += __shfl_xor_sync(quad, sum, 1);
            sum += __shfl_xor_sync(quad, sum, 2);
            if (t == 0) xsum[s * Mp + m] = sum;
            if (!real) continue;
            uint4 f01 = make_uint4(__byte_perm(v0[u].x, v0[u].z, 0x5410), __byte_perm(v1[u].x, v1[u].z, 0x5410),
                                   __byte_perm(v0[u].x, v0[u].z, 0x7632), __byte_perm(v1[u].x, v1[u].z, 0x7632));
            uint4 f23 = make_uint4(__byte_perm(v0[u].y, v0[u].w, 0x5410), __byte_perm(v1[u].y, v1[u].w, 0x5410),
                                   __byte_perm(v0[u].y, v0[u].w, 0x7632), __byte_perm(v1[u].y, v1[u].w, 0x7632));
            if (BF16) {
                asm("mul.rn.bf16x2 %0, %0, %1;" : "+r"(f01.x) : "r"(0x5F805F80u));      // 2^64
                asm("mul.rn.bf16x2 %0, %0, %1;" : "+r"(f01.y) : "r"(0x5F805F80u));
                asm("mul.rn.bf16x2 %0, %0, %1;" : "+r"(f23.x) : "r"(0x5F805F80u));
                asm("mul.rn.bf16x2 %0, %0, %1;" : "+r"(f23.y) : "r"(0x5F805F80u));
                asm("mul.rn.bf16x2 %0, %0, %1;" : "+r"(f01.z) : "r"(0x5D805D80u));      // 2^60
                asm("mul.rn.bf16x2 %0, %0, %1;" : "+r"(f01.w) : "r"(0x5D805D80u));
                asm("mul.rn.bf16x2 %0, %0, %1;" : "+r"(f23.z) : "r"(0x5D805D80u));
                asm("mul.rn.bf16x2 %0, %0, %1;" : "+r"(f23.w) : "r"(0x5D805D80u));
            } else {
                const __half2 sixteenth = __float2half2_rn(0.0625f);
                *reinterpret_cast<__half2 *>(&f01.z) = __hmul2(*reinterpret_cast<__half2 *>(&f01.z), sixteenth);
                *reinterpret_cast<__half2 *>(&f01.w) = __hmul2(*reinterpret_cast<__half2 *>(&f01.w), sixteenth);
                *reinterpret_cast<__half2 *>(&f23.z) = __hmul2(*reinterpret_cast<__half2 *>(&f23.z), sixteenth);
                *reinterpret_cast<__half2 *>(&f23.w) = __hmul2(*reinterpret_cast<__half2 *>(&f23.w), sixteenth);
            }
            const int i = (s * a.M + m) * 4 + t;
            xb[i * 2 + (m & 1)] = f01;
            xb[i * 2 + ((m & 1) ^ 1)] = f23;
        }
    }
}

template <int NT, bool BF16, bool kFull /* M == 8 * NT: every lane has a token, strides are constants */,
          int GSH /* log2(group / 64): 0, 1 or 2 - a run of 8 segments holds 8, 4 or 2 groups per row */>
__global__ void __launch_bounds__(kRingWarps * 32, 1) qmv_mma_ring_kernel(const MmaArgs a) {
    extern __shared__ __align__(1024) unsigned char smem_mma[];
    uint4 *xb = reinterpret_cast<uint4 *>(smem_mma);
    unsigned char *ring_all = smem_mma + kStageBytes;                                   // [warps][2][kRunBytes]
    float *red = reinterpret_cast<float *>(ring_all + kRingWarps * 2 * kRunBytes);      // [warps][32][NT*4]
    float *xsum = red + kRingWarps * 32 * NT * 4;                // [block_segs][Mp]: sum of x per segment and token
    unsigned char *zeros = reinterpret_cast<unsigned char *>(xsum) + (NT == 1 ? 4096 : 2048);   // 32 bytes

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int ksh = a.ksplit_shift, KS = 1 << ksh, slots = kRingWarps >> ksh, slot = warp >> ksh, ks = warp & (KS - 1);
    const int tile_begin = static_cast<int>((static_cast<long long>(blockIdx.x) * a.tiles) / gridDim.x);
    const int tile_end = static_cast<int>((static_cast<long long>(blockIdx.x + 1) * a.tiles) / gridDim.x);
    const int block_segs = a.block_segs;
    const int chunk = block_segs >> ksh;                 // consecutive segments of a staged block owned by this warp
    const int runs = chunk >> 3;                         // runs of 8 segments per block
    const int nblocks = (a.nseg + block_segs - 1) / block_segs;
    const int Mtok = kFull ? NT * 8 : a.M;
    const int Mp = kFull ? NT * 8 : (a.M + 1) & ~1;
    unsigned char *ring_p = ring_all + warp * 2 * kRunBytes;
    const uint32_t ring = static_cast<uint32_t>(__cvta_generic_to_shared(ring_p));
    const unsigned char *smem0 = smem_mma;               // shared-memory loads below are plain loads at byte offsets from here
    const uint32_t xb_s = 0;

    asm volatile("griddepcontrol.launch_dependents;");

    // ---- copy side: lane l moves chunk (l & 15) of rows 2i + (l >> 4), i = 0..7, and 16 bytes of scales
    //      (even lanes) or biases (odd lanes) of row l >> 1.  Chunk c of row r lands at c ^ ((r & 3) << 1). ----
    const int c_row = lane >> 4, c_chunk = lane & 15, c_srow = lane >> 1;
    const char *c_sb = static_cast<const char *>((lane & 1) ? a.biases : a.scales);
    const size_t w_pitch = static_cast<size_t>(a.wpr) * 4, sb_pitch = static_cast<size_t>(a.gpr) * 2;
    auto issue = [&](int tile, int s_run, int buf) {
        const uint32_t dst = ring + buf * kRunBytes;
        const int row0 = tile * 16;
        const char *src0 = reinterpret_cast<const char *>(a.w) + static_cast<size_t>(s_run) * 32 + c_chunk * 16;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int row = 2 * i + c_row;
            const int gr = min(row0 + row, a.N - 1);                    // rows past N re-read the last row
            cp_async16(dst + row * 256 + ((c_chunk ^ ((row & 3) << 1)) << 4), src0 + gr * w_pitch);
        }
        const int gr = min(row0 + c_srow, a.N - 1);
        const uint32_t sdst = dst + kRunWBytes + (lane & 1) * 256 + c_srow * 16;
        const char *ssrc = c_sb + gr * sb_pitch + static_cast<size_t>(s_run >> GSH) * 2;
        if (GSH == 0) cp_async16(sdst, ssrc);
        else if (GSH == 1) cp_async_small<8>(sdst, ssrc);
        else cp_async_small<4>(sdst, ssrc);
    };
    // the runs of this warp in the order (tile, block, run); the copies run one run ahead, across tiles
    int it_n = 0, kb_n = 0, r_n = -1, s_n = 0, tile_n = tile_begin + slot;
    bool have_n = false;
    auto advance = [&]() {
        have_n = false;
        for (;;) {
            if (++r_n == runs) {
                r_n = 0;
                if (++kb_n == nblocks) {
                    kb_n = 0;
                    ++it_n;
                    tile_n += slots;
                }
            }
            if (it_n >= a.iters || tile_n >= tile_end) break;
            s_n = kb_n * block_segs + ks * chunk + r_n * 8;
            if (s_n < a.nseg) {
                have_n = true;
                break;
            }
        }
    };
    advance();
    if (have_n) issue(tile_n, s_n, 0);
    asm volatile("cp.async.commit_group;" ::: "memory");
    // the weights do not depend on the previous kernel of the stream; the activations and the stores do
    asm volatile("griddepcontrol.wait;" ::: "memory");

    const uint32_t lane_w = g * 256 + ((g & 3) << 5) + t * 8;           // fragment address within a run: ^ (p << 5)
    // B fragments of this lane: token nt*8 + g, quad-lane t.  Lanes without a token read 32 bytes of zeros with
    // stride 0 instead of branching; the same for the sums of tokens 2t, 2t+1.
    const uint32_t zero_s = static_cast<uint32_t>(zeros - smem_mma);
    uint32_t lane_x[NT], x_stride[NT], lane_xs[NT], xs_stride[NT];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        const bool has = kFull || nt * 8 + g < Mtok;
        lane_x[nt] = has ? xb_s + ((nt * 8 + g) * 4 + t) * 32 + ((g & 1) << 4) : zero_s;    // + segment * M * 128; halves at ^ 16
        x_stride[nt] = has ? Mtok * 128 : 0;
        const bool has_s = kFull || nt * 8 + 2 * t < Mp;
        lane_xs[nt] = has_s ? static_cast<uint32_t>(reinterpret_cast<unsigned char *>(xsum + nt * 8 + 2 * t) - smem_mma) : zero_s;   // + segment * Mp * 4
        xs_stride[nt] = has_s ? Mp * 4 : 0;
    }
    if (threadIdx.x < 8) reinterpret_cast<uint32_t *>(zeros)[threadIdx.x] = 0u;     // visible after the first barrier below
    auto load_frags = [&](int sl, uint4 (&bf)[2][NT]) {
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            const uint32_t addr = lane_x[nt] + sl * x_stride[nt];
            bf[0][nt] = *reinterpret_cast<const uint4 *>(smem0 + addr);
            bf[1][nt] = *reinterpret_cast<const uint4 *>(smem0 + (addr ^ 16));
        }
    };
    int buf = 0;
    for (int it = 0; it < a.iters; ++it) {
        const int tile = tile_begin + it * slots + slot;
        const bool active = tile < tile_end;
        float acc[NT][4];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int q = 0; q < 4; ++q) acc[nt][q] = 0.0f;

        for (int kb = 0; kb < nblocks; ++kb) {
            if (it == 0 || nblocks > 1) {                // one block holding all of K is kept across tiles
                const int nsb = min(block_segs, a.nseg - kb * block_segs);
                __syncthreads();
                stage_x_ring<BF16>(a, xb, xsum, Mp, kb * block_segs, nsb);     // fragments and per-segment sums, once per block
                __syncthreads();
            }
            if (!active) continue;
            for (int r = 0; r < runs; ++r) {
                const int sl0 = ks * chunk + r * 8;                      // first segment of the run within the block
                if (kb * block_segs + sl0 >= a.nseg) break;
                __syncwarp();                                            // every lane is done with the other buffer
                advance();
                if (have_n) issue(tile_n, s_n, buf ^ 1);
                asm volatile("cp.async.commit_group;" ::: "memory");
                asm volatile("cp.async.wait_group 1;" ::: "memory");     // this run has landed (this lane's copies)
                __syncwarp();                                            // ... and every other lane's
                const unsigned char *rb = ring_p + buf * kRunBytes;
                const uint4 v0 = *reinterpret_cast<const uint4 *>(rb + kRunWBytes + g * 16), v1 = *reinterpret_cast<const uint4 *>(rb + kRunWBytes + (g + 8) * 16);
                const uint4 v2 = *reinterpret_cast<const uint4 *>(rb + kRunWBytes + 256 + g * 16), v3 = *reinterpret_cast<const uint4 *>(rb + kRunWBytes + 256 + (g + 8) * 16);
                const uint32_t sp[4][4] = {{v0.x, v0.y, v0.z, v0.w}, {v1.x, v1.y, v1.z, v1.w},
                                           {v2.x, v2.y, v2.z, v2.w}, {v3.x, v3.y, v3.z, v3.w}};   // [s_lo, s_hi, b_lo, b_hi][pair]
                const unsigned char *wrun = rb;
#pragma unroll
                for (int p = 0; p < 8; ++p) {
                    const uint2 cl = *reinterpret_cast<const uint2 *>(wrun + (lane_w ^ (p << 5)));
                    const uint2 ch = *reinterpret_cast<const uint2 *>(wrun + (lane_w ^ (p << 5)) + 8 * 256);
                    uint4 bf[2][NT];
                    load_frags(sl0 + p, bf);
                    float d[NT][4], xs[NT][2];
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) {
                        const float2 v = *reinterpret_cast<const float2 *>(smem0 + lane_xs[nt] + (sl0 + p) * xs_stride[nt]);
                        xs[nt][0] = v.x;
                        xs[nt][1] = v.y;
                    }
                    // the codes are the A operand as they sit in the words: a 16-bit float with exponent field 0 is linear
                    // in its low bits, so `word & 0x000F000F` is two operands q * c and `word & 0x00F000F0` two operands
                    // 16 q * c (met by x / 16); one shift by 8 gives the other four nibbles
                    const uint32_t wl[2][4] = {{cl.x, ch.x, cl.y, ch.y}, {cl.x >> 8, ch.x >> 8, cl.y >> 8, ch.y >> 8}};
#define MTC_STEP(J, ZERO)                                                                                 \
    {                                                                                                     \
        constexpr uint32_t msk = ((J) & 1) ? 0x00F000F0u : 0x000F000Fu;                                   \
        const uint32_t af[4] = {wl[(J) >> 1][0] & msk, wl[(J) >> 1][1] & msk, wl[(J) >> 1][2] & msk, wl[(J) >> 1][3] & msk}; \
        _Pragma("unroll") for (int nt = 0; nt < NT; ++nt) {                                               \
            const uint4 f = bf[(J) >> 1][nt];                                                             \
            mma16816<BF16, ZERO>(d[nt], af, ((J) & 1) ? f.z : f.x, ((J) & 1) ? f.w : f.y);                \
        }                                                                                                 \
    }
                    MTC_STEP(0, true)
                    MTC_STEP(1, false)
                    MTC_STEP(2, false)
                    MTC_STEP(3, false)
#undef MTC_STEP
                    const int gi = p >> GSH, q = gi >> 1;        // group of this segment within the run, its 32-bit pair
                    float s_lo, s_hi, o_lo, o_hi;
                    if (BF16) {
                        s_lo = __uint_as_float((gi & 1) ? (sp[0][q] & 0xFFFF0000u) : (sp[0][q] << 16));
                        s_hi = __uint_as_float((gi & 1) ? (sp[1][q] & 0xFFFF0000u) : (sp[1][q] << 16));
                        o_lo = __uint_as_float((gi & 1) ? (sp[2][q] & 0xFFFF0000u) : (sp[2][q] << 16));
                        o_hi = __uint_as_float((gi & 1) ? (sp[3][q] & 0xFFFF0000u) : (sp[3][q] << 16));
                    } else {
                        const __half2 h0 = *reinterpret_cast<const __half2 *>(&sp[0][q]), h1 = *reinterpret_cast<const __half2 *>(&sp[1][q]);
                        const __half2 h2 = *reinterpret_cast<const __half2 *>(&sp[2][q]), h3 = *reinterpret_cast<const __half2 *>(&sp[3][q]);
                        s_lo = (gi & 1) ? __high2float(h0) : __low2float(h0);
                        s_hi = (gi & 1) ? __high2float(h1) : __low2float(h1);
                        o_lo = (gi & 1) ? __high2float(h2) : __low2float(h2);
                        o_hi = (gi & 1) ? __high2float(h3) : __low2float(h3);
                    }
                    // c * 2^(pre-scale) leaves with the scale: f16 codes are q * 2^-24; bf16 codes q * 2^-133 against x * 2^64
                    constexpr float post = BF16 ? 5.9029581035870565e20f /* 2^69 */ : 16777216.0f /* 2^24 */;
                    s_lo *= post;
                    s_hi *= post;
                    const float b_lo = o_lo, b_hi = o_hi;
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) {
                        acc[nt][0] = fmaf(s_lo, d[nt][0], fmaf(b_lo, xs[nt][0], acc[nt][0]));
                        acc[nt][1] = fmaf(s_lo, d[nt][1], fmaf(b_lo, xs[nt][1], acc[nt][1]));
                        acc[nt][2] = fmaf(s_hi, d[nt][2], fmaf(b_hi, xs[nt][0], acc[nt][2]));
                        acc[nt][3] = fmaf(s_hi, d[nt][3], fmaf(b_hi, xs[nt][1], acc[nt][3]));
                    }
                }
                buf ^= 1;
            }
        }

        if (KS > 1) {   // split-K: the warps of a slot add up in shared memory
            float *mine = red + (warp * 32 + lane) * (NT * 4);
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int q = 0; q < 4; ++q) mine[nt * 4 + q] = acc[nt][q];
            __syncthreads();
            if (ks == 0) {
                for (int o = 1; o < KS; ++o) {
                    const float *other = red + ((warp + o) * 32 + lane) * (NT * 4);
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                        for (int q = 0; q < 4; ++q) acc[nt][q] += other[nt * 4 + q];
                }
            }
            __syncthreads();   // the partial sums are rewritten by the next tile
        }
        if (active && ks == 0) {
            const int n_lo = tile * 16 + g, n_hi = n_lo + 8;
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const int m0 = nt * 8 + 2 * t;
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const int m = m0 + (q & 1), n = (q & 2) ? n_hi : n_lo;
                    if (m < a.M && n < a.N) st_from_f32(a.out, static_cast<size_t>(m) * a.N + n, acc[nt][q], BF16 ? MTC_BF16 : MTC_F16);
                }
            }
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
}

template <int NT>
constexpr size_t ring_smem_bytes() {
    return static_cast<size_t>(kStageBytes) + static_cast<size_t>(kRingWarps) * 2 * kRunBytes +
           static_cast<size_t>(kRingWarps) * 32 * NT * 4 * sizeof(float) + (NT == 1 ? 4096 : 2048) + 64;
}

template <int NT, bool BF16, int GSH>
cudaError_t launch_ring(Ctx *ctx, cudaStream_t st, MmaArgs a) {
    const int sms = ctx->sm_count;
    a.tiles = (a.N + 15) / 16;
    int grid = a.tiles < sms ? a.tiles : sms;
    const int max_tiles = (a.tiles + grid - 1) / grid;
    // K split over the warps of a CTA: the split with the fewest runs on the busiest warp (then the fewest
    // barriers), ties to the smaller.  A staged block holds kStageBytes / (M * 128) segments at most and is a
    // multiple of 8 segments per warp of the split.
    const int cap = kStageBytes / (a.M * 128);
    int best_ksh = 0, best_block = 0;
    long best_cost = -1;
    for (int ksh = 0; (1 << ksh) <= kRingWarps && (8 << ksh) <= cap; ++ksh) {
        const int unit = 8 << ksh;
        int block = (a.nseg + unit - 1) / unit * unit;
        if (block > cap) block = cap / unit * unit;
        const int nblocks = (a.nseg + block - 1) / block;
        const int slots = kRingWarps >> ksh;
        const long iters = (max_tiles + slots - 1) / slots;
        const long cost = iters * nblocks * ((block >> ksh) / 8) * 16 + iters * nblocks;
        if (best_cost < 0 || cost < best_cost) {
            best_cost = cost;
            best_ksh = ksh;
            best_block = block;
        }
    }
    a.block_segs = best_block;
    a.ksplit_shift = best_ksh;
    const int slots = kRingWarps >> best_ksh;
    a.iters = (max_tiles + slots - 1) / slots;
    constexpr size_t smem = ring_smem_bytes<NT>();
    static PerDeviceAttr attr_full, attr_part;
    cudaError_t e = attr_full.set(qmv_mma_ring_kernel<NT, BF16, true, GSH>, smem);
    if (e == cudaSuccess) e = attr_part.set(qmv_mma_ring_kernel<NT, BF16, false, GSH>, smem);
    if (e != cudaSuccess) return e;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kRingWarps * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (a.M == NT * 8) return cudaLaunchKernelEx(&cfg, qmv_mma_ring_kernel<NT, BF16, true, GSH>, a);
    return cudaLaunchKernelEx(&cfg, qmv_mma_ring_kernel<NT, BF16, false, GSH>, a);
}

template <int NT>
constexpr size_t mma_smem_bytes() {
    return static_cast<size_t>(kStageBytes) + 2 * static_cast<size_t>(kMmaWarps) * 32 * NT * 4 * sizeof(float);
}

template <int NT, bool BF16>
cudaError_t launch_mma(Ctx *ctx, cudaStream_t st, MmaArgs a) {
    const int sms = ctx->sm_count;
    constexpr int kBlockSegs = kStageBytes / (NT * 1024);
    a.tiles = (a.N + 15) / 16;
    // split K over the warps of a CTA while every warp keeps a full round of segments per staged block and
    // the grid is short of two CTAs per SM
    int ksh = 0;
    while ((2 << ksh) <= kMmaWarps && (a.tiles << ksh) < sms * 2 * kMmaWarps && a.nseg >= (2 << ksh) * kMmaPF &&
           (kBlockSegs >> (ksh + 1)) >= kMmaPF)
        ++ksh;
    a.ksplit_shift = ksh;
    const int slots = kMmaWarps >> ksh;
    int grid = (a.tiles + slots - 1) / slots;
    if (grid > sms * 2) grid = sms * 2;
    if (grid < 1) grid = 1;
    const int max_tiles = (a.tiles + grid - 1) / grid;
    a.iters = (max_tiles + slots - 1) / slots;
    constexpr size_t smem = mma_smem_bytes<NT>();
    auto kernel = qmv_mma_kernel<NT, BF16>;
    static PerDeviceAttr smem_attr;
    cudaError_t e = smem_attr.set(qmv_mma_kernel<NT, BF16>, smem);
    if (e != cudaSuccess) return e;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kMmaWarps * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, a);
}

}  // namespace

bool qmv_mma_supported(int M, int N, int K, int bits, int group_size, int dt, const void *w, const void *x) {
    const auto al = [](const void *p, size_t a) { return reinterpret_cast<uintptr_t>(p) % a == 0; };
    return bits == 4 && M >= 2 && M <= 16 && N > 0 && (dt == MTC_BF16 || dt == MTC_F16) && K % 64 == 0 &&
           group_size >= 64 && (group_size & (group_size - 1)) == 0 && K % group_size == 0 && al(w, 16) && al(x, 16);
}

cudaError_t launch_qmv_mma(Ctx *ctx, cudaStream_t st, const void *w, const void *scales, const void *biases, const void *x,
                           void *out, int M, int N, int K, int group_size, int dt) {
    MmaArgs a{};
    a.w = static_cast<const uint32_t *>(w);
    a.scales = scales;
    a.biases = biases;
    a.x = x;
    a.out = out;
    a.M = M; a.N = N; a.K = K; a.dt = dt;
    a.gs_shift = 0;
    while ((1 << a.gs_shift) < group_size) ++a.gs_shift;
    a.wpr = K / 8;
    a.gpr = K / group_size;
    a.nseg = K / 64;
    const auto al16 = [](const void *p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; };
    if (group_size <= 256 && K % 512 == 0 && al16(scales) && al16(biases)) {
#define MTC_RING(GSH_)                                                                                              \
    if (dt == MTC_BF16) return M <= 8 ? launch_ring<1, true, GSH_>(ctx, st, a) : launch_ring<2, true, GSH_>(ctx, st, a); \
    return M <= 8 ? launch_ring<1, false, GSH_>(ctx, st, a) : launch_ring<2, false, GSH_>(ctx, st, a);
        if (group_size == 64) { MTC_RING(0) }
        if (group_size == 128) { MTC_RING(1) }
        { MTC_RING(2) }
#undef MTC_RING
    }
    if (dt == MTC_BF16) return M <= 8 ? launch_mma<1, true>(ctx, st, a) : launch_mma<2, true>(ctx, st, a);
    return M <= 8 ? launch_mma<1, false>(ctx, st, a) : launch_mma<2, false>(ctx, st, a);
}

}  // namespace mtc
