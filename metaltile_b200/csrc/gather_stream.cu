// gather_stream — the grouped (mixture-of-experts) quantized product for SMALL expert groups as a weight stream:
//
//   out[r, n] = sum_k (q(e, n, k) * scale[e, n, k/G] + bias[e, n, k/G]) * x[r, k],   e = the expert that owns row r
//
// x rows are sorted by expert (expert_offsets, CSR).  Stands in for mt_moe_gather_qmm_int4{,_m8,_m16,_m32}
// (crates/metaltile-std/src/ffai/moe.rs:358-1363) when an expert sees a few dozen rows: then the layer is bound by
// reading every expert's packed matrix once, exactly like a decode projection, and the kernel is built like the decode
// stream (qmv_stream.cu): every warp copies its own 16-row slices of the packed matrix into a private shared-memory
// ring with 16-byte asynchronous copies and multiplies them on the warp-level tensor cores with the integer codes as
// the A operand (a 16-bit float with exponent field 0 is linear in its low bits - no conversion, 5 integer instructions
// per 8 codes), here against up to four 8-row token tiles at once, so that the extraction is paid once per 32 rows.
//
// Work.  A PASS is (expert, up to TB of its rows); its activations sit in shared memory for every warp of the CTA, in
// MMA fragment order.  A pass has ceil(n_out / 32) row tiles; a tile is one warp's unit of work (all of K, so no
// cross-warp sums): 32 weight rows against up to 32 token rows, so that every activation fragment read from shared
// memory meets two code fragments and every code fragment four activation fragments.  The (pass, tile) pairs, weighted by the token tiles of their pass, are dealt to the CTAs as
// contiguous ranges of equal weight; a warp's copy side runs ahead of its arithmetic across tiles and passes.
//
// A preparation kernel writes the activations once in fragment order (pre-scaled as the decode kernel stages them:
// bf16 times 2^64, the nibbles at bits 4-7 against x / 16) with the per-segment sums, and builds the table of passes
// from expert_offsets, so staging a pass is a plain asynchronous copy.
#include "common.cuh"

namespace mtc {
namespace {

constexpr int kGW = 8;                         // warps per CTA; one CTA per SM (a warp holds a 32 x 32 block of sums)
constexpr int kGTileRows = 32;                 // weight rows of a tile: two MMA row blocks that share every activation fragment
constexpr int kGThreads = kGW * 32;
constexpr int kGRunSegs = 4;                   // 64-code segments per run: 256 codes, 128 bytes per weight row
constexpr int kGPitch = 144;                   // 128 bytes of a run + 16: rows two apart land 8 banks apart
constexpr int kGSlotW = kGTileRows * kGPitch;  // packed words of a run: 32 rows
constexpr int kGSlotBytes = kGSlotW + 512;     // + scales [32 rows x 8 B], biases [32 rows x 8 B]
constexpr int kGMaxPasses = 4096;
constexpr uint32_t kGOffX = 128;

struct GPass {
    int expert, tok0, ntok;
    int cost0;            // weight of the passes before this one (a pass weighs 2 + its token tiles, per row tile)
};
struct GTable {
    int n_pass, total_cost, overflow, pad;
    GPass pass[kGMaxPasses];
};

struct GArgs {
    const uint32_t *w;
    const void *scales, *biases;
    const uint32_t *w2;              // a second matrix set of the same shape that reads the same rows (gate and up), or null
    const void *scales2, *biases2;
    void *out2;
    int tpe1;                        // row tiles of the first matrix: tile indices from tpe1 on belong to the second
    const unsigned char *xfrag;      // [m_total][K / 64][4][2] units of 16 bytes
    const float *xsum;               // [m_total][K / 64]
    const GTable *table;
    void *out;
    uint32_t *status;
    int n_out, K, TB;
    int tiles_per_expert;            // ceil(n_out / 32)
    int rowbytes, gpr2;              // bytes per weight row, bytes per row of scales
    uint32_t off_xsum, off_ring;
};

__device__ __forceinline__ uint32_t gs_u32(const void *p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void g_cp16(uint32_t dst, const void *src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void g_cp8(uint32_t dst, const void *src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void g_cp4(uint32_t dst, const void *src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void g_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int DEPTH>
__device__ __forceinline__ void g_wait_oldest() {       // all but the newest DEPTH-1 groups have landed
    if (DEPTH == 2) asm volatile("cp.async.wait_group 1;" ::: "memory");
    else if (DEPTH == 3) asm volatile("cp.async.wait_group 2;" ::: "memory");
    else asm volatile("cp.async.wait_group 3;" ::: "memory");
}

template <bool BF16, bool kZero>
__device__ __forceinline__ void g_hmma(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
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

template <bool BF16>
__device__ __forceinline__ float g_f32_of_half(uint32_t word, int hi) {
    if (BF16) return __uint_as_float(hi ? (word & 0xFFFF0000u) : (word << 16));
    const __half2 v = *reinterpret_cast<const __half2 *>(&word);
    return hi ? __high2float(v) : __low2float(v);
}

// ---- preparation: the table of passes, and the activations in fragment order ---------------------------------------
//
// Block 0 walks expert_offsets: expert e with r rows gives ceil(r / TB) passes.  Offsets that are not monotone or reach
// past m_total are clamped (the rows they would have named are left out) and reported in the status word (0x901).
// Every block converts rows: the four lanes of a quad share (row, segment); lane t reads x[16t .. 16t+15] of the
// segment and writes two 16-byte units: fragments 0,1 (nibbles 0,4 and 1,5) and 2,3 (nibbles 2,6 and 3,7).
// MODE 0: row m of x.  MODE 1: row row_src[m] of x (the permutation of mt_moe_permute, moe.rs:222-281, without the copy).
// MODE 2: silu(x[m]) * x2[m] rounded to the activation type first (mt_swiglu, crates/metaltile-std/src/mlx/swiglu.rs:45-57,
// with the arithmetic of the stand-alone kernel: g / (1 + expf(-g)) * u in f32).
template <bool BF16, int MODE>
__global__ void __launch_bounds__(256) gather_prep_kernel(const void *x, const void *x2, const uint32_t *row_src, int n_src_rows,
                                                          const uint32_t *offsets, int n_experts, int m_total, int K, int TB,
                                                          unsigned char *xfrag, float *xsum, GTable *table, uint32_t *status) {
    if (blockIdx.x == 0 && threadIdx.x < 32) {
        const int lane = threadIdx.x;
        int n_pass = 0, cost = 0;
        bool bad = false, over = false;
        for (int e0 = 0; e0 < n_experts; e0 += 32) {
            const int e = e0 + lane;
            int lo = 0, hi = 0;
            if (e < n_experts) {
                const uint32_t a = offsets[e], b = offsets[e + 1];
                lo = static_cast<int>(min(a, static_cast<uint32_t>(m_total)));
                hi = static_cast<int>(min(b, static_cast<uint32_t>(m_total)));
                if (a > static_cast<uint32_t>(m_total) || b > static_cast<uint32_t>(m_total) || b < a) bad = true;
                if (hi < lo) hi = lo;
            }
            const int rows = hi - lo, np = (rows + TB - 1) / TB;
            const int full = rows / TB, rem = rows - full * TB;
            const int c = full * (2 + (TB + 7) / 8) + (rem ? 2 + (rem + 7) / 8 : 0);
            int pp = np, pc = c;                       // inclusive scans over these 32 experts
            for (int d = 1; d < 32; d <<= 1) {
                const int up = __shfl_up_sync(0xffffffffu, pp, d), uc = __shfl_up_sync(0xffffffffu, pc, d);
                if (lane >= d) {
                    pp += up;
                    pc += uc;
                }
            }
            int p0 = n_pass + pp - np, c0 = cost + pc - c;
            for (int i = 0; i < np; ++i) {
                const int nt = min(TB, rows - i * TB);
                if (p0 + i < kGMaxPasses) table->pass[p0 + i] = GPass{e, lo + i * TB, nt, c0};
                else over = true;
                c0 += 2 + (nt + 7) / 8;
            }
            n_pass += __shfl_sync(0xffffffffu, pp, 31);
            cost += __shfl_sync(0xffffffffu, pc, 31);
        }
        bad = __any_sync(0xffffffffu, bad);
        over = __any_sync(0xffffffffu, over);
        if (lane == 0) {
            table->n_pass = over ? 0 : n_pass;         // a table that does not fit runs nothing: the caller is told
            table->total_cost = over ? 0 : cost;
            table->overflow = over ? 1 : 0;
            if (bad) atomicCAS(status, 0u, 0x901u);
            if (over) atomicCAS(status, 0u, 0x902u);
        }
    }
    const int nseg = K >> 6;
    const int t = threadIdx.x & 3;
    const long long quads = static_cast<long long>(m_total) * nseg;
    for (long long q = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 2; q < ((quads + 7) & ~7ll);
         q += (static_cast<long long>(gridDim.x) * blockDim.x) >> 2) {
        const bool on = q < quads;                     // whole warps stay in the loop: the sums use shuffles
        const long long m = on ? q / nseg : 0;
        const int s = on ? static_cast<int>(q - m * nseg) : 0;
        uint4 v0 = make_uint4(0u, 0u, 0u, 0u), v1 = v0;
        if (on) {
            size_t src = static_cast<size_t>(m);
            if (MODE == 1) {
                const uint32_t r = __ldg(row_src + m);
                if (r >= static_cast<uint32_t>(n_src_rows)) atomicCAS(status, 0u, 0x903u);     // not a row of x: row 0 is read instead
                src = r < static_cast<uint32_t>(n_src_rows) ? r : 0;
            }
            const uint4 *p = reinterpret_cast<const uint4 *>(static_cast<const uint16_t *>(x) + src * K + s * 64 + 16 * t);
            v0 = __ldg(p);
            v1 = __ldg(p + 1);
        }
        uint32_t u[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
        if (MODE == 2 && on) {
            const uint4 *p2 = reinterpret_cast<const uint4 *>(static_cast<const uint16_t *>(x2) + static_cast<size_t>(m) * K + s * 64 + 16 * t);
            const uint4 w0 = __ldg(p2), w1 = __ldg(p2 + 1);
            const uint32_t uu[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                float g0, g1, u0, u1;
                if (BF16) {
                    g0 = __uint_as_float(u[i] << 16); g1 = __uint_as_float(u[i] & 0xFFFF0000u);
                    u0 = __uint_as_float(uu[i] << 16); u1 = __uint_as_float(uu[i] & 0xFFFF0000u);
                } else {
                    const float2 gf = __half22float2(*reinterpret_cast<const __half2 *>(&u[i]));
                    const float2 uf = __half22float2(*reinterpret_cast<const __half2 *>(&uu[i]));
                    g0 = gf.x; g1 = gf.y; u0 = uf.x; u1 = uf.y;
                }
                const float r0 = (g0 / (1.0f + expf(-g0))) * u0, r1 = (g1 / (1.0f + expf(-g1))) * u1;
                if (BF16) {
                    const __nv_bfloat162 p2v = __floats2bfloat162_rn(r0, r1);
                    u[i] = *reinterpret_cast<const uint32_t *>(&p2v);
                } else {
                    const __half2 p2v = __floats2half2_rn(r0, r1);
                    u[i] = *reinterpret_cast<const uint32_t *>(&p2v);
                }
            }
        }
        uint32_t e[8], o[8];
        float sum = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            if (BF16) {
                const float lo = __uint_as_float(u[i] << 16), hi = __uint_as_float(u[i] & 0xFFFF0000u);
                sum += lo + hi;
                e[i] = (__float_as_uint(lo * 18446744073709551616.0f) >> 16) | (__float_as_uint(hi * 18446744073709551616.0f) & 0xFFFF0000u);
                o[i] = (__float_as_uint(lo * 1152921504606846976.0f) >> 16) | (__float_as_uint(hi * 1152921504606846976.0f) & 0xFFFF0000u);
            } else {
                const __half2 h2 = *reinterpret_cast<const __half2 *>(&u[i]);
                const float2 f = __half22float2(h2);
                sum += f.x + f.y;
                e[i] = u[i];
                const __half2 sc = __hmul2(h2, __float2half2_rn(0.0625f));
                o[i] = *reinterpret_cast<const uint32_t *>(&sc);
            }
        }
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        if (on) {
            uint4 *dst = reinterpret_cast<uint4 *>(xfrag) + ((static_cast<size_t>(m) * nseg + s) * 4 + t) * 2;
            dst[0] = make_uint4(__byte_perm(e[0], e[2], 0x5410), __byte_perm(e[4], e[6], 0x5410),
                                __byte_perm(o[0], o[2], 0x7632), __byte_perm(o[4], o[6], 0x7632));
            dst[1] = make_uint4(__byte_perm(e[1], e[3], 0x5410), __byte_perm(e[5], e[7], 0x5410),
                                __byte_perm(o[1], o[3], 0x7632), __byte_perm(o[5], o[7], 0x7632));
            if (t == 0) xsum[static_cast<size_t>(m) * nseg + s] = sum;
        }
    }
}

// ---- the gather kernel ------------------------------------------------------------------------------------------

// Row tiles [ta, tb) of pass `ps` that belong to the cost range [lo, hi).  Work is dealt in UNITS of kGW tiles (one per
// warp), so that no warp idles at the end of a pass while the others finish: unit i sits at cost0 * UPE + i * c.
__device__ __forceinline__ void g_tile_range(const GPass &ps, long long lo, long long hi, int TPE, int &ta, int &tb) {
    const int c = 2 + ((ps.ntok + 7) >> 3);
    const int UPE = (TPE + kGW - 1) / kGW;
    const long long base = static_cast<long long>(ps.cost0) * UPE;
    const int ua = lo <= base ? 0 : static_cast<int>(min(static_cast<long long>(UPE), (lo - base + c - 1) / c));
    const int ub = hi <= base ? 0 : static_cast<int>(min(static_cast<long long>(UPE), (hi - base + c - 1) / c));
    ta = min(ua * kGW, TPE);
    tb = min(ub * kGW, TPE);
}

// The integer codes of one 64-code segment of 16 rows as the four A fragments of its MMAs.
struct GFrag {
    uint32_t a[4][4];
};
__device__ __forceinline__ void g_extract(const unsigned char *lo, const unsigned char *hi, GFrag &f) {
    constexpr uint32_t m0 = 0x000F000Fu, m1 = 0x00F000F0u;
    const uint2 cl = *reinterpret_cast<const uint2 *>(lo);
    const uint2 ch = *reinterpret_cast<const uint2 *>(hi);
    f.a[0][0] = cl.x & m0; f.a[0][1] = ch.x & m0; f.a[0][2] = cl.y & m0; f.a[0][3] = ch.y & m0;       // nibbles 0, 4
    f.a[1][0] = cl.x & m1; f.a[1][1] = ch.x & m1; f.a[1][2] = cl.y & m1; f.a[1][3] = ch.y & m1;       // nibbles 1, 5 (x 16)
    const uint32_t c0 = cl.x >> 8, c1 = ch.x >> 8, c2 = cl.y >> 8, c3 = ch.y >> 8;
    f.a[2][0] = c0 & m0; f.a[2][1] = c1 & m0; f.a[2][2] = c2 & m0; f.a[2][3] = c3 & m0;               // nibbles 2, 6
    f.a[3][0] = c0 & m1; f.a[3][1] = c1 & m1; f.a[3][2] = c2 & m1; f.a[3][3] = c3 & m1;               // nibbles 3, 7 (x 16)
}

// One 64-code segment of a 32-row tile (two 16-row halves) against NT token tiles; P (0..3) is its place in the run.
// Every activation fragment is read from shared memory once and meets both halves; every code fragment meets all NT tiles.
//   acc[h][nt][i] += scale * c * sum(q x) + bias * sum(x);  i = 0,1: row 16 h + pi(g), tokens 8 nt + 2t, + 1;  i = 2,3: 8 rows on
template <bool BF16, int GSH, int NT, int P>
__device__ __forceinline__ void g_segment(const unsigned char *w_lo, const uint2 (&sc)[2][4], const unsigned char *xa,
                                          const unsigned char *xb, const float *xs, float (&acc)[2][NT][4]) {
    GFrag f[2];
    g_extract(w_lo + P * 32, w_lo + 8 * kGPitch + P * 32, f[0]);
    g_extract(w_lo + 16 * kGPitch + P * 32, w_lo + 24 * kGPitch + P * 32, f[1]);
    constexpr int gi = P >> GSH;
    // c * 2^(pre-scale) leaves with the scale: f16 codes are q * 2^-24; bf16 codes q * 2^-133 against x * 2^64
    const float post = BF16 ? 5.9029581035870565e20f /* 2^69 */ : 16777216.0f /* 2^24 */;
    float s_lo[2], s_hi[2], b_lo[2], b_hi[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        s_lo[h] = g_f32_of_half<BF16>(gi >> 1 ? sc[h][0].y : sc[h][0].x, gi & 1) * post;
        s_hi[h] = g_f32_of_half<BF16>(gi >> 1 ? sc[h][1].y : sc[h][1].x, gi & 1) * post;
        b_lo[h] = g_f32_of_half<BF16>(gi >> 1 ? sc[h][2].y : sc[h][2].x, gi & 1);
        b_hi[h] = g_f32_of_half<BF16>(gi >> 1 ? sc[h][3].y : sc[h][3].x, gi & 1);
    }
    // the MMAs of one step (nibble class) go to 2 NT different accumulators: consecutive MMAs never depend on each other
    uint4 f01[NT], f23[NT];
    float2 x_sum[NT];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        f01[nt] = *reinterpret_cast<const uint4 *>(xa + nt * 1024);
        f23[nt] = *reinterpret_cast<const uint4 *>(xb + nt * 1024);
        x_sum[nt] = *reinterpret_cast<const float2 *>(xs + nt * 8);
    }
    float d[NT][2][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int h = 0; h < 2; ++h) g_hmma<BF16, true>(d[nt][h], f[h].a[0][0], f[h].a[0][1], f[h].a[0][2], f[h].a[0][3], f01[nt].x, f01[nt].y);
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int h = 0; h < 2; ++h) g_hmma<BF16, false>(d[nt][h], f[h].a[1][0], f[h].a[1][1], f[h].a[1][2], f[h].a[1][3], f01[nt].z, f01[nt].w);
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int h = 0; h < 2; ++h) g_hmma<BF16, false>(d[nt][h], f[h].a[2][0], f[h].a[2][1], f[h].a[2][2], f[h].a[2][3], f23[nt].x, f23[nt].y);
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int h = 0; h < 2; ++h) g_hmma<BF16, false>(d[nt][h], f[h].a[3][0], f[h].a[3][1], f[h].a[3][2], f[h].a[3][3], f23[nt].z, f23[nt].w);
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            acc[h][nt][0] = fmaf(s_lo[h], d[nt][h][0], fmaf(b_lo[h], x_sum[nt].x, acc[h][nt][0]));
            acc[h][nt][1] = fmaf(s_lo[h], d[nt][h][1], fmaf(b_lo[h], x_sum[nt].y, acc[h][nt][1]));
            acc[h][nt][2] = fmaf(s_hi[h], d[nt][h][2], fmaf(b_hi[h], x_sum[nt].x, acc[h][nt][2]));
            acc[h][nt][3] = fmaf(s_hi[h], d[nt][h][3], fmaf(b_hi[h], x_sum[nt].y, acc[h][nt][3]));
        }
    }
}

// Position of a warp on the copy side, which runs DEPTH - 1 runs ahead of its arithmetic.
struct GCopy {
    size_t woff, sboff;       // this pass's expert: byte offsets of its packed words and of its scales / biases
    int pp, tile, tb, run;
    bool valid;
};

template <bool BF16, int GSH, int DEPTH>
__global__ void __launch_bounds__(kGThreads, 1) gather_stream_kernel(const __grid_constant__ GArgs a) {
    extern __shared__ __align__(128) unsigned char gsm[];
    int *ctl = reinterpret_cast<int *>(gsm);            // [0] first pass, [1] last pass of this CTA
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const GTable *tb_ = a.table;
    const int n_pass = tb_->n_pass, TPE = a.tiles_per_expert;
    const long long total = static_cast<long long>(tb_->total_cost) * ((TPE + kGW - 1) / kGW);
    const long long lo = total * blockIdx.x / gridDim.x, hi = total * (blockIdx.x + 1) / gridDim.x;
    const int runs = a.K >> 8;
    if (threadIdx.x == 0) {
        ctl[0] = n_pass;
        ctl[1] = -1;
    }
    __syncthreads();
    for (int p = threadIdx.x; p < n_pass; p += kGThreads) {
        int ta, tb;
        g_tile_range(tb_->pass[p], lo, hi, TPE, ta, tb);
        if (tb > ta) {
            atomicMin(&ctl[0], p);
            atomicMax(&ctl[1], p);
        }
    }
    __syncthreads();
    const int p_first = ctl[0], p_last = ctl[1];
    if (p_last < p_first) return;                        // nothing for this CTA (uniform)

    // ---- copy side ----
    unsigned char *ring_p = gsm + a.off_ring + static_cast<size_t>(warp) * DEPTH * kGSlotBytes;
    const uint32_t ring = gs_u32(ring_p);
    const size_t w_expert = static_cast<size_t>(a.n_out) * a.rowbytes, sb_expert = static_cast<size_t>(a.n_out) * a.gpr2;
    const char *const w_mat[2] = {reinterpret_cast<const char *>(a.w), reinterpret_cast<const char *>(a.w2)};
    const char *const sb_mat[2] = {static_cast<const char *>(lane < 16 ? a.scales : a.biases),
                                   static_cast<const char *>(lane < 16 ? a.scales2 : a.biases2)};
    GCopy cit;
    cit.pp = p_first;
    cit.valid = false;
    auto copy_enter = [&]() {
        for (; cit.pp <= p_last; ++cit.pp) {
            const GPass ps = tb_->pass[cit.pp];
            int ta, tb;
            g_tile_range(ps, lo, hi, TPE, ta, tb);
            if (ta + warp < tb) {
                cit.tile = ta + warp;
                cit.tb = tb;
                cit.run = 0;
                cit.woff = ps.expert * w_expert;
                cit.sboff = ps.expert * sb_expert;
                cit.valid = true;
                return;
            }
        }
        cit.valid = false;
    };
    // One run of a tile: 32 rows x 128 bytes of packed words (8 copies of 16 bytes per lane: lane -> row 4q + (lane >> 3),
    // chunk lane & 7) and 32 rows x 8 (4) bytes of scales and of biases (two copies per lane).  Rows past the end of the
    // matrix re-read its last row, so every byte of the slot is defined.
    auto copy_next = [&](uint32_t slot) {
        if (cit.valid) {
            const int second = cit.tile >= a.tpe1 ? 1 : 0;
            const int r0 = (cit.tile - (second ? a.tpe1 : 0)) * kGTileRows, last = a.n_out - 1;
            const int crow = lane >> 3, cch = lane & 7;
            const char *src = w_mat[second] + cit.woff + static_cast<size_t>(cit.run) * 128 + cch * 16;
            const uint32_t dst = slot + crow * kGPitch + cch * 16;
#pragma unroll
            for (int q = 0; q < 8; ++q) g_cp16(dst + q * 4 * kGPitch, src + static_cast<size_t>(min(r0 + crow + 4 * q, last)) * a.rowbytes);
#pragma unroll
            for (int q = 0; q < 2; ++q) {
                const int r = (lane & 15) + 16 * q;
                const uint32_t sdst = slot + kGSlotW + (lane >> 4) * 256 + r * 8;
                const char *ssrc = sb_mat[second] + cit.sboff + static_cast<size_t>(min(r0 + r, last)) * a.gpr2;
                if (GSH == 0) g_cp8(sdst, ssrc + static_cast<size_t>(cit.run) * 8);
                else g_cp4(sdst, ssrc + static_cast<size_t>(cit.run) * 4);
            }
            if (++cit.run == runs) {
                cit.run = 0;
                cit.tile += kGW;
                if (cit.tile >= cit.tb) {
                    ++cit.pp;
                    copy_enter();
                }
            }
        }
        g_commit();
    };
    copy_enter();
#pragma unroll 1
    for (int p = 0; p < DEPTH - 1; ++p) copy_next(ring + p * kGSlotBytes);
    int islot = DEPTH - 1, cslot = 0;

    // ---- arithmetic side ----
    const int pi = 2 * (g & 3) + (g >> 2);                        // tile row of MMA row g (and 8 + pi of MMA row g + 8)
    const uint32_t a_lo = pi * kGPitch + t * 8;
    const int TB = a.TB, nseg = a.K >> 6, upr = a.K >> 3;
    const uint32_t segstride = TB * 128;
    const unsigned char *x0 = gsm + kGOffX + g * 128 + t * 32 + (g & 1) * 16;
    const unsigned char *x1 = gsm + kGOffX + g * 128 + t * 32 + ((g & 1) ^ 1) * 16;
    const float *xs0 = reinterpret_cast<const float *>(gsm + a.off_xsum) + 2 * t;
    const uint32_t xdst = gs_u32(gsm + kGOffX), sdst0 = gs_u32(gsm + a.off_xsum);

    auto run_tiles = [&](auto nt_tag, const GPass &ps, int ta, int tb) {
        constexpr int NT = decltype(nt_tag)::value;
#pragma unroll 1
        for (int tile = ta + warp; tile < tb; tile += kGW) {
            float acc[2][NT][4];
#pragma unroll
            for (int h = 0; h < 2; ++h)
#pragma unroll
                for (int i = 0; i < NT; ++i) acc[h][i][0] = acc[h][i][1] = acc[h][i][2] = acc[h][i][3] = 0.0f;
#pragma unroll 1
            for (int run = 0; run < runs; ++run) {
                __syncwarp();                                    // every lane is done with the slot about to be refilled
                copy_next(ring + islot * kGSlotBytes);
                g_wait_oldest<DEPTH>();                          // this run has landed (this lane's copies)
                __syncwarp();                                    // ... and every other lane's
                const unsigned char *slot = ring_p + cslot * kGSlotBytes;
                uint2 sc[2][4];                                  // per half: scales of its two rows, biases of its two rows
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const unsigned char *sp = slot + kGSlotW + (16 * h + pi) * 8;
                    sc[h][0] = *reinterpret_cast<const uint2 *>(sp);
                    sc[h][1] = *reinterpret_cast<const uint2 *>(sp + 64);
                    sc[h][2] = *reinterpret_cast<const uint2 *>(sp + 256);
                    sc[h][3] = *reinterpret_cast<const uint2 *>(sp + 256 + 64);
                }
                const uint32_t so = run * kGRunSegs;
                const unsigned char *xa = x0 + so * segstride, *xb = x1 + so * segstride;
                const float *xs = xs0 + so * TB;
                const unsigned char *w_lo = slot + a_lo;
                g_segment<BF16, GSH, NT, 0>(w_lo, sc, xa, xb, xs, acc);
                g_segment<BF16, GSH, NT, 1>(w_lo, sc, xa + segstride, xb + segstride, xs + TB, acc);
                g_segment<BF16, GSH, NT, 2>(w_lo, sc, xa + 2 * segstride, xb + 2 * segstride, xs + 2 * TB, acc);
                g_segment<BF16, GSH, NT, 3>(w_lo, sc, xa + 3 * segstride, xb + 3 * segstride, xs + 3 * TB, acc);
                if (++cslot == DEPTH) cslot = 0;
                if (++islot == DEPTH) islot = 0;
            }
            const int dt = BF16 ? MTC_BF16 : MTC_F16;
            const bool second = tile >= a.tpe1;
            void *const outp = second ? a.out2 : a.out;
            const int trow = (tile - (second ? a.tpe1 : 0)) * kGTileRows;
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int ra = trow + 16 * h + pi, rb = ra + 8;
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
                    for (int j = 0; j < 2; ++j) {
                        const int tok = 8 * nt + 2 * t + j;
                        if (tok < ps.ntok) {
                            const size_t o = static_cast<size_t>(ps.tok0 + tok) * a.n_out;
                            if (ra < a.n_out) st_from_f32(outp, o + ra, acc[h][nt][j], dt);
                            if (rb < a.n_out) st_from_f32(outp, o + rb, acc[h][nt][2 + j], dt);
                        }
                    }
                }
            }
        }
    };

#pragma unroll 1
    for (int pp = p_first; pp <= p_last; ++pp) {
        const GPass ps = tb_->pass[pp];
        int ta, tb;
        g_tile_range(ps, lo, hi, TPE, ta, tb);
        if (pp != p_first) __syncthreads();                      // every warp is done with the previous pass's activations
        for (int idx = threadIdx.x; idx < ps.ntok * upr; idx += kGThreads) {
            const int m = idx / upr, r = idx - m * upr;
            const int s = r >> 3, tt = (r >> 1) & 3, h = r & 1;
            g_cp16(xdst + ((((s * TB + m) * 4 + tt) * 2 + (h ^ (m & 1))) << 4), a.xfrag + (static_cast<size_t>(ps.tok0 + m) * upr + r) * 16);
        }
        for (int idx = threadIdx.x; idx < ps.ntok * nseg; idx += kGThreads) {
            const int m = idx / nseg, s = idx - m * nseg;
            g_cp4(sdst0 + ((s * TB + m) << 2), a.xsum + static_cast<size_t>(ps.tok0 + m) * nseg + s);
        }
        g_commit();
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();
        const int NT = (ps.ntok + 7) >> 3;
        if (NT <= 1) run_tiles(std::integral_constant<int, 1>{}, ps, ta, tb);
        else if (NT == 2) run_tiles(std::integral_constant<int, 2>{}, ps, ta, tb);
        else if (NT == 3) run_tiles(std::integral_constant<int, 3>{}, ps, ta, tb);
        else run_tiles(std::integral_constant<int, 4>{}, ps, ta, tb);
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
}

inline size_t g_up256(size_t v) { return (v + 255) / 256 * 256; }

struct GPlan {
    int TB = 0, depth = 0;
    size_t smem = 0;
    uint32_t off_xsum = 0, off_ring = 0;
};

GPlan g_plan(int K) {
    GPlan p;
    p.TB = K <= 2048 ? 32 : K <= 4096 ? 16 : 8;
    const size_t xfrag = static_cast<size_t>(p.TB) * K * 2, xsum = static_cast<size_t>(p.TB) * (K / 64) * 4;
    p.off_xsum = static_cast<uint32_t>(kGOffX + xfrag);
    p.off_ring = static_cast<uint32_t>((p.off_xsum + xsum + 127) / 128 * 128);
    for (int d = 4; d >= 2; --d) {
        const size_t need = p.off_ring + static_cast<size_t>(kGW) * d * kGSlotBytes;
        if (need <= 227 * 1024) {
            p.depth = d;
            p.smem = need;
            break;
        }
    }
    return p;
}

template <bool BF16, int GSH, int DEPTH>
cudaError_t g_launch(const GArgs &a, int grid, size_t smem, cudaStream_t st) {
    static PerDeviceAttr attr;
    cudaError_t e = attr.set(gather_stream_kernel<BF16, GSH, DEPTH>, 227 * 1024);
    if (e != cudaSuccess) return e;
    gather_stream_kernel<BF16, GSH, DEPTH><<<grid, kGThreads, smem, st>>>(a);
    return cudaGetLastError();
}

template <bool BF16, int GSH>
cudaError_t g_launch_depth(const GArgs &a, int depth, int grid, size_t smem, cudaStream_t st) {
    if (depth == 4) return g_launch<BF16, GSH, 4>(a, grid, smem, st);
    if (depth == 3) return g_launch<BF16, GSH, 3>(a, grid, smem, st);
    return g_launch<BF16, GSH, 2>(a, grid, smem, st);
}

}  // namespace

bool gather_stream_supported(int m_total, int n_out, int K, int n_experts, int bits, int group_size, int dtype, const void *w,
                             const void *scales, const void *biases, const void *x) {
    if (bits != 4 || (dtype != MTC_F16 && dtype != MTC_BF16) || (group_size != 64 && group_size != 128)) return false;
    if (m_total <= 0 || n_out <= 0 || K <= 0 || K % 256 != 0 || K > 8192 || n_experts <= 0) return false;
    const GPlan p = g_plan(K);
    if (p.depth == 0) return false;
    if (static_cast<long long>(n_experts) + m_total / p.TB > kGMaxPasses) return false;
    auto al = [](const void *q, uintptr_t n) { return q == nullptr || reinterpret_cast<uintptr_t>(q) % n == 0; };
    return al(w, 16) && al(x, 16) && al(scales, 8) && al(biases, 8);
}

size_t gather_stream_scratch_bytes(int m_total, int K) {
    return g_up256(static_cast<size_t>(m_total) * K * 2) + g_up256(static_cast<size_t>(m_total) * (K / 64) * 4) + g_up256(sizeof(GTable));
}

// x rows sorted by expert (expert_offsets [n_experts + 1]) -> mats[i].out [m_total, n_out] for one matrix set or for two
// that read the same rows (gate and up); `scratch` holds gather_stream_scratch_bytes(m_total, K) bytes and is used by the
// two launches only (stream order).  row_src: row m of the product reads x[row_src[m]] (x has n_src_rows rows);
// x2: the rows are silu(x) * x2 (both [m_total, K]).  At most one of row_src and x2.
cudaError_t launch_gather_stream(Ctx *ctx, cudaStream_t st, const void *x, const void *x2, const uint32_t *row_src, int n_src_rows,
                                 const GatherMats *mats, int n_mats, const uint32_t *expert_offsets, int m_total, int n_out, int K,
                                 int n_experts, int group_size, int dtype, void *scratch) {
    const GPlan p = g_plan(K);
    if (p.depth == 0 || n_mats < 1 || n_mats > 2 || (x2 && row_src)) return cudaErrorInvalidValue;
    unsigned char *xfrag = static_cast<unsigned char *>(scratch);
    float *xsum = reinterpret_cast<float *>(xfrag + g_up256(static_cast<size_t>(m_total) * K * 2));
    GTable *table = reinterpret_cast<GTable *>(reinterpret_cast<unsigned char *>(xsum) + g_up256(static_cast<size_t>(m_total) * (K / 64) * 4));
    const bool bf16 = dtype == MTC_BF16;
    const long long threads = static_cast<long long>(m_total) * (K / 64) * 4;
    int pgrid = static_cast<int>(std::min<long long>((threads + 255) / 256, 8ll * ctx->sm_count));
    if (pgrid < 1) pgrid = 1;
    auto prep = [&](auto kern) {
        kern<<<pgrid, 256, 0, st>>>(x, x2, row_src, n_src_rows, expert_offsets, n_experts, m_total, K, p.TB, xfrag, xsum, table, ctx->d_status);
    };
    if (x2) {
        if (bf16) prep(gather_prep_kernel<true, 2>); else prep(gather_prep_kernel<false, 2>);
    } else if (row_src) {
        if (bf16) prep(gather_prep_kernel<true, 1>); else prep(gather_prep_kernel<false, 1>);
    } else {
        if (bf16) prep(gather_prep_kernel<true, 0>); else prep(gather_prep_kernel<false, 0>);
    }
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    GArgs a{};
    a.w = static_cast<const uint32_t *>(mats[0].w);
    a.scales = mats[0].scales;
    a.biases = mats[0].biases;
    a.out = mats[0].out;
    a.tpe1 = (n_out + kGTileRows - 1) / kGTileRows;
    a.tiles_per_expert = a.tpe1 * n_mats;
    if (n_mats == 2) {
        a.w2 = static_cast<const uint32_t *>(mats[1].w);
        a.scales2 = mats[1].scales;
        a.biases2 = mats[1].biases;
        a.out2 = mats[1].out;
    } else {                              // never selected: tile indices stay below tpe1
        a.w2 = a.w;
        a.scales2 = a.scales;
        a.biases2 = a.biases;
        a.out2 = a.out;
    }
    a.xfrag = xfrag;
    a.xsum = xsum;
    a.table = table;
    a.status = ctx->d_status;
    a.n_out = n_out;
    a.K = K;
    a.TB = p.TB;
    a.rowbytes = K / 2;
    a.gpr2 = K / group_size * 2;
    a.off_xsum = p.off_xsum;
    a.off_ring = p.off_ring;
    const int grid = ctx->sm_count;
    if (bf16) return group_size == 64 ? g_launch_depth<true, 0>(a, p.depth, grid, p.smem, st) : g_launch_depth<true, 1>(a, p.depth, grid, p.smem, st);
    return group_size == 64 ? g_launch_depth<false, 0>(a, p.depth, grid, p.smem, st) : g_launch_depth<false, 1>(a, p.depth, grid, p.smem, st);
}

}  // namespace mtc
