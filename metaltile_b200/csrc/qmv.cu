// qmv — affine group-quantized matrix-vector / small-M matmul on CUDA cores (sm_100a).
//
//   out[m, n] = sum_k (q(n,k) * scale[n, k/G] + bias[n, k/G]) * x[m, k]      (f32 accumulate)
//
// Stands in for mt_qmv, mt_qmm{,_bm2,_bm4}, the generic mt_qmv_b*/mt_qmm_b* family
// (crates/metaltile-std/src/mlx/quantized.rs:7-308,343-1441,4273-4392) and the
// 2-bit dequant_gemv (crates/metaltile-std/src/ffai/dequant_gemv.rs:52-105).
//
// Design (HBM-bound, no tensor cores):
//   * a warp owns R = 4 weight rows at a time; lane l owns "chunks" l, l+32, ... of
//     the row, a chunk being 16 or 32 consecutive codes loaded with one vector load
//     (128-bit for 4/8-bit, 64-bit for 2-bit, 3 or 5 words for the 3/5/6-bit
//     streams, whose period is exactly one chunk so no code straddles a lane);
//   * codes are never converted with I2F: `word & (mask << p)` reinterpreted as
//     f32 is the subnormal-or-tiny number q * 2^(p-149) exactly (bits 0..23 of an
//     f32 are linear in the integer they hold), and x is staged once per CTA in
//     shared memory as f32 pre-multiplied by 2^(64-p).  One LOP3 + one FFMA per
//     (code, m); a funnel shift every 24 bits brings later codes below bit 24;
//   * the reference's algebraic split (quantized.rs:29-32):
//     acc += scale * sum(q*x) + bias * sum(x) per chunk; sum(x) comes from the same
//     staging pass;
//   * x tiles live in shared memory in a lane-interleaved layout so every
//     LDS.128 of a warp is conflict-free;
//   * rows are dealt round-robin over CTAs so all 148 SMs stream at once; small N
//     splits K over the warps of a CTA (intra-CTA split-K, reduced in shared
//     memory, no global scratch).
// Domain note: the 2^64 pre-scale keeps every product exact for |x| < 2^63; beyond
// that the staged value overflows to inf where the reference would stay finite.
#include "common.cuh"

namespace mtc {
namespace {

template <int BITS>
struct Pack {
    static constexpr int WORDS = BITS == 2 ? 2 : (BITS == 4 || BITS == 8) ? 4 : (BITS == 6 ? 3 : BITS);
    static constexpr int CODES = WORDS * 32 / BITS;  // 2,3,4,5-bit: 32; 6,8-bit: 16
    static constexpr int CPW = 24 / BITS;            // codes per 24-bit window
    static constexpr int NWIN = (CODES + CPW - 1) / CPW;
    static constexpr uint32_t MASK = (1u << BITS) - 1u;
};

constexpr int kPreExp = 64;  // x is staged as x * 2^(kPreExp - p)

constexpr int kMaxPeers = 8;

struct QmvArgs {
    const uint32_t *w;
    const void *scales, *biases, *x;
    void *out;
    int M, N, K, gs, dt;
    int gs_shift;      // log2(gs) (the vectorised kernels need a power-of-two group)
    int wpr, gpr;      // words per weight row, groups per row
    int nchunks, njb;  // chunks per row, ceil(nchunks / 32)
    int kb_jb, nkb;    // chunk-iterations per staged K block, number of K blocks
    int ksplit;        // warps sharing one row group
    int groups, iters; // row groups (ceil(N/R)), row-group iterations per CTA slot
    int gpc;           // consecutive row groups owned by one CTA (its weights are one contiguous range)
    // fused RMSNorm (ffai_rms_norm_qgemv, crates/metaltile-std/src/ffai/rms_norm_qgemv.rs:51-107; M = 1): the staged
    // activation is x[k] * norm_w[k] * inv_rms in f32, inv_rms = rsqrt(mean(x^2) + eps); null = plain x
    const void *norm_w;
    float eps;
};

// Further copies of the output tile (peer GPUs' buffers: the all-gather is the store).  A second kernel parameter of
// the multi-destination instantiations only: the single-destination kernels keep their parameter block and code
// (measured: carrying the pointers and the store loop in every instantiation cost the decode set 6.5 %).
template <bool kMulti>
struct QmvTail {};
template <>
struct QmvTail<true> {
    int n_extra;
    void *extra[kMaxPeers - 1];
};

template <int WORDS>
__device__ __forceinline__ void load_words(const uint32_t *p, uint32_t (&w)[WORDS]) {
    if constexpr (WORDS == 4) {
        asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                     : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3]) : "l"(p));
    } else if constexpr (WORDS == 2) {
        asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];"
                     : "=r"(w[0]), "=r"(w[1]) : "l"(p));
    } else {
#pragma unroll
        for (int i = 0; i < WORDS; ++i) w[i] = __ldg(p + i);  // neighbours share sectors: keep in L1
    }
}

__device__ __forceinline__ float comp(const float4 &v, int i) {
    return i == 0 ? v.x : i == 1 ? v.y : i == 2 ? v.z : v.w;
}

// Stage one K block of x (all MT rows) into shared memory.  A lane-step unit is V consecutive base
// chunks; unit u = (iteration jb, lane ln), part vv:
//   xs   : f32, element (unit, vv, code i, row m) at float4 index
//          ((jb * V + vv) * (CODES*MT/4) + (i*MT+m)/4) * 32 + ln, component (i*MT+m)%4,
//          value x[m, k] * 2^(kPreExp - (i % CPW) * BITS);
//   xsum : plain sum of the base chunk's x values, at ((jb*32 + ln) * V + vv) * MT + m.
// CODES consecutive elements of a T array (f32, f16 or bf16; 16-byte aligned position) as f32.
template <int CODES>
__device__ __forceinline__ void load_vals(const void *src, size_t base, int dt, float (&v)[CODES]) {
    if (dt == MTC_F32) {
        const float4 *p = reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(src) + base);
#pragma unroll
        for (int q = 0; q < CODES / 4; ++q) {
            float4 t = __ldg(p + q);
            v[4 * q] = t.x; v[4 * q + 1] = t.y; v[4 * q + 2] = t.z; v[4 * q + 3] = t.w;
        }
    } else {
        const uint4 *p = reinterpret_cast<const uint4 *>(reinterpret_cast<const uint16_t *>(src) + base);
#pragma unroll
        for (int q = 0; q < CODES / 8; ++q) {
            uint4 t = __ldg(p + q);
            uint32_t u[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
            for (int h = 0; h < 4; ++h) {
                if (dt == MTC_BF16) {
                    v[8 * q + 2 * h] = __uint_as_float(u[h] << 16);
                    v[8 * q + 2 * h + 1] = __uint_as_float(u[h] & 0xFFFF0000u);
                } else {
                    float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&u[h]));
                    v[8 * q + 2 * h] = f.x;
                    v[8 * q + 2 * h + 1] = f.y;
                }
            }
        }
    }
}

template <int BITS, int MT, int V>
__device__ __forceinline__ void stage_x(const QmvArgs &a, float *xs, float *xsum, int chunk0, int nch, float inv_rms = 1.0f) {
    using P = Pack<BITS>;
    constexpr int E4 = P::CODES * MT / 4;   // float4 per base chunk
    for (int t = threadIdx.x; t < nch * MT; t += blockDim.x) {
        const int c = t / MT, m = t - c * MT;
        // base chunk c belongs to lane-step unit c / V: iteration jb = unit / 32, lane ln = unit % 32, part vv
        const int unit = c / V, vv = c - unit * V;
        const int jb = unit >> 5, ln = unit & 31;
        const size_t k0 = static_cast<size_t>(chunk0 + c) * P::CODES;
        {
            float v[P::CODES];
            if (m < a.M) {
                load_vals<P::CODES>(a.x, static_cast<size_t>(m) * a.K + k0, a.dt, v);
                if (a.norm_w) {
                    float nw[P::CODES];
                    load_vals<P::CODES>(a.norm_w, k0, a.dt, nw);
#pragma unroll
                    for (int i = 0; i < P::CODES; ++i) v[i] = v[i] * nw[i] * inv_rms;
                }
            } else {
#pragma unroll
                for (int i = 0; i < P::CODES; ++i) v[i] = 0.0f;
            }
            float s = 0.0f;
#pragma unroll
            for (int i = 0; i < P::CODES; ++i) s += v[i];
            xsum[((jb * 32 + ln) * V + vv) * MT + m] = s;
#pragma unroll
            for (int i = 0; i < P::CODES; ++i) {
                const int p = (i % P::CPW) * BITS;
                v[i] *= __uint_as_float(static_cast<uint32_t>(kPreExp - p + 127) << 23);
            }
            if constexpr (MT == 1) {
                float4 *dst = reinterpret_cast<float4 *>(xs) + (static_cast<size_t>(jb) * V + vv) * E4 * 32 + ln;
#pragma unroll
                for (int q = 0; q < P::CODES / 4; ++q)
                    dst[q * 32] = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
            } else {
#pragma unroll
                for (int i = 0; i < P::CODES; ++i) {
                    const int lin = i * MT + m;
                    xs[(((static_cast<size_t>(jb) * V + vv) * E4 + lin / 4) * 32 + ln) * 4 + (lin & 3)] = v[i];
                }
            }
        }
    }
}

// Raw (unconverted) scale / bias element: touching a prefetched register before its load has
// landed would stall the whole warp, so conversion to f32 waits until the chunk is consumed.
__device__ __forceinline__ uint32_t ld_raw(const void *p, size_t i, int dt) {
    if (dt == MTC_F32) return __ldg(reinterpret_cast<const uint32_t *>(p) + i);
    return __ldg(reinterpret_cast<const unsigned short *>(p) + i);
}
__device__ __forceinline__ float raw_to_f32(uint32_t raw, int dt) {
    if (dt == MTC_F32) return __uint_as_float(raw);
    if (dt == MTC_BF16) return __uint_as_float(raw << 16);
    return __half2float(__ushort_as_half(static_cast<unsigned short>(raw)));
}

// One chunk of R rows against the staged x: acc[r][m] += scale_r * sum_i q_ri * xs_mi (xs = pre-scaled x, so the
// sum carries a factor 2^(kPreExp-149) that reduce_store removes), accb[r][m] += bias_r * sum_i x_mi.
template <int BITS, int MT, int R>
__device__ __forceinline__ void consume_chunk(const uint32_t (&wreg)[R][Pack<BITS>::WORDS], const float (&sc)[R],
                                              const float (&bi)[R], const float4 *xv, const float *xsp,
                                              float (&acc)[R][MT], float (&accb)[R][MT]) {
    using P = Pack<BITS>;
    float dot[R][MT];
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int m = 0; m < MT; ++m) dot[r][m] = 0.0f;
    float4 xq = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int wi = 0; wi < P::NWIN; ++wi) {
        constexpr int kWinBits = P::CPW * BITS;
        const int word = (wi * kWinBits) / 32, sh = (wi * kWinBits) % 32;
        uint32_t v[R];
#pragma unroll
        for (int r = 0; r < R; ++r) {
            if (sh == 0) v[r] = wreg[r][word];
            else if (word + 1 < P::WORDS) v[r] = __funnelshift_r(wreg[r][word], wreg[r][word + 1], sh);
            else v[r] = wreg[r][word] >> sh;
        }
#pragma unroll
        for (int c = 0; c < P::CPW; ++c) {
            const int i = wi * P::CPW + c;
            if (i < P::CODES) {
                float f[R];
#pragma unroll
                for (int r = 0; r < R; ++r) f[r] = __uint_as_float(v[r] & (P::MASK << (c * BITS)));
#pragma unroll
                for (int m = 0; m < MT; ++m) {
                    const int lin = i * MT + m;
                    if ((lin & 3) == 0) xq = xv[(lin >> 2) * 32];
                    const float xval = comp(xq, lin & 3);
#pragma unroll
                    for (int r = 0; r < R; ++r) dot[r][m] = fmaf(f[r], xval, dot[r][m]);
                }
            }
        }
    }
#pragma unroll
    for (int m = 0; m < MT; ++m) {
        const float sx = xsp[m];
#pragma unroll
        for (int r = 0; r < R; ++r) {
            acc[r][m] = fmaf(sc[r], dot[r][m], acc[r][m]);     // still carries the 2^(kPreExp-149) factor
            accb[r][m] = fmaf(bi[r], sx, accb[r][m]);
        }
    }
}

// K reduction over the lanes of a warp, then (split-K) over the warps sharing the row group,
// then the store.  Contains __syncthreads when KS > 1: callers keep it CTA-uniform.
template <int MT, int R, bool kMulti>
__device__ __forceinline__ void reduce_store(const QmvArgs &a, const QmvTail<kMulti> &tail, float (&acc)[R][MT],
                                             float (&accb)[R][MT], float *red, int KS, int ks, int warp, int lane,
                                             bool active, int n0) {
    const float kPost = __uint_as_float(static_cast<uint32_t>(149 - kPreExp + 127) << 23);
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            float v = fmaf(acc[r][m], kPost, accb[r][m]);
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            acc[r][m] = v;
        }
    if (KS > 1) {
        if (lane == 0) {
#pragma unroll
            for (int r = 0; r < R; ++r)
#pragma unroll
                for (int m = 0; m < MT; ++m) red[(warp * R + r) * MT + m] = acc[r][m];
        }
        __syncthreads();
        if (ks == 0 && lane == 0) {
#pragma unroll
            for (int r = 0; r < R; ++r)
#pragma unroll
                for (int m = 0; m < MT; ++m)
                    for (int q = 1; q < KS; ++q) acc[r][m] += red[((warp + q) * R + r) * MT + m];
        }
        __syncthreads();
    }
    if (active && ks == 0 && lane == 0) {
#pragma unroll
        for (int r = 0; r < R; ++r) {
            if (n0 + r < a.N) {
#pragma unroll
                for (int m = 0; m < MT; ++m)
                    if (m < a.M) {
                        st_from_f32(a.out, static_cast<size_t>(m) * a.N + n0 + r, acc[r][m], a.dt);
                        if constexpr (kMulti) {
                            for (int e = 0; e < tail.n_extra; ++e)
                                st_from_f32(tail.extra[e], static_cast<size_t>(m) * a.N + n0 + r, acc[r][m], a.dt);
                        }
                    }
            }
        }
    }
}

// Pipelined kernel: the whole K extent of x fits the shared-memory stage (nkb == 1).  A lane-step
// unit is R rows x V consecutive base chunks (for 4-bit, V = 2: 64 codes = 32 bytes per lane and
// row, one scale/bias pair at group 64).  Each warp walks its (row group, iteration) units in one
// flat sequence and keeps PF units of packed words and raw scale/bias bits in flight in registers;
// the first PF units are requested before x is staged, so the DRAM latency of the weights overlaps
// the staging pass.  Prefetched registers are not touched (not even converted) before their turn.
template <int BITS, int MT, int R, int V, int PF, bool kMulti = false>
__global__ void __launch_bounds__(256, (MT <= 2 ? 2 : 1)) qmv_pipe_kernel(const QmvArgs a, const QmvTail<kMulti> tail) {
    using P = Pack<BITS>;
    constexpr int E4 = P::CODES * MT / 4;
    extern __shared__ __align__(16) float smem[];
    float *xs = smem;
    float *xsum = xs + static_cast<size_t>(a.njb) * 32 * V * P::CODES * MT;
    float *red = xsum + static_cast<size_t>(a.njb) * 32 * V * MT;

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const int KS = a.ksplit, slots = nwarps / KS, slot = warp / KS, ks = warp % KS;
    const int njb_w = a.njb / KS;          // host guarantees KS | njb
    const int U = a.iters * njb_w;
    // balanced contiguous partition of the row groups over the CTAs
    const int g_begin = static_cast<int>((static_cast<long long>(blockIdx.x) * a.groups) / gridDim.x);
    const int g_end = static_cast<int>((static_cast<long long>(blockIdx.x + 1) * a.groups) / gridDim.x);
    const int nunits = a.nchunks / V;      // lane-step units per row
    const int esz = a.dt == MTC_F32 ? 4 : 2;

    uint32_t wbuf[PF][V][R][P::WORDS];
    uint32_t sraw[PF][R], braw[PF][R];      // one scale/bias pair per unit and row (host: gs >= V * CODES)

    int l_g = g_begin + slot, l_jbi = 0, l_u = 0;                   // loader position
    auto issue = [&](uint32_t (&wd)[V][R][P::WORDS], uint32_t (&sr)[R], uint32_t (&br)[R]) {
        const int un = (ks + l_jbi * KS) * 32 + lane;               // unit index within the row
        if (l_u < U && l_g < g_end && un < nunits) {
            const int n0 = l_g * R;
            const int rmax = a.N - 1 - n0;                          // rows past N re-read the last row
            const uint32_t *wp = a.w + static_cast<size_t>(n0) * a.wpr + static_cast<size_t>(un) * (V * P::WORDS);
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const uint32_t *wr = wp + static_cast<size_t>(min(r, rmax)) * a.wpr;
#pragma unroll
                for (int v = 0; v < V; ++v) load_words<P::WORDS>(wr + v * P::WORDS, wd[v][r]);
            }
            const int grp = (un * (V * P::CODES)) >> a.gs_shift;
            const char *sp = static_cast<const char *>(a.scales) + (static_cast<size_t>(n0) * a.gpr + grp) * esz;
            const char *bp = static_cast<const char *>(a.biases) + (static_cast<size_t>(n0) * a.gpr + grp) * esz;
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const size_t ro = static_cast<size_t>(min(r, rmax)) * a.gpr * esz;
                if (esz == 4) {
                    sr[r] = __ldg(reinterpret_cast<const uint32_t *>(sp + ro));
                    br[r] = __ldg(reinterpret_cast<const uint32_t *>(bp + ro));
                } else {
                    sr[r] = __ldg(reinterpret_cast<const unsigned short *>(sp + ro));
                    br[r] = __ldg(reinterpret_cast<const unsigned short *>(bp + ro));
                }
            }
        }
        ++l_u;
        if (++l_jbi == njb_w) { l_jbi = 0; l_g += slots; }
    };

#pragma unroll
    for (int p = 0; p < PF; ++p) issue(wbuf[p], sraw[p], braw[p]);

    // Programmatic dependent launch: weights, scales and biases are constants of the model, so the
    // requests above may run ahead of the previous kernel in the stream; x (and every store) must
    // wait for it.  The next kernel may start its own prefetch from here on.
    asm volatile("griddepcontrol.launch_dependents;");
    asm volatile("griddepcontrol.wait;" ::: "memory");

    float inv_rms = 1.0f;
    if (a.norm_w) {
        // sum of squares of the (single) activation row over the CTA, then every thread holds inv_rms
        float ssq = 0.0f;
        for (int k = threadIdx.x; k < a.K; k += blockDim.x) {
            const float v = ld_as_f32(a.x, static_cast<size_t>(k), a.dt);
            ssq = fmaf(v, v, ssq);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ssq += __shfl_xor_sync(0xffffffffu, ssq, o);
        if (lane == 0) red[warp] = ssq;
        __syncthreads();
        float tot = 0.0f;
        for (int wi = 0; wi < nwarps; ++wi) tot += red[wi];
        inv_rms = 1.0f / sqrtf(tot / static_cast<float>(a.K) + a.eps);
        __syncthreads();                 // `red` is free again before the row-group sums use it
    }
    stage_x<BITS, MT, V>(a, xs, xsum, 0, a.nchunks, inv_rms);
    __syncthreads();

    float acc[R][MT], accb[R][MT];
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int m = 0; m < MT; ++m) acc[r][m] = accb[r][m] = 0.0f;

    int c_g = g_begin + slot, c_jbi = 0;                            // consumer position
    for (int u0 = 0; u0 < U; u0 += PF) {
#pragma unroll
        for (int p = 0; p < PF; ++p) {
            if (u0 + p < U) {
                const int jb = ks + c_jbi * KS;
                const int un = jb * 32 + lane;
                const bool active = c_g < g_end;
                if (active && un < nunits) {
                    float sc[R], bi[R];
                    if (a.dt == MTC_BF16) {
#pragma unroll
                        for (int r = 0; r < R; ++r) {
                            sc[r] = __uint_as_float(sraw[p][r] << 16);
                            bi[r] = __uint_as_float(braw[p][r] << 16);
                        }
                    } else if (a.dt == MTC_F32) {
#pragma unroll
                        for (int r = 0; r < R; ++r) {
                            sc[r] = __uint_as_float(sraw[p][r]);
                            bi[r] = __uint_as_float(braw[p][r]);
                        }
                    } else {
#pragma unroll
                        for (int r = 0; r < R; ++r) {
                            sc[r] = __half2float(__ushort_as_half(static_cast<unsigned short>(sraw[p][r])));
                            bi[r] = __half2float(__ushort_as_half(static_cast<unsigned short>(braw[p][r])));
                        }
                    }
                    const float4 *xv = reinterpret_cast<const float4 *>(xs) + static_cast<size_t>(jb) * (V * E4) * 32 + lane;
                    const float *xsp = xsum + (jb * 32 + lane) * (V * MT);
#pragma unroll
                    for (int v = 0; v < V; ++v)
                        consume_chunk<BITS, MT, R>(wbuf[p][v], sc, bi, xv + v * E4 * 32, xsp + v * MT, acc, accb);
                }
                issue(wbuf[p], sraw[p], braw[p]);
                if (c_jbi == njb_w - 1) {
                    reduce_store<MT, R, kMulti>(a, tail, acc, accb, red, KS, ks, warp, lane, active, c_g * R);
#pragma unroll
                    for (int r = 0; r < R; ++r)
#pragma unroll
                        for (int m = 0; m < MT; ++m) acc[r][m] = accb[r][m] = 0.0f;
                }
                if (++c_jbi == njb_w) { c_jbi = 0; c_g += slots; }
            }
        }
    }
}

// Blocked kernel: x for the whole K does not fit the stage (large M * K); K is walked in blocks
// that are re-staged for every row-group iteration.
template <int BITS, int MT, int R>
__global__ void __launch_bounds__(256) qmv_kernel(const QmvArgs a) {
    using P = Pack<BITS>;
    constexpr int E4 = P::CODES * MT / 4;
    extern __shared__ __align__(16) float smem[];
    float *xs = smem;
    float *xsum = xs + static_cast<size_t>(a.kb_jb) * 32 * P::CODES * MT;
    float *red = xsum + static_cast<size_t>(a.kb_jb) * 32 * MT;

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const int KS = a.ksplit, slots = nwarps / KS, slot = warp / KS, ks = warp % KS;

    for (int it = 0; it < a.iters; ++it) {
        const int g = blockIdx.x * a.gpc + it * slots + slot;
        const bool active = it * slots + slot < a.gpc && g < a.groups;
        const int n0 = g * R;
        float acc[R][MT], accb[R][MT];
#pragma unroll
        for (int r = 0; r < R; ++r)
#pragma unroll
            for (int m = 0; m < MT; ++m) acc[r][m] = accb[r][m] = 0.0f;

        for (int kb = 0; kb < a.nkb; ++kb) {
            const int jb_lo = kb * a.kb_jb;
            const int jb_hi = min(jb_lo + a.kb_jb, a.njb);
            __syncthreads();
            stage_x<BITS, MT, 1>(a, xs, xsum, jb_lo * 32, min(jb_hi * 32, a.nchunks) - jb_lo * 32);
            __syncthreads();
            if (!active) continue;
            for (int jb = jb_lo + ks; jb < jb_hi; jb += KS) {
                const int j = jb * 32 + lane;
                if (j >= a.nchunks) continue;
                uint32_t wreg[R][P::WORDS];
                float sc[R], bi[R];
                const int grp = (j * P::CODES) >> a.gs_shift;
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    const int row = min(n0 + r, a.N - 1);
                    load_words<P::WORDS>(a.w + static_cast<size_t>(row) * a.wpr + static_cast<size_t>(j) * P::WORDS,
                                         wreg[r]);
                }
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    const int row = min(n0 + r, a.N - 1);
                    sc[r] = ld_as_f32(a.scales, static_cast<size_t>(row) * a.gpr + grp, a.dt);
                    bi[r] = ld_as_f32(a.biases, static_cast<size_t>(row) * a.gpr + grp, a.dt);
                }
                const int jbl = jb - jb_lo;
                const float4 *xv = reinterpret_cast<const float4 *>(xs) + static_cast<size_t>(jbl) * E4 * 32 + lane;
                consume_chunk<BITS, MT, R>(wreg, sc, bi, xv, xsum + (jbl * 32 + lane) * MT, acc, accb);
            }
        }
        reduce_store<MT, R, false>(a, QmvTail<false>{}, acc, accb, red, KS, ks, warp, lane, active, n0);
    }
}

// Any-shape fallback (unaligned pointers, group sizes that are not a multiple of the
// chunk, K not a multiple of the chunk): one warp per weight row, lanes stride over k,
// scalar two-word extraction like the reference's generic kernels
// (crates/metaltile-std/src/mlx/quantized.rs:4300-4325,4357-4390).
__global__ void __launch_bounds__(256)
qmv_generic_kernel(const uint32_t *w, const void *scales, const void *biases, const void *x, void *out,
                   int M, int N, int K, int bits, int gs, int dt) {
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= N) return;
    const size_t wpr = static_cast<size_t>(K) * bits / 32, gpr = K / gs;
    const uint32_t *wr = w + row * wpr;
    for (int m = 0; m < M; ++m) {
        float acc = 0.0f;
        for (int k = lane; k < K; k += 32) {
            const float s = ld_as_f32(scales, row * gpr + k / gs, dt);
            const float b = ld_as_f32(biases, row * gpr + k / gs, dt);
            const float q = static_cast<float>(code_at(wr, k, bits));
            acc = fmaf(fmaf(q, s, b), ld_as_f32(x, static_cast<size_t>(m) * K + k, dt), acc);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        if (lane == 0) st_from_f32(out, static_cast<size_t>(m) * N + row, acc, dt);
    }
}

__global__ void unpack_codes_kernel(const uint32_t *w, uint8_t *codes, int N, int K, int bits) {
    const size_t wpr = static_cast<size_t>(K) * bits / 32;
    const size_t total = static_cast<size_t>(N) * K;
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const size_t r = i / K;
        codes[i] = static_cast<uint8_t>(code_at(w + r * wpr, static_cast<uint32_t>(i - r * K), bits));
    }
}

constexpr int kRows = 4;
constexpr int kWarps = 8;
constexpr size_t kSmemBlocked = 80 * 1024;   // stage of the K-blocked kernel
constexpr size_t kSmemPipe = 200 * 1024;     // whole-K stage of the pipelined kernel (1 CTA / SM at the limit)

// Lane-step width V (base chunks per lane and step) and prefetch depth PF per M tile.
template <int BITS, int MT>
struct Shape {
    static constexpr int V = (MT == 1 && BITS != 5) ? 2 : 1;
    static constexpr int PF = MT <= 4 ? 2 : 1;
};

template <int BITS, int MT, int V>
cudaError_t launch_pipe(Ctx *ctx, cudaStream_t st, QmvArgs a, size_t per_jb, size_t red_bytes,
                        const QmvTail<true> *tail = nullptr) {
    using P = Pack<BITS>;
    constexpr int PF = Shape<BITS, MT>::PF;
    const int sms = ctx->sm_count;
    a.njb = (a.nchunks / V + 31) / 32;     // iterations of 32 lane-step units
    a.nkb = 1;
    a.kb_jb = a.njb;
    const size_t smem = per_jb * V * a.njb + red_bytes;
    auto kern = qmv_pipe_kernel<BITS, MT, kRows, V, PF>;
    int occ = 1;
    cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kern, kWarps * 32, smem);
    if (e != cudaSuccess) return e;
    if (occ < 1) occ = 1;
    if (occ > 2) occ = 2;
    if (ctx->qmv_max_occ > 0 && occ > ctx->qmv_max_occ) occ = ctx->qmv_max_occ;
    // split K over the warps of a CTA until the resident warp slots (occ CTAs of kWarps per SM) are used
    int ks = 1;
    while (ks < kWarps && a.groups * ks * 2 <= sms * occ * kWarps && a.njb % (ks * 2) == 0) ks *= 2;
    a.ksplit = ks;
    const int slots = kWarps / ks;
    int per_sm = (a.groups + sms * slots - 1) / (sms * slots);     // CTAs per SM if every slot took one group
    if (per_sm > occ) per_sm = occ;
    if (per_sm < 1) per_sm = 1;
    int grid = a.groups < sms * per_sm ? a.groups : sms * per_sm;
    if (grid < 1) grid = 1;
    a.gpc = (a.groups + grid - 1) / grid;                          // largest share of any CTA
    a.iters = (a.gpc + slots - 1) / slots;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kWarps * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if constexpr (MT == 1) {
        if (tail) {        // multi-destination instantiation: same configuration, one more parameter
            auto mk = qmv_pipe_kernel<BITS, MT, kRows, V, PF, true>;
            static PerDeviceAttr attr;
            e = attr.set(mk, kSmemPipe + 4096);
            if (e != cudaSuccess) return e;
            return cudaLaunchKernelEx(&cfg, mk, a, *tail);
        }
    }
    return cudaLaunchKernelEx(&cfg, kern, a, QmvTail<false>{});
}

template <int BITS, int MT>
cudaError_t launch_tile(Ctx *ctx, cudaStream_t st, QmvArgs a, const QmvTail<true> *tail) {
    using P = Pack<BITS>;
    constexpr int V = Shape<BITS, MT>::V;
    a.nchunks = a.K / P::CODES;
    a.groups = (a.N + kRows - 1) / kRows;
    const int sms = ctx->sm_count;
    const size_t per_jb = (static_cast<size_t>(32) * P::CODES * MT + 32 * MT) * sizeof(float);  // per 32 base chunks
    const size_t red_bytes = static_cast<size_t>(kWarps) * kRows * MT * sizeof(float);
    const size_t whole_k = per_jb * ((a.nchunks + 31) / 32 + 1) + red_bytes;
    if (a.norm_w && (MT != 1 || whole_k > kSmemPipe)) return cudaErrorNotSupported;   // fused RMSNorm: M = 1, whole K staged
    if (whole_k <= kSmemPipe) {
        if (V > 1 && a.nchunks % V == 0 && a.gs >= V * P::CODES) return launch_pipe<BITS, MT, V>(ctx, st, a, per_jb, red_bytes, tail);
        return launch_pipe<BITS, MT, 1>(ctx, st, a, per_jb, red_bytes, tail);
    }
    if (tail) return cudaErrorNotSupported;     // several destinations: whole K staged only
    a.njb = (a.nchunks + 31) / 32;

    int max_jb = static_cast<int>((kSmemBlocked - red_bytes) / per_jb);
    if (max_jb < 1) max_jb = 1;
    a.nkb = (a.njb + max_jb - 1) / max_jb;
    a.kb_jb = (a.njb + a.nkb - 1) / a.nkb;
    a.ksplit = 1;
    const size_t smem = per_jb * a.kb_jb + red_bytes;
    int grid = (a.groups + kWarps - 1) / kWarps;
    if (grid > sms * 2) grid = sms * 2;
    a.gpc = (a.groups + grid - 1) / grid;
    grid = (a.groups + a.gpc - 1) / a.gpc;
    a.iters = (a.gpc + kWarps - 1) / kWarps;
    qmv_kernel<BITS, MT, kRows><<<grid, kWarps * 32, smem, st>>>(a);
    return cudaGetLastError();
}

template <int BITS>
cudaError_t launch_bits(Ctx *ctx, cudaStream_t st, const QmvArgs &a, const QmvTail<true> *tail) {
    if (a.M == 1) return launch_tile<BITS, 1>(ctx, st, a, tail);
    if (tail) return cudaErrorNotSupported;     // several destinations: M = 1 (the sharded decode case)
    if (a.M == 2) return launch_tile<BITS, 2>(ctx, st, a, nullptr);
    if (a.M <= 4) return launch_tile<BITS, 4>(ctx, st, a, nullptr);
    if (a.M <= 8) return launch_tile<BITS, 8>(ctx, st, a, nullptr);
    return launch_tile<BITS, 16>(ctx, st, a, nullptr);
}

template <int BITS>
cudaError_t set_attrs_bits() {
    cudaError_t e;
#define MTC_SET(MT_)                                                                                     \
    e = cudaFuncSetAttribute(qmv_kernel<BITS, MT_, kRows>, cudaFuncAttributeMaxDynamicSharedMemorySize,         \
                             static_cast<int>(kSmemBlocked + 4096));                                            \
    if (e != cudaSuccess) return e;                                                                            \
    e = cudaFuncSetAttribute(qmv_pipe_kernel<BITS, MT_, kRows, 1, Shape<BITS, MT_>::PF>,                        \
                             cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kSmemPipe + 4096)); \
    if (e != cudaSuccess) return e;                                                                            \
    e = cudaFuncSetAttribute(qmv_pipe_kernel<BITS, MT_, kRows, Shape<BITS, MT_>::V, Shape<BITS, MT_>::PF>,      \
                             cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kSmemPipe + 4096)); \
    if (e != cudaSuccess) return e;
    MTC_SET(1) MTC_SET(2) MTC_SET(4) MTC_SET(8) MTC_SET(16)
#undef MTC_SET
    return cudaSuccess;
}

}  // namespace

// Opt every instantiation into > 48 KB of dynamic shared memory (once per device, from mtc_init).
cudaError_t qmv_init_device() {
    cudaError_t e;
    if ((e = set_attrs_bits<2>()) != cudaSuccess) return e;
    if ((e = set_attrs_bits<3>()) != cudaSuccess) return e;
    if ((e = set_attrs_bits<4>()) != cudaSuccess) return e;
    if ((e = set_attrs_bits<5>()) != cudaSuccess) return e;
    if ((e = set_attrs_bits<6>()) != cudaSuccess) return e;
    return set_attrs_bits<8>();
}

cudaError_t launch_qmv(Ctx *ctx, cudaStream_t st, const void *w, const void *scales, const void *biases,
                       const void *x, void *out, int M, int N, int K, int bits, int group_size, int dt,
                       std::string *why, void *const *extra_outs, int n_extra, const void *norm_w, float eps) {
    if (n_extra < 0 || n_extra > kMaxPeers - 1 || (n_extra > 0 && !extra_outs)) {
        if (why) *why = "qmv: at most 8 output copies";
        return cudaErrorInvalidValue;
    }
    const bool bits_ok = bits == 2 || bits == 3 || bits == 4 || bits == 5 || bits == 6 || bits == 8;
    if (!bits_ok || M < 0 || N < 0 || K <= 0 || group_size <= 0 || K % group_size != 0 ||
        (static_cast<long long>(K) * bits) % 32 != 0) {
        if (why) *why = "qmv: need bits in {2,3,4,5,6,8}, group_size | K, K*bits % 32 == 0";
        return cudaErrorInvalidValue;
    }
    if (M == 0 || N == 0) return cudaSuccess;
    const int codes = (bits == 6 || bits == 8) ? 16 : 32;
    const size_t esz = dtype_size(dt);
    const auto aligned = [](const void *p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; };
    const bool pow2 = (group_size & (group_size - 1)) == 0;
    const bool fast = pow2 && K % codes == 0 && group_size % codes == 0 && aligned(w, 16) && aligned(x, 16) &&
                      (static_cast<size_t>(K) * esz) % 16 == 0 && aligned(scales, esz) && aligned(biases, esz) &&
                      (static_cast<size_t>(K) * bits / 8) % (bits == 2 ? 8 : (bits == 4 || bits == 8) ? 16 : 4) == 0;
    if (!fast && n_extra > 0) {
        if (why) *why = "qmv with several outputs needs the vectorised path (power-of-two group, aligned pointers)";
        return cudaErrorInvalidValue;
    }
    if (norm_w && (!fast || M != 1 || !aligned(norm_w, 16))) return cudaErrorNotSupported;   // the caller normalises separately
    if (!fast) {
        const int wpb = 8;
        qmv_generic_kernel<<<(N + wpb - 1) / wpb, wpb * 32, 0, st>>>(
            static_cast<const uint32_t *>(w), scales, biases, x, out, M, N, K, bits, group_size, dt);
        return cudaGetLastError();
    }
    for (int m0 = 0; m0 < M; m0 += 16) {
        QmvArgs a{};
        a.w = static_cast<const uint32_t *>(w);
        a.scales = scales;
        a.biases = biases;
        a.x = static_cast<const char *>(x) + static_cast<size_t>(m0) * K * esz;
        a.out = static_cast<char *>(out) + static_cast<size_t>(m0) * N * esz;
        QmvTail<true> tail{};
        tail.n_extra = n_extra;
        for (int e = 0; e < n_extra; ++e) tail.extra[e] = static_cast<char *>(extra_outs[e]) + static_cast<size_t>(m0) * N * esz;
        const QmvTail<true> *tp = n_extra > 0 ? &tail : nullptr;
        a.M = M - m0 < 16 ? M - m0 : 16;
        a.N = N;
        a.K = K;
        a.gs = group_size;
        a.gs_shift = 0;
        while ((1 << a.gs_shift) < group_size) ++a.gs_shift;
        a.dt = dt;
        a.wpr = K * bits / 32;
        a.gpr = K / group_size;
        a.norm_w = norm_w;
        a.eps = eps;
        cudaError_t e;
        switch (bits) {
            case 2: e = launch_bits<2>(ctx, st, a, tp); break;
            case 3: e = launch_bits<3>(ctx, st, a, tp); break;
            case 4: e = launch_bits<4>(ctx, st, a, tp); break;
            case 5: e = launch_bits<5>(ctx, st, a, tp); break;
            case 6: e = launch_bits<6>(ctx, st, a, tp); break;
            default: e = launch_bits<8>(ctx, st, a, tp); break;
        }
        if (e == cudaErrorNotSupported && norm_w) return e;
        if (e == cudaErrorNotSupported && why) *why = "qmv with several outputs: M = 1 with the whole K staged in shared memory only";
        if (e == cudaErrorNotSupported) return cudaErrorInvalidValue;
        if (e != cudaSuccess) return e;
    }
    return cudaSuccess;
}

// x * norm_w * inv_rms of one row, rounded to the activation type: the unfused form for shapes the fused kernel does not take
__global__ void __launch_bounds__(256) rms_norm_row_kernel(const void *x, const void *norm_w, void *out, int K, float eps, int dt) {
    __shared__ float red[8];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float ssq = 0.0f;
    for (int k = threadIdx.x; k < K; k += blockDim.x) {
        const float v = ld_as_f32(x, static_cast<size_t>(k), dt);
        ssq = fmaf(v, v, ssq);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ssq += __shfl_xor_sync(0xffffffffu, ssq, o);
    if (lane == 0) red[warp] = ssq;
    __syncthreads();
    float tot = 0.0f;
    for (int wi = 0; wi < 8; ++wi) tot += red[wi];
    const float inv_rms = 1.0f / sqrtf(tot / static_cast<float>(K) + eps);
    for (int k = threadIdx.x; k < K; k += blockDim.x)
        st_from_f32(out, static_cast<size_t>(k), ld_as_f32(x, static_cast<size_t>(k), dt) * ld_as_f32(norm_w, static_cast<size_t>(k), dt) * inv_rms, dt);
}

cudaError_t launch_rms_norm_row(cudaStream_t st, const void *x, const void *norm_w, void *out, int K, float eps, int dt) {
    rms_norm_row_kernel<<<1, 256, 0, st>>>(x, norm_w, out, K, eps, dt);
    return cudaGetLastError();
}

cudaError_t launch_unpack_codes(cudaStream_t st, const void *w, void *codes, int N, int K, int bits) {
    if (N <= 0 || K <= 0) return cudaSuccess;
    unpack_codes_kernel<<<kNumSMsB200 * 4, 256, 0, st>>>(static_cast<const uint32_t *>(w),
                                                          static_cast<uint8_t *>(codes), N, K, bits);
    return cudaGetLastError();
}

}  // namespace mtc
