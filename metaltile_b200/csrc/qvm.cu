// qvm — the quantized vector-matrix product, the dual of qmv: the weight matrix is stored transposed, [K, N], codes packed
// along N, and the groups run along K:
//
//   out[m, c] = sum_d (q(d, c) * scale[d / G, c] + bias[d / G, c]) * x[m, d]
//
// w u32[K, N*bits/32] (row d = LSB-first bit-stream of N codes), scales / biases T[K/G, N], x T[M, K], out T[M, N].
// Stands in for mt_qvm_b{3,4,5,6,8} and mt_qvm_int4_fast (crates/metaltile-std/src/mlx/quantized.rs:4397-4530,4582-4700).
//
// HBM-bound: every packed word is read once per row of x.  A lane owns the columns of one packed word (2 / 4 / 8-bit:
// 16 / 8 / 4 columns) or of one 32-column period of the bit-stream (3 / 5 / 6-bit: b words), so a warp reads whole
// lines of a weight row; a warp walks whole groups of K rows and uses the algebraic split per group,
//   acc[c] += scale[g, c] * sum_d q(d, c) x[d]  +  bias[g, c] * sum_d x[d],
// the 8 warps of a CTA take different groups of the same column tile and add up in shared memory in a fixed order, and
// K is split over CTAs (partial sums in a context scratch block, added in a fixed order by a second small kernel), so
// results are deterministic.
#include "common.cuh"

namespace mtc {
namespace {

constexpr int kQvWarps = 8;

template <int BITS>
struct QvShape {
    static constexpr bool kStream = BITS == 3 || BITS == 5 || BITS == 6;
    static constexpr int WPT = kStream ? BITS : 1;              // words per lane and weight row
    static constexpr int CPT = kStream ? 32 : 32 / BITS;        // columns per lane
};

// Code j of a lane's words as an unshifted bit field below bit 24, and the position p of its lowest bit there.
template <int BITS>
struct QvCode {
    static constexpr uint32_t MASK = (1u << BITS) - 1u;
    __device__ static constexpr int pos(int j) {
        const int sh = (j * BITS) & 31;
        if (sh + BITS > 32) return 0;                      // straddles two words: assembled at bit 0
        return sh + BITS <= 24 ? sh : sh - 16;             // high fields are taken from the word shifted down by 16
    }
    template <int W>
    __device__ __forceinline__ static uint32_t field(const uint32_t (&w)[W], int j) {      // j: compile-time after unrolling
        const int bit = j * BITS, wi = bit >> 5, sh = bit & 31;
        if (sh + BITS > 32) return ((w[wi] >> sh) | (w[wi + 1] << (32 - sh))) & MASK;
        if (sh + BITS <= 24) return w[wi] & (MASK << sh);
        return (w[wi] >> 16) & (MASK << (sh - 16));
    }
};

constexpr int kQvTickets = 4096;               // arrival counters at the head of the partial-sum block (one per column tile and x row)

// NW consecutive 32-bit words from a 16-byte (NW % 4 == 0) or 8-byte (NW == 2) aligned address, read-only path
template <int NW>
__device__ __forceinline__ void qv_ld(const void *p, uint32_t (&o)[NW]) {
    static_assert(NW == 2 || NW % 4 == 0, "vector loads of 8 or 16 bytes");
    if (NW == 2) {
        const uint2 v = __ldg(static_cast<const uint2 *>(p));
        o[0] = v.x;
        o[1] = v.y;
    } else {
#pragma unroll
        for (int i = 0; i < NW / 4; ++i) {
            const uint4 v = __ldg(static_cast<const uint4 *>(p) + i);
            o[4 * i] = v.x; o[4 * i + 1] = v.y; o[4 * i + 2] = v.z; o[4 * i + 3] = v.w;
        }
    }
}
// element i (compile-time after unrolling) of a vector of DT values held as words
template <int DT, int NW>
__device__ __forceinline__ float qv_elem(const uint32_t (&v)[NW], int i) {
    if (DT == MTC_F32) return __uint_as_float(v[i]);
    const uint32_t wd = v[i >> 1];
    if (DT == MTC_BF16) return __uint_as_float((i & 1) ? (wd & 0xFFFF0000u) : (wd << 16));
    const __half2 h = *reinterpret_cast<const __half2 *>(&wd);
    return (i & 1) ? __high2float(h) : __low2float(h);
}

// What a lane needs for one slab of R rows: its packed words of every row, the R activations, and the scales and biases
// of its columns in the slab's group - all fetched with 8- or 16-byte loads before any of it is used.
template <int BITS, int DT>
struct QvSlab {
    using S = QvShape<BITS>;
    static constexpr int R = S::kStream ? 8 : 16;
    static constexpr int ESZ = DT == MTC_F32 ? 4 : 2;
    static constexpr int XW = R * ESZ / 4, SW = S::CPT * ESZ / 4;
    uint32_t w[R][S::WPT];
    uint32_t x[XW], sc[SW], bi[SW];
    int g;
};

template <int BITS, int DT>
__global__ void __launch_bounds__(kQvWarps * 32, 2) qvm_kernel(const uint32_t *w, const void *scales, const void *biases, const void *x,
                                                               float *partial, uint32_t *tickets, void *out, int M, int N, int K, int gs, int KC) {
    using S = QvShape<BITS>;
    using Slab = QvSlab<BITS, DT>;
    constexpr int R = Slab::R, ESZ = Slab::ESZ;
    __shared__ float red[kQvWarps][32 * S::CPT + 1];
    __shared__ uint32_t s_last;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int tile = blockIdx.x, kc = blockIdx.y, m = blockIdx.z;
    const int col0 = (tile * 32 + lane) * S::CPT;                  // first column of this lane
    const bool on = col0 < N;                                      // N % CPT == 0: a lane is in or out as a whole
    const int wpr = N * BITS / 32, n_groups = K / gs;
    const uint32_t *wl = w + (static_cast<size_t>(tile) * 32 + lane) * S::WPT;
    const char *xrow = static_cast<const char *>(x) + static_cast<size_t>(m) * K * ESZ;
    const char *sc0 = static_cast<const char *>(scales) + static_cast<size_t>(col0) * ESZ;
    const char *bi0 = static_cast<const char *>(biases) + static_cast<size_t>(col0) * ESZ;
    float acc[S::CPT];
#pragma unroll
    for (int j = 0; j < S::CPT; ++j) acc[j] = 0.0f;
    // a warp's unit of work is a slab of R consecutive rows of one group; a matrix has K / R units per column tile to
    // spread over warps and CTAs.  The loads of a warp's next slab are issued before its current slab is multiplied.
    const int upg = gs / R, n_units = n_groups * upg;              // gs % R == 0 (host)
    const int ustep = KC * kQvWarps;
    auto fetch = [&](int u, Slab &sl) {
        const int g = u / upg, d0 = g * gs + (u - g * upg) * R;
        sl.g = g;
        const uint32_t *wp = wl + static_cast<size_t>(d0) * wpr;
#pragma unroll
        for (int r = 0; r < R; ++r) {
#pragma unroll
            for (int i = 0; i < S::WPT; ++i) sl.w[r][i] = __ldg(wp + i);
            wp += wpr;
        }
        qv_ld<Slab::XW>(xrow + static_cast<size_t>(d0) * ESZ, sl.x);
        qv_ld<Slab::SW>(sc0 + static_cast<size_t>(g) * N * ESZ, sl.sc);
        qv_ld<Slab::SW>(bi0 + static_cast<size_t>(g) * N * ESZ, sl.bi);
    };
    // No integer-to-float conversion: the bits of a code, left where they sit in the word (below bit 24), read as an
    // f32 are q * 2^(p - 149) exactly - the subnormals and the first binade are one linear ramp, multiplied at full
    // rate - and x is pre-multiplied by 2^64 (exact; |x| < 2^63) so that products are normal numbers; the factor
    // 2^(85 - p) of column j leaves with the group's scale.  One LOP3 and one FFMA per code.
    auto multiply = [&](const Slab &sl) {
        float raw[S::CPT];
#pragma unroll
        for (int j = 0; j < S::CPT; ++j) raw[j] = 0.0f;
        float xs = 0.0f;
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const float xv = qv_elem<DT>(sl.x, r);
            xs += xv;
            const float xp = xv * 18446744073709551616.0f;                   // 2^64
#pragma unroll
            for (int j = 0; j < S::CPT; ++j) raw[j] = fmaf(xp, __uint_as_float(QvCode<BITS>::field(sl.w[r], j)), raw[j]);
        }
#pragma unroll
        for (int j = 0; j < S::CPT; ++j) {
            const float post = __uint_as_float(static_cast<uint32_t>(127 + 85 - QvCode<BITS>::pos(j)) << 23);     // 2^(85 - p)
            acc[j] = fmaf(qv_elem<DT>(sl.sc, j) * post, raw[j], fmaf(qv_elem<DT>(sl.bi, j), xs, acc[j]));
        }
    };
    if (on) {
        int u = kc * kQvWarps + warp;
        if (S::kStream || BITS == 2) {                             // 3 / 5 / 6-bit (b words per row) and 2-bit (16 columns): one slab in registers
            for (; u < n_units; u += ustep) {
                Slab sl;
                fetch(u, sl);
                multiply(sl);
            }
        } else if (u < n_units) {
            Slab sa, sb;
            fetch(u, sa);
            for (;;) {
                u += ustep;
                if (u < n_units) fetch(u, sb);
                multiply(sa);
                if (u >= n_units) break;
                u += ustep;
                if (u < n_units) fetch(u, sa);
                multiply(sb);
                if (u >= n_units) break;
            }
        }
    }
#pragma unroll
    for (int j = 0; j < S::CPT; ++j) red[warp][j * 32 + lane] = acc[j];
    __syncthreads();
    // column (tile * 32 + l) * CPT + j of the tile: summed over the warps in warp order
    for (int idx = threadIdx.x; idx < 32 * S::CPT; idx += kQvWarps * 32) {
        const int j = idx >> 5, l = idx & 31;
        const int c = (tile * 32 + l) * S::CPT + j;
        if (c >= N) continue;
        float v = 0.0f;
#pragma unroll
        for (int q = 0; q < kQvWarps; ++q) v += red[q][idx];
        if (KC == 1) st_from_f32(out, static_cast<size_t>(m) * N + c, v, DT);
        else partial[(static_cast<size_t>(kc) * M + m) * N + c] = v;
    }
    if (KC == 1 || tickets == nullptr) return;
    // K chunks: the CTA that arrives last for (column tile, x row) adds the chunks in chunk order (deterministic) and
    // leaves the counter at zero for the next launch.  Nothing waits for anything.
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const uint32_t old = atomicAdd(tickets + static_cast<size_t>(m) * gridDim.x + tile, 1u);
        s_last = old == static_cast<uint32_t>(KC - 1) ? 1u : 0u;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    for (int idx = threadIdx.x; idx < 32 * S::CPT; idx += kQvWarps * 32) {
        const int j = idx >> 5, l = idx & 31;
        const int c = (tile * 32 + l) * S::CPT + j;
        if (c >= N) continue;
        float v = 0.0f;
        const float *src = partial + static_cast<size_t>(m) * N + c;
        const size_t stride = static_cast<size_t>(M) * N;
        for (int q0 = 0; q0 < KC; q0 += 8) {                       // eight loads in flight, added in chunk order
            float pv[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) pv[i] = q0 + i < KC ? __ldcg(src + (q0 + i) * stride) : 0.0f;
#pragma unroll
            for (int i = 0; i < 8; ++i) v += pv[i];
        }
        st_from_f32(out, static_cast<size_t>(m) * N + c, v, DT);
    }
    if (threadIdx.x == 0) tickets[static_cast<size_t>(m) * gridDim.x + tile] = 0u;
}

__global__ void __launch_bounds__(256) qvm_sum_kernel(const float *partial, void *out, size_t mn, int KC, int dt) {
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < mn; i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        float v = 0.0f;
        for (int q0 = 0; q0 < KC; q0 += 8) {                       // eight loads in flight, added in chunk order
            float pv[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) pv[j] = q0 + j < KC ? partial[static_cast<size_t>(q0 + j) * mn + i] : 0.0f;
#pragma unroll
            for (int j = 0; j < 8; ++j) v += pv[j];
        }
        st_from_f32(out, i, v, dt);
    }
}

// any N, any group size: one thread per output element, rows of w walked one by one
__global__ void __launch_bounds__(256) qvm_generic_kernel(const uint32_t *w, const void *scales, const void *biases, const void *x,
                                                          void *out, int M, int N, int K, int gs, int bits, int dt) {
    const size_t mn = static_cast<size_t>(M) * N, wpr = static_cast<size_t>(N) * bits / 32;
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < mn; i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const int m = static_cast<int>(i / N), c = static_cast<int>(i - static_cast<size_t>(m) * N);
        float acc = 0.0f;
        for (int d = 0; d < K; ++d) {
            const float q = static_cast<float>(code_at(w + d * wpr, static_cast<uint32_t>(c), bits));
            const size_t si = static_cast<size_t>(d / gs) * N + c;
            acc = fmaf(fmaf(q, ld_as_f32(scales, si, dt), ld_as_f32(biases, si, dt)), ld_as_f32(x, static_cast<size_t>(m) * K + d, dt), acc);
        }
        st_from_f32(out, i, acc, dt);
    }
}

template <int BITS>
cudaError_t qvm_launch(cudaStream_t st, const void *w, const void *scales, const void *biases, const void *x, float *partial,
                       uint32_t *tickets, void *out, int M, int N, int K, int gs, int KC, int dt) {
    using S = QvShape<BITS>;
    const int tiles = (N + 32 * S::CPT - 1) / (32 * S::CPT);
    const dim3 grid(tiles, KC, M), block(kQvWarps * 32);
    const uint32_t *wp = static_cast<const uint32_t *>(w);
    if (dt == MTC_F32) qvm_kernel<BITS, MTC_F32><<<grid, block, 0, st>>>(wp, scales, biases, x, partial, tickets, out, M, N, K, gs, KC);
    else if (dt == MTC_F16) qvm_kernel<BITS, MTC_F16><<<grid, block, 0, st>>>(wp, scales, biases, x, partial, tickets, out, M, N, K, gs, KC);
    else qvm_kernel<BITS, MTC_BF16><<<grid, block, 0, st>>>(wp, scales, biases, x, partial, tickets, out, M, N, K, gs, KC);
    return cudaGetLastError();
}

}  // namespace

// Split of K over CTAs for these sizes (1 = a CTA owns all of K for its column tile): as many CTAs as are resident at once.
int qvm_k_chunks(int sms, int N, int K, int bits, int group_size) {
    const int cpt = (bits == 3 || bits == 5 || bits == 6) ? 32 : 32 / bits;
    const int tiles = (N + 32 * cpt - 1) / (32 * cpt);
    const int units = K / ((bits == 3 || bits == 5 || bits == 6) ? 8 : 16);      // slabs of R rows
    int kc = 2 * sms / tiles;                 // never more CTAs than are resident at once (two per SM): a few CTAs in a second round would double the time
    const int most = (units + kQvWarps - 1) / kQvWarps;
    if (kc > most) kc = most;
    if (kc > 32) kc = 32;                     // the chunks of a column tile are added by one CTA
    return kc < 1 ? 1 : kc;
}

bool qvm_fast_supported(int N, int K, int bits, int group_size) {
    const int cpt = (bits == 3 || bits == 5 || bits == 6) ? 32 : 32 / bits;
    return N % cpt == 0 && K % group_size == 0 && group_size % 16 == 0 && (bits == 2 || bits == 3 || bits == 4 || bits == 5 || bits == 6 || bits == 8);
}

size_t qvm_scratch_bytes(int M, int N, int KC) {
    return KC > 1 ? kQvTickets * sizeof(uint32_t) + static_cast<size_t>(KC) * M * N * sizeof(float) : 0;
}

// scratch: qvm_scratch_bytes when KC > 1 (qvm_k_chunks), else unused; its first kQvTickets words are arrival counters
// that are zero between launches (the caller zeroes them when the block is allocated)
cudaError_t launch_qvm(Ctx *ctx, cudaStream_t st, const void *w, const void *scales, const void *biases, const void *x, void *out,
                       int M, int N, int K, int bits, int group_size, int dt, void *scratch, int KC) {
    if (M <= 0 || N <= 0) return cudaSuccess;
    const auto al16 = [](const void *p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; };
    const bool vec_ok = al16(w) && al16(scales) && al16(biases) && al16(x) && (static_cast<size_t>(K) * dtype_size(dt)) % 16 == 0;
    if (!qvm_fast_supported(N, K, bits, group_size) || M > 65535 || !vec_ok) {
        const size_t mn = static_cast<size_t>(M) * N;
        size_t grid = (mn + 255) / 256;
        if (grid > static_cast<size_t>(ctx->sm_count) * 16) grid = static_cast<size_t>(ctx->sm_count) * 16;
        qvm_generic_kernel<<<static_cast<int>(grid), 256, 0, st>>>(static_cast<const uint32_t *>(w), scales, biases, x, out, M, N, K,
                                                                    group_size, bits, dt);
        return cudaGetLastError();
    }
    if (KC > 1 && !scratch) return cudaErrorInvalidValue;
    const int cpt = (bits == 3 || bits == 5 || bits == 6) ? 32 : 32 / bits;
    const long long n_tickets = static_cast<long long>((N + 32 * cpt - 1) / (32 * cpt)) * M;
    uint32_t *tickets = KC > 1 && n_tickets <= kQvTickets ? static_cast<uint32_t *>(scratch) : nullptr;   // else a second kernel adds the chunks
    float *partial = KC > 1 ? reinterpret_cast<float *>(static_cast<uint32_t *>(scratch) + kQvTickets) : nullptr;
    cudaError_t e;
    switch (bits) {
        case 2: e = qvm_launch<2>(st, w, scales, biases, x, partial, tickets, out, M, N, K, group_size, KC, dt); break;
        case 3: e = qvm_launch<3>(st, w, scales, biases, x, partial, tickets, out, M, N, K, group_size, KC, dt); break;
        case 4: e = qvm_launch<4>(st, w, scales, biases, x, partial, tickets, out, M, N, K, group_size, KC, dt); break;
        case 5: e = qvm_launch<5>(st, w, scales, biases, x, partial, tickets, out, M, N, K, group_size, KC, dt); break;
        case 6: e = qvm_launch<6>(st, w, scales, biases, x, partial, tickets, out, M, N, K, group_size, KC, dt); break;
        default: e = qvm_launch<8>(st, w, scales, biases, x, partial, tickets, out, M, N, K, group_size, KC, dt); break;
    }
    if (e != cudaSuccess || KC == 1 || tickets) return e;
    const size_t mn = static_cast<size_t>(M) * N;
    size_t grid = (mn + 255) / 256;
    if (grid > static_cast<size_t>(ctx->sm_count) * 8) grid = static_cast<size_t>(ctx->sm_count) * 8;
    qvm_sum_kernel<<<static_cast<int>(grid), 256, 0, st>>>(partial, out, mn, KC, dt);
    return cudaGetLastError();
}

}  // namespace mtc
