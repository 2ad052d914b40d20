// qmm / gather_qmm — prefill and MoE matmuls on the sm_100a tensor cores.
//
//   dense : out[m, n]  = sum_k x[m, k] * w(n, k)                      (mt_qmm_mma family)
//   gather: out[t, n]  = sum_k x[t, k] * w(E(t), n, k), rows sorted by expert (mt_moe_gather_qmm_*)
//
// Stands in for mt_qmm_mma and its int8/int2/bit-stream variants
// (crates/metaltile-std/src/mlx/quantized.rs:2106-2362,2731,3330,4720-5012) and for the MoE gather
// kernels (crates/metaltile-std/src/ffai/moe.rs:358-605,2256-2835).  Like the reference's MMA kernels
// the weight tile is dequantised to the activation type on chip and fed to the matrix unit with f32
// accumulation (quantized.rs:2245-2252); unlike them neither M nor the rows of an expert need padding.
//
// The product is computed transposed: D^T[n, t] = W_tile[128 x K] * X_chunk[TN x K]^T, so the
// dequantised weights are the A operand (always a full 128-row MMA, however few tokens there are) and
// the activations are the B operand (TN = 16..256 token rows, straight from TMA).
//
// One persistent CTA per SM, 512 threads, warp-specialised:
//   warp 0      producer   one lane issues TMA (cp.async.bulk.tensor, 128B swizzle) loads of the X
//                          chunk [TN x 64] into a 4-stage shared-memory ring
//   warp 1      MMA        one lane issues tcgen05.mma (M=128, N=TN, K=16, kind::f16), accumulators in
//                          TMEM, double buffered (2 x 256 columns)
//   warp 2      TMEM allocation / deallocation
//   warps 4-7   epilogue   tcgen05.ld of the finished accumulator, f32 -> T, transposed stores to out
//   warps 8-15  dequant    256 threads = 128 weight rows x 2 halves of a 64-wide k block: packed words
//                          come straight from global memory into registers one k block ahead, every
//                          code is extracted with one LOP3 ((win & mask<<p) | 1.0f, minus 1.0f =
//                          q * 2^(p-23)), w = q*scale + bias in f32, rounded to f16, written as the
//                          K-major 128B-swizzled A operand tile the MMA reads
// Stage hand-off uses mbarriers; tcgen05.commit releases a stage when its MMAs have read it.  Every
// wait is bounded: on expiry the kernel records a code in the context's status word, all roles leave
// their loops, TMEM is released and the kernel returns.
//
// Work items (weight-row tile, expert, first token row, token count) are enumerated arithmetically
// for the dense case and read from a list in scratch memory for the gather case; that list is built
// on the device from expert_offsets by build_items_kernel.
#include <cuda.h>

#include "common.cuh"

namespace mtc {
namespace {

constexpr int BMW = 128;         // weight rows per tile (TMEM lanes, MMA M)
constexpr int BK = 64;           // k per stage: 64 x 16-bit = one 128B swizzle row
constexpr int TN_MAX = 256;      // token rows per tile (TMEM columns of one accumulator, MMA N)
constexpr int MAX_STAGES = 8;    // ring depth: as many stages as fit in RING_BYTES, at most this
constexpr int RING_BYTES = 224 * 1024;      // stages of the ring, then the raw staging buffers; SmemCtrl follows
constexpr int SB_PER_RAW = 4;               // k blocks per raw super-block: 256 codes = 32*BITS bytes per weight row
constexpr int RAW_SB_BYTES = 2 * BMW * 16;  // scales then biases of a super-block: 16 bytes per row each
constexpr int A_BYTES = BMW * BK * 2;       // 16 KB, dequantised weights
constexpr int B_BYTES = TN_MAX * BK * 2;    // 32 KB, activations
constexpr int NUM_THREADS = 512;
constexpr int DEQ_WARP0 = 8, DEQ_THREADS = 256;
constexpr int EPI_WARP0 = 4;
constexpr uint32_t kSpinLimit = 1u << 22;   // bounded waits: ~seconds, then give up
struct QmmParams {
    const uint32_t *w;
    const void *scales, *biases;
    void *out;
    void *outs[8];               // destinations of the result block (outs[0] == out); further ones may be peers' memory
    int n_outs;
    long long out_ld;            // elements between consecutive token rows of a destination (N, or the width of a wider matrix)
    uint32_t *status;
    const int4 *items;           // gather: {n_tile, expert, row_start, row_count}; dense: nullptr
    const int *item_count;       // gather: device counter; dense: nullptr
    int dense_items;             // dense: number of items = n_tiles * m_chunks
    int m_chunks;                // dense: token chunks per weight-row tile
    int M;                       // dense: rows of x; gather: total rows of x
    int N, K, gs_shift;          // N: weight rows per expert (output columns)
    int op_f16;                  // MMA operand format: 1 = f16, 0 = bf16 (dequantised W and the X tensor map)
    int sb_dt;                   // element type of scales / biases (MTC_F16 or MTC_BF16)
    int out_dt;                  // element type of out
    const float *tok_scale;      // per-token power-of-two factor applied in the epilogue, or nullptr
    int wpr, gpr;                // words / groups per weight row
    int TN;                      // token rows per item (TMA box rows, MMA N)
    int nst;                     // ring depth
    uint32_t hint_ns;            // base suspend-time hint of the waits (0: plain polling)
    int raw;                     // 1: packed words reach the dequant warps through shared memory (cp.async, whole lines)
    uint32_t raw_off, raw_tile;  // byte offset of the raw buffers in shared memory; bytes of one tile of one buffer
    int wide_items;              // wide: items [0, wide_items) cover two token chunks, each later pair of items one such unit
    int wide;                    // 1: a dense item covers up to 2 TN token rows: one dequantised W stage meets two X chunks, both
                                 //    accumulators belong to the item (the dequant work per flop halves; no epilogue overlap)
    int n_tiles;                 // dense: weight-row tiles
    int ksplit;                  // dense, one token chunk: K slices per weight-row tile (each an item of its own); 1 = none
    int kb_per;                  // k blocks per item (K / BK / ksplit)
    float *partial;              // ksplit > 1: f32 partial sums [ksplit][M][N], added by ksplit_sum_kernel
    int pdl_roles;               // programmatic dependent launch: 1 = only the roles that touch what an earlier kernel of the
                                 //    stream may have written (producer: x; epilogue: token factors, out) wait for it, the
                                 //    dequant warps start on the weights at once; 0 = every thread waits first
    uint32_t idesc;
};

struct __align__(8) SmemCtrl {
    uint64_t full[MAX_STAGES];   // the X stage has landed (TMA transaction bytes) and the dequant warps finished the W stage
    uint64_t empty[MAX_STAGES];  // MMAs that read the stage have completed
    uint64_t acc_full[2];        // accumulator buffer complete
    uint64_t acc_empty[2];       // epilogue drained the accumulator buffer
    uint64_t raw_full[2];        // every dequant warp's copies of a raw super-block have landed
    uint32_t tmem_base;
    volatile uint32_t abort;
};

// ---- PTX wrappers -------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// try_wait with a suspend-time hint: the thread may sleep in hardware for up to `ns` before it reports failure
__device__ __forceinline__ bool mbar_try_hint(uint64_t *bar, uint32_t parity, uint32_t ns) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity), "r"(ns) : "memory");
    return ok != 0;
}
// Bounded wait.  Returns false (and raises the CTA's abort flag + the global status word) when the
// barrier did not complete within kSpinLimit polls or another role already aborted.  `sleep_ns` > 0 lets
// the hardware suspend the thread between polls: without it the fourteen waiting threads of a CTA issue
// more poll instructions than the dequant warps issue useful ones (ncu: SYNCS + BRA + BREAK were 60 % of all
// instructions executed).
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, SmemCtrl *ctl, uint32_t *status, uint32_t code,
                                          uint32_t sleep_ns = 0) {
    for (uint32_t i = 0; i < kSpinLimit; ++i) {
        if (sleep_ns ? mbar_try_hint(bar, parity, sleep_ns) : mbar_try(bar, parity)) return true;
        if ((i & 63u) == 63u && ctl->abort) return false;
    }
    ctl->abort = 1;
    atomicCAS(status, 0u, code);
    return false;
}
// Whole-warp wait: lane 0 polls, the result is broadcast.
__device__ __forceinline__ bool mbar_wait_warp(uint64_t *bar, uint32_t parity, SmemCtrl *ctl, uint32_t *status, uint32_t code,
                                               uint32_t sleep_ns) {
    uint32_t ok = 1;
    if ((threadIdx.x & 31) == 0) ok = mbar_wait(bar, parity, ctl, status, code, sleep_ns) ? 1u : 0u;
    ok = __shfl_sync(0xffffffffu, ok, 0);
    return ok != 0;
}

__device__ __forceinline__ void tma_load_2d(void *dst, const CUtensorMap *map, int c0, int c1, uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(smem_u32(bar)) : "memory");
}

// Shared-memory matrix descriptor: K-major operand, 128-byte swizzle, 8-row atoms 1024 B apart.
__device__ __forceinline__ uint64_t make_desc_sw128(uint32_t saddr) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4);   // start address  [0,14)
    d |= static_cast<uint64_t>(1) << 16;                   // leading byte offset (unused with 128B swizzle)
    d |= static_cast<uint64_t>(1024 >> 4) << 32;           // stride byte offset [32,46)
    d |= static_cast<uint64_t>(1) << 46;                   // descriptor version (sm_100)
    d |= static_cast<uint64_t>(2) << 61;                   // SWIZZLE_128B
    return d;
}

__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
    return pred != 0;
}
__device__ __forceinline__ void umma_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ uint32_t pack_f16x2(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));   // first source -> upper half
    return r;
}
// (win & mask) | 1.0f in one LOP3: the constant 1.0f sits in a register, the mask is an immediate
__device__ __forceinline__ float code_plus_one(uint32_t win, uint32_t mask, uint32_t one) {
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(win), "r"(mask), "r"(one));
    return __uint_as_float(r);
}
__device__ __forceinline__ void st_shared_v4(uint32_t saddr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(saddr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

__device__ __forceinline__ void cp_async_16(uint32_t dst, const void *src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
template <int BYTES>
__device__ __forceinline__ void cp_async_small(uint32_t dst, const void *src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], %2;" ::"r"(dst), "l"(src), "n"(BYTES) : "memory");
}
// BITS consecutive words from shared memory, with the widest loads the 4*BITS-byte pieces are aligned for
template <int BITS>
__device__ __forceinline__ void lds_words(uint32_t addr, uint32_t (&w)[BITS]) {
    if constexpr (BITS % 4 == 0) {
#pragma unroll
        for (int i = 0; i < BITS / 4; ++i)
            asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(w[4 * i]), "=r"(w[4 * i + 1]), "=r"(w[4 * i + 2]), "=r"(w[4 * i + 3]) : "r"(addr + 16 * i));
    } else if constexpr (BITS % 2 == 0) {
#pragma unroll
        for (int i = 0; i < BITS / 2; ++i)
            asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(w[2 * i]), "=r"(w[2 * i + 1]) : "r"(addr + 8 * i));
    } else {
#pragma unroll
        for (int i = 0; i < BITS; ++i) asm volatile("ld.shared.u32 %0, [%1];" : "=r"(w[i]) : "r"(addr + 4 * i));
    }
}

// ---- dequantisation of half a W row segment (32 codes = BITS words) into 4 swizzled 16-byte chunks --
template <int BITS>
struct QPack {
    static constexpr int CPW = 23 / BITS;       // codes per window: a window must fit the 23 mantissa bits
    static constexpr uint32_t MASK = (1u << BITS) - 1u;
};

// 32 codes (BITS words) of one weight row, straight from global memory
template <int BITS>
__device__ __forceinline__ void load_half_words(const uint32_t *p, uint32_t (&w)[BITS], bool valid) {
    if (!valid) {
#pragma unroll
        for (int i = 0; i < BITS; ++i) w[i] = 0u;
        return;
    }
    if constexpr (BITS % 4 == 0) {          // 4-, 8-bit: 16-byte pieces
#pragma unroll
        for (int i = 0; i < BITS / 4; ++i) {
            const uint4 v = __ldg(reinterpret_cast<const uint4 *>(p) + i);
            w[4 * i] = v.x; w[4 * i + 1] = v.y; w[4 * i + 2] = v.z; w[4 * i + 3] = v.w;
        }
    } else if constexpr (BITS % 2 == 0) {   // 2-, 6-bit: 8-byte pieces
#pragma unroll
        for (int i = 0; i < BITS / 2; ++i) {
            const uint2 v = __ldg(reinterpret_cast<const uint2 *>(p) + i);
            w[2 * i] = v.x; w[2 * i + 1] = v.y;
        }
    } else {                                // 3-, 5-bit: single words
#pragma unroll
        for (int i = 0; i < BITS; ++i) w[i] = __ldg(p + i);
    }
}

// dst[c] = shared-memory address of the c-th of this thread's four 16-byte chunks (swizzle applied by the caller)
// 4- and 8-bit codes in packed-half arithmetic.  `byte-permute | 0x6400` makes two f16 values 1024 + q without a
// conversion, HSUB2 removes the 1024 exactly, and one HFMA2 per two codes gives round_f16(q*scale + bias) - the
// value the f32 path rounds to, up to double rounding - already in the operand's type: ~2 instructions per code
// instead of ~3.5.  The caller uses it only when the scale is a normal f16 number.
template <int BITS>
__device__ __forceinline__ void dequant_half_h2(const uint32_t (&w)[BITS], float s, float b, const uint32_t (&dst)[4],
                                                uint32_t stage_off) {
    static_assert(BITS == 4 || BITS == 8, "packed-half path: 4- and 8-bit codes");
    const __half2 s2 = __float2half2_rn(s), b2 = __float2half2_rn(b);
    const __half2 k1024 = __half2half2(__ushort_as_half(0x6400));
    uint32_t magic = 0x64006400u;
    asm volatile("" : "+r"(magic));          // in a register, so that mask-and-or is a single LOP3
    auto finish = [&](uint32_t t) {
        const __half2 q = __hsub2(*reinterpret_cast<const __half2 *>(&t), k1024);
        const __half2 v = __hfma2(q, s2, b2);
        return *reinterpret_cast<const uint32_t *>(&v);
    };
    if (BITS == 4) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {        // word i = codes 8i..8i+7 = one 16-byte chunk of the tile row
            const uint32_t lo = w[i], hi = w[i] >> 4;      // byte j of lo / hi has code 2j / 2j+1 in its low nibble
            uint32_t o[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint32_t t = __byte_perm(lo, hi, ((4 + j) << 8) | j);          // code 2j -> bits 0..3, code 2j+1 -> bits 16..19
                uint32_t r;
                asm("lop3.b32 %0, %1, 0x000F000F, %2, 0xEA;" : "=r"(r) : "r"(t), "r"(magic));
                o[j] = finish(r);
            }
            st_shared_v4(dst[i] + stage_off, o[0], o[1], o[2], o[3]);
        }
    } else {
#pragma unroll
        for (int i = 0; i < 4; ++i) {        // words 2i, 2i+1 = codes 8i..8i+7
            uint32_t o[4];
#pragma unroll
            for (int j = 0; j < 4; ++j)      // two bytes of word 2i + j/2 under the 0x64 exponent bytes
                o[j] = finish(__byte_perm(w[2 * i + (j >> 1)], 0x64646464u, (j & 1) ? 0x4342 : 0x4140));
            st_shared_v4(dst[i] + stage_off, o[0], o[1], o[2], o[3]);
        }
    }
}

template <int BITS>
__device__ __forceinline__ void dequant_half(const uint32_t (&w)[BITS], float s, float b, const uint32_t (&dst)[4],
                                             uint32_t stage_off) {
    using Q = QPack<BITS>;
    if constexpr (BITS == 4 || BITS == 8) {
        // scale a normal f16 number (its exact value survives the conversion), bias within f16 range
        if (fabsf(s) >= 6.104e-5f && fabsf(s) <= 65504.0f && fabsf(b) <= 65504.0f) {
            dequant_half_h2<BITS>(w, s, b, dst, stage_off);
            return;
        }
    }
    // a code at bit p of a window becomes q * 2^(p-23) after the magic subtract: fold 2^(23-p) into the scale
    float sp[Q::CPW];
#pragma unroll
    for (int c = 0; c < Q::CPW; ++c) sp[c] = s * __uint_as_float(static_cast<uint32_t>(23 - c * BITS + 127) << 23);
    uint32_t one = 0x3F800000u;
    asm volatile("" : "+r"(one));            // keep 1.0f in a register so the extraction is a single LOP3
    float vals[8];
#pragma unroll
    for (int i = 0; i < 32; ++i) {
        const int wi = i / Q::CPW, c = i % Q::CPW;
        const int sbit = wi * Q::CPW * BITS, word = sbit / 32, sh = sbit % 32;
        uint32_t win;
        if (sh == 0) win = w[word];
        else if (word + 1 < BITS) win = __funnelshift_r(w[word], w[word + 1], sh);
        else win = w[word] >> sh;
        const float f = code_plus_one(win, Q::MASK << (c * BITS), one) - 1.0f;
        vals[i & 7] = fmaf(f, sp[c], b);
        if ((i & 7) == 7)
            st_shared_v4(dst[i >> 3] + stage_off, pack_f16x2(vals[0], vals[1]), pack_f16x2(vals[2], vals[3]),
                         pack_f16x2(vals[4], vals[5]), pack_f16x2(vals[6], vals[7]));
    }
}

// 16-bit scale (or bias) of k block j (0..3) of a super-block for the thread's 32-code half h, out of the row's line:
// group 32: entry 2j + h; group 64: entry j; group 128: entry j / 2.  j is a compile-time constant where this is used.
__device__ __forceinline__ uint32_t sb_half(const uint4 &v, int j, int h, int gs_shift) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    if (gs_shift == 5) return (w[j] >> (16 * h)) & 0xFFFFu;
    if (gs_shift == 6) return (w[j >> 1] >> (16 * (j & 1))) & 0xFFFFu;
    return (w[0] >> (16 * ((j >> 1) & 1))) & 0xFFFFu;
}

struct Item {
    int n_tile, expert, row0, rows;
    int nc;                                 // token chunks of TN rows covered (1 or 2): one accumulator each
    int kb0, ks;                            // first k block and index of the K slice (0, 0 unless the launch splits K)
};

template <bool KSPLIT>
__device__ __forceinline__ Item get_item(const QmmParams &p, int i) {
    Item it;
    it.kb0 = 0;
    it.ks = 0;
    if (p.items) {
        const int4 v = __ldg(p.items + i);
        it.n_tile = v.x; it.expert = v.y & 0xFFFFFF; it.row0 = v.z; it.rows = v.w;
        it.nc = 1;
    } else if (p.wide) {
        // dense, wide: m_chunks items of up to 2 TN token rows per weight-row tile, adjacent so that CTAs running at
        // the same time share the tile's packed words in L2
        // the wide items that do not fill a whole round of the grid (items >= wide_items) run as two single-chunk
        // items each, so that the last round is a short one
        const int u = i < p.wide_items ? i : p.wide_items + ((i - p.wide_items) >> 1);
        const int half = i < p.wide_items ? 0 : ((i - p.wide_items) & 1);
        const int unit = u / p.m_chunks, chunk = u - unit * p.m_chunks;
        it.expert = 0;
        it.n_tile = unit;
        it.row0 = chunk * 2 * p.TN + half * p.TN;
        it.rows = i < p.wide_items ? min(2 * p.TN, p.M - it.row0) : min(p.TN, p.M - it.row0);
        it.nc = it.rows > p.TN ? 2 : 1;
    } else {
        // dense: the token chunks of one weight-row tile are adjacent, so CTAs running at the same time share its
        // packed words in L2
        // K slices of one tile are adjacent items too
        const int b = KSPLIT ? i / p.ksplit : i;
        if (KSPLIT) {
            it.ks = i - b * p.ksplit;
            it.kb0 = it.ks * p.kb_per;
        }
        const int unit = b / p.m_chunks, chunk = b - unit * p.m_chunks;
        it.nc = 1;
        it.expert = 0;
        it.n_tile = unit;
        it.row0 = chunk * p.TN;
        it.rows = min(p.TN, p.M - it.row0);
    }
    return it;
}

// KSPLIT: the launch cuts K into slices (items carry a first k block, the epilogue writes f32 partial sums); a
// separate instantiation, so that the code of every other launch is what it was without the feature.
template <int BITS, bool KSPLIT>
__global__ void __launch_bounds__(NUM_THREADS, 1)
qmm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_x, const QmmParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    const int nst = p.nst;
    const uint32_t w_stage = A_BYTES;                                   // one dequantised W tile per stage
    const uint32_t x_stage = static_cast<uint32_t>(p.TN) * BK * 2;      // one X chunk; multiple of 2 KB
    const uint32_t x_slot = (p.wide ? 2 : 1) * x_stage;                 // one or two X chunks per stage
    uint8_t *sW = smem;                                  // nst x w_stage: dequantised weights (A operand)
    uint8_t *sX = smem + nst * w_stage;                  // nst x x_slot: activations (B operand)
    SmemCtrl *ctl = reinterpret_cast<SmemCtrl *>(smem + RING_BYTES);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int num_kb = KSPLIT ? p.kb_per : p.K / BK;       // k blocks per item
    const int num_items = p.items ? __ldg(p.item_count) : p.dense_items;
    const uint32_t x_bytes = static_cast<uint32_t>(p.TN) * BK * 2;

    if (threadIdx.x == 0) {
        for (int s = 0; s < MAX_STAGES; ++s) {
            mbar_init(&ctl->full[s], 1 + DEQ_THREADS / 32);
            mbar_init(&ctl->empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&ctl->acc_full[b], 1);
            mbar_init(&ctl->acc_empty[b], 4);
            mbar_init(&ctl->raw_full[b], DEQ_THREADS / 32);
        }
        ctl->abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 2) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&ctl->tmem_base)), "r"(512));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = ctl->tmem_base;
    asm volatile("griddepcontrol.launch_dependents;");
    if (!p.pdl_roles) asm volatile("griddepcontrol.wait;" ::: "memory");

    if (warp == 0) {
        // ---------------- producer: TMA loads of the X chunk ----------------
        if (lane == 0) {
            int s = 0;
            uint32_t ph = 0;                              // stage and ring-pass parity, advanced without a division
            bool ok = true;
            if (p.pdl_roles) asm volatile("griddepcontrol.wait;" ::: "memory");      // x may come from the previous kernel
            for (int i = blockIdx.x; i < num_items && ok; i += gridDim.x) {
                const Item item = get_item<KSPLIT>(p, i);
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!(ok = mbar_wait(&ctl->empty[s], ph ^ 1, ctl, p.status, 0x101, p.hint_ns))) break;
                    mbar_expect_tx(&ctl->full[s], x_bytes * item.nc);
                    for (int c = 0; c < item.nc; ++c)
                        tma_load_2d(sX + s * x_slot + c * x_stage, &tmap_x, ((KSPLIT ? item.kb0 : 0) + kb) * BK, item.row0 + c * p.TN, &ctl->full[s]);
                    if (++s == nst) {
                        s = 0;
                        ph ^= 1;
                    }
                }
            }
            if (!ok) {   // let copies already in flight land before the CTA tears down
                for (int s = 0; s < nst; ++s)
                    for (uint32_t j = 0; j < 4096 && !mbar_try(&ctl->full[s], 0) && !mbar_try(&ctl->full[s], 1); ++j) {}
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        // The whole warp runs the loop so that stage counters, descriptors and accumulator addresses are
        // warp-uniform values; one elected lane issues.  (With the loop under `if (lane == 0)` every operand of
        // every tcgen05.mma was moved to a uniform register first and two barriers were polled one after the other:
        // 1100 cycles per k block whatever the tile width, measured - the issuer, not the tensor pipe or the
        // producers, set the pace of the kernel.)
        {
            uint32_t tile_i = 0;
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            const bool leader = elect_one();
            const uint64_t adesc0 = make_desc_sw128(smem_u32(sW)), bdesc0 = make_desc_sw128(smem_u32(sX));
            const uint32_t a_step = w_stage >> 4, b_step = x_slot >> 4;       // descriptor address units per stage
            for (int i = blockIdx.x; i < num_items && ok; i += gridDim.x, ++tile_i) {
                const Item item = get_item<KSPLIT>(p, i);
                // wide items: both 256-column accumulators belong to one item (no double buffering);
                // otherwise the two accumulators alternate so that the epilogue overlaps the next item
                const bool both = p.wide != 0;
                const int buf = both ? 0 : (tile_i & 1);
                const uint32_t acc_ph = (both ? tile_i : (tile_i >> 1)) & 1;
                if (!(ok = mbar_wait_warp(&ctl->acc_empty[buf], acc_ph ^ 1, ctl, p.status, 0x201, 0))) break;
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + buf * TN_MAX;
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!(ok = mbar_wait_warp(&ctl->full[s], ph, ctl, p.status, 0x202, 0))) break;
                    tc_fence_after();
                    if (leader) {
                        const uint64_t bdesc = bdesc0 + static_cast<uint64_t>(s * b_step);
                        const uint64_t adesc = adesc0 + static_cast<uint64_t>(s * a_step);
                        for (int c = 0; c < item.nc; ++c) {          // token chunk c accumulates in TMEM half c
                            const uint64_t bd = bdesc + static_cast<uint64_t>(c * (x_stage >> 4));
#pragma unroll
                            for (int k = 0; k < BK / 16; ++k)       // 16 elements = 32 bytes further along the swizzled row
                                umma_f16(tmem_d + c * TN_MAX, adesc + 2 * k, bd + 2 * k, p.idesc, (kb | k) ? 1u : 0u);
                        }
                        umma_commit(&ctl->empty[s]);         // frees the stage when these MMAs have read it
                    }
                    __syncwarp();
                    if (++s == nst) {
                        s = 0;
                        ph ^= 1;
                    }
                }
                if (ok && leader) umma_commit(&ctl->acc_full[buf]);
                __syncwarp();
            }
        }
    } else if (warp >= EPI_WARP0 && warp < EPI_WARP0 + 4) {
        // ---------------- epilogue: TMEM -> registers -> out (transposed) ----------------
        const int q = warp - EPI_WARP0;          // == warp % 4: the TMEM lane quarter this warp may read
        uint32_t tile_i = 0;
        bool ok = true;
        if (p.pdl_roles) asm volatile("griddepcontrol.wait;" ::: "memory");          // token factors; nothing is stored before this
        for (int i = blockIdx.x; i < num_items && ok; i += gridDim.x, ++tile_i) {
            const bool both = p.wide != 0;
            const int buf = both ? 0 : (tile_i & 1);
            const uint32_t acc_ph = (both ? tile_i : (tile_i >> 1)) & 1;
            const Item item = get_item<KSPLIT>(p, i);
            if (!(ok = mbar_wait_warp(&ctl->acc_full[buf], acc_ph, ctl, p.status, 0x301, p.hint_ns))) break;
            tc_fence_after();
            const int n = item.n_tile * BMW + q * 32 + lane;     // output column owned by this thread
            const bool n_ok = n < p.N;
            for (int hh = 0; hh < item.nc; ++hh) {               // accumulators of this item: 1 or 2
                const int c = hh;
                const int row_base = item.row0 + c * p.TN;
                const int rows_h = item.nc == 2 ? min(p.TN, item.rows - c * p.TN) : item.rows;
                const int cols = (rows_h + 15) & ~15;
                for (int c0 = 0; c0 < cols; c0 += 16) {
                    float ts[16];                  // per-token factors first, so their latency hides behind the TMEM load
#pragma unroll
                    for (int j = 0; j < 16; ++j)
                        ts[j] = (p.tok_scale && c0 + j < rows_h) ? __ldg(p.tok_scale + row_base + c0 + j) : 1.0f;
                    uint32_t v[16];
                    tmem_ld16(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + (buf + hh) * TN_MAX + c0, v);
                    if (KSPLIT && n_ok) {
                        // a K slice: f32 partial sums, 128-byte segments per warp and token row
                        float *o = p.partial + (static_cast<size_t>(item.ks) * p.M + row_base + c0) * p.N + n;
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            if (c0 + j < rows_h) o[static_cast<size_t>(j) * p.N] = __uint_as_float(v[j]) * ts[j];
                    } else if (n_ok) {
                        // lanes of a warp hold 32 consecutive columns of the same output row: 64-byte segments
                        unsigned short hv[16];
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            const float f = __uint_as_float(v[j]) * ts[j];
                            hv[j] = p.out_dt == MTC_F16 ? __half_as_ushort(__float2half_rn(f)) : __bfloat16_as_ushort(__float2bfloat16_rn(f));
                        }
                        for (int d = 0; d < p.n_outs; ++d) {
                            unsigned short *o = static_cast<unsigned short *>(p.outs[d]) + static_cast<size_t>(row_base + c0) * p.out_ld + n;
#pragma unroll
                            for (int j = 0; j < 16; ++j)
                                if (c0 + j < rows_h) o[static_cast<size_t>(j) * p.out_ld] = hv[j];
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&ctl->acc_empty[buf]);
        }
    } else if (warp >= DEQ_WARP0) {
        // ---------------- dequant: packed W rows -> swizzled A operand tile ----------------
        const int t = threadIdx.x - DEQ_WARP0 * 32;
        const int r = t & (BMW - 1);                       // row of the W tile
        const int h = t >> 7;                              // which 32-code half of the 64-wide k block
        const int r7 = r & 7;
        uint32_t dst[4];                                   // this thread's four swizzled 16-byte chunks in stage 0
#pragma unroll
        for (int c = 0; c < 4; ++c)
            dst[c] = smem_u32(sW) + (r >> 3) * 1024 + r7 * 128 + (((h * 4 + c) ^ r7) << 4);
        int s = 0;
        uint32_t ph = 0;                                  // stage and ring-pass parity, advanced without a division
        bool ok = true;
        if (p.raw) {
            // Packed words through shared memory.  A thread that loads its own row's 16 bytes per k block makes
            // every warp-load touch 32 cache lines (plus 64 for the scale and the bias): measured, the L1 tag stage,
            // not the arithmetic, set the pace of a k block (0.8 us whatever the tile width or the ring depth).  Here
            // the 256 dequant threads copy a super-block of 4 k blocks of the tile - 32*BITS contiguous bytes per
            // row, 16 bytes per thread and copy, two rows per warp-copy - with cp.async into one of two raw
            // buffers, one super-block ahead and across items, and read their pieces back from shared memory.
            constexpr int ROW_BYTES = 32 * BITS, PITCH = ROW_BYTES + 16, CPR = 2 * BITS;   // padded rows: conflict-free reads
            const uint32_t raw0 = smem_u32(smem) + p.raw_off;
            const uint32_t buf_bytes = p.raw_tile;
            const int num_sb = num_kb / SB_PER_RAW;
            const int sb_bytes = (2 * SB_PER_RAW * BK) >> p.gs_shift;       // scale bytes of a row per super-block: 16, 8 or 4
            const int srow = t & (BMW - 1), sarr = t >> 7;                  // this thread copies scales (0) or biases (1) of a row
            auto issue = [&](const Item &im, int sb_rel, int buf) {
                const int sbk = (KSPLIT ? im.kb0 / SB_PER_RAW : 0) + sb_rel;      // super-block of the row
                const uint32_t dstt = raw0 + buf * buf_bytes;
                const int n0 = im.n_tile * BMW;
                const size_t erow = static_cast<size_t>(im.expert) * p.N;
#pragma unroll
                for (int c = 0; c < BITS; ++c) {
                    const int ch = c * DEQ_THREADS + t, row = ch / CPR, col = ch - row * CPR;
                    const size_t grow = erow + min(n0 + row, p.N - 1);          // rows past N copy the last row; never stored
                    cp_async_16(dstt + row * PITCH + col * 16,
                                reinterpret_cast<const char *>(p.w + grow * p.wpr) + static_cast<size_t>(sbk) * ROW_BYTES + col * 16);
                }
                const size_t grow = erow + min(n0 + srow, p.N - 1);
                const char *src = static_cast<const char *>(sarr ? p.biases : p.scales) + (grow * p.gpr) * 2 +
                                  static_cast<size_t>(sbk) * sb_bytes;
                const uint32_t d = dstt + BMW * PITCH + sarr * (BMW * 16) + srow * 16;
                if (sb_bytes == 16) cp_async_16(d, src);
                else if (sb_bytes == 8) cp_async_small<8>(d, src);
                else cp_async_small<4>(d, src);
            };
            // request stream: (item, super-block) pairs in processing order
            int i_n = blockIdx.x, sb_n = 0;
            Item item_n{};
            if (i_n < num_items) {
                item_n = get_item<KSPLIT>(p, i_n);
                issue(item_n, 0, 0);
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
            uint32_t q = 0;
            for (int i = blockIdx.x; i < num_items && ok; i += gridDim.x) {
                const Item item = get_item<KSPLIT>(p, i);
                for (int sbk = 0; sbk < num_sb && ok; ++sbk, ++q) {
                    const int buf = q & 1;
                    // this super-block has landed: my copies, then every warp's (which also says that every warp is
                    // done reading the other buffer)
                    asm volatile("cp.async.wait_group 0;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&ctl->raw_full[buf]);
                    if (!(ok = mbar_wait_warp(&ctl->raw_full[buf], (q >> 1) & 1, ctl, p.status, 0x402, 0))) break;
                    // the next one, into the other buffer
                    if (++sb_n == num_sb) {
                        sb_n = 0;
                        i_n += gridDim.x;
                        if (i_n < num_items) item_n = get_item<KSPLIT>(p, i_n);
                    }
                    if (i_n < num_items) issue(item_n, sb_n, buf ^ 1);
                    asm volatile("cp.async.commit_group;" ::: "memory");
                    // the row's scales and biases of the whole super-block: one 16-byte load each (4, 8 or 16 bytes are in use)
                    uint4 sline, bline;
                    {
                        const uint32_t sb_addr = raw0 + buf * buf_bytes + BMW * PITCH + r * 16;
                        asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(sline.x), "=r"(sline.y), "=r"(sline.z), "=r"(sline.w) : "r"(sb_addr));
                        asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(bline.x), "=r"(bline.y), "=r"(bline.z), "=r"(bline.w) : "r"(sb_addr + BMW * 16));
                    }
#pragma unroll
                    for (int j = 0; j < SB_PER_RAW; ++j) {
                        if (!(ok = mbar_wait_warp(&ctl->empty[s], ph ^ 1, ctl, p.status, 0x401, 0))) break;
                        {
                            const uint32_t base = raw0 + buf * buf_bytes;
                            uint32_t wv[BITS];
                            lds_words<BITS>(base + r * PITCH + (2 * j + h) * (4 * BITS), wv);
                            const unsigned short sr = static_cast<unsigned short>(sb_half(sline, j, h, p.gs_shift));
                            const unsigned short br = static_cast<unsigned short>(sb_half(bline, j, h, p.gs_shift));
                            float sc, bi;
                            if (p.sb_dt == MTC_F16) {
                                sc = __half2float(__ushort_as_half(sr));
                                bi = __half2float(__ushort_as_half(br));
                            } else {
                                sc = __uint_as_float(static_cast<uint32_t>(sr) << 16);
                                bi = __uint_as_float(static_cast<uint32_t>(br) << 16);
                            }
                            dequant_half<BITS>(wv, sc, bi, dst, s * w_stage);
                        }
                        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy stores -> async proxy (MMA)
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&ctl->full[s]);
                        if (++s == nst) {
                            s = 0;
                            ph ^= 1;
                        }
                    }
                }
            }
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        } else
        for (int i = blockIdx.x; i < num_items && ok; i += gridDim.x) {
            const Item item = get_item<KSPLIT>(p, i);
            const int n = item.n_tile * BMW + r;
            const bool valid = n < p.N;
            const size_t grow = static_cast<size_t>(item.expert) * p.N + (valid ? n : 0);
            const uint32_t *wrow = p.w + grow * p.wpr + h * BITS;
            const unsigned short *sc16 = static_cast<const unsigned short *>(p.scales) + grow * p.gpr;
            const unsigned short *bi16 = static_cast<const unsigned short *>(p.biases) + grow * p.gpr;
            uint32_t wnext[BITS];
            uint32_t sn = 0, bn = 0;                       // raw 16-bit scale / bias, converted when used
            auto request = [&](int kb) {
                load_half_words<BITS>(wrow + static_cast<size_t>(kb) * (2 * BITS), wnext, valid);
                if (valid) {
                    const int g = (kb * BK + h * 32) >> p.gs_shift;
                    sn = __ldg(sc16 + g);
                    bn = __ldg(bi16 + g);
                }
            };
            const int kb0 = KSPLIT ? item.kb0 : 0;
            request(kb0);
            for (int kb = 0; kb < num_kb; ++kb) {
                uint32_t wcur[BITS];
#pragma unroll
                for (int j = 0; j < BITS; ++j) wcur[j] = wnext[j];
                const uint32_t sr = sn, br = bn;
                if (kb + 1 < num_kb) request(kb0 + kb + 1);      // the next k block is requested before this one is converted
                // the stage is free once empty[s] has completed (the producer waits on the same barrier)
                if (!(ok = mbar_wait_warp(&ctl->empty[s], ph ^ 1, ctl, p.status, 0x401, 0))) break;
                float sc, bi;
                if (p.sb_dt == MTC_F16) {
                    sc = __half2float(__ushort_as_half(static_cast<unsigned short>(sr)));
                    bi = __half2float(__ushort_as_half(static_cast<unsigned short>(br)));
                } else {
                    sc = __uint_as_float(sr << 16);
                    bi = __uint_as_float(br << 16);
                }
                dequant_half<BITS>(wcur, sc, bi, dst, s * w_stage);
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy stores -> async proxy (MMA)
                __syncwarp();
                if (lane == 0) mbar_arrive(&ctl->full[s]);
                if (++s == nst) {
                    s = 0;
                    ph ^= 1;
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 2) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512));
    }
}

// bf16 activations -> f16 with one power-of-two factor per row.  bf16 keeps 8 significant bits, so
// x * 2^-e is exact in f16 (11 bits) once the row maximum is brought to [2^14, 2^15); elements more than
// 2^38 below the row maximum lose bits, which changes nothing measurable.  The MMA then runs on f16
// operands, whose 3 extra mantissa bits keep the dequantised weights 8x closer to the f32 oracle than
// bf16 weights would be; the epilogue multiplies the accumulator by 2^e again.
__global__ void __launch_bounds__(256) rows_to_f16_kernel(const __nv_bfloat16 *x, __half *y, float *row_scale, int rows, int K) {
    asm volatile("griddepcontrol.launch_dependents;");      // the product kernel may start on the weights meanwhile
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    const uint4 *src = reinterpret_cast<const uint4 *>(x + static_cast<size_t>(row) * K);
    uint4 *dst = reinterpret_cast<uint4 *>(y + static_cast<size_t>(row) * K);
    const int nvec = K / 8;
    uint32_t amax = 0;                       // max of |x| as bf16 bit patterns (monotone for finite values)
    for (int i = lane; i < nvec; i += 32) {
        const uint4 v = __ldg(src + i);
        const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            amax = max(amax, u[j] & 0x7FFFu);
            amax = max(amax, (u[j] >> 16) & 0x7FFFu);
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = max(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const int ex = static_cast<int>(amax >> 7);                    // biased exponent of the row maximum
    int e = (ex == 0 || ex == 0xFF) ? 0 : ex - 127 - 14;           // zero rows and inf/nan rows stay unscaled
    e = max(e, -126);                                              // 2^-e and 2^e must both be normal f32 numbers
    const float down = __uint_as_float(static_cast<uint32_t>(127 - e) << 23);
    if (lane == 0) row_scale[row] = __uint_as_float(static_cast<uint32_t>(127 + e) << 23);
    for (int i = lane; i < nvec; i += 32) {
        const uint4 v = __ldg(src + i);
        const uint32_t u[4] = {v.x, v.y, v.z, v.w};
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const __half2 h = __floats2half2_rn(__uint_as_float(u[j] << 16) * down, __uint_as_float(u[j] & 0xFFFF0000u) * down);
            o[j] = *reinterpret_cast<const uint32_t *>(&h);
        }
        dst[i] = make_uint4(o[0], o[1], o[2], o[3]);
    }
}

// Work list of the gather case, built on the device from the CSR expert_offsets (or, when only the
// per-row expert ids are given, from those: rows are sorted by expert, so offsets[e] is the first
// row whose id is >= e).  Layout of the scratch block: int count; int pad[3]; int4 items[].
// Expert-major order: the token chunks and weight-row tiles of one expert are adjacent, so the
// CTAs working at the same time share that expert's X rows in L2.
// Offsets that reach past total_rows are clamped to it (the rows they would have named do not exist: nothing is read or
// written for them) and reported in the status word, 0x901, like offsets that run backwards (those experts get no rows).
__global__ void build_items_kernel(const uint32_t *expert_offsets, const uint32_t *indices, int total_rows, int n_experts,
                                   int n_tiles, int TN, int *count_out, int4 *items, int max_items, uint32_t *status) {
    extern __shared__ int sh[];          // [n_experts + 1] offsets, then [n_experts + 1] item bases
    int *off = sh, *base = sh + n_experts + 1;
    for (int e = threadIdx.x; e <= n_experts; e += blockDim.x) {
        if (expert_offsets) {
            const uint32_t o = expert_offsets[e];
            if (o > static_cast<uint32_t>(total_rows) || (e > 0 && o < expert_offsets[e - 1])) atomicCAS(status, 0u, 0x901u);
            off[e] = static_cast<int>(min(o, static_cast<uint32_t>(total_rows)));
        } else {                          // lower bound of e in the sorted per-row ids
            int lo = 0, hi = total_rows;
            while (lo < hi) {
                const int mid = (lo + hi) >> 1;
                if (indices[mid] < static_cast<uint32_t>(e)) lo = mid + 1; else hi = mid;
            }
            off[e] = lo;
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int acc = 0;
        for (int e = 0; e < n_experts; ++e) {
            base[e] = acc;
            const int rows = max(off[e + 1] - off[e], 0);
            acc += ((rows + TN - 1) / TN) * n_tiles;
        }
        base[n_experts] = acc;
        *count_out = acc < max_items ? acc : max_items;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < n_experts; e += blockDim.x) {
        const int rows = max(off[e + 1] - off[e], 0);
        const int chunks = (rows + TN - 1) / TN;
        int idx = base[e];
        for (int c = 0; c < chunks; ++c)
            for (int nt = 0; nt < n_tiles; ++nt, ++idx)
                if (idx < max_items) items[idx] = make_int4(nt, e, off[e] + c * TN, min(TN, rows - c * TN));
    }
}

// ---- host side ----------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void *ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
    return fn;
}

template <int BITS>
constexpr size_t qmm_smem_bytes() {
    return RING_BYTES + sizeof(SmemCtrl) + 1024;
}

template <int BITS>
cudaError_t launch_bits(cudaStream_t st, const CUtensorMap &tmap, const QmmParams &p, int grid) {
    constexpr size_t smem = qmm_smem_bytes<BITS>();
    static_assert(smem <= 227 * 1024, "shared memory per CTA");
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(NUM_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute la[1];
    la[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    la[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = la;
    cfg.numAttrs = 1;
    if (p.ksplit > 1) {
        auto kern = qmm_tcgen05_kernel<BITS, true>;
        static PerDeviceAttr attr;
        cudaError_t e = attr.set(kern, smem);
        if (e != cudaSuccess) return e;
        return cudaLaunchKernelEx(&cfg, kern, tmap, p);
    }
    auto kern = qmm_tcgen05_kernel<BITS, false>;
    static PerDeviceAttr attr;
    cudaError_t e = attr.set(kern, smem);
    if (e != cudaSuccess) return e;
    return cudaLaunchKernelEx(&cfg, kern, tmap, p);
}

cudaError_t launch_any(int bits, cudaStream_t st, const CUtensorMap &tmap, const QmmParams &p, int grid) {
    switch (bits) {
        case 2: return launch_bits<2>(st, tmap, p, grid);
        case 3: return launch_bits<3>(st, tmap, p, grid);
        case 4: return launch_bits<4>(st, tmap, p, grid);
        case 5: return launch_bits<5>(st, tmap, p, grid);
        case 6: return launch_bits<6>(st, tmap, p, grid);
        default: return launch_bits<8>(st, tmap, p, grid);
    }
}

// X as a 2-D tensor [rows, K] of 16-bit elements, box 64 x TN, 128-byte swizzle; rows past the end read as zero.
cudaError_t make_x_map(CUtensorMap *tmap, const void *x, int rows, int K, int TN, int op_f16, std::string *why) {
    EncodeTiledFn encode = get_encode_fn();
    if (!encode) {
        if (why) *why = "cuTensorMapEncodeTiled is not available from the driver";
        return cudaErrorNotSupported;
    }
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(K), static_cast<cuuint64_t>(rows)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(K) * 2};
    const cuuint32_t box[2] = {BK, static_cast<cuuint32_t>(TN)};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = encode(tmap, op_f16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                        const_cast<void *>(x), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        if (why) *why = "cuTensorMapEncodeTiled failed with code " + std::to_string(static_cast<int>(r));
        return cudaErrorInvalidValue;
    }
    return cudaSuccess;
}

// Ring depth and raw staging buffers for p.TN / p.wide.  The raw path needs whole super-blocks (K % 256 == 0), 4 to 16
// bytes of scales per row and super-block (group 32, 64 or 128) and 16-byte aligned scale / bias arrays; it takes
// two buffers per weight tile out of the ring, which costs nothing: measured, a ring deeper than 2 stages does not
// change the time of any shape.
void plan_smem(QmmParams &p, Ctx *ctx, int bits) {
    const int stage = A_BYTES + (p.wide ? 2 : 1) * p.TN * BK * 2;
    const auto al16 = [](const void *ptr) { return reinterpret_cast<uintptr_t>(ptr) % 16 == 0; };
    p.raw_tile = static_cast<uint32_t>(BMW * (32 * bits + 16) + RAW_SB_BYTES);
    const int raw_total = 2 * static_cast<int>(p.raw_tile);
    p.raw = ctx->qmm_raw != 0 && p.K % (SB_PER_RAW * BK) == 0 && p.gs_shift >= 5 && p.gs_shift <= 7 && al16(p.scales) &&
            al16(p.biases) && (RING_BYTES - raw_total) / stage >= 2;
    p.nst = (RING_BYTES - (p.raw ? raw_total : 0)) / stage;
    if (p.nst > MAX_STAGES) p.nst = MAX_STAGES;
    if (ctx->qmm_max_stages > 0 && p.nst > ctx->qmm_max_stages) p.nst = ctx->qmm_max_stages;
    p.raw_off = static_cast<uint32_t>(p.nst * stage);
}

void fill_common(QmmParams &p, Ctx *ctx, const void *w, const void *scales, const void *biases, void *out, int N, int K,
                 int bits, int group_size, int dt, int TN) {
    p.w = static_cast<const uint32_t *>(w);
    p.scales = scales;
    p.biases = biases;
    p.out = out;
    p.outs[0] = out;
    p.n_outs = 1;
    p.out_ld = N;
    p.status = ctx->d_status;
    p.N = N; p.K = K;
    p.sb_dt = dt;
    p.out_dt = dt;
    p.op_f16 = 1;   // bf16 activations are converted to scaled f16 first (see rows_to_f16_kernel)
    p.gs_shift = 0;
    while ((1 << p.gs_shift) < group_size) ++p.gs_shift;
    p.wpr = K * bits / 32;
    p.gpr = K / group_size;
    p.TN = TN;
    p.wide = 0;
    p.ksplit = 1;
    p.kb_per = K / BK;
    p.partial = nullptr;
    p.pdl_roles = 0;               // the dense launcher turns it on: a gather launch reads a work list the previous kernel built
    plan_smem(p, ctx, bits);
    p.hint_ns = static_cast<uint32_t>(ctx->qmm_wait_hint_ns);
    const uint32_t fmt = p.op_f16 ? 0u : 1u;           // both operands carry the same 16-bit format
    p.idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | (static_cast<uint32_t>(TN >> 3) << 17) |
              (static_cast<uint32_t>(BMW >> 4) << 24);
}

// bf16 activations: stage a scaled f16 copy of x in the context's conversion buffer.
cudaError_t stage_x(Ctx *ctx, cudaStream_t st, const void *x, int rows, int K, int dt, const void **x_op,
                    const float **tok_scale, std::string *why) {
    *x_op = x;
    *tok_scale = nullptr;
    if (dt == MTC_F16) return cudaSuccess;
    const size_t need = ((static_cast<size_t>(rows) * K * 2 + 255) & ~static_cast<size_t>(255)) + static_cast<size_t>(rows) * sizeof(float);
    cudaError_t ge = grow_block(ctx, st, &ctx->d_xconv, &ctx->xconv_bytes, need, why);
    if (ge != cudaSuccess) return ge;
    __half *y = static_cast<__half *>(ctx->d_xconv);
    float *scale = reinterpret_cast<float *>(static_cast<char *>(ctx->d_xconv) + ((static_cast<size_t>(rows) * K * 2 + 255) & ~static_cast<size_t>(255)));
    rows_to_f16_kernel<<<(rows + 7) / 8, 256, 0, st>>>(static_cast<const __nv_bfloat16 *>(x), y, scale, rows, K);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    *x_op = y;
    *tok_scale = scale;
    return cudaSuccess;
}

// out[i] = sum over the K slices of partial[s][i], in slice order
__global__ void __launch_bounds__(256) ksplit_sum_kernel(const float *partial, void *out, size_t mn, int S, int dt) {
    asm volatile("griddepcontrol.wait;" ::: "memory");       // launched while the product kernel runs
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < mn; i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        float pv[16];
#pragma unroll
        for (int q = 0; q < 16; ++q) pv[q] = q < S ? partial[static_cast<size_t>(q) * mn + i] : 0.0f;
        float v = pv[0];
#pragma unroll
        for (int q = 1; q < 16; ++q) v += pv[q];
        st_from_f32(out, i, v, dt);
    }
}

}  // namespace

bool qmm_tcgen05_supported(int M, int N, int K, int bits, int group_size, int dt, const void *w, const void *x,
                           const void *out) {
    const bool bits_ok = bits == 2 || bits == 3 || bits == 4 || bits == 5 || bits == 6 || bits == 8;
    const bool gs_ok = group_size >= 32 && (group_size & (group_size - 1)) == 0 && K % group_size == 0;
    const auto al = [](const void *ptr, size_t a) { return reinterpret_cast<uintptr_t>(ptr) % a == 0; };
    return bits_ok && gs_ok && (dt == MTC_F16 || dt == MTC_BF16) && M > 0 && N > 0 && K % BK == 0 && al(w, 16) &&
           al(x, 16) && al(out, 2);
}

cudaError_t launch_qmm_tcgen05(Ctx *ctx, cudaStream_t st, const void *w, const void *scales, const void *biases,
                               const void *x, void *out, int M, int N, int K, int bits, int group_size, int dt,
                               std::string *why, void *const *outs, int n_outs, long long out_ld) {
    int TN = ctx->qmm_force_tn > 0 ? ctx->qmm_force_tn : (M >= TN_MAX ? TN_MAX : ((M + 15) / 16) * 16);
    const void *x_op = nullptr;
    const float *tok_scale = nullptr;
    cudaError_t e = stage_x(ctx, st, x, M, K, dt, &x_op, &tok_scale, why);
    if (e != cudaSuccess) return e;
    CUtensorMap tmap;
    e = make_x_map(&tmap, x_op, M, K, TN, 1, why);
    if (e != cudaSuccess) return e;
    QmmParams p{};
    fill_common(p, ctx, w, scales, biases, out, N, K, bits, group_size, dt, TN);
    p.tok_scale = tok_scale;
    if (outs) {                         // the result is a column block of wider row-major matrices, possibly on other GPUs
        for (int i = 0; i < n_outs && i < 8; ++i) p.outs[i] = outs[i];
        p.out = outs[0];
        p.n_outs = n_outs;
        p.out_ld = out_ld;
    }
    p.M = M;
    p.m_chunks = (M + TN - 1) / TN;
    p.n_tiles = (N + BMW - 1) / BMW;
    p.pdl_roles = ctx->pdl_early_weights ? 1 : 0;
    const int sms = ctx->sm_count;
    {
        // Two token chunks per item: the dequantised W stage, which sets the pace of a k block, is built once per
        // 2 TN token rows instead of once per TN.
        // Worth it when it saves rounds of the grid: a k block of a wide item costs ~1.55 x one of a single-chunk item
        // (measured), so 7 rounds of single chunks against 3 wide rounds + a short one is a win, one round against one
        // wide round on half the SMs is not.
        bool wide_pays = false;
        if (ctx->qmm_wide && TN == TN_MAX && M > TN_MAX) {
            const int single = p.n_tiles * p.m_chunks, units = p.n_tiles * ((M + 2 * TN - 1) / (2 * TN));
            const double cost_single = static_cast<double>((single + sms - 1) / sms);
            const int left = units % sms;
            const bool two_halves = M % (2 * TN) == 0 || M % (2 * TN) > TN;
            const bool split_tail = units > sms && left > 0 && 2 * left <= sms && two_halves;
            const double cost_wide = 1.55 * (units / sms) + (left == 0 ? 0.0 : (split_tail ? 1.0 : 1.55));
            wide_pays = cost_wide < cost_single || ctx->qmm_wide == 2;      // 2: whenever the shape allows (tests)
        }
        if (wide_pays) {
            p.wide = 1;
            plan_smem(p, ctx, bits);
            if (p.nst < 2) {
                p.wide = 0;
                plan_smem(p, ctx, bits);
            } else {
                p.m_chunks = (M + 2 * TN - 1) / (2 * TN);
            }
        }
        p.dense_items = p.n_tiles * p.m_chunks;
        if (p.wide) {
            // a k block costs the same whatever the token count, so the leftover of the last round is cheaper as
            // single-chunk items on twice as many SMs - when those still fit in one round and every unit has two halves
            const int units = p.n_tiles * p.m_chunks, left = units % sms;
            const bool two_halves = M % (2 * TN) == 0 || M % (2 * TN) > TN;
            p.wide_items = units;
            if (units > sms && left > 0 && 2 * left <= sms && two_halves) {
                p.wide_items = units - left;
                p.dense_items = p.wide_items + 2 * left;
            }
        }
    }
    // Few weight-row tiles and one token chunk: the tiles alone would leave most SMs idle, so K is cut into slices that
    // run as items of their own (f32 partial sums, added in slice order by a second small kernel).
    if (ctx->qmm_ksplit && !p.wide && p.m_chunks == 1 && !outs && 2 * p.n_tiles <= sms) {
        const int nkb = K / BK, unit = p.raw ? SB_PER_RAW : 1;
        int S = sms / p.n_tiles;
        if (S > 16) S = 16;
        while (S > 1 && (nkb % (S * unit) != 0 || nkb / S < 4)) --S;
        if (S > 1) {
            cudaError_t ge = grow_block(ctx, st, &ctx->d_ksplit, &ctx->ksplit_bytes, static_cast<size_t>(S) * M * N * sizeof(float), why);
            if (ge != cudaSuccess) return ge;
            p.ksplit = S;
            p.kb_per = nkb / S;
            p.partial = static_cast<float *>(ctx->d_ksplit);
            p.dense_items *= S;
        }
    }
    const int grid = p.dense_items < sms ? p.dense_items : sms;
    e = launch_any(bits, st, tmap, p, grid);
    if (e != cudaSuccess || p.ksplit == 1) return e;
    const size_t mn = static_cast<size_t>(M) * N;
    size_t sgrid = (mn + 255) / 256;
    if (sgrid > static_cast<size_t>(sms) * 8) sgrid = static_cast<size_t>(sms) * 8;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(static_cast<unsigned>(sgrid));
    cfg.blockDim = dim3(256);
    cfg.stream = st;
    cudaLaunchAttribute la[1];
    la[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    la[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = la;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, ksplit_sum_kernel, static_cast<const float *>(p.partial), out, mn, p.ksplit, dt);
}

// scratch bytes the gather work list needs for these sizes
size_t gather_items_bytes(int total_rows, int n_experts, int N, int TN) {
    const size_t n_tiles = (N + BMW - 1) / BMW;
    const size_t max_items = n_tiles * (static_cast<size_t>(total_rows) / TN + n_experts + 1);
    return 16 + max_items * sizeof(int4);
}

cudaError_t launch_gather_qmm_tcgen05(Ctx *ctx, cudaStream_t st, const void *x, const void *w, const void *scales,
                                      const void *biases, const uint32_t *expert_offsets, const uint32_t *indices,
                                      void *out, int total_rows, int N, int K, int n_experts, int bits, int group_size,
                                      int dt, void *scratch, size_t scratch_bytes, std::string *why) {
    // token rows per item: about twice the mean rows per expert, so most experts are one chunk
    int TN = ctx->qmm_force_tn;
    if (TN <= 0) {
        const int mean = (total_rows + n_experts - 1) / n_experts;
        TN = ((2 * mean + 15) / 16) * 16;
        if (TN < 32) TN = 32;
        if (TN > TN_MAX) TN = TN_MAX;
    }
    const size_t need = gather_items_bytes(total_rows, n_experts, N, TN);
    if (!scratch || scratch_bytes < need) {
        if (why) *why = "gather_qmm: work-list scratch too small";
        return cudaErrorInvalidValue;
    }
    const int n_tiles = (N + BMW - 1) / BMW;
    const int max_items = static_cast<int>((scratch_bytes - 16) / sizeof(int4));
    int *count = static_cast<int *>(scratch);
    int4 *items = reinterpret_cast<int4 *>(static_cast<char *>(scratch) + 16);
    build_items_kernel<<<1, 256, 2 * (n_experts + 1) * sizeof(int), st>>>(expert_offsets, indices, total_rows, n_experts,
                                                                         n_tiles, TN, count, items, max_items, ctx->d_status);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    const void *x_op = nullptr;
    const float *tok_scale = nullptr;
    e = stage_x(ctx, st, x, total_rows, K, dt, &x_op, &tok_scale, why);
    if (e != cudaSuccess) return e;
    CUtensorMap tmap;
    e = make_x_map(&tmap, x_op, total_rows, K, TN, 1, why);
    if (e != cudaSuccess) return e;
    QmmParams p{};
    fill_common(p, ctx, w, scales, biases, out, N, K, bits, group_size, dt, TN);
    p.tok_scale = tok_scale;
    p.M = total_rows;
    p.items = items;
    p.item_count = count;
    return launch_any(bits, st, tmap, p, ctx->sm_count);
}

// ---- gather_qmm for callers that cannot allocate ---------------------------------------------------
// Some hosts of this library may not call cudaMalloc at the point where they run a MoE layer:
// allocator-managed processes where every device byte is accounted for at start-up, and latency-critical
// loops that must not take the allocator's lock or meet an out-of-memory error in the middle of a step.  mtc_gather_qmm_static does the same
// work as mtc_gather_qmm on the tensor-core path but takes its scratch (the work list and the scaled-f16
// copy of bf16 activations) from one fixed array that lives in the library image: every GPU that loads
// the library holds these bytes until the process exits.  Limits below; sizes beyond them are refused.
constexpr size_t kStaticItems = 16384;                        // work items (16 bytes each)
constexpr size_t kStaticXElems = 8u << 20;                    // bf16 activations staged as f16: m_total * k_in elements
constexpr size_t kStaticRows = 65536;                         // rows of x (one f32 factor each)
constexpr size_t kStaticListBytes = 16 + kStaticItems * sizeof(int4);
constexpr size_t kStaticXOff = (kStaticListBytes + 255) & ~static_cast<size_t>(255);
constexpr size_t kStaticScaleOff = kStaticXOff + kStaticXElems * 2;
constexpr size_t kStaticBytes = kStaticScaleOff + kStaticRows * sizeof(float);

static __device__ __align__(256) unsigned char g_gather_static[kStaticBytes];

// The array's name is a host-side handle, not a device address: the address each device gave it is
// looked up once per device (with that device current) and cached.
cudaError_t gather_static_base(unsigned char **base) {
    static unsigned char *cache[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    if (!cache[dev]) {
        void *ptr = nullptr;
        e = cudaGetSymbolAddress(&ptr, g_gather_static);
        if (e != cudaSuccess) return e;
        cache[dev] = static_cast<unsigned char *>(ptr);
    }
    *base = cache[dev];
    return cudaSuccess;
}

cudaError_t launch_gather_qmm_static(Ctx *ctx, cudaStream_t st, const void *x, const void *w, const void *scales,
                                     const void *biases, const uint32_t *expert_offsets, const uint32_t *indices,
                                     void *out, int total_rows, int N, int K, int n_experts, int bits, int group_size,
                                     int dt, std::string *why) {
    int TN = ctx->qmm_force_tn;
    if (TN <= 0) {
        const int mean = (total_rows + n_experts - 1) / n_experts;
        TN = ((2 * mean + 15) / 16) * 16;
        if (TN < 32) TN = 32;
        if (TN > TN_MAX) TN = TN_MAX;
    }
    if (gather_items_bytes(total_rows, n_experts, N, TN) > kStaticListBytes) {
        if (why) *why = "gather_qmm_static: more than " + std::to_string(kStaticItems) + " work items (n_out/128 * (m_total/chunk + n_experts))";
        return cudaErrorInvalidValue;
    }
    if (dt == MTC_BF16 && (static_cast<size_t>(total_rows) * K > kStaticXElems || static_cast<size_t>(total_rows) > kStaticRows)) {
        if (why) *why = "gather_qmm_static: bf16 activations are limited to m_total * k_in <= " + std::to_string(kStaticXElems) +
                        " elements and m_total <= " + std::to_string(kStaticRows);
        return cudaErrorInvalidValue;
    }
    unsigned char *base = nullptr;
    cudaError_t e = gather_static_base(&base);
    if (e != cudaSuccess) return e;
    const int n_tiles = (N + BMW - 1) / BMW;
    int *count = reinterpret_cast<int *>(base);
    int4 *items = reinterpret_cast<int4 *>(base + 16);
    // the list and its count are rewritten by every call; nothing in the array has to start at zero
    build_items_kernel<<<1, 256, 2 * (n_experts + 1) * sizeof(int), st>>>(expert_offsets, indices, total_rows, n_experts,
                                                                         n_tiles, TN, count, items, static_cast<int>(kStaticItems), ctx->d_status);
    if ((e = cudaGetLastError()) != cudaSuccess) return e;
    const void *x_op = x;
    const float *tok_scale = nullptr;
    if (dt == MTC_BF16) {
        __half *y = reinterpret_cast<__half *>(base + kStaticXOff);
        float *scale = reinterpret_cast<float *>(base + kStaticScaleOff);
        rows_to_f16_kernel<<<(total_rows + 7) / 8, 256, 0, st>>>(static_cast<const __nv_bfloat16 *>(x), y, scale, total_rows, K);
        if ((e = cudaGetLastError()) != cudaSuccess) return e;
        x_op = y;
        tok_scale = scale;
    }
    CUtensorMap tmap;
    e = make_x_map(&tmap, x_op, total_rows, K, TN, 1, why);
    if (e != cudaSuccess) return e;
    QmmParams p{};
    fill_common(p, ctx, w, scales, biases, out, N, K, bits, group_size, dt, TN);
    p.tok_scale = tok_scale;
    p.M = total_rows;
    p.items = items;
    p.item_count = count;
    return launch_any(bits, st, tmap, p, ctx->sm_count);
}

}  // namespace mtc
