/*
 * mt_oracle.c — CPU restatement of metaltile's scalar reference for the affine
 * group-quantized matmul family.  TEST INFRASTRUCTURE ONLY: it is the checker
 * the CUDA path is compared against and the timed CPU baseline; nothing in the
 * product library links, loads or calls it.
 *
 * Every function cites the reference source it follows (paths are relative to
 * the metaltile repository root).  The reference is Rust and computes in f32
 * with no fused multiply-add; build this file with -ffp-contract=off so that
 * `(q*s + b) * x` rounds after every operation exactly as the Rust code does.
 *
 * Parity pinning: the reference stores no numeric golden outputs (its tests
 * recompute the oracle from closed-form inputs).  This restatement is pinned
 * against (1) the literal expectations the reference's tests do hold (top-k tie
 * break, k = 1 weight, NaN/Inf invariants, worked bit layouts) and (2) an
 * independent pure-numpy restatement whose outputs on the reference's
 * registered test shapes are committed under tests/golden/.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

/* ---- dtype rounding ------------------------------------------------------ */

/* bf16 round-to-nearest-even, same bit recipe as
 * crates/metaltile-std/src/runner.rs:521-525 (`f32_to_bf16`), which agrees with
 * crate `half`'s bf16::from_f32 for every finite input; NaN is kept quiet. */
static inline uint16_t f32_to_bf16_bits(float v) {
    uint32_t x;
    memcpy(&x, &v, 4);
    if ((x & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((x >> 16) | 0x0040u);
    uint32_t r = x + 0x7FFFu + ((x >> 16) & 1u);
    return (uint16_t)(r >> 16);
}
static inline float bf16_bits_to_f32(uint16_t h) {
    uint32_t x = (uint32_t)h << 16;
    float f;
    memcpy(&f, &x, 4);
    return f;
}

/* IEEE binary16 round-to-nearest-even with subnormals, the behaviour of
 * `half::f16::from_f32` used by crates/metaltile-std/src/utils.rs:26-30.
 * (runner.rs:498-519 flushes subnormals to zero; the test path uses `half`.) */
static inline uint16_t f32_to_f16_bits(float v) {
    uint32_t x;
    memcpy(&x, &v, 4);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t ax = x & 0x7FFFFFFFu;
    if (ax > 0x7F800000u) return (uint16_t)(sign | 0x7E00u);       /* NaN */
    if (ax >= 0x47800000u) return (uint16_t)(sign | 0x7C00u);      /* >= 65536 -> inf */
    if (ax < 0x33000000u) return (uint16_t)sign;                   /* < 2^-25 -> 0 */
    int32_t e = (int32_t)(ax >> 23) - 127;
    uint32_t m = (ax & 0x7FFFFFu) | 0x800000u;
    uint32_t shift, half_bits;
    if (e < -14) {                      /* subnormal result */
        shift = (uint32_t)(13 + (-14 - e));
        half_bits = 0;
    } else {
        shift = 13;
        half_bits = ((uint32_t)(e + 15) << 10) - 0x400u; /* implicit bit adds back */
    }
    uint32_t q = m >> shift;
    uint32_t rem = m & ((1u << shift) - 1u);
    uint32_t halfway = 1u << (shift - 1);
    if (rem > halfway || (rem == halfway && (q & 1u))) q++;
    uint32_t h = half_bits + q;         /* carries propagate into the exponent */
    if (h >= 0x7C00u) h = 0x7C00u;
    return (uint16_t)(sign | h);
}
static inline float f16_bits_to_f32(uint16_t h) {
    uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
    uint32_t e = (h >> 10) & 0x1Fu;
    uint32_t m = h & 0x3FFu;
    uint32_t x;
    if (e == 0) {
        if (m == 0) {
            x = sign;
        } else {
            int s = 0;
            while (!(m & 0x400u)) { m <<= 1; s++; }
            m &= 0x3FFu;
            x = sign | ((uint32_t)(113 - s) << 23) | (m << 13);
        }
    } else if (e == 31) {
        x = sign | 0x7F800000u | (m << 13);
    } else {
        x = sign | ((e + 112u) << 23) | (m << 13);
    }
    float f;
    memcpy(&f, &x, 4);
    return f;
}

/* dtype ids shared with include/mtcuda.h: 0 = f32, 1 = f16, 2 = bf16. */
static inline float round_dt(float v, int dt) {
    if (dt == 1) return f16_bits_to_f32(f32_to_f16_bits(v));
    if (dt == 2) return bf16_bits_to_f32(f32_to_bf16_bits(v));
    return v;
}

/* pack_f32 followed by unpack_f32 (crates/metaltile-std/src/utils.rs:26-66):
 * the conditioning the reference applies to scales, biases, x and to the
 * expected output (crates/metaltile-std/src/mlx/quantized.rs:5428-5431,5441). */
void mto_round_through(const float *in, float *out, size_t n, int dt) {
    for (size_t i = 0; i < n; i++) out[i] = round_dt(in[i], dt);
}
void mto_f32_to_bits16(const float *in, uint16_t *out, size_t n, int dt) {
    for (size_t i = 0; i < n; i++)
        out[i] = dt == 1 ? f32_to_f16_bits(in[i]) : f32_to_bf16_bits(in[i]);
}
void mto_bits16_to_f32(const uint16_t *in, float *out, size_t n, int dt) {
    for (size_t i = 0; i < n; i++)
        out[i] = dt == 1 ? f16_bits_to_f32(in[i]) : bf16_bits_to_f32(in[i]);
}

/* ---- packed codes -------------------------------------------------------- */

/* Code (row, k) of a row that is a contiguous LSB-first bit-stream of
 * `words_per_row` u32 words: the `bits` bits starting at bit k*bits, possibly
 * straddling two words.  Follows the two-word extract of
 * crates/metaltile-std/src/mlx/quantized.rs:4366-4379 and `dequant_matrix` in
 * crates/metaltile-std/tests/quantized_family_gpu_correctness.rs:115-149.  For
 * bits in {2,4,8} no code straddles and this equals the pack-aligned form
 * `(word >> ((k % pf) * bits)) & mask` of quantized.rs:5395-5396. */
static inline uint32_t code_at(const uint32_t *row, size_t k, uint32_t bits) {
    size_t bit_off = k * bits;
    size_t word = bit_off >> 5;
    uint32_t sh = (uint32_t)(bit_off & 31u);
    uint64_t lo = (uint64_t)row[word] >> sh;
    uint64_t hi = (32u - sh < bits) ? ((uint64_t)row[word + 1] << (32u - sh)) : 0;
    return (uint32_t)((lo | hi) & ((1ull << bits) - 1ull));
}

/* Row packer: crates/metaltile-std/tests/quantized_family_gpu_correctness.rs:52-69
 * (`pack_codes`).  `words` must be zeroed, length ceil(n*bits/32). */
void mto_pack_row(const uint32_t *codes, size_t n, uint32_t bits, uint32_t *words) {
    uint32_t mask = (uint32_t)((1ull << bits) - 1ull);
    for (size_t i = 0; i < n; i++) {
        size_t bit_off = i * bits;
        size_t word = bit_off >> 5;
        uint32_t sh = (uint32_t)(bit_off & 31u);
        uint32_t c = codes[i] & mask;
        words[word] |= c << sh;
        if (32u - sh < bits) words[word + 1] |= c >> (32u - sh);
    }
}

/* Pack / unpack an [n_rows, k] matrix; each row starts on a word boundary
 * (quantized.rs:4354-4355: u32_per_row = k*bits/32). */
void mto_pack_matrix(const uint32_t *codes, size_t n_rows, size_t k, uint32_t bits,
                     uint32_t *words) {
    size_t wpr = (k * bits + 31) / 32;
    memset(words, 0, n_rows * wpr * sizeof(uint32_t));
    for (size_t r = 0; r < n_rows; r++) mto_pack_row(codes + r * k, k, bits, words + r * wpr);
}
void mto_unpack_matrix(const uint32_t *words, size_t n_rows, size_t k, uint32_t bits,
                       uint8_t *codes) {
    size_t wpr = (k * bits + 31) / 32;
#pragma omp parallel for schedule(static)
    for (size_t r = 0; r < n_rows; r++)
        for (size_t j = 0; j < k; j++)
            codes[r * k + j] = (uint8_t)code_at(words + r * wpr, j, bits);
}

/* ---- qmv / qmm ----------------------------------------------------------- */

/* qmm_oracle, crates/metaltile-std/src/mlx/quantized.rs:5374-5404: one f32
 * accumulator per output, k ascending, `acc += (q*scale + bias) * x`.
 * scales/biases/x are f32 values that the caller has already rounded through
 * the activation dtype; out is the raw f32 accumulator (round it with
 * mto_round_through to obtain the expected buffer of quantized.rs:5441).
 * Rows n0 <= n < n1 only, so a bounded slice can be timed or checked.
 * `threads` <= 0 keeps the OpenMP default. */
void mto_qmm_rows(const uint32_t *w, const float *scales, const float *biases, const float *x,
                  float *out, size_t m, size_t n, size_t k, uint32_t bits, size_t group_size,
                  size_t n0, size_t n1, int threads) {
    size_t wpr = k * bits / 32;
    size_t gpr = k / group_size;
#ifdef _OPENMP
    if (threads > 0) omp_set_num_threads(threads);
#endif
#pragma omp parallel for schedule(static)
    for (size_t nc = n0; nc < n1; nc++) {
        const uint32_t *row = w + nc * wpr;
        for (size_t mr = 0; mr < m; mr++) {
            float acc = 0.0f;
            for (size_t j = 0; j < k; j++) {
                size_t g = j / group_size;
                float q = (float)code_at(row, j, bits);
                acc += (q * scales[nc * gpr + g] + biases[nc * gpr + g]) * x[mr * k + j];
            }
            out[mr * n + nc] = acc;
        }
    }
}

void mto_qmm(const uint32_t *w, const float *scales, const float *biases, const float *x,
             float *out, size_t m, size_t n, size_t k, uint32_t bits, size_t group_size,
             int threads) {
    mto_qmm_rows(w, scales, biases, x, out, m, n, k, bits, group_size, 0, n, threads);
}

/* Dequantised weights as the oracle sees them (`dequant_matrix`,
 * tests/quantized_family_gpu_correctness.rs:115-149). */
void mto_dequant(const uint32_t *w, const float *scales, const float *biases, float *out,
                 size_t n, size_t k, uint32_t bits, size_t group_size) {
    size_t wpr = k * bits / 32;
    size_t gpr = k / group_size;
#pragma omp parallel for schedule(static)
    for (size_t r = 0; r < n; r++)
        for (size_t j = 0; j < k; j++) {
            size_t g = j / group_size;
            out[r * k + j] =
                (float)code_at(w + r * wpr, j, bits) * scales[r * gpr + g] + biases[r * gpr + g];
        }
}

/* ---- MoE ----------------------------------------------------------------- */

/* cpu_gather_qmm_int4, crates/metaltile-std/src/ffai/moe.rs:3577-3622, widened
 * to any bit width with the same bit-stream extraction (the b{3,5,6,8} gather
 * kernels, moe.rs:461-599).  Row t uses the first expert e with
 * t < expert_offsets[e+1]; when `indices` is non-NULL it names the expert of
 * each row directly (the MMA form, moe.rs:2256-2533).  Weights are stacked
 * [E, n_out, k_in*bits/32]; scales/biases [E, n_out, k_in/group]. */
void mto_gather_qmm(const float *x, const uint32_t *w, const float *scales, const float *biases,
                    const uint32_t *expert_offsets, const uint32_t *indices, float *out,
                    size_t t_rows, size_t k_in, size_t n_out, size_t n_experts, uint32_t bits,
                    size_t group_size, int threads) {
    size_t wpr = k_in * bits / 32;
    size_t gpr = k_in / group_size;
#ifdef _OPENMP
    if (threads > 0) omp_set_num_threads(threads);
#endif
#pragma omp parallel for schedule(dynamic, 8)
    for (size_t row = 0; row < t_rows; row++) {
        size_t expert = 0;
        if (indices) {
            expert = indices[row];
        } else {
            for (size_t e = 0; e < n_experts; e++)
                if ((uint32_t)row < expert_offsets[e + 1]) { expert = e; break; }
        }
        for (size_t mo = 0; mo < n_out; mo++) {
            const uint32_t *wrow = w + (expert * n_out + mo) * wpr;
            const float *srow = scales + (expert * n_out + mo) * gpr;
            const float *brow = biases + (expert * n_out + mo) * gpr;
            float acc = 0.0f;
            for (size_t j = 0; j < k_in; j++) {
                float q = (float)code_at(wrow, j, bits);
                float wv = q * srow[j / group_size] + brow[j / group_size];
                acc += wv * x[row * k_in + j];
            }
            out[row * n_out + mo] = acc;
        }
    }
}

/* cpu_topk_reference, crates/metaltile-std/tests/moe_gpu_correctness.rs:55-93
 * (norm_topk_prob = 1: softmax over the chosen k with max subtraction), and
 * the norm_topk_prob = 0 mode of the kernel, crates/metaltile-std/src/ffai/moe.rs:166-185
 * (weight = exp(z - max_all) / sum over ALL experts).  k passes of strict `>`
 * scanning ascending index, so ties go to the lower index and NaN never wins;
 * when nothing beats -inf the pick is index 0, as in the reference. */
void mto_router_topk(const float *logits, uint32_t *indices, float *weights, size_t n_rows,
                     size_t n_experts, size_t k, int norm_topk_prob) {
    for (size_t row = 0; row < n_rows; row++) {
        const float *z = logits + row * n_experts;
        uint32_t chosen[64];
        float vals[64];
        for (size_t it = 0; it < k; it++) {
            float best = -INFINITY;
            size_t best_idx = 0;
            for (size_t j = 0; j < n_experts; j++) {
                int taken = 0;
                for (size_t p = 0; p < it; p++) taken |= (chosen[p] == (uint32_t)j);
                if (taken) continue;
                if (z[j] > best) { best = z[j]; best_idx = j; }
            }
            chosen[it] = (uint32_t)best_idx;
            vals[it] = best;
        }
        if (norm_topk_prob) {
            float mx = -INFINITY;
            for (size_t j = 0; j < k; j++) mx = vals[j] > mx ? vals[j] : mx;
            float e[64], sum = 0.0f;
            for (size_t j = 0; j < k; j++) { e[j] = expf(vals[j] - mx); sum += e[j]; }
            for (size_t j = 0; j < k; j++) weights[row * k + j] = e[j] / sum;
        } else {
            float mx = -INFINITY;
            for (size_t j = 0; j < n_experts; j++) mx = z[j] > mx ? z[j] : mx;
            float sum = 0.0f;
            for (size_t j = 0; j < n_experts; j++) sum += expf(z[j] - mx);
            for (size_t j = 0; j < k; j++) weights[row * k + j] = expf(vals[j] - mx) / sum;
        }
        for (size_t j = 0; j < k; j++) indices[row * k + j] = chosen[j];
    }
}

/* MoE sort.  The reference leaves this step to its caller
 * (crates/metaltile-std/src/ffai/moe.rs:253-271 states only the contract), so
 * the definition is this project's: stable sort of flat slots f = token*k + slot
 * by (expert[f], f).  sort_token_idx[p] = f_p / k, inv_perm[f_p] = p,
 * expert_offsets[e] = #{f : expert[f] < e}, row_expert[p] = expert[f_p]. */
void mto_moe_sort(const uint32_t *topk_idx, size_t n_tokens, size_t k, size_t n_experts,
                  uint32_t *sort_token_idx, uint32_t *inv_perm, uint32_t *expert_offsets,
                  uint32_t *row_expert) {
    size_t total = n_tokens * k;
    for (size_t e = 0; e <= n_experts; e++) expert_offsets[e] = 0;
    for (size_t f = 0; f < total; f++) expert_offsets[topk_idx[f] + 1]++;
    for (size_t e = 0; e < n_experts; e++) expert_offsets[e + 1] += expert_offsets[e];
    uint32_t *cursor = (uint32_t *)malloc(n_experts * sizeof(uint32_t));
    for (size_t e = 0; e < n_experts; e++) cursor[e] = expert_offsets[e];
    for (size_t f = 0; f < total; f++) {
        uint32_t e = topk_idx[f];
        uint32_t p = cursor[e]++;
        sort_token_idx[p] = (uint32_t)(f / k);
        inv_perm[f] = p;
        if (row_expert) row_expert[p] = e;
    }
    free(cursor);
}

/* mt_moe_permute, crates/metaltile-std/src/ffai/moe.rs:283-302: row copy. */
void mto_moe_permute(const float *tokens, const uint32_t *sort_token_idx, float *permuted,
                     size_t n_rows, size_t hidden) {
    for (size_t p = 0; p < n_rows; p++)
        memcpy(permuted + p * hidden, tokens + (size_t)sort_token_idx[p] * hidden,
               hidden * sizeof(float));
}

/* mt_moe_unpermute, crates/metaltile-std/src/ffai/moe.rs:222-249 and the inline
 * reference of tests/moe_gpu_correctness.rs:186-198: f32 accumulate, j ascending. */
void mto_moe_unpermute(const float *expert_out, const uint32_t *inv_perm, const float *weights,
                       float *out, size_t n_tokens, size_t hidden, size_t k) {
#pragma omp parallel for schedule(static)
    for (size_t t = 0; t < n_tokens; t++)
        for (size_t h = 0; h < hidden; h++) {
            float acc = 0.0f;
            for (size_t j = 0; j < k; j++)
                acc += weights[t * k + j] * expert_out[(size_t)inv_perm[t * k + j] * hidden + h];
            out[t * hidden + h] = acc;
        }
}

/* mt_swiglu, crates/metaltile-std/src/mlx/swiglu.rs:45-57: silu(g) * u in f32,
 * silu(g) = g / (1 + exp(-g)). */
void mto_swiglu(const float *gate, const float *up, float *out, size_t n) {
    for (size_t i = 0; i < n; i++) {
        float g = gate[i];
        float s = g / (1.0f + expf(-g));
        out[i] = s * up[i];
    }
}

/* The normalised activation of ffai_rms_norm_qgemv, crates/metaltile-std/src/ffai/rms_norm_qgemv.rs:51-107, with the
 * arithmetic of the reference's own CPU check (crates/metaltile-std/tests/rms_norm_qgemv_gpu_correctness.rs:59-90):
 *   ssq = sum x[d]^2 (one f32 accumulator, d ascending);  inv_rms = 1 / sqrt(ssq / K + eps);
 *   normed[d] = (x[d] * norm_weight[d]) * inv_rms      - f32, never rounded to the activation type.
 * The fused product is then mto_qmm_rows on `normed` as a one-row x. */
void mto_rms_normed(const float *x, const float *norm_weight, float *normed, size_t k, float eps) {
    float ssq = 0.0f;
    for (size_t d = 0; d < k; d++) ssq += x[d] * x[d];
    float inv_rms = 1.0f / sqrtf(ssq / (float)k + eps);
    for (size_t d = 0; d < k; d++) normed[d] = x[d] * norm_weight[d] * inv_rms;
}

/* mt_affine_quantize_int{2,3,4,5,6,8}, crates/metaltile-std/src/mlx/quantized.rs:3629-3667,3707-3750,3793-3860,3871-4070
 * (one template, checked by :5268-5339 and tests/affine_int356_quantize_gpu_correctness.rs): per group of `group_size`
 * values  scale = (max - min) / (2^bits - 1), 1 when that is below 1e-7;  bias = min;
 *         q = trunc(clamp((v - bias) * (1 / scale) + 0.5, 0, 2^bits - 1))      - every operation rounded to f32, no FMA;
 * codes packed LSB-first as one bit-stream per group (group_size * bits is a multiple of 32); scales and biases are
 * returned in f32 (the kernels store them rounded to the activation type). */
void mto_affine_quantize(const float *w, uint32_t *out, float *scales, float *biases, size_t n_groups, size_t group_size,
                         uint32_t bits) {
    const float n_bins = (float)((1u << bits) - 1u);
    const size_t wpg = group_size * bits / 32;
    for (size_t g = 0; g < n_groups; g++) {
        const float *v = w + g * group_size;
        float mn = INFINITY, mx = -INFINITY;
        for (size_t i = 0; i < group_size; i++) {
            if (v[i] < mn) mn = v[i];
            if (v[i] > mx) mx = v[i];
        }
        float raw = (mx - mn) / n_bins;
        float scale = raw < 1.0e-7f ? 1.0f : raw;
        float inv = 1.0f / scale;
        scales[g] = scale;
        biases[g] = mn;
        uint32_t *o = out + g * wpg;
        for (size_t i = 0; i < wpg; i++) o[i] = 0u;
        for (size_t i = 0; i < group_size; i++) {
            float t = v[i] - mn;
            float qf = t * inv;
            qf = qf + 0.5f;
            if (qf > n_bins) qf = n_bins;
            if (qf < 0.0f) qf = 0.0f;
            uint32_t q = (uint32_t)qf;
            size_t bit = i * bits;
            o[bit >> 5] |= q << (bit & 31u);
            if ((bit & 31u) + bits > 32u) o[(bit >> 5) + 1] |= q >> (32u - (bit & 31u));
        }
    }
}

/* mt_affine_dequantize_int{2,3,4,5,6,8}, quantized.rs:3575-3604,3681-3705,3762-3791,4081-4214 (expected values of
 * :5216-5251): out[i] = scale[i / group_size] * q_i + bias[i / group_size] in f32, codes read from the LSB-first stream. */
void mto_affine_dequantize(const uint32_t *w, const float *scales, const float *biases, float *out, size_t n_elem,
                           size_t group_size, uint32_t bits) {
    const uint32_t mask = (1u << bits) - 1u;
    for (size_t i = 0; i < n_elem; i++) {
        size_t bit = i * bits;
        uint32_t q = w[bit >> 5] >> (bit & 31u);
        if ((bit & 31u) + bits > 32u) q |= w[(bit >> 5) + 1] << (32u - (bit & 31u));
        q &= mask;
        float prod = scales[i / group_size] * (float)q;
        out[i] = prod + biases[i / group_size];
    }
}

/* dequant_gather_int{2,3,4,5,6,8}, crates/metaltile-std/src/ffai/dequant_gather.rs:44-94 (CPU check :150-190): row
 * indices[t] of a quantized table, dequantized: out[t, d] = q * scale[row, d / G] + bias[row, d / G] in f32. */
void mto_dequant_gather(const uint32_t *weight, const float *scales, const float *biases, const uint32_t *indices, float *out,
                        size_t n_tokens, size_t hidden, size_t group_size, uint32_t bits) {
    const size_t wpr = hidden * bits / 32, gpr = hidden / group_size;
    const uint32_t mask = (1u << bits) - 1u;
    for (size_t t = 0; t < n_tokens; t++) {
        const size_t row = indices[t];
        const uint32_t *rw = weight + row * wpr;
        for (size_t d = 0; d < hidden; d++) {
            size_t bit = d * bits;
            uint32_t q = rw[bit >> 5] >> (bit & 31u);
            if ((bit & 31u) + bits > 32u) q |= rw[(bit >> 5) + 1] << (32u - (bit & 31u));
            q &= mask;
            float prod = (float)q * scales[row * gpr + d / group_size];
            out[t * hidden + d] = prod + biases[row * gpr + d / group_size];
        }
    }
}

/* mt_qvm_b{3,4,5,6,8} / mt_qvm_int4_fast, crates/metaltile-std/src/mlx/quantized.rs:4397-4530 with the CPU check
 * qvm_oracle (:5613-5635) generalised to every width: the weight matrix is [K, N], row d an LSB-first bit-stream of N codes,
 * scales / biases [K / G, N] (groups along K):
 *     out[m, c] = sum_d (q(d, c) * scale[d / G, c] + bias[d / G, c]) * x[m, d]     (one f32 accumulator, d ascending). */
void mto_qvm(const uint32_t *w, const float *scales, const float *biases, const float *x, float *out, size_t m, size_t n, size_t k,
             uint32_t bits, size_t group_size) {
    const size_t wpr = n * bits / 32;
    const uint32_t mask = (1u << bits) - 1u;
#pragma omp parallel for schedule(static)
    for (size_t c = 0; c < n; c++) {
        for (size_t mr = 0; mr < m; mr++) {
            float acc = 0.0f;
            for (size_t d = 0; d < k; d++) {
                const uint32_t *rw = w + d * wpr;
                size_t bit = c * bits;
                uint32_t q = rw[bit >> 5] >> (bit & 31u);
                if ((bit & 31u) + bits > 32u) q |= rw[(bit >> 5) + 1] << (32u - (bit & 31u));
                q &= mask;
                size_t g = d / group_size;
                float wv = (float)q * scales[g * n + c];
                wv = wv + biases[g * n + c];
                float p = wv * x[mr * k + d];
                acc = acc + p;
            }
            out[mr * n + c] = acc;
        }
    }
}

/* ffai_moe_down_swiglu_accum_int4_chain8, crates/metaltile-std/src/ffai/moe_down_swiglu_accum.rs:158-318 with the CPU check
 * `oracle` (:355-402): the M = 1 MoE decode tail for n_slots routed experts,
 *     out[row] = sum_k sum_d (sw[k] * (q(e_k, row, d) * scale + bias)) * inner_k[d],   inner_k[d] = silu(gate_k[d]) * up_k[d],
 * one f32 accumulator, slots, packs and nibbles ascending; gates / ups are [n_slots, in_dim]. */
void mto_moe_down_swiglu_accum(const float *gates, const float *ups, const uint32_t *experts, const float *slot_w, const uint32_t *w,
                               const float *scales, const float *biases, float *out, size_t n_slots, size_t in_dim, size_t out_dim,
                               size_t group_size) {
    const size_t ppr = in_dim / 8, gpr = in_dim / group_size;
    float *inner = (float *)malloc(n_slots * in_dim * sizeof(float));
    for (size_t i = 0; i < n_slots * in_dim; i++) {
        float g = gates[i];
        float silu = g / (1.0f + expf(-g));
        inner[i] = silu * ups[i];
    }
    for (size_t row = 0; row < out_dim; row++) {
        float acc = 0.0f;
        for (size_t k = 0; k < n_slots; k++) {
            const size_t e = experts[k];
            const uint32_t *rw = w + (e * out_dim + row) * ppr;
            const float *rs = scales + (e * out_dim + row) * gpr, *rb = biases + (e * out_dim + row) * gpr;
            for (size_t d = 0; d < in_dim; d++) {
                float q = (float)((rw[d >> 3] >> ((d & 7u) * 4u)) & 0xFu);
                float dq = q * rs[d / group_size];
                dq = dq + rb[d / group_size];
                float t = slot_w[k] * dq;
                t = t * inner[k * in_dim + d];
                acc = acc + t;
            }
        }
        out[row] = acc;
    }
    free(inner);
}

int mto_max_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
