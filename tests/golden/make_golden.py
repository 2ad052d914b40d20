"""Generate the golden fixtures in this directory (``python tests/golden/make_golden.py``).

The reference (metaltile, Rust + Metal) cannot be built or run in this
environment, and its tests hold no stored numeric outputs: each test builds
closed-form inputs and recomputes a scalar f32 oracle.  This script restates
those input formulas and that oracle a second time, in numpy, independently of
``oracle/mt_oracle.c`` (nothing from ``oracle/`` is imported here), and stores
inputs + expected outputs as ``.npz``.  The test-suite then requires the C
oracle to reproduce every stored output bit for bit, so two independent
restatements of the reference have to agree before either is trusted.

Arithmetic notes: all oracle sums run k-ascending with one f32 accumulator per
output and no fused multiply-add; numpy float32 array ops round after every
operation, which is the same thing element-wise.

Reference sources restated here
  synth_packed_w / qx_setup ... crates/metaltile-std/src/mlx/quantized.rs:5355-5369,5411-5446
  qmm_oracle ................. crates/metaltile-std/src/mlx/quantized.rs:5374-5404
  registered shapes .......... crates/metaltile-std/src/mlx/quantized.rs:5449-5605
  pack_codes / quantize_* .... crates/metaltile-std/tests/quantized_family_gpu_correctness.rs:52-149,200-211
  int4 gather setup + oracle . crates/metaltile-std/src/ffai/moe.rs:3577-3651
  cpu_topk_reference ......... crates/metaltile-std/tests/moe_gpu_correctness.rs:55-93
  top-k literal cases ........ crates/metaltile-std/tests/moe_gpu_correctness.rs:96-108,288-335,441-470,524-597
  unpermute reference ........ crates/metaltile-std/tests/moe_gpu_correctness.rs:164-198
  swiglu setup ............... crates/metaltile-std/src/mlx/swiglu.rs:65-72
  batched q/k/v decode ....... crates/metaltile-std/tests/batched_qkv_qgemv_gpu_correctness.rs:30-127,167-181,312-321
  batched 4-way decode ....... crates/metaltile-std/src/ffai/batched_4_qgemv.rs:342-440
  affine quantize / dequantize crates/metaltile-std/src/mlx/quantized.rs:3629-3667,5216-5330
  dequantizing gather ........ crates/metaltile-std/src/ffai/dequant_gather.rs:119-243
  fused RMSNorm + decode ..... crates/metaltile-std/tests/rms_norm_qgemv_gpu_correctness.rs:35-177,232-294
"""
from __future__ import annotations

import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
f32 = np.float32


# ---- dtype rounding (independent of the C code) --------------------------------
def round_bf16(a):
    a = np.asarray(a, dtype=np.float32)
    x = a.view(np.uint32).astype(np.uint64)
    r = (x + 0x7FFF + ((x >> 16) & 1)) & 0xFFFFFFFF
    return ((r >> 16) << 16).astype(np.uint32).view(np.float32)


def round_dt(a, dt):
    a = np.asarray(a, dtype=np.float32)
    if dt == "f32":
        return a.copy()
    if dt == "f16":
        with np.errstate(over="ignore"):
            return a.astype(np.float16).astype(np.float32)
    return round_bf16(a)


# ---- packing -------------------------------------------------------------------
def pack_rows(codes, bits):
    """LSB-first bit-stream per row, python ints so nothing can overflow."""
    rows, k = codes.shape
    wpr = (k * bits + 31) // 32
    out = np.zeros((rows, wpr), dtype=np.uint32)
    for r in range(rows):
        stream = 0
        for i in range(k):
            stream |= (int(codes[r, i]) & ((1 << bits) - 1)) << (i * bits)
        for wi in range(wpr):
            out[r, wi] = (stream >> (32 * wi)) & 0xFFFFFFFF
    return out


def unpack_rows(words, k, bits):
    rows = words.shape[0]
    out = np.zeros((rows, k), dtype=np.uint32)
    for r in range(rows):
        stream = 0
        for wi in range(words.shape[1]):
            stream |= int(words[r, wi]) << (32 * wi)
        for i in range(k):
            out[r, i] = (stream >> (i * bits)) & ((1 << bits) - 1)
    return out


def synth_packed_w(n, k, bits):
    pf = 32 // bits
    mask = (1 << bits) - 1
    n_packs = n * k // pf
    words = np.zeros(n_packs, dtype=np.uint32)
    for p in range(n_packs):
        v = 0
        for s in range(pf):
            code = ((p * 2654435761) + s) & 0xFFFFFFFF & mask
            v |= code << (s * bits)
        words[p] = v
    return words.reshape(n, k // pf)


# ---- the oracle, second restatement ---------------------------------------------
def qmm_ref(codes, scales, biases, x, group_size):
    """codes [n,k] ints, scales/biases [n,k/g] f32, x [m,k] f32 -> [m,n] f32."""
    n, k = codes.shape
    m = x.shape[0]
    out = np.zeros((m, n), dtype=np.float32)
    q = codes.astype(np.float32)
    for mr in range(m):
        acc = np.zeros(n, dtype=np.float32)
        for j in range(k):
            g = j // group_size
            wv = (q[:, j] * scales[:, g]).astype(f32) + biases[:, g]
            acc = (acc + (wv.astype(f32) * x[mr, j]).astype(f32)).astype(f32)
        out[mr] = acc
    return out


def qx_case(m, n, k, bits, group_size, dt):
    gspr = k // group_size
    w = synth_packed_w(n, k, bits)
    i = np.arange(n * gspr)
    scales_f = (f32(0.004) + (i % 7).astype(f32) * f32(0.0008)).astype(f32)
    biases_f = (((i % 5).astype(f32) - f32(2.0)) * f32(0.0009)).astype(f32)
    ix = np.arange(m * k)
    x_f = (((ix % 11).astype(f32) - f32(5.0)) * f32(0.01)).astype(f32)
    s = round_dt(scales_f, dt).reshape(n, gspr)
    b = round_dt(biases_f, dt).reshape(n, gspr)
    x = round_dt(x_f, dt).reshape(m, k)
    codes = unpack_rows(w, k, bits)
    acc = qmm_ref(codes, s, b, x, group_size)
    return dict(w=w, scales=scales_f.reshape(n, gspr), biases=biases_f.reshape(n, gspr),
                x=x_f.reshape(m, k), codes=codes.astype(np.uint8), acc=acc,
                expected=round_dt(acc, dt), meta=np.array([m, n, k, bits, group_size]))


def quantize_group(group, bits):
    max_code = f32((1 << bits) - 1)
    mn, mx = f32(group.min()), f32(group.max())
    scale = f32(1.0) if abs(f32(mx - mn)) < 1e-10 else f32(f32(mx - mn) / max_code)
    t = ((group - mn).astype(f32) / scale).astype(f32)
    # Rust f32::round is half away from zero on the exact value of t; t >= 0 here
    # and t + 0.5 is exact in float64.
    r = np.floor(t.astype(np.float64) + 0.5).astype(f32)
    codes = np.clip(r, 0, max_code).astype(np.uint32)
    return codes, scale, mn


def family_case(bits, dt):
    """run_qmv_test of quantized_family_gpu_correctness.rs:200-211 (n=64,k=256,g=64)."""
    n, k, gs = 64, 256, 64
    i = np.arange(n * k)
    w = ((((i * 31 + 7) % 53).astype(f32) - f32(26.0)) * f32(0.03)).astype(f32).reshape(n, k)
    d = np.arange(k)
    x = ((((d * 17 + 3) % 19).astype(f32) - f32(9.0)) * f32(0.05)).astype(f32)
    codes = np.zeros((n, k), dtype=np.uint32)
    scales = np.zeros((n, k // gs), dtype=np.float32)
    biases = np.zeros((n, k // gs), dtype=np.float32)
    for r in range(n):
        for g in range(k // gs):
            c, s, b = quantize_group(w[r, g * gs:(g + 1) * gs], bits)
            codes[r, g * gs:(g + 1) * gs] = c
            scales[r, g] = s
            biases[r, g] = b
    words = pack_rows(codes, bits)
    assert np.array_equal(unpack_rows(words, k, bits), codes)
    s, b, xr = round_dt(scales, dt), round_dt(biases, dt), round_dt(x, dt).reshape(1, k)
    acc = qmm_ref(codes, s, b, xr, gs)
    return dict(w=words, scales=scales, biases=biases, x=x.reshape(1, k), codes=codes.astype(np.uint8),
                acc=acc, expected=round_dt(acc, dt), meta=np.array([1, n, k, bits, gs]))


def gather_case(dt):
    """int4_setup of crates/metaltile-std/src/ffai/moe.rs:3627-3668."""
    n_experts, k_in, m_out, gs, t_rows = 3, 64, 8, 32, 6
    offsets = np.array([0, 2, 5, 6], dtype=np.uint32)
    i = np.arange(n_experts * m_out * k_in, dtype=np.uint64)
    codes = ((i * 7 + 3) & 0xF).astype(np.uint32).reshape(n_experts * m_out, k_in)
    words = pack_rows(codes, 4)
    ng = k_in // gs
    j = np.arange(n_experts * m_out * ng)
    scales_f = (f32(0.01) + f32(0.001) * j.astype(f32)).astype(f32)
    biases_f = (f32(-0.05) + f32(0.002) * j.astype(f32)).astype(f32)
    ix = np.arange(t_rows * k_in)
    # Rust: 0.1 * ((i as f32 * 0.17).sin()); f32 sin of an f32 argument.  numpy's
    # float32 sin and Rust's (libm sinf) may differ in the last bit, which only
    # perturbs the INPUT; the stored x is what both sides consume.
    x_f = (f32(0.1) * np.sin((ix.astype(f32) * f32(0.17)).astype(f32)).astype(f32)).astype(f32)
    s = round_dt(scales_f, dt).reshape(n_experts * m_out, ng)
    b = round_dt(biases_f, dt).reshape(n_experts * m_out, ng)
    x = round_dt(x_f, dt).reshape(t_rows, k_in)
    acc = np.zeros((t_rows, m_out), dtype=np.float32)
    for row in range(t_rows):
        e = next(e for e in range(n_experts) if row < offsets[e + 1])
        rows = slice(e * m_out, (e + 1) * m_out)
        acc[row] = qmm_ref(codes[rows], s[rows], b[rows], x[row:row + 1], gs)[0]
    return dict(w=words.reshape(n_experts, m_out, k_in // 8), scales=scales_f.reshape(n_experts, m_out, ng),
                biases=biases_f.reshape(n_experts, m_out, ng), x=x_f.reshape(t_rows, k_in),
                expert_offsets=offsets, acc=acc, expected=round_dt(acc, dt),
                meta=np.array([t_rows, k_in, m_out, n_experts, 4, gs]))


def topk_ref(logits, k, norm=1):
    rows, ne = logits.shape
    idx = np.zeros((rows, k), dtype=np.uint32)
    wts = np.zeros((rows, k), dtype=np.float32)
    for r in range(rows):
        chosen, vals = [], []
        for _ in range(k):
            best, bi = f32(-np.inf), 0
            for j in range(ne):
                if j in chosen:
                    continue
                if logits[r, j] > best:
                    best, bi = logits[r, j], j
            chosen.append(bi)
            vals.append(best)
        vals = np.array(vals, dtype=np.float32)
        if norm:
            mx = vals.max()
            e = np.exp((vals - mx).astype(f32)).astype(f32)
            ssum = f32(0)
            for v in e:
                ssum = f32(ssum + v)
            wts[r] = e / ssum
        else:
            mx = logits[r].max()
            ssum = f32(0)
            for v in np.exp((logits[r] - mx).astype(f32)).astype(f32):
                ssum = f32(ssum + v)
            wts[r] = np.exp((vals - mx).astype(f32)).astype(f32) / ssum
        idx[r] = chosen
    return idx, wts


def xorshift_source(n, seed, scale, off):
    """`source` of batched_qkv_qgemv_gpu_correctness.rs:100-110: xorshift64 (13, 7, 17) on a u64, value
    ((s % 20000) / 20000 - 0.5) * scale + off in f32."""
    s = seed
    mask = (1 << 64) - 1
    vals = np.empty(n, dtype=np.float32)
    for i in range(n):
        s ^= (s << 13) & mask
        s ^= s >> 7
        s ^= (s << 17) & mask
        v = f32(f32(s % 20000) / f32(20000.0))
        vals[i] = f32(f32(f32(v - f32(0.5)) * f32(scale)) + f32(off))
    return vals


def quantize_int4_matrix(rows, out_dim, in_dim, gs):
    """quantize_matrix / quantize_int4_row of the same file (:30-70): per group min / (max - min) / 15, round half away."""
    codes = np.zeros((out_dim, in_dim), dtype=np.uint32)
    scales = np.zeros((out_dim, in_dim // gs), dtype=np.float32)
    biases = np.zeros((out_dim, in_dim // gs), dtype=np.float32)
    w = rows.reshape(out_dim, in_dim)
    for r in range(out_dim):
        for g in range(in_dim // gs):
            c, sc, mn = quantize_group(w[r, g * gs:(g + 1) * gs], 4)
            codes[r, g * gs:(g + 1) * gs] = c
            scales[r, g] = sc
            biases[r, g] = mn
    return codes, scales, biases


def batched_case(dt, in_dim, gs, outs, seeds):
    """Fused decode projections that share x: run_case (:112-127) and test_batched_4_qgemv_fast (batched_4_qgemv.rs:421-440).
    The expected vector is naive_gemv per matrix with scales, biases and x rounded through the dtype."""
    x = round_dt(xorshift_source(in_dim, 0x11, 2.0, 0.05), dt).reshape(1, in_dim)
    d = dict(x=x, meta=np.array([in_dim, gs] + list(outs)))
    for i, (n, seed) in enumerate(zip(outs, seeds)):
        codes, sc, bi = quantize_int4_matrix(xorshift_source(n * in_dim, seed, 3.0, 0.0), n, in_dim, gs)
        words = pack_rows(codes, 4)
        acc = qmm_ref(codes, round_dt(sc, dt), round_dt(bi, dt), x, gs)
        d[f"w{i}"], d[f"scales{i}"], d[f"biases{i}"], d[f"acc{i}"] = words, sc, bi, acc.reshape(-1)
    return d


def rms_norm_case(dt, in_dim, gs, out_dim, eps=1e-5):
    """run_case / run_case_fast of crates/metaltile-std/tests/rms_norm_qgemv_gpu_correctness.rs:138-177,232-276 with the
    CPU check `naive` (:59-90): normed = x * norm_weight * inv_rms in f32, inv_rms = 1 / sqrt(ssq / K + eps)."""
    x = round_dt(xorshift_source(in_dim, 0xA1, 2.0, 0.1), dt)
    nw = round_dt(xorshift_source(in_dim, 0xB2, 0.4, 1.0), dt)
    codes, sc, bi = quantize_int4_matrix(xorshift_source(out_dim * in_dim, 0xC3, 3.0, 0.0), out_dim, in_dim, gs)
    ssq = f32(0.0)
    for v in x:
        ssq = f32(ssq + f32(v * v))
    inv_rms = f32(f32(1.0) / f32(np.sqrt(f32(f32(ssq / f32(in_dim)) + f32(eps)))))
    normed = ((x * nw).astype(f32) * inv_rms).astype(f32)
    acc = qmm_ref(codes, round_dt(sc, dt), round_dt(bi, dt), normed.reshape(1, in_dim), gs)
    return dict(x=x, norm_weight=nw, w=pack_rows(codes, 4), scales=sc, biases=bi, normed=normed, acc=acc.reshape(-1),
                eps=np.array([eps], dtype=np.float32), meta=np.array([in_dim, gs, out_dim]))


def affine_dequant_case(bits, gs, n_groups, dt):
    """dequant_setup of crates/metaltile-std/src/mlx/quantized.rs:5216-5251."""
    pf = 32 // bits
    n_elem = n_groups * gs
    w = ((np.arange(n_elem // pf, dtype=np.uint64) * 2654435761) & 0xFFFFFFFF).astype(np.uint32)
    scales = (f32(0.05) + np.arange(n_groups).astype(f32) * f32(0.01)).astype(f32)
    biases = (f32(-0.2) + np.arange(n_groups).astype(f32) * f32(0.03)).astype(f32)
    sd, bd = round_dt(scales, dt), round_dt(biases, dt)
    q = unpack_rows(w.reshape(1, -1), n_elem, bits).reshape(-1).astype(f32)
    g = np.arange(n_elem) // gs
    expected = ((sd[g] * q).astype(f32) + bd[g]).astype(f32)
    return dict(w=w, scales=scales, biases=biases, expected=expected, meta=np.array([bits, gs, n_groups]))


def affine_quant_case(bits, gs, n_groups, dt):
    """quantize_setup of quantized.rs:5268-5305 (scales and biases are what the reference pins); the codes follow the
    kernels' formula (:3657-3664) with every operation rounded to f32: trunc(clamp((v - min) * (1 / scale) + 0.5))."""
    n_bins = f32((1 << bits) - 1)
    n_elem = n_groups * gs
    w = (((np.arange(n_elem) % 37).astype(f32) - f32(18.0)) * f32(0.05)).astype(f32)
    wd = round_dt(w, dt).reshape(n_groups, gs)
    mn, mx = wd.min(axis=1), wd.max(axis=1)
    raw = ((mx - mn).astype(f32) / n_bins).astype(f32)
    scales = np.where(raw < f32(1.0e-7), f32(1.0), raw).astype(f32)
    inv = (f32(1.0) / scales).astype(f32)
    qf = (((wd - mn[:, None]).astype(f32) * inv[:, None]).astype(f32) + f32(0.5)).astype(f32)
    codes = np.clip(qf, f32(0.0), n_bins).astype(np.uint32)
    words = pack_rows(codes, bits).reshape(-1)
    return dict(w=w, scales=scales, biases=mn.astype(f32), codes=codes.astype(np.uint8), words=words, meta=np.array([bits, gs, n_groups]))


def dequant_gather_case(bits, hidden, gs, dt):
    """gather_setup of crates/metaltile-std/src/ffai/dequant_gather.rs:119-215."""
    vocab, ng = 8, hidden // gs
    r, d = np.meshgrid(np.arange(vocab, dtype=np.uint64), np.arange(hidden, dtype=np.uint64), indexing="ij")
    codes = ((((r * hidden + d) & 0xFFFFFFFF) * 2654435761 + d) & 0xFFFFFFFF).astype(np.uint32) & np.uint32((1 << bits) - 1)
    w = pack_rows(codes, bits)
    i = np.arange(vocab * ng)
    scales = (f32(0.02) + (i % 7).astype(f32) * f32(0.01)).astype(f32).reshape(vocab, ng)
    biases = (((i % 5).astype(f32) - f32(2.0)) * f32(0.05)).astype(f32).reshape(vocab, ng)
    idx = np.array([3, 0, 7, 1, 4, 4], dtype=np.uint32)
    s, b = round_dt(scales, dt), round_dt(biases, dt)
    g = np.arange(hidden) // gs
    expected = np.stack([((codes[t].astype(f32) * s[t][g]).astype(f32) + b[t][g]).astype(f32) for t in idx])
    return dict(weight=w, scales=scales, biases=biases, indices=idx, expected=expected, meta=np.array([bits, hidden, gs, vocab]))


def qvm_case(dt):
    """test_qvm_int4_fast of crates/metaltile-std/src/mlx/quantized.rs:5637-5663 with qvm_oracle (:5613-5635)."""
    n, k, gs = 32, 512, 64
    w = synth_packed_w(k, n, 4)                       # [K, N] transposed: K rows of N codes
    i = np.arange((k // gs) * n)
    scales = (f32(0.004) + (i % 7).astype(f32) * f32(0.0008)).astype(f32).reshape(k // gs, n)
    biases = (((i % 5).astype(f32) - f32(2.0)) * f32(0.0009)).astype(f32).reshape(k // gs, n)
    x = (((np.arange(k) % 11).astype(f32) - f32(5.0)) * f32(0.01)).astype(f32)
    s, b, xr = round_dt(scales, dt), round_dt(biases, dt), round_dt(x, dt)
    codes = unpack_rows(w, n, 4).astype(f32)          # [K, N]
    acc = np.zeros(n, dtype=np.float32)
    for d in range(k):
        wv = ((codes[d] * s[d // gs]).astype(f32) + b[d // gs]).astype(f32)
        acc = (acc + (wv * xr[d]).astype(f32)).astype(f32)
    return dict(w=w, scales=scales, biases=biases, x=x.reshape(1, k), acc=acc, meta=np.array([n, k, gs]))


def expert_indexed_case(dt):
    """test_dequant_gemv_int4_expert_indexed of crates/metaltile-std/src/ffai/dequant_gemv_expert_indexed.rs:129-208."""
    ne, od, idim, gs, expert = 4, 4, 256, 64, 2
    idx = np.arange(ne * od * idim, dtype=np.uint64)
    codes = (((idx & 0xFFFFFFFF) * 2654435761) & 0xFFFFFFFF).astype(np.uint32) & np.uint32(15)
    w = pack_rows(codes.reshape(ne * od, idim), 4)
    i = np.arange(ne * od * (idim // gs))
    scales = (f32(0.004) + (i % 7).astype(f32) * f32(0.0008)).astype(f32)
    biases = (((i % 5).astype(f32) - f32(2.0)) * f32(0.0009)).astype(f32)
    x = (((np.arange(idim) % 11).astype(f32) - f32(5.0)) * f32(0.01)).astype(f32)
    s, b, xr = round_dt(scales, dt).reshape(ne * od, -1), round_dt(biases, dt).reshape(ne * od, -1), round_dt(x, dt)
    sl = slice(expert * od, (expert + 1) * od)
    acc = qmm_ref(codes.reshape(ne * od, idim)[sl], s[sl], b[sl], xr.reshape(1, idim), gs).reshape(-1)
    return dict(w=w, scales=scales, biases=biases, x=x, acc=acc, meta=np.array([ne, od, idim, gs, expert]))


def moe_decode_tail_case(dt):
    """test_moe_down_swiglu_accum_int4_chain8 of crates/metaltile-std/src/ffai/moe_down_swiglu_accum.rs:355-487 (setup(4, 64, 8, 32))."""
    ne, idim, od, gs, ns = 4, 64, 8, 32, 8
    kd = np.arange(ns * idim).astype(f32)
    gates = (np.sin((kd * f32(0.017)).astype(f32)).astype(f32) * f32(0.5)).astype(f32).reshape(ns, idim)
    ups = (np.cos((kd * f32(0.021)).astype(f32)).astype(f32) * f32(0.5)).astype(f32).reshape(ns, idim)
    experts = (np.arange(ns) % ne).astype(np.uint32)
    sw = (f32(0.1) + np.arange(ns).astype(f32) * f32(0.05)).astype(f32)
    codes = ((np.arange(ne * od * idim, dtype=np.uint64) * 7 + 3) & 15).astype(np.uint32).reshape(ne * od, idim)
    w = pack_rows(codes, 4)
    i = np.arange(ne * od * (idim // gs)).astype(f32)
    scales = (f32(0.005) + (f32(0.001) * np.sin((i * f32(0.03)).astype(f32)).astype(f32)).astype(f32)).astype(f32)
    biases = (f32(-0.02) + (f32(0.005) * np.cos((i * f32(0.07)).astype(f32)).astype(f32)).astype(f32)).astype(f32)
    g_r, u_r, sw_r = round_dt(gates, dt), round_dt(ups, dt), round_dt(sw, dt)
    s_r, b_r = round_dt(scales, dt).reshape(ne * od, -1), round_dt(biases, dt).reshape(ne * od, -1)
    silu = (g_r / (f32(1.0) + np.exp(-g_r).astype(f32)).astype(f32)).astype(f32)
    inner = (silu * u_r).astype(f32)
    out = np.zeros(od, dtype=np.float32)
    cf = codes.astype(f32)
    for row in range(od):
        acc = f32(0.0)
        for k in range(ns):
            r = int(experts[k]) * od + row
            for d in range(idim):
                dq = f32(f32(cf[r, d] * s_r[r, d // gs]) + b_r[r, d // gs])
                acc = f32(acc + f32(f32(sw_r[k] * dq) * inner[k, d]))
        out[row] = acc
    return dict(gates=gates, ups=ups, experts=experts, slot_weights=sw, w=w, scales=scales, biases=biases, acc=out,
                meta=np.array([ne, idim, od, gs, ns]))


def save_new(path, **arrays):
    """Write a fixture unless the file already holds exactly these arrays (keeps unchanged fixtures byte-stable)."""
    if os.path.exists(path):
        old = dict(np.load(path))
        if old.keys() == arrays.keys() and all(np.array_equal(old[k], np.asarray(v), equal_nan=True) for k, v in arrays.items()):
            return
    np.savez_compressed(path, **arrays)


def main():
    out = {}
    # fused decode projections (N1): the reference's own cases
    for dt, in_dim, gs, oq, ok in (("f32", 256, 64, 16, 4), ("f32", 512, 128, 12, 6), ("f16", 256, 64, 16, 4),
                                   ("bf16", 256, 64, 16, 4), ("f32", 512, 64, 16, 8), ("f16", 512, 64, 16, 8),
                                   ("bf16", 512, 64, 16, 8)):
        save_new(os.path.join(HERE, f"batched_qkv_k{in_dim}_g{gs}_q{oq}_kv{ok}_{dt}.npz"),
                 **batched_case(dt, in_dim, gs, (oq, ok, ok), (0x22, 0x33, 0x44)))
    for dt, in_dim, gs, od in (("f32", 256, 64, 8), ("f32", 512, 128, 6), ("f16", 256, 64, 8), ("bf16", 256, 64, 8),
                               ("f32", 512, 64, 16), ("f16", 512, 64, 16), ("bf16", 512, 64, 16), ("f32", 1024, 64, 32)):
        save_new(os.path.join(HERE, f"rms_norm_qgemv_k{in_dim}_g{gs}_n{od}_{dt}.npz"), **rms_norm_case(dt, in_dim, gs, od))
    for dt in ("f32", "f16", "bf16"):
        for bits, gs, ng in ((4, 64, 8), (8, 64, 4), (2, 64, 16)):                     # quantized.rs:5253-5265
            save_new(os.path.join(HERE, f"test_affine_dequantize_int{bits}_{dt}.npz"), **affine_dequant_case(bits, gs, ng, dt))
        save_new(os.path.join(HERE, f"qvm_int4_fast_{dt}.npz"), **qvm_case(dt))
        save_new(os.path.join(HERE, f"expert_indexed_gemv_{dt}.npz"), **expert_indexed_case(dt))
        save_new(os.path.join(HERE, f"moe_down_swiglu_accum_{dt}.npz"), **moe_decode_tail_case(dt))
        for bits, hidden, gs in ((2, 256, 64), (4, 256, 64), (8, 256, 64), (3, 64, 32), (5, 64, 32), (6, 64, 32)):   # dequant_gather.rs:217-243
            save_new(os.path.join(HERE, f"test_dequant_gather_int{bits}_{dt}.npz"), **dequant_gather_case(bits, hidden, gs, dt))
        for bits, gs in ((2, 64), (3, 32), (4, 64), (5, 32), (6, 32), (8, 64)):          # quantized.rs:5307-5330
            save_new(os.path.join(HERE, f"test_affine_quantize_int{bits}_{dt}.npz"), **affine_quant_case(bits, gs, 8, dt))
    for dt in ("f32", "f16", "bf16"):
        save_new(os.path.join(HERE, f"test_batched_4_qgemv_fast_{dt}.npz"),
                 **batched_case(dt, 512, 64, (16, 8, 8, 8), (0x22, 0x33, 0x44, 0x55)))
    for dt in ("f32", "f16", "bf16"):
        # registered #[test_kernel] shapes (quantized.rs:5449-5605)
        for name, (m, n, k, bits, gs) in {
            "test_qmv": (1, 32, 512, 4, 64),
            "test_qmv_int8_fast": (1, 32, 512, 8, 64),
            "test_qmm": (8, 16, 512, 4, 64),
            "test_qmm_int8_fast": (8, 16, 512, 8, 64),
            "test_qmm_mma": (32, 64, 512, 4, 64),
            "test_qmm_mma_m16": (16, 64, 512, 4, 64),
            "test_qmm_mma_int8": (32, 64, 512, 8, 64),
            "test_qmm_mma_int2": (32, 64, 512, 2, 64),
        }.items():
            save_new(os.path.join(HERE, f"{name}_{dt}.npz"), **qx_case(m, n, k, bits, gs, dt))
        save_new(os.path.join(HERE, f"test_moe_gather_qmm_int4_{dt}.npz"), **gather_case(dt))
    for bits in (3, 4, 5, 6, 8):
        for dt in ("f32", "bf16"):
            save_new(os.path.join(HERE, f"family_qmv_b{bits}_{dt}.npz"), **family_case(bits, dt))

    # router top-k cases (moe_gpu_correctness.rs)
    i = np.arange(8 * 64).astype(f32)
    lg = (np.fmod((i * f32(0.13)).astype(f32), f32(7.0)) - f32(3.5) + (i * f32(0.001)).astype(f32)).astype(f32)
    lg = lg.reshape(8, 64)
    idx, wts = topk_ref(lg, 4)
    out["topk_base_logits"], out["topk_base_idx"], out["topk_base_w"] = lg, idx, wts
    i = np.arange(4 * 32).astype(f32)
    lg = (np.fmod((i * f32(0.7)).astype(f32), f32(5.0)) - f32(2.5) + (i * f32(0.01)).astype(f32)).astype(f32)
    lg = lg.reshape(4, 32)
    idx, wts = topk_ref(lg, 1)
    out["topk_k1_logits"], out["topk_k1_idx"], out["topk_k1_w"] = lg, idx, wts
    lg = np.zeros((1, 8), dtype=np.float32)
    lg[0, 2] = 10.0
    lg[0, 5] = 10.0
    lg[0, 3] = 8.0
    out["topk_tie_logits"] = lg
    out["topk_tie_idx"] = np.array([[2, 5]], dtype=np.uint32)  # literal: moe_gpu_correctness.rs:334
    i = np.arange(4 * 32).astype(f32)
    lg = (np.fmod((i * f32(0.31)).astype(f32), f32(9.0)) - f32(4.5)).astype(f32).reshape(4, 32)
    idx, wts = topk_ref(lg, 4, norm=0)
    out["topk_next_logits"], out["topk_next_idx"], out["topk_next_w"] = lg, idx, wts
    lg = np.tile((np.arange(16).astype(f32) * f32(0.1)).astype(f32), (4, 1))
    lg[0, 5] = np.nan
    lg[1, 7] = np.inf
    lg[2, 3] = -np.inf
    lg[3, 2] = np.nan
    lg[3, 11] = np.inf
    out["topk_naninf_logits"] = lg
    out["topk_naninf_idx"] = topk_ref(lg, 4)[0]

    # unpermute (moe_gpu_correctness.rs:164-198): identity inv_perm, normalised weights
    n_rows, hidden, k = 4, 256, 4
    i = np.arange(n_rows * k * hidden).astype(f32)
    eo = (np.fmod((i * f32(0.07)).astype(f32), f32(11.0)) - f32(5.5)).astype(f32).reshape(n_rows * k, hidden)
    raw = (f32(0.1) + (np.arange(n_rows * k).astype(f32) * f32(0.03)).astype(f32)).astype(f32).reshape(n_rows, k)
    wts = np.zeros_like(raw)
    for r in range(n_rows):
        ssum = f32(0)
        for v in raw[r]:
            ssum = f32(ssum + v)
        wts[r] = raw[r] / ssum
    inv = np.arange(n_rows * k, dtype=np.uint32).reshape(n_rows, k)
    ref = np.zeros((n_rows, hidden), dtype=np.float32)
    for t in range(n_rows):
        acc = np.zeros(hidden, dtype=np.float32)
        for j in range(k):
            acc = (acc + (wts[t, j] * eo[inv[t, j]]).astype(f32)).astype(f32)
        ref[t] = acc
    out["unperm_eo"], out["unperm_w"], out["unperm_inv"], out["unperm_out"] = eo, wts, inv, ref

    # swiglu (swiglu.rs:65-72), f32
    n = 1024
    g = ((np.arange(n) % 17).astype(f32) * f32(0.35) - f32(3.0)).astype(f32)
    u = ((np.arange(n) % 13).astype(f32) * f32(0.2) - f32(1.0)).astype(f32)
    out["swiglu_gate"], out["swiglu_up"] = g, u
    out["swiglu_out"] = ((g / (f32(1.0) + np.exp(-g).astype(f32)).astype(f32)).astype(f32) * u).astype(f32)

    # worked bit layouts: 3- and 6-bit streams, first period of a row
    c3 = np.arange(32, dtype=np.uint32).reshape(1, 32) % 8
    out["layout_b3_codes"], out["layout_b3_words"] = c3, pack_rows(c3, 3)
    c6 = (np.arange(16, dtype=np.uint32).reshape(1, 16) * 5 + 3) % 64
    out["layout_b6_codes"], out["layout_b6_words"] = c6, pack_rows(c6, 6)
    c4 = np.arange(8, dtype=np.uint32).reshape(1, 8) + 1
    out["layout_b4_codes"], out["layout_b4_words"] = c4, pack_rows(c4, 4)  # 0x87654321
    np.savez_compressed(os.path.join(HERE, "moe_and_layout.npz"), **out)
    print("wrote fixtures to", HERE)


if __name__ == "__main__":
    main()
