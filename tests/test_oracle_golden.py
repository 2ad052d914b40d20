"""The C oracle must reproduce, bit for bit, the fixtures written by the independent
numpy restatement in tests/golden/make_golden.py, and the literal expectations the
reference's own tests hold."""
import glob
import os

import numpy as np
import pytest

import oracle

DT = {"f32": oracle.F32, "f16": oracle.F16, "bf16": oracle.BF16}


def _load(path):
    return dict(np.load(path))


def _bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


QX = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "test_q*.npz")) +
            glob.glob(os.path.join(os.path.dirname(__file__), "golden", "family_qmv_*.npz")))


@pytest.mark.parametrize("path", QX, ids=[os.path.basename(p)[:-4] for p in QX])
def test_qmm_oracle_matches_fixture(path):
    fx = _load(path)
    dt = DT[os.path.basename(path)[:-4].rsplit("_", 1)[1]]
    m, n, k, bits, gs = (int(v) for v in fx["meta"])
    # bit-exact integer codes
    assert np.array_equal(oracle.unpack_matrix(fx["w"], k, bits), fx["codes"])
    assert np.array_equal(oracle.pack_matrix(fx["codes"], bits), fx["w"].reshape(n, -1))
    s = oracle.round_through(fx["scales"], dt)
    b = oracle.round_through(fx["biases"], dt)
    x = oracle.round_through(fx["x"], dt)
    acc = oracle.qmm(fx["w"], s, b, x, m, n, k, bits, gs)
    assert np.array_equal(_bits(acc), _bits(fx["acc"]))
    assert np.array_equal(_bits(oracle.round_through(acc, dt)), _bits(fx["expected"]))
    # M = 1 of qmm is qmv (tests/qmm_gpu_correctness.rs:341-393): row 0 alone gives the same numbers
    acc0 = oracle.qmm(fx["w"], s, b, x[:1], 1, n, k, bits, gs)
    assert np.array_equal(_bits(acc0[0]), _bits(acc[0]))
    # a row slice equals the same rows of the full result
    part = oracle.qmm(fx["w"], s, b, x, m, n, k, bits, gs, rows=(n // 4, n // 2))
    assert np.array_equal(_bits(part[:, n // 4:n // 2]), _bits(acc[:, n // 4:n // 2]))
    # dequant view agrees with code*scale+bias
    deq = oracle.dequant(fx["w"], s, b, n, k, bits, gs)
    ref = fx["codes"].astype(np.float32) * np.repeat(s.reshape(n, -1), gs, axis=1) \
        + np.repeat(b.reshape(n, -1), gs, axis=1)
    assert np.array_equal(_bits(deq), _bits(ref.astype(np.float32)))


@pytest.mark.parametrize("dt", ["f32", "f16", "bf16"])
def test_gather_oracle_matches_fixture(golden_dir, dt):
    fx = _load(os.path.join(golden_dir, f"test_moe_gather_qmm_int4_{dt}.npz"))
    t_rows, k_in, m_out, ne, bits, gs = (int(v) for v in fx["meta"])
    s = oracle.round_through(fx["scales"], DT[dt])
    b = oracle.round_through(fx["biases"], DT[dt])
    x = oracle.round_through(fx["x"], DT[dt])
    acc = oracle.gather_qmm(x, fx["w"], s, b, t_rows, k_in, m_out, ne, bits, gs,
                            expert_offsets=fx["expert_offsets"])
    assert np.array_equal(_bits(acc), _bits(fx["acc"]))
    # per-row index form gives the same result as the CSR form
    idx = np.array([0, 0, 1, 1, 1, 2], dtype=np.uint32)
    acc2 = oracle.gather_qmm(x, fx["w"], s, b, t_rows, k_in, m_out, ne, bits, gs, indices=idx)
    assert np.array_equal(_bits(acc2), _bits(acc))


@pytest.fixture(scope="module")
def moe(golden_dir):
    return _load(os.path.join(golden_dir, "moe_and_layout.npz"))


def test_router_topk_fixtures(moe):
    idx, w = oracle.router_topk(moe["topk_base_logits"], 64, 4)
    assert np.array_equal(idx, moe["topk_base_idx"])
    np.testing.assert_allclose(w, moe["topk_base_w"], rtol=0, atol=1e-6)
    idx, w = oracle.router_topk(moe["topk_k1_logits"], 32, 1)
    assert np.array_equal(idx, moe["topk_k1_idx"])
    assert np.all(np.abs(w - 1.0) < 1e-6)            # moe_gpu_correctness.rs:297-300
    idx, _ = oracle.router_topk(moe["topk_tie_logits"], 8, 2)
    assert idx.tolist() == [[2, 5]]                  # moe_gpu_correctness.rs:334
    idx, w = oracle.router_topk(moe["topk_next_logits"], 32, 4, norm_topk_prob=0)
    assert np.array_equal(idx, moe["topk_next_idx"])
    np.testing.assert_allclose(w, moe["topk_next_w"], rtol=0, atol=1e-6)
    assert np.all(w.sum(axis=1) < 1.0)


def test_router_topk_nan_inf_invariants(moe):
    """moe_gpu_correctness.rs:524-597."""
    idx, _ = oracle.router_topk(moe["topk_naninf_logits"], 16, 4)
    assert np.array_equal(idx, moe["topk_naninf_idx"])
    for r in range(4):
        assert len(set(idx[r].tolist())) == 4
    assert idx[1, 0] == 7 and idx[3, 0] == 11
    assert 3 not in idx[2] and 5 not in idx[0] and 2 not in idx[3]


def test_unpermute_and_swiglu_fixtures(moe):
    out = oracle.moe_unpermute(moe["unperm_eo"], moe["unperm_inv"], moe["unperm_w"])
    assert np.array_equal(_bits(out), _bits(moe["unperm_out"]))
    sw = oracle.swiglu(moe["swiglu_gate"], moe["swiglu_up"])
    np.testing.assert_allclose(sw, moe["swiglu_out"], rtol=2e-7, atol=1e-7)  # expf vs numpy exp: 1 ulp


def test_worked_bit_layouts(moe):
    assert np.array_equal(oracle.pack_matrix(moe["layout_b3_codes"], 3), moe["layout_b3_words"])
    assert np.array_equal(oracle.pack_matrix(moe["layout_b6_codes"], 6), moe["layout_b6_words"])
    w4 = oracle.pack_matrix(moe["layout_b4_codes"], 4)
    assert w4.tolist() == [[0x87654321]]             # low nibble first along K
    # 3-bit period: code 10 straddles words 0/1, code 21 straddles words 1/2
    c = np.zeros((1, 32), dtype=np.uint32)
    c[0, 10] = 0b101
    w = oracle.pack_matrix(c, 3)
    assert w[0, 0] == (0b01 << 30) and w[0, 1] == 0b1 and w[0, 2] == 0
    c = np.zeros((1, 32), dtype=np.uint32)
    c[0, 21] = 0b110
    w = oracle.pack_matrix(c, 3)
    assert w[0, 1] == (0b0 << 31) and w[0, 2] == 0b11
    c[0, 21] = 0b111
    w = oracle.pack_matrix(c, 3)
    assert w[0, 1] == (1 << 31) and w[0, 2] == 0b11


def test_moe_sort_definition():
    rng = np.random.default_rng(0)
    n_tokens, k, ne = 37, 4, 9
    topk = np.stack([rng.permutation(ne)[:k] for _ in range(n_tokens)]).astype(np.uint32)
    sti, inv, off, rex = oracle.moe_sort(topk, ne)
    flat = topk.reshape(-1)
    order = np.lexsort((np.arange(flat.size), flat))      # stable by (expert, flat slot)
    assert np.array_equal(sti, (order // k).astype(np.uint32))
    assert np.array_equal(rex, flat[order])
    assert np.array_equal(inv.reshape(-1)[order], np.arange(flat.size))
    assert np.array_equal(off, np.concatenate([[0], np.cumsum(np.bincount(flat, minlength=ne))]))
    # permute is a bit-exact row copy (moe_gpu_correctness.rs:627-672)
    tok = rng.standard_normal((n_tokens, 16)).astype(np.float32)
    assert np.array_equal(oracle.moe_permute(tok, sti), tok[sti])


def test_rounding_matches_torch():
    import torch
    rng = np.random.default_rng(1)
    a = np.concatenate([rng.standard_normal(20000).astype(np.float32) * s for s in (1e-8, 1e-4, 1, 300, 7e4)])
    a = np.concatenate([a, np.array([0.0, -0.0, 65504.0, 65520.0, 65519.9, 6.1e-5, 5.96e-8, 2.98e-8,
                                     2.9802325e-08, 1.0000001, 3.3895314e38], dtype=np.float32)])
    t = torch.from_numpy(a)
    for dt, tdt in ((oracle.BF16, torch.bfloat16), (oracle.F16, torch.float16)):
        ref = t.to(tdt).to(torch.float32).numpy()
        got = oracle.round_through(a, dt)
        assert np.array_equal(_bits(got), _bits(ref))
        bits = oracle.to_bits16(a, dt)
        assert np.array_equal(bits.view(np.int16), t.to(tdt).view(torch.int16).numpy())
        assert np.array_equal(_bits(oracle.from_bits16(bits, dt)), _bits(ref))


BATCHED = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "batched_qkv_*.npz")) +
                 glob.glob(os.path.join(os.path.dirname(__file__), "golden", "test_batched_4_*.npz")))


@pytest.mark.parametrize("path", BATCHED, ids=[os.path.basename(p)[:-4] for p in BATCHED])
def test_batched_decode_fixtures(path):
    """Fused decode projections (batched_qkv_qgemv_gpu_correctness.rs:112-127, batched_4_qgemv.rs:421-440): the C oracle
    reproduces every matrix's naive_gemv accumulator bit for bit."""
    fx = _load(path)
    dt = DT[os.path.basename(path)[:-4].rsplit("_", 1)[1]]
    in_dim, gs, outs = int(fx["meta"][0]), int(fx["meta"][1]), [int(v) for v in fx["meta"][2:]]
    assert len(outs) in (3, 4)
    for i, n in enumerate(outs):
        s, b = oracle.round_through(fx[f"scales{i}"], dt), oracle.round_through(fx[f"biases{i}"], dt)
        codes = oracle.unpack_matrix(fx[f"w{i}"], in_dim, 4)
        assert codes.max() <= 15 and fx[f"w{i}"].shape == (n, in_dim // 8)
        acc = oracle.qmm(fx[f"w{i}"], s, b, fx["x"], 1, n, in_dim, 4, gs)
        assert np.array_equal(_bits(acc.reshape(-1)), _bits(fx[f"acc{i}"]))


RMS = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "rms_norm_qgemv_*.npz")))


@pytest.mark.parametrize("path", RMS, ids=[os.path.basename(p)[:-4] for p in RMS])
def test_rms_norm_qgemv_fixtures(path):
    """Fused RMSNorm + decode projection (rms_norm_qgemv_gpu_correctness.rs:59-90,138-177): the C oracle reproduces the
    normalised activation and the accumulator bit for bit."""
    fx = _load(path)
    dt = DT[os.path.basename(path)[:-4].rsplit("_", 1)[1]]
    in_dim, gs, n = (int(v) for v in fx["meta"])
    eps = float(fx["eps"][0])
    assert np.array_equal(_bits(oracle.rms_normed(fx["x"], fx["norm_weight"], eps)), _bits(fx["normed"]))
    s, b = oracle.round_through(fx["scales"], dt), oracle.round_through(fx["biases"], dt)
    acc = oracle.rms_norm_qmv(fx["w"], s, b, fx["x"], fx["norm_weight"], eps, n, in_dim, 4, gs)
    assert np.array_equal(_bits(acc.reshape(-1)), _bits(fx["acc"]))


AFFINE_DQ = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "test_affine_dequantize_*.npz")))
AFFINE_Q = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "test_affine_quantize_*.npz")))


@pytest.mark.parametrize("path", AFFINE_DQ, ids=[os.path.basename(p)[:-4] for p in AFFINE_DQ])
def test_affine_dequantize_fixtures(path):
    """test_affine_dequantize_int{2,4,8} (crates/metaltile-std/src/mlx/quantized.rs:5216-5265): expected values bit for bit."""
    fx = _load(path)
    dt = DT[os.path.basename(path)[:-4].rsplit("_", 1)[1]]
    bits, gs, ng = (int(v) for v in fx["meta"])
    got = oracle.affine_dequantize(fx["w"], oracle.round_through(fx["scales"], dt), oracle.round_through(fx["biases"], dt), ng * gs, bits, gs)
    assert np.array_equal(_bits(got), _bits(fx["expected"]))


@pytest.mark.parametrize("path", AFFINE_Q, ids=[os.path.basename(p)[:-4] for p in AFFINE_Q])
def test_affine_quantize_fixtures(path):
    """test_affine_quantize_int{2,3,4,5,6,8} (quantized.rs:5268-5330): scales and biases (what the reference pins) and the
    packed codes of the kernels' formula, bit for bit; and the quantize -> dequantize round trip stays within half a step."""
    fx = _load(path)
    dt = DT[os.path.basename(path)[:-4].rsplit("_", 1)[1]]
    bits, gs, ng = (int(v) for v in fx["meta"])
    wd = oracle.round_through(fx["w"], dt)
    words, sc, bi = oracle.affine_quantize(wd, bits, gs)
    assert np.array_equal(_bits(sc), _bits(fx["scales"])) and np.array_equal(_bits(bi), _bits(fx["biases"]))
    assert np.array_equal(words, fx["words"])
    assert np.array_equal(oracle.unpack_matrix(words.reshape(ng, -1), gs, bits), fx["codes"])
    back = oracle.affine_dequantize(words, sc, bi, ng * gs, bits, gs).reshape(ng, gs)
    assert np.all(np.abs(back - wd.reshape(ng, gs)) <= 0.5 * sc[:, None] * (1 + 1e-5))


DQ_GATHER = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "test_dequant_gather_*.npz")))


@pytest.mark.parametrize("path", DQ_GATHER, ids=[os.path.basename(p)[:-4] for p in DQ_GATHER])
def test_dequant_gather_fixtures(path):
    """test_dequant_gather_int{2,3,4,5,6,8} (crates/metaltile-std/src/ffai/dequant_gather.rs:119-243): bit for bit."""
    fx = _load(path)
    dt = DT[os.path.basename(path)[:-4].rsplit("_", 1)[1]]
    bits, hidden, gs, _ = (int(v) for v in fx["meta"])
    got = oracle.dequant_gather(fx["weight"], oracle.round_through(fx["scales"], dt), oracle.round_through(fx["biases"], dt),
                                fx["indices"], hidden, bits, gs)
    assert np.array_equal(_bits(got), _bits(fx["expected"]))


@pytest.mark.parametrize("dt", ["f32", "f16", "bf16"])
def test_qvm_fixture(golden_dir, dt):
    """test_qvm_int4_fast (crates/metaltile-std/src/mlx/quantized.rs:5607-5663): the transposed-weight product bit for bit."""
    fx = _load(os.path.join(golden_dir, f"qvm_int4_fast_{dt}.npz"))
    n, k, gs = (int(v) for v in fx["meta"])
    d = DT[dt]
    acc = oracle.qvm(fx["w"], oracle.round_through(fx["scales"], d), oracle.round_through(fx["biases"], d), oracle.round_through(fx["x"], d),
                     1, n, k, 4, gs)
    assert np.array_equal(_bits(acc.reshape(-1)), _bits(fx["acc"]))


@pytest.mark.parametrize("dt", ["f32", "f16", "bf16"])
def test_moe_decode_tail_fixtures(golden_dir, dt):
    """test_dequant_gemv_int4_expert_indexed (ffai/dequant_gemv_expert_indexed.rs:129-208) and
    test_moe_down_swiglu_accum_int4_chain8 (ffai/moe_down_swiglu_accum.rs:355-487).  The expert-indexed product is the plain
    product on the chosen expert's slab, bit for bit; the fused tail agrees with the numpy restatement to within the last
    bits of expf (numpy's float32 exp and libm's expf are not the same function)."""
    d = DT[dt]
    fx = _load(os.path.join(golden_dir, f"expert_indexed_gemv_{dt}.npz"))
    ne, od, idim, gs, e = (int(v) for v in fx["meta"])
    s, b = oracle.round_through(fx["scales"], d).reshape(ne * od, -1), oracle.round_through(fx["biases"], d).reshape(ne * od, -1)
    sl = slice(e * od, (e + 1) * od)
    acc = oracle.qmm(fx["w"][sl], s[sl], b[sl], oracle.round_through(fx["x"], d).reshape(1, idim), 1, od, idim, 4, gs)
    assert np.array_equal(_bits(acc.reshape(-1)), _bits(fx["acc"]))
    fx = _load(os.path.join(golden_dir, f"moe_down_swiglu_accum_{dt}.npz"))
    ne, idim, od, gs, ns = (int(v) for v in fx["meta"])
    rt = lambda a: oracle.round_through(a, d)
    got = oracle.moe_down_swiglu_accum(rt(fx["gates"]), rt(fx["ups"]), fx["experts"], rt(fx["slot_weights"]), fx["w"], rt(fx["scales"]),
                                       rt(fx["biases"]), idim, od, gs)
    assert np.max(np.abs(got - fx["acc"])) <= 1e-6 * max(1.0, float(np.max(np.abs(fx["acc"]))))
