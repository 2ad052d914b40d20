"""The codec either side of the quantized matmuls on the GPU: mt_affine_quantize_int* / mt_affine_dequantize_int*
(crates/metaltile-std/src/mlx/quantized.rs:3575-4214) against the reference's own cases and against the oracle.
Integer codes, scales, biases and dequantized values are compared for equality."""
import os

import numpy as np
import pytest

import oracle
from helpers import ODT, TOL, bytes_to_f32, dt_bytes, rel_err, to_dev

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


@pytest.fixture(scope="module")
def ctx():
    from metaltile_b200 import ops
    return ops.context(0)


@pytest.mark.parametrize("dt", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("bits", [2, 4, 8])
def test_reference_dequantize_cases(ctx, bits, dt):
    """test_affine_dequantize_int{2,4,8} (quantized.rs:5216-5265) under the reference's kernel and buffer names."""
    fx = dict(np.load(os.path.join(GOLDEN, f"test_affine_dequantize_int{bits}_{dt}.npz")))
    _, gs, ng = (int(v) for v in fx["meta"])
    n = ng * gs
    bufs = {"w": fx["w"].tobytes(), "scales": dt_bytes(fx["scales"], dt), "biases": dt_bytes(fx["biases"], dt),
            "out": bytes(n * (4 if dt == "f32" else 2))}
    res = ctx.dispatch_with_grid(f"mt_affine_dequantize_int{bits}", bufs, {"group_size": gs}, (n * bits // 32, 1, 1), (64, 1, 1), dtype=dt)
    got = bytes_to_f32(res.outputs["out"], dt)
    assert np.array_equal(got, oracle.round_through(fx["expected"], ODT[dt]))


@pytest.mark.parametrize("dt", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("bits", [2, 3, 4, 5, 6, 8])
def test_reference_quantize_cases(ctx, bits, dt):
    """test_affine_quantize_int{2,3,4,5,6,8} (quantized.rs:5268-5330): the scales and biases the reference pins, and the
    packed codes of its formula, all for equality."""
    fx = dict(np.load(os.path.join(GOLDEN, f"test_affine_quantize_int{bits}_{dt}.npz")))
    _, gs, ng = (int(v) for v in fx["meta"])
    n, esz = ng * gs, (4 if dt == "f32" else 2)
    bufs = {"w": dt_bytes(fx["w"], dt), "out": bytes(n * bits // 8), "scales": bytes(ng * esz), "biases": bytes(ng * esz)}
    res = ctx.dispatch_with_grid(f"mt_affine_quantize_int{bits}", bufs, {"group_size": gs}, (ng, 1, 1), (32, 1, 1), dtype=dt,
                                 outputs=("out", "scales", "biases"))
    assert np.array_equal(bytes_to_f32(res.outputs["scales"], dt), oracle.round_through(fx["scales"], ODT[dt]))
    assert np.array_equal(bytes_to_f32(res.outputs["biases"], dt), oracle.round_through(fx["biases"], ODT[dt]))
    assert np.array_equal(np.frombuffer(res.outputs["out"], dtype=np.uint32), fx["words"])


@pytest.mark.parametrize("bits,gs,dt", [(4, 64, "bf16"), (3, 32, "f16"), (8, 128, "bf16"), (5, 32, "f32"), (6, 64, "bf16"), (2, 64, "f16"),
                                        (2, 48, "bf16"), (4, 8, "f32")])
def test_quantize_then_matmul_on_device(ctx, bits, gs, dt):
    """Real float weights packed on the device: codes, scales and biases equal the oracle's, the inverse equals the
    oracle's, and the decode product of the packed matrix matches the oracle's product (the last two shapes have groups
    that are not a multiple of 32: the one-thread-per-group form)."""
    import torch
    from metaltile_b200 import ops, synth
    n, k = 512, 1536
    wf = oracle.round_through(0.05 * synth.activations(n, k, seed=40 + bits), ODT[dt])
    wd = to_dev(wf, dt)
    q, s, b = ops.affine_quantize(wd, bits, gs, ctx=ctx)
    back = ops.affine_dequantize(q, s, b, bits, gs, ctx=ctx)
    torch.cuda.synchronize()
    oq, osc, obi = oracle.affine_quantize(wf, bits, gs)
    assert np.array_equal(q.cpu().numpy().view(np.uint32).reshape(-1), oq)
    s_h, b_h = s.float().cpu().numpy().reshape(-1), b.float().cpu().numpy().reshape(-1)
    assert np.array_equal(s_h, oracle.round_through(osc, ODT[dt])) and np.array_equal(b_h, oracle.round_through(obi, ODT[dt]))
    ref_back = oracle.round_through(oracle.affine_dequantize(oq, s_h, b_h, n * k, bits, gs), ODT[dt])
    assert np.array_equal(back.float().cpu().numpy().reshape(-1), ref_back)
    # half a quantization step (plus the rounding of scale and bias to the activation type)
    assert np.all(np.abs(back.float().cpu().numpy() - wf) <= (0.5 * np.repeat(s_h, gs).reshape(n, k) * 1.02 + 2e-3))
    if k % gs == 0 and gs >= 32:
        x = oracle.round_through(synth.activations(1, k, seed=3), ODT[dt])
        got = ops.qmv(q, s, b, to_dev(x, dt), bits, gs, ctx=ctx)
        torch.cuda.synchronize()
        ref = oracle.qmm(oq.reshape(n, -1), s_h.reshape(n, -1), b_h.reshape(n, -1), x, 1, n, k, bits, gs)
        assert rel_err(got.float().cpu().numpy(), ref) <= TOL[dt]
    assert ctx.status_word() == 0


def test_codec_refuses_partial_groups(ctx):
    import torch
    from metaltile_b200 import MetalTileError
    w = torch.zeros(100, dtype=torch.float32, device="cuda")
    out = torch.zeros(64, dtype=torch.int32, device="cuda")
    sb = torch.zeros(8, dtype=torch.float32, device="cuda")
    with pytest.raises(MetalTileError) as ei:               # 100 is not a whole number of groups of 64
        ctx.affine_quantize(w.data_ptr(), out.data_ptr(), sb.data_ptr(), sb.data_ptr(), 100, 4, 64, "f32")
    assert ei.value.variant == "Unsupported"
    with pytest.raises(MetalTileError) as ei:               # 3-bit groups of 8 are not whole words
        ctx.affine_dequantize(out.data_ptr(), sb.data_ptr(), sb.data_ptr(), w.data_ptr(), 64, 3, 8, "f32")
    assert ei.value.variant == "Unsupported"


@pytest.mark.parametrize("dt", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("bits,hidden,gs", [(2, 256, 64), (4, 256, 64), (8, 256, 64), (3, 64, 32), (5, 64, 32), (6, 64, 32)])
def test_reference_dequant_gather_cases(ctx, bits, hidden, gs, dt):
    """test_dequant_gather_int{2,3,4,5,6,8} (crates/metaltile-std/src/ffai/dequant_gather.rs:119-243) under the reference's
    kernel and buffer names: a non-monotonic gather that repeats a row."""
    fx = dict(np.load(os.path.join(GOLDEN, f"test_dequant_gather_int{bits}_{dt}.npz")))
    n_tok = fx["indices"].size
    bufs = {"weight": fx["weight"].tobytes(), "scales": dt_bytes(fx["scales"], dt), "biases": dt_bytes(fx["biases"], dt),
            "indices": fx["indices"].astype(np.uint32).tobytes(), "out": bytes(n_tok * hidden * (4 if dt == "f32" else 2))}
    res = ctx.dispatch_with_grid(f"dequant_gather_int{bits}", bufs, {"hidden": hidden, "group_size": gs}, (n_tok * hidden // 256 + 1, 1, 1),
                                 (256, 1, 1), dtype=dt)
    got = bytes_to_f32(res.outputs["out"], dt).reshape(n_tok, hidden)
    assert np.array_equal(got, oracle.round_through(fx["expected"], ODT[dt]))


@pytest.mark.parametrize("bits,hidden,gs,dt", [(4, 4096, 64, "bf16"), (3, 1024, 32, "f16"), (8, 2048, 128, "f32"), (4, 72, 24, "bf16")])
def test_embedding_gather_at_size(ctx, bits, hidden, gs, dt):
    """A quantized embedding table with 1000 rows, 777 lookups (repeats, first and last row); the last shape has a hidden
    size and a group that are not multiples of 32: the one-thread-per-element form.  Equal to the oracle."""
    import torch
    from metaltile_b200 import ops, synth
    vocab, n_tok = 1000, 777
    w, s, b = synth.quantized_matrix(vocab, hidden, bits, gs, seed=50 + bits)
    s, b = oracle.round_through(s, ODT[dt]), oracle.round_through(b, ODT[dt])
    rng = np.random.default_rng(bits)
    idx = rng.integers(0, vocab, n_tok).astype(np.uint32)
    idx[:3] = (0, vocab - 1, vocab - 1)
    got = ops.dequant_gather(to_dev(w), to_dev(s, dt), to_dev(b, dt), to_dev(idx), bits, gs, ctx=ctx)
    torch.cuda.synchronize()
    ref = oracle.round_through(oracle.dequant_gather(w, s, b, idx, hidden, bits, gs), ODT[dt])
    assert ctx.status_word() == 0
    assert np.array_equal(got.float().cpu().numpy(), ref)


def test_embedding_gather_reports_a_bad_index(ctx):
    import torch
    from metaltile_b200 import MetalTileError, ops, synth
    w, s, b = synth.quantized_matrix(16, 256, 4, 64, seed=1)
    idx = np.array([1, 99, 2], dtype=np.uint32)             # 99 is outside the table: row 0 is read, 0x904 reported
    try:
        got = ops.dequant_gather(to_dev(w), to_dev(s, "bf16"), to_dev(b, "bf16"), to_dev(idx), 4, 64, ctx=ctx)
        with pytest.raises(MetalTileError):
            ctx.sync(torch.cuda.current_stream().cuda_stream)
        assert ctx.status_word() == 0x904
    finally:
        ctx.status_clear()
    assert torch.equal(got[1], ops.dequant_gather(to_dev(w), to_dev(s, "bf16"), to_dev(b, "bf16"), to_dev(np.array([0], dtype=np.uint32)), 4, 64, ctx=ctx)[0])


@pytest.mark.parametrize("dt", ["f32", "f16", "bf16"])
def test_reference_qvm_case(ctx, dt):
    """test_qvm_int4_fast (crates/metaltile-std/src/mlx/quantized.rs:5637-5663) under the reference's names, with its
    tolerances (5e-3 / 5e-2 / 2e-1) and this build's."""
    fx = dict(np.load(os.path.join(GOLDEN, f"qvm_int4_fast_{dt}.npz")))
    n, k, gs = (int(v) for v in fx["meta"])
    bufs = {"w": fx["w"].tobytes(), "scales": dt_bytes(fx["scales"], dt), "biases": dt_bytes(fx["biases"], dt), "x": dt_bytes(fx["x"], dt),
            "out": bytes(n * (4 if dt == "f32" else 2))}
    for kernel, consts in (("mt_qvm_int4_fast", {"k": k, "n": n, "gs_per_col": k // gs}), ("mt_qvm_b4", {"k": k, "n": n, "group_size": gs})):
        res = ctx.dispatch_with_grid(kernel, bufs, consts, (n // 8, 1, 1), (64, 1, 1), dtype=dt)
        got = bytes_to_f32(res.outputs["out"], dt)
        assert np.any(got != 0.0)
        assert rel_err(got.reshape(1, -1), fx["acc"].reshape(1, -1)) <= TOL[dt]
        assert float(np.max(np.abs(got - fx["acc"]))) <= {"f32": 5e-3, "f16": 5e-2, "bf16": 2e-1}[dt]


@pytest.mark.parametrize("m,n,k,bits,gs,dt", [
    (1, 4096, 4096, 4, 64, "bf16"), (1, 1024, 2048, 8, 64, "f16"), (2, 512, 1024, 3, 32, "bf16"), (1, 320, 768, 5, 128, "f32"),
    (3, 96, 256, 6, 64, "bf16"), (1, 4096, 512, 2, 64, "f16"), (1, 40, 192, 4, 48, "f32"), (1, 24, 128, 4, 64, "bf16"),
])
def test_qvm_matches_oracle(ctx, m, n, k, bits, gs, dt):
    """The vector-matrix product over transposed weights against the oracle: every width, several token rows, K split over
    CTAs and not, a column count that leaves lanes idle (40, 24), a group that is not a power of two; twice for equality."""
    import torch
    from metaltile_b200 import ops, synth
    w = synth.words(k * n * bits // 32, seed=60 + bits).reshape(k, -1)                          # [K, N] codes packed along N
    sc = oracle.round_through(0.002 + 0.018 * np.random.default_rng(bits).random((k // gs, n), dtype=np.float32), ODT[dt])
    bi = oracle.round_through(-8.0 * sc, ODT[dt])
    x = oracle.round_through(synth.activations(m, k, seed=7), ODT[dt])
    got = ops.qvm(to_dev(w), to_dev(sc, dt), to_dev(bi, dt), to_dev(x, dt), bits, gs, ctx=ctx)
    again = ops.qvm(to_dev(w), to_dev(sc, dt), to_dev(bi, dt), to_dev(x, dt), bits, gs, ctx=ctx)
    torch.cuda.synchronize()
    ref = oracle.qvm(w, sc, bi, x, m, n, k, bits, gs)
    assert ctx.status_word() == 0
    assert torch.equal(got, again)
    assert rel_err(got.float().cpu().numpy(), ref) <= TOL[dt]
