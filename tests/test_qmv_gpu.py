"""Parity of the CUDA qmv path with the CPU oracle (all calls go through the C ABI)."""
import os

import numpy as np
import pytest

import oracle
from helpers import DT_NAMES, ODT, TOL, bytes_to_f32, dense_case, dt_bytes, rel_err, to_dev

pytestmark = pytest.mark.gpu

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


@pytest.fixture(scope="module")
def ctx():
    from metaltile_b200 import ops
    return ops.context(0)


def run_qmv(w, s, b, x, bits, gs, dt, fn="qmv"):
    import torch
    from metaltile_b200 import ops
    out = getattr(ops, fn)(to_dev(w), to_dev(s, dt), to_dev(b, dt), to_dev(x, dt), bits, gs)
    torch.cuda.synchronize()
    return out.float().cpu().numpy()


# ---- the reference's registered #[test_kernel] cases, by kernel name, host buffers ----
REGISTERED = {
    "test_qmv": ("mt_qmv", "gs_per_row", False),
    "test_qmv_int8_fast": ("mt_qmv_int8_fast", "gs_per_row", False),
    "test_qmm": ("mt_qmm", "gs_per_row", True),
    "test_qmm_int8_fast": ("mt_qmm_int8_fast", "gs_per_row", True),
    "test_qmm_mma": ("mt_qmm_mma", "gs_per_row", True),
    "test_qmm_mma_m16": ("mt_qmm_mma_m16", "gs_per_row", True),
    "test_qmm_mma_int8": ("mt_qmm_mma_int8", "gs_per_row", True),
    "test_qmm_mma_int2": ("mt_qmm_mma_int2", "gs_per_row", True),
}


@pytest.mark.parametrize("dt", DT_NAMES)
@pytest.mark.parametrize("case", sorted(REGISTERED))
def test_registered_cases_via_dispatch(ctx, case, dt):
    fx = dict(np.load(os.path.join(GOLDEN, f"{case}_{dt}.npz")))
    kernel, gs_const, has_n = REGISTERED[case]
    m, n, k, bits, gs = (int(v) for v in fx["meta"])
    bufs = {"w": fx["w"].tobytes(), "scales": dt_bytes(fx["scales"], dt), "biases": dt_bytes(fx["biases"], dt),
            "x": dt_bytes(fx["x"], dt), "out": bytes(m * n * (4 if dt == "f32" else 2)),
            "k": k.to_bytes(4, "little"), gs_const: (k // gs).to_bytes(4, "little")}
    if has_n:
        bufs["n"] = n.to_bytes(4, "little")
    res = ctx.dispatch_with_grid(kernel, bufs, {}, (max(n // 8, 1), 1, 1), (64, 1, 1), dtype=dt)
    got = bytes_to_f32(res.outputs["out"], dt).reshape(m, n)
    assert np.any(got != 0.0)
    assert rel_err(got, fx["expected"]) <= TOL[dt]
    assert res.elapsed_us > 0.0


@pytest.mark.parametrize("dt", ["f32", "bf16"])
@pytest.mark.parametrize("bits", [3, 4, 5, 6, 8])
def test_family_cases_via_dispatch(ctx, bits, dt):
    """mt_qmv_b* with quantised real weights (tests/quantized_family_gpu_correctness.rs:200-233)."""
    fx = dict(np.load(os.path.join(GOLDEN, f"family_qmv_b{bits}_{dt}.npz")))
    m, n, k, _, gs = (int(v) for v in fx["meta"])
    bufs = {"w": fx["w"].tobytes(), "scales": dt_bytes(fx["scales"], dt), "biases": dt_bytes(fx["biases"], dt),
            "x": dt_bytes(fx["x"], dt), "out": bytes(m * n * (4 if dt == "f32" else 2))}
    res = ctx.dispatch_with_grid(f"mt_qmv_b{bits}", bufs, {"k": k, "n": n, "group_size": gs}, (n, 1, 1),
                                 (32, 1, 1), dtype=dt)
    got = bytes_to_f32(res.outputs["out"], dt).reshape(m, n)
    assert np.any(got != 0.0)
    assert rel_err(got, fx["expected"]) <= TOL[dt]


@pytest.mark.parametrize("bits", [2, 3, 4, 5, 6, 8])
def test_unpacked_codes_bit_exact(bits):
    import torch
    from metaltile_b200 import ops, synth
    n, k = 257, 4096
    w = synth.words(n * k * bits // 32, seed=3).reshape(n, -1)
    got = ops.unpack_codes(to_dev(w), k, bits)
    torch.cuda.synchronize()
    assert np.array_equal(got.cpu().numpy(), oracle.unpack_matrix(w, k, bits))


def test_config0_qmv_4bit_g64_4096(ctx):
    """The headline case: bf16 x[1,4096], W 4096x4096 4-bit g64, seed 0."""
    w, s, b, x = dense_case(1, 4096, 4096, 4, 64, "bf16", seed=0)
    ref = oracle.qmm(w, s, b, x, 1, 4096, 4096, 4, 64)
    got = run_qmv(w, s, b, x, 4, 64, "bf16")
    assert rel_err(got, ref) <= TOL["bf16"]
    # tighter diagnosis: before the final bf16 rounding the kernel is within f32 round-off of the
    # oracle, so got must equal round_bf16(ref) except for values on a rounding boundary
    exp = oracle.round_through(ref, oracle.BF16)
    assert np.mean(got == exp) > 0.99
    ctx.set_option("qmv_stream", 0)            # the CUDA-core kernel on the same case
    try:
        cores = run_qmv(w, s, b, x, 4, 64, "bf16")
    finally:
        ctx.set_option("qmv_stream", 1)
    assert rel_err(cores, ref) <= TOL["bf16"]
    assert np.mean(cores == exp) > 0.99


SWEEP = [(bits, gs, m, kn, dt)
         for bits in (2, 3, 4, 6, 8) for gs in (32, 64, 128) for m in (1, 4, 8, 16)
         for kn in (2048, 4096, 8192) for dt in DT_NAMES]
_CASES = {}


def _sweep_weights(bits, gs, kn):
    """One weight matrix per (bits, group, size), shared by the M and dtype cells of the sweep (generated once)."""
    key = (bits, gs, kn)
    if key not in _CASES:
        _CASES.clear()                      # the cells are ordered by (bits, gs, ..): keep one matrix at a time
        from metaltile_b200 import synth
        w, s, b = synth.quantized_matrix(kn, kn, bits, gs, 0, bits)
        _CASES[key] = (w, s, b, to_dev(w))
    return _CASES[key]


@pytest.mark.parametrize("bits,gs,m,kn,dt", sorted(SWEEP, key=lambda c: (c[0], c[1], c[3])))
def test_sweep(bits, gs, m, kn, dt):
    """The benchmark's sweep grid: bits x group x M x K = N x dtype.  At 2048 every output is compared with the
    oracle; at 4096 and 8192 the first, a middle and the last band of 32 weight rows (the CPU oracle is a scalar
    loop), which covers the first and last row group of the first, a middle and the last CTA of every kernel."""
    from metaltile_b200 import ops, synth
    import torch
    w, s, b, wd = _sweep_weights(bits, gs, kn)
    x = synth.activations(m, kn, 0, bits)
    s, b, x = (oracle.round_through(a, ODT[dt]) for a in (s, b, x))
    out = ops.qmv(wd, to_dev(s, dt), to_dev(b, dt), to_dev(x, dt), bits, gs)
    torch.cuda.synchronize()
    got = out.float().cpu().numpy()
    bands = [(0, kn)] if kn == 2048 else [(0, 32), (kn // 2 + 5, kn // 2 + 37), (kn - 32, kn)]
    for (n0, n1) in bands:
        ref = oracle.qmm(w, s, b, x, m, kn, kn, bits, gs, rows=(n0, n1))
        assert rel_err(got[:, n0:n1], ref[:, n0:n1]) <= TOL[dt], (n0, n1)


@pytest.mark.parametrize("bits,gs,m,kn,dt", [
    (4, 64, 1, 8192, "bf16"), (4, 64, 16, 4096, "bf16"), (3, 32, 8, 4096, "f16"), (6, 128, 4, 8192, "f32"),
    (2, 64, 1, 8192, "f32"), (8, 32, 16, 4096, "f32"), (5, 64, 3, 4096, "bf16"),
])
def test_sweep_large(bits, gs, m, kn, dt):
    w, s, b, x = dense_case(m, kn, kn, bits, gs, dt, seed=0, salt=7)
    ref = oracle.qmm(w, s, b, x, m, kn, kn, bits, gs)
    got = run_qmv(w, s, b, x, bits, gs, dt)
    assert rel_err(got, ref) <= TOL[dt]


@pytest.mark.parametrize("m,n,k,bits,gs,dt", [
    (1, 1024, 4096, 4, 64, "bf16"),     # Llama kv projection: split-K path
    (8, 1024, 4096, 4, 64, "bf16"),
    (1, 14336, 4096, 4, 64, "bf16"),    # gate/up
    (1, 4096, 14336, 4, 64, "bf16"),    # down: K = 14336
    (8, 4096, 14336, 4, 64, "bf16"),
    (1, 128, 4096, 4, 64, "bf16"),      # an 8-way shard of kv
    (1, 2048, 768, 4, 64, "bf16"),      # MoE down shape
    (5, 37, 96, 4, 32, "f32"),          # ragged N, tiny K
    (3, 7, 32, 8, 32, "f16"),
    (17, 64, 256, 4, 64, "bf16"),       # M > 16: two M tiles
    (33, 40, 512, 3, 64, "f32"),
    (2, 9, 1536, 6, 128, "bf16"),
])
def test_shapes_and_edges(m, n, k, bits, gs, dt):
    w, s, b, x = dense_case(m, n, k, bits, gs, dt, seed=1, salt=m + n)
    ref = oracle.qmm(w, s, b, x, m, n, k, bits, gs)
    got = run_qmv(w, s, b, x, bits, gs, dt)
    assert got.shape == (m, n)
    assert rel_err(got, ref) <= TOL[dt]


@pytest.mark.parametrize("m,n,k,gs,dt", [
    (2, 4096, 4096, 64, "bf16"), (3, 37, 64, 64, "f16"),        # one segment, ragged N
    (7, 1000, 2112, 64, "bf16"),                                # 33 segments: two staged blocks, the second ragged
    (8, 16, 4096, 128, "f16"), (9, 1024, 4096, 64, "bf16"),     # 9 tokens: two token tiles
    (15, 250, 8192, 256, "bf16"), (16, 14336, 4096, 64, "f16"), (16, 4096, 14336, 64, "bf16"),
    (12, 8, 128, 64, "bf16"),                                   # fewer rows than one 16-row tile
])
def test_small_m_tensor_core_path(ctx, m, n, k, gs, dt):
    """2 <= M <= 16 with 4-bit codes runs on warp-level MMAs (the register / cp.async ring kernels of qmv_mma.cu once
    the streaming kernel is switched off); same oracle, and within round-off of the CUDA-core kernel for the same call."""
    assert ctx.qmm_route(m, n, k, 4, gs, dt) in ("qmv_mma_sync", "qmv_stream")
    w, s, b, x = dense_case(m, n, k, 4, gs, dt, seed=6, salt=m * 31 + n)
    ref = oracle.qmm(w, s, b, x, m, n, k, 4, gs)
    assert rel_err(run_qmv(w, s, b, x, 4, gs, dt), ref) <= TOL[dt]          # the default route
    ctx.set_option("qmv_stream", 0)
    try:
        got = run_qmv(w, s, b, x, 4, gs, dt)
        assert got.shape == (m, n)
        assert rel_err(got, ref) <= TOL[dt]
        ctx.set_option("qmv_small_m_mma", 0)
        try:
            cores = run_qmv(w, s, b, x, 4, gs, dt)
        finally:
            ctx.set_option("qmv_small_m_mma", 1)
    finally:
        ctx.set_option("qmv_stream", 1)
    assert rel_err(cores, ref) <= TOL[dt]
    assert rel_err(got, cores) <= TOL[dt]


@pytest.mark.parametrize("n,k,dt", [(4096, 4096, "bf16"), (100, 14336, "f16"), (1024, 512, "bf16")])
def test_single_row_through_tensor_core_path(ctx, n, k, dt):
    """Option value 2 sends M = 1 down the same path; K = 14336 stays resident as one staged block."""
    w, s, b, x = dense_case(1, n, k, 4, 64, dt, seed=8, salt=n)
    ref = oracle.qmm(w, s, b, x, 1, n, k, 4, 64)
    ctx.set_option("qmv_small_m_mma", 2)
    ctx.set_option("qmv_stream", 0)
    try:
        got = run_qmv(w, s, b, x, 4, 64, dt)
    finally:
        ctx.set_option("qmv_small_m_mma", 1)
        ctx.set_option("qmv_stream", 1)
    assert rel_err(got, ref) <= TOL[dt]


def test_small_m_tensor_core_exact_integers(ctx):
    """Integer-valued scales, biases and activations: every product and sum is exact in f32, so the MMA
    path must reproduce the oracle bit for bit (checks the code-to-slot permutation of the operands)."""
    from metaltile_b200 import synth
    m, n, k, gs = 5, 48, 256, 64
    w = synth.words(n * k * 4 // 32, seed=9).reshape(n, -1)
    rng = np.random.default_rng(9)
    s = rng.integers(1, 4, size=(n, k // gs)).astype(np.float32)
    b = rng.integers(-3, 4, size=(n, k // gs)).astype(np.float32)
    x = rng.integers(-2, 3, size=(m, k)).astype(np.float32)
    ref = oracle.qmm(w, s, b, x, m, n, k, 4, gs)
    got = run_qmv(w, s, b, x, 4, gs, "f16")
    assert np.array_equal(got, oracle.round_through(ref, oracle.F16))


def test_multi_output_store_and_single_rank_barrier(ctx):
    """mtc_qmv_multi writes the same tile to every destination (the sharded path's all-gather is these stores);
    with one rank the barrier kernel only meets its own flag, raises the epoch and leaves the status word clear."""
    import torch
    from metaltile_b200.ops import _TORCH_DT
    for m, n, k, dt in [(1, 1024, 4096, "bf16"), (1, 200, 512, "f32"), (1, 4096, 14336, "f16")]:
        w, s, b, x = dense_case(m, n, k, 4, 64, dt, seed=15, salt=n)
        wd, sd, bd, xd = to_dev(w), to_dev(s, dt), to_dev(b, dt), to_dev(x, dt)
        outs = [torch.zeros((m, n), dtype=xd.dtype, device="cuda") for _ in range(3)]
        ctx.qmv_multi(wd.data_ptr(), sd.data_ptr(), bd.data_ptr(), xd.data_ptr(), [o.data_ptr() for o in outs], m, n, k, 4, 64,
                      _TORCH_DT[xd.dtype], stream=torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        ref = oracle.qmm(w, s, b, x, m, n, k, 4, 64)
        assert rel_err(outs[0].float().cpu().numpy(), ref) <= TOL[dt]
        assert torch.equal(outs[1], outs[0]) and torch.equal(outs[2], outs[0])
    flags = torch.zeros(64, dtype=torch.int32, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    for _ in range(3):
        ctx.peer_barrier([flags.data_ptr()], 0, flags.data_ptr(), flags.data_ptr() + 128, stream=st)
    torch.cuda.synchronize()
    assert int(flags[0]) == 3 and int(flags[32]) == 3          # own flag word and the epoch counter
    assert ctx.status_word() == 0
    from metaltile_b200 import MetalTileError
    with pytest.raises(MetalTileError):
        ctx.peer_barrier([flags.data_ptr()] * 9, 0, flags.data_ptr(), flags.data_ptr() + 128, stream=st)
    ctx.set_option("qmv_stream", 0)
    try:
        with pytest.raises(MetalTileError) as ei:      # on the CUDA-core kernel several destinations are the M = 1 case only
            ctx.qmv_multi(wd.data_ptr(), sd.data_ptr(), bd.data_ptr(), xd.data_ptr(), [o.data_ptr() for o in outs], 3, n, k, 4, 64,
                          _TORCH_DT[xd.dtype], stream=st)
        assert ei.value.variant == "Unsupported"
    finally:
        ctx.set_option("qmv_stream", 1)


def test_generic_fallback_paths(ctx):
    """Group sizes below the chunk and unaligned pointers take the any-shape kernel."""
    import torch
    from metaltile_b200 import ops
    # group_size 16 with 4-bit codes (chunk = 32 codes)
    w, s, b, x = dense_case(2, 33, 128, 4, 16, "f32", seed=2)
    ref = oracle.qmm(w, s, b, x, 2, 33, 128, 4, 16)
    assert rel_err(run_qmv(w, s, b, x, 4, 16, "f32"), ref) <= TOL["f32"]
    # weights at a 4-byte (not 16-byte) aligned address
    w, s, b, x = dense_case(1, 64, 256, 4, 64, "bf16", seed=2)
    ref = oracle.qmm(w, s, b, x, 1, 64, 256, 4, 64)
    flat = torch.zeros(w.size + 1, dtype=torch.int32, device="cuda")
    flat[1:] = to_dev(w).reshape(-1)
    wv = flat[1:].view(64, -1)
    assert wv.data_ptr() % 16 != 0
    out = ops.qmv(wv, to_dev(s, "bf16"), to_dev(b, "bf16"), to_dev(x, "bf16"), 4, 64)
    torch.cuda.synchronize()
    assert rel_err(out.float().cpu().numpy(), ref) <= TOL["bf16"]


def test_m1_equals_row_of_batched(ctx):
    """M = 1 of qmm is qmv (tests/qmm_gpu_correctness.rs:341-393)."""
    w, s, b, x = dense_case(8, 512, 1024, 4, 64, "f32", seed=4)
    full = run_qmv(w, s, b, x, 4, 64, "f32", fn="qmm")
    for r in (0, 5):
        one = run_qmv(w, s, b, x[r:r + 1], 4, 64, "f32")
        assert rel_err(one[0], full[r]) <= 1e-5


def test_linearity_at_full_size(ctx):
    """qmv(x1 + x2) = qmv(x1) + qmv(x2) up to round-off, at K = N = 8192 (size-independent property)."""
    w, s, b, x = dense_case(2, 8192, 8192, 4, 64, "f32", seed=5)
    xs = np.stack([x[0], x[1], x[0] + x[1]])
    got = run_qmv(w, s, b, xs, 4, 64, "f32")
    assert rel_err(got[2], got[0] + got[1]) <= 1e-4


def test_empty_inputs(ctx):
    import torch
    from metaltile_b200 import ops
    w, s, b, x = dense_case(1, 8, 64, 4, 64, "f32")
    out = ops.qmv(to_dev(w), to_dev(s), to_dev(b), to_dev(x[:0]), 4, 64)
    torch.cuda.synchronize()
    assert out.shape == (0, 8)


def test_error_behaviour(ctx):
    from metaltile_b200 import MetalTileError
    w, s, b, x = dense_case(1, 8, 64, 4, 64, "f32")
    good = {"w": w.tobytes(), "scales": s.tobytes(), "biases": b.tobytes(), "x": x.tobytes(), "out": bytes(32)}
    with pytest.raises(MetalTileError) as ei:
        ctx.dispatch_with_grid("mt_not_a_kernel", good, {"k": 64, "gs_per_row": 1})
    assert ei.value.variant == "FunctionNotFound"
    with pytest.raises(MetalTileError) as ei:       # undersized buffer (buffer_plan.rs:68-76)
        ctx.dispatch_with_grid("mt_qmm", dict(good, w=w.tobytes()[:-4]), {"k": 64, "n": 8, "gs_per_row": 1})
    assert ei.value.variant == "BufferSize"
    with pytest.raises(MetalTileError) as ei:       # missing constexpr
        ctx.dispatch_with_grid("mt_qmm", good, {"k": 64, "gs_per_row": 1})
    assert ei.value.variant == "Buffer"
    with pytest.raises(MetalTileError) as ei:       # unsupported width
        ctx.qmv(1, 1, 1, 1, 1, 1, 8, 64, 7, 64, "f32")
    assert ei.value.variant == "Unsupported"
    assert ctx.status_word() == 0


RMS_CASES = [("ffai_rms_norm_qgemv", 256, 64, 8, "f32"), ("ffai_rms_norm_qgemv", 512, 128, 6, "f32"), ("ffai_rms_norm_qgemv", 256, 64, 8, "f16"),
             ("ffai_rms_norm_qgemv", 256, 64, 8, "bf16"), ("ffai_rms_norm_qgemv_fast", 512, 64, 16, "f32"),
             ("ffai_rms_norm_qgemv_fast", 512, 64, 16, "f16"), ("ffai_rms_norm_qgemv_fast", 512, 64, 16, "bf16"),
             ("ffai_rms_norm_qgemv_fast", 1024, 64, 32, "f32")]


@pytest.mark.parametrize("kernel,in_dim,gs,n,dt", RMS_CASES)
def test_rms_norm_qgemv_via_dispatch(ctx, kernel, in_dim, gs, n, dt):
    """The reference's own cases of the fused RMSNorm + decode projection under its kernel and buffer names
    (crates/metaltile-std/tests/rms_norm_qgemv_gpu_correctness.rs:93-124,179-294), with its tolerances and this build's."""
    fx = dict(np.load(os.path.join(GOLDEN, f"rms_norm_qgemv_k{in_dim}_g{gs}_n{n}_{dt}.npz")))
    bufs = {"x": dt_bytes(fx["x"], dt), "norm_weight": dt_bytes(fx["norm_weight"], dt), "weight": fx["w"].tobytes(),
            "scales": dt_bytes(fx["scales"], dt), "biases": dt_bytes(fx["biases"], dt), "output": bytes(n * (4 if dt == "f32" else 2)),
            "eps_buf": fx["eps"].astype(np.float32).tobytes()}
    res = ctx.dispatch_with_grid(kernel, bufs, {"in_dim": in_dim, "group_size": gs}, (n, 1, 1), (128, 1, 1), dtype=dt, outputs=("output",))
    got = bytes_to_f32(res.outputs["output"], dt)
    exp = fx["acc"]
    assert np.any(got != 0.0)
    ref_tol = {"f32": 5e-3, "f16": 2e-2, "bf16": 5e-2}[dt]
    assert float(np.max(np.abs(got - exp) / np.maximum(np.abs(exp), 1e-3))) <= ref_tol
    assert rel_err(got.reshape(1, -1), exp.reshape(1, -1)) <= TOL[dt]


@pytest.mark.parametrize("n,k,gs,dt", [(4096, 4096, 64, "bf16"), (1024, 4096, 128, "f16"), (300, 2048, 64, "f32"), (64, 480, 96, "bf16")])
def test_rms_norm_qmv_typed(ctx, n, k, gs, dt):
    """mtc_rms_norm_qmv at decode sizes against the oracle (the normalised activation stays f32); the last case has a group
    that is not a power of two: the unfused form (normalise into a row of the activation type, then the plain product)."""
    import torch
    from metaltile_b200 import ops, synth
    w, s, b, x = dense_case(1, n, k, 4, gs, dt, seed=31)
    nw = oracle.round_through(1.0 + 0.2 * synth.activations(1, k, seed=32), {"f32": oracle.F32, "f16": oracle.F16, "bf16": oracle.BF16}[dt])
    eps = 1e-5
    got = ops.rms_norm_qmv(to_dev(w), to_dev(s, dt), to_dev(b, dt), to_dev(x, dt).reshape(-1), to_dev(nw, dt).reshape(-1), eps, 4, gs, ctx=ctx)
    torch.cuda.synchronize()
    ref = oracle.rms_norm_qmv(w, s, b, x.reshape(-1), nw.reshape(-1), eps, n, k, 4, gs)
    assert ctx.status_word() == 0
    assert rel_err(got.float().cpu().numpy(), ref) <= TOL[dt]


@pytest.mark.parametrize("m", [2, 5, 16])
def test_small_m_tensor_core_path_special_activations(ctx, m):
    """The ring kernel stages bf16 activations times 2^64 (and x / 16 for the nibbles at bits 4-7): zeros of both signs,
    bf16 subnormals, tiny and large magnitudes must come through exactly."""
    import torch
    from metaltile_b200 import ops
    n, k = 96, 4096
    assert ctx.qmm_route(m, n, k, 4, 64, "bf16") == "qmv_mma_sync"
    w, s, b, x = dense_case(m, n, k, 4, 64, "bf16", seed=14)
    special = np.array([0x0000, 0x8000, 0x0001, 0x8001, 0x007F, 0x0080, 0x8080, 0x0100, 0x1F80, 0x5D80, 0xDD80, 0x3F80], dtype=np.uint32)
    bits = (special[np.arange(m * k) % len(special)] << 16).astype(np.uint32).reshape(m, k)
    x = bits.view(np.float32).copy()
    x[:, 5::11] = oracle.round_through(np.random.default_rng(15).standard_normal(x[:, 5::11].shape).astype(np.float32), oracle.BF16)
    ref = oracle.qmm(w, s, b, x, m, n, k, 4, 64)
    xd = torch.from_numpy((np.ascontiguousarray(x).view(np.uint32) >> 16).astype(np.int16)).cuda().view(torch.bfloat16)
    got = ops.qmv(to_dev(w), to_dev(s, "bf16"), to_dev(b, "bf16"), xd, 4, 64, ctx=ctx)
    torch.cuda.synchronize()
    got = got.float().cpu().numpy()
    assert ctx.status_word() == 0 and np.all(np.isfinite(got))
    assert rel_err(got, ref) <= TOL["bf16"]
    assert np.mean(got == oracle.round_through(ref, oracle.BF16)) > 0.98
