"""Parity of the streaming decode kernel (qmv_stream.cu) with the CPU oracle: single projections through
mtc_qmv, projections that share x through mtc_qmv_batched, and prepared chains through mtc_chain_*."""
import numpy as np
import pytest

import oracle
from helpers import ODT, TOL, dense_case, rel_err, to_dev

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    """The context with the streaming kernel taking every M <= 8 it supports (option value 2; the default routes only
    M = 1 to it), so that the multi-token cases below exercise that kernel."""
    from metaltile_b200 import ops
    c = ops.context(0)
    c.set_option("qmv_stream", 2)
    yield c
    c.set_option("qmv_stream", 1)


def _bands(n, width=32):
    """First, middle and last row band of a matrix: what the oracle computes for the large shapes."""
    if n <= 3 * width:
        return [(0, n)]
    mid = (n // 2) // 16 * 16 + 5
    return [(0, width), (mid, mid + width), (n - width, n)]


def _check(got, w, s, b, x, m, n, k, bits, gs, dt):
    for (n0, n1) in _bands(n):
        ref = oracle.qmm(w, s, b, x, m, n, k, bits, gs, rows=(n0, n1))
        assert rel_err(got[:, n0:n1], ref[:, n0:n1]) <= TOL[dt], (n0, n1)


@pytest.mark.parametrize("m,n,k,gs,dt", [
    (1, 4096, 4096, 64, "bf16"), (1, 4096, 4096, 64, "f16"), (1, 1024, 4096, 64, "bf16"), (1, 14336, 4096, 64, "bf16"),
    (1, 4096, 14336, 64, "bf16"), (1, 8192, 8192, 64, "bf16"), (1, 2048, 2048, 128, "f16"), (1, 4096, 4096, 128, "bf16"),
    (2, 4096, 4096, 64, "bf16"), (3, 1000, 2048, 64, "f16"), (4, 4096, 4096, 64, "bf16"), (5, 777, 1024, 128, "bf16"),
    (8, 4096, 4096, 64, "bf16"), (8, 4096, 4096, 64, "f16"), (7, 37, 512, 64, "bf16"), (1, 5, 512, 64, "f16"),
    (1, 128, 4096, 64, "bf16"), (8, 1024, 4096, 128, "f16"), (1, 2048, 1536, 64, "bf16"), (6, 300, 512, 64, "bf16"),
    (1, 31, 3584, 128, "bf16"), (2, 16, 14336, 64, "f16"),
])
@pytest.mark.parametrize("engine", ["tcgen05", "stream"])
def test_stream_matches_oracle(ctx, m, n, k, gs, dt, engine):
    """The two decode kernels for M <= 8: the warp-level MMA stream kernel (the default) and the kernel with the codes
    as the A operand in tensor memory (tcgen05; option `qmv_tc` = 1; shapes whose activations do not fit its shared
    memory fall through to the stream kernel)."""
    import torch
    from metaltile_b200 import ops
    w, s, b, x = dense_case(m, n, k, 4, gs, dt, seed=2, salt=m + n % 7)
    # a single projection takes this kernel by default from 8 Mi codes on (fused launches and option value 2: any size)
    assert ctx.qmm_route(1, n, k, 4, gs, dt) == ("qmv_stream" if n * k >= 8 << 20 else "qmv_cuda_core")
    ctx.set_option("qmv_tc", 1 if engine == "tcgen05" else 0)
    try:
        got = ops.qmv(to_dev(w), to_dev(s, dt), to_dev(b, dt), to_dev(x, dt), 4, gs, ctx=ctx)
        torch.cuda.synchronize()
    finally:
        ctx.set_option("qmv_tc", 0)
    assert ctx.status_word() == 0
    _check(got.float().cpu().numpy(), w, s, b, x, m, n, k, 4, gs, dt)


def test_tcgen05_decode_twice_and_exact(ctx):
    """Back-to-back launches reuse the arrival counters (left at zero by the kernel) and the partial-sum planes; the
    result equals the rounded oracle almost everywhere (exact products, f32 sums)."""
    import torch
    from metaltile_b200 import ops
    m, n, k = 1, 1000, 4096
    w, s, b, x = dense_case(m, n, k, 4, 64, "bf16", seed=12)
    ref = oracle.qmm(w, s, b, x, m, n, k, 4, 64)
    args = (to_dev(w), to_dev(s, "bf16"), to_dev(b, "bf16"), to_dev(x, "bf16"), 4, 64)
    ctx.set_option("qmv_tc", 1)
    try:
        outs = [ops.qmv(*args, ctx=ctx) for _ in range(3)]
        torch.cuda.synchronize()
    finally:
        ctx.set_option("qmv_tc", 0)
    assert ctx.status_word() == 0
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
    exp = oracle.round_through(ref, oracle.BF16)
    assert np.mean(outs[0].float().cpu().numpy() == exp) > 0.99


def test_stream_is_exact_before_rounding(ctx):
    """Codes times activations are exact products accumulated in f32: the result equals the rounded oracle
    almost everywhere (differences only where the oracle sits on a rounding boundary)."""
    import torch
    from metaltile_b200 import ops
    m, n, k = 1, 512, 4096
    w, s, b, x = dense_case(m, n, k, 4, 64, "bf16", seed=0)
    ref = oracle.qmm(w, s, b, x, m, n, k, 4, 64)
    got = ops.qmv(to_dev(w), to_dev(s, "bf16"), to_dev(b, "bf16"), to_dev(x, "bf16"), 4, 64, ctx=ctx)
    torch.cuda.synchronize()
    exp = oracle.round_through(ref, oracle.BF16)
    assert np.mean(got.float().cpu().numpy() == exp) > 0.99


def bits_of(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


@pytest.mark.parametrize("m", [1, 3])
def test_stream_staging_of_special_activations(ctx, m):
    """The activations are staged times 2^64 (bf16): zeros of both signs, bf16 subnormals, tiny and large magnitudes must
    come through exactly - the result is compared with the oracle on an x made of such values."""
    import torch
    from metaltile_b200 import ops
    n, k = 64, 4096
    w, s, b, x = dense_case(m, n, k, 4, 64, "bf16", seed=4)
    special = np.array([0x0000, 0x8000, 0x0001, 0x8001, 0x007F, 0x0080, 0x8080, 0x0100, 0x1F80, 0x5D80, 0xDD80, 0x3F80],
                       dtype=np.uint32)                       # +-0, smallest / largest subnormal, smallest normals, 2^-64, +-2^60, 1
    bits = (special[np.arange(m * k) % len(special)] << 16).astype(np.uint32).reshape(m, k)
    x = bits.view(np.float32).copy()
    x[:, 7::13] = oracle.round_through(np.random.default_rng(5).standard_normal(x[:, 7::13].shape).astype(np.float32), oracle.BF16)
    ref = oracle.qmm(w, s, b, x, m, n, k, 4, 64)
    xd = torch.from_numpy((bits_of(x) >> 16).astype(np.int16)).cuda().view(torch.bfloat16)      # the exact bit patterns
    got = ops.qmv(to_dev(w), to_dev(s, "bf16"), to_dev(b, "bf16"), xd, 4, 64, ctx=ctx)
    torch.cuda.synchronize()
    assert ctx.status_word() == 0
    got = got.float().cpu().numpy()
    assert np.all(np.isfinite(got)) and rel_err(got, ref) <= TOL["bf16"]
    exp = oracle.round_through(ref, oracle.BF16)
    assert np.mean(got == exp) > 0.98


def test_stream_equals_the_cuda_core_kernel_within_rounding(ctx):
    import torch
    from metaltile_b200 import ops
    m, n, k = 1, 4096, 4096
    w, s, b, x = dense_case(m, n, k, 4, 64, "bf16", seed=5)
    args = (to_dev(w), to_dev(s, "bf16"), to_dev(b, "bf16"), to_dev(x, "bf16"), 4, 64)
    a = ops.qmv(*args, ctx=ctx)                    # the warp-level MMA stream kernel
    ctx.set_option("qmv_tc", 1)
    try:
        t2 = ops.qmv(*args, ctx=ctx)               # the tcgen05 decode kernel
    finally:
        ctx.set_option("qmv_tc", 0)
    ctx.set_option("qmv_stream", 0)
    try:
        c = ops.qmv(*args, ctx=ctx)                # the CUDA-core kernel
    finally:
        ctx.set_option("qmv_stream", 2)
    assert torch.mean((a == t2).float()).item() > 0.98
    torch.cuda.synchronize()
    assert rel_err(a.float().cpu().numpy(), c.float().cpu().numpy()) <= 1e-2
    assert torch.mean((a == c).float()).item() > 0.98


@pytest.mark.parametrize("dt", ["bf16", "f16"])
@pytest.mark.parametrize("m", [1, 4])
def test_batched_qkv_is_three_qmv(ctx, m, dt):
    """q, k, v in one launch == three oracle products side by side
    (ffai_batched_qkv_qgemv, crates/metaltile-std/src/ffai/batched_qkv_qgemv.rs:1-35)."""
    import torch
    from metaltile_b200 import ops
    k, ns = 4096, (4096, 1024, 1024)
    x = oracle.round_through(__import__("metaltile_b200").synth.activations(m, k, seed=3), ODT[dt])
    mats, refs = [], []
    for i, n in enumerate(ns):
        w, s, b, _ = dense_case(m, n, k, 4, 64, dt, seed=3, salt=10 + i)
        mats.append((to_dev(w), to_dev(s, dt), to_dev(b, dt)))
        refs.append((w, s, b, n))
    out = ops.qmv_batched(mats, to_dev(x, dt), 4, 64, ctx=ctx)
    torch.cuda.synchronize()
    assert ctx.status_word() == 0
    tiles = [out[:, 0:4096], out[:, 4096:5120], out[:, 5120:6144]] if m == 1 else out
    for t, (w, s, b, n) in zip(tiles, refs):
        _check(t.float().cpu().numpy(), w, s, b, x, m, n, k, 4, 64, dt)
    # and bit-identical to three separate launches of the same kernel
    for t, (wd, sd, bd) in zip(tiles, mats):
        one = ops.qmv(wd, sd, bd, to_dev(x, dt), 4, 64, ctx=ctx)
        assert torch.equal(one, t.reshape(one.shape))


def _layer(dt, seed, k_small=4096, k_big=14336, scale=8):
    """A decode layer's projection list at 1/scale of the Llama-3-8B widths (same structure, same phases)."""
    shapes = [("q", k_small, 4096 // scale, 0), ("k", k_small, 1024 // scale, 0), ("v", k_small, 1024 // scale, 0),
              ("o", k_small, 4096 // scale, 1), ("gate", k_small, 14336 // scale, 2), ("up", k_small, 14336 // scale, 2),
              ("down", k_big, 4096 // scale, 3)]
    mats = []
    for i, (_, k, n, ph) in enumerate(shapes):
        w, s, b, _ = dense_case(1, n, k, 4, 64, dt, seed=seed, salt=20 + i)
        mats.append((w, s, b, k, n, ph))
    return mats


@pytest.mark.parametrize("dt", ["bf16", "f16"])
def test_chain_matches_oracle_per_projection(ctx, dt):
    """Two layers (8 phases, 14 projections) in one persistent launch, run twice: every projection equals its
    oracle, and the second run (counters reset by the first) reproduces the first bit for bit."""
    import torch
    from metaltile_b200 import ops, synth
    from metaltile_b200.ops import _projection
    m = 1
    layers = [_layer(dt, 4), _layer(dt, 5)]
    xs = {k: oracle.round_through(synth.activations(m, k, seed=9, salt=k), ODT[dt]) for k in (4096, 14336)}
    xd = {k: to_dev(v, dt) for k, v in xs.items()}
    projs, keep, outs = [], [], []
    for li, mats in enumerate(layers):
        for (w, s, b, k, n, ph) in mats:
            wd, sd, bd = to_dev(w), to_dev(s, dt), to_dev(b, dt)
            o = torch.zeros((m, n), dtype=xd[k].dtype, device="cuda")
            keep.append((wd, sd, bd))
            outs.append((o, w, s, b, k, n))
            projs.append(_projection(wd, sd, bd, xd[k], 4, 64, [o], phase=li * 4 + ph))
    chain = ctx.chain_create(projs)
    assert chain.fused
    chain.run(torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert ctx.status_word() == 0
    first = [o.clone() for (o, *_r) in outs]
    for (o, w, s, b, k, n) in outs:
        _check(o.float().cpu().numpy(), w, s, b, xs[k], m, n, k, 4, 64, dt)
        o.zero_()
    chain.run(torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert ctx.status_word() == 0
    for f, (o, *_r) in zip(first, outs):
        assert torch.equal(f, o)
    chain.close()


def test_chain_phases_order_dependent_projections(ctx):
    """Phase p + 1 reads what phase p wrote: y1 = W1 x, y2 = W2 y1 in one launch equals two separate launches."""
    import torch
    from metaltile_b200 import ops
    from metaltile_b200.ops import _projection
    dt, k = "bf16", 2048
    w1, s1, b1, x = dense_case(1, k, k, 4, 64, dt, seed=6, salt=1)
    w2, s2, b2, _ = dense_case(1, 1024, k, 4, 64, dt, seed=6, salt=2)
    d = [to_dev(w1), to_dev(s1, dt), to_dev(b1, dt), to_dev(w2), to_dev(s2, dt), to_dev(b2, dt)]
    xd = to_dev(x, dt)
    y1 = torch.zeros((1, k), dtype=torch.bfloat16, device="cuda")
    y2 = torch.zeros((1, 1024), dtype=torch.bfloat16, device="cuda")
    chain = ctx.chain_create([_projection(d[0], d[1], d[2], xd, 4, 64, [y1], phase=0),
                              _projection(d[3], d[4], d[5], y1, 4, 64, [y2], phase=1)])
    assert chain.fused
    for _ in range(3):
        y1.zero_()
        y2.zero_()
        chain.run(torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        r1 = ops.qmv(d[0], d[1], d[2], xd, 4, 64, ctx=ctx)
        r2 = ops.qmv(d[3], d[4], d[5], r1, 4, 64, ctx=ctx)
        torch.cuda.synchronize()
        assert torch.equal(y1, r1) and torch.equal(y2, r2)
    assert ctx.status_word() == 0
    chain.close()


def test_chain_outside_the_contract_falls_back_to_launches(ctx):
    """A 3-bit projection cannot run on the streaming kernel: the chain still runs, one launch per projection."""
    import torch
    from metaltile_b200.ops import _projection
    dt = "bf16"
    w, s, b, x = dense_case(2, 96, 512, 3, 32, dt, seed=8)
    wd, sd, bd, xd = to_dev(w), to_dev(s, dt), to_dev(b, dt), to_dev(x, dt)
    o = torch.zeros((2, 96), dtype=torch.bfloat16, device="cuda")
    chain = ctx.chain_create([_projection(wd, sd, bd, xd, 3, 32, [o])])
    assert not chain.fused
    chain.run(torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    ref = oracle.qmm(w, s, b, x, 2, 96, 512, 3, 32)
    assert rel_err(o.float().cpu().numpy(), ref) <= TOL[dt]
    chain.close()


def test_chain_rejects_bad_phases(ctx):
    import torch
    from metaltile_b200.context import MetalTileError
    from metaltile_b200.ops import _projection
    dt = "bf16"
    w, s, b, x = dense_case(1, 64, 256, 4, 64, dt, seed=8)
    wd, sd, bd, xd = to_dev(w), to_dev(s, dt), to_dev(b, dt), to_dev(x, dt)
    o = torch.zeros((1, 64), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(MetalTileError) as ei:
        ctx.chain_create([_projection(wd, sd, bd, xd, 4, 64, [o], phase=1)])
    assert ei.value.variant == "Invalid"
    with pytest.raises(MetalTileError):
        ctx.chain_create([_projection(wd, sd, bd, xd, 4, 64, [o], phase=0), _projection(wd, sd, bd, xd, 4, 64, [o], phase=2)])


def test_chain_in_a_cuda_graph(ctx):
    """The chain launch is capturable: graph replays give the same bytes as a direct run."""
    import torch
    from metaltile_b200.ops import _projection
    dt = "bf16"
    mats = _layer(dt, 11, scale=16)
    from metaltile_b200 import synth
    xs = {k: to_dev(oracle.round_through(synth.activations(1, k, seed=1, salt=k), ODT[dt]), dt) for k in (4096, 14336)}
    keep, outs, projs = [], [], []
    for (w, s, b, k, n, ph) in mats:
        wd, sd, bd = to_dev(w), to_dev(s, dt), to_dev(b, dt)
        o = torch.zeros((1, n), dtype=torch.bfloat16, device="cuda")
        keep.append((wd, sd, bd))
        outs.append(o)
        projs.append(_projection(wd, sd, bd, xs[k], 4, 64, [o], phase=ph))
    chain = ctx.chain_create(projs)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        chain.run(side.cuda_stream)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    direct = [o.clone() for o in outs]
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        chain.run(torch.cuda.current_stream().cuda_stream)
    for _ in range(3):
        for o in outs:
            o.zero_()
        g.replay()
        torch.cuda.synchronize()
        for a, o in zip(direct, outs):
            assert torch.equal(a, o)
    assert ctx.status_word() == 0
    chain.close()


def _batched_fixture(name):
    import os
    return dict(np.load(os.path.join(os.path.dirname(__file__), "golden", name)))


# the reference's tolerances: max |a - e| / max(|e|, 1e-3) (batched_qkv_qgemv_gpu_correctness.rs:159-181)
REF_TOL = {"f32": 5e-3, "f16": 2e-2, "bf16": 5e-2}


def _ref_rel(got, exp):
    return float(np.max(np.abs(got - exp) / np.maximum(np.abs(exp), 1e-3)))


@pytest.mark.parametrize("kernel,fixture,dt", [
    ("ffai_batched_qkv_qgemv", "batched_qkv_k256_g64_q16_kv4", "f32"), ("ffai_batched_qkv_qgemv", "batched_qkv_k512_g128_q12_kv6", "f32"),
    ("ffai_batched_qkv_qgemv", "batched_qkv_k256_g64_q16_kv4", "f16"), ("ffai_batched_qkv_qgemv", "batched_qkv_k256_g64_q16_kv4", "bf16"),
    ("ffai_batched_qkv_qgemv_fast", "batched_qkv_k512_g64_q16_kv8", "f32"), ("ffai_batched_qkv_qgemv_fast", "batched_qkv_k512_g64_q16_kv8", "f16"),
    ("ffai_batched_qkv_qgemv_fast", "batched_qkv_k512_g64_q16_kv8", "bf16"),
])
def test_batched_qkv_via_dispatch(ctx, kernel, fixture, dt):
    """The reference's own cases of the fused q / k / v decode projection under its kernel and buffer names: one
    concatenated `out` (batched_qkv_qgemv_gpu_correctness.rs:112-181,312-321)."""
    from helpers import bytes_to_f32, dt_bytes
    fx = _batched_fixture(f"{fixture}_{dt}.npz")
    in_dim, gs, (oq, ok, ov) = int(fx["meta"][0]), int(fx["meta"][1]), (int(v) for v in fx["meta"][2:])
    bufs = {"x": dt_bytes(fx["x"], dt), "out": bytes((oq + ok + ov) * (4 if dt == "f32" else 2))}
    for i, sfx in enumerate("qkv"):
        bufs[f"w_{sfx}"], bufs[f"scales_{sfx}"], bufs[f"biases_{sfx}"] = fx[f"w{i}"].tobytes(), dt_bytes(fx[f"scales{i}"], dt), dt_bytes(fx[f"biases{i}"], dt)
    consts = {"out_q": oq, "out_k": ok, "out_v": ov, "in_dim": in_dim, "group_size": gs}
    res = ctx.dispatch_with_grid(kernel, bufs, consts, (max(oq, ok, ov), 1, 3), (128, 1, 1), dtype=dt)
    got = bytes_to_f32(res.outputs["out"], dt)
    exp = oracle.round_through(np.concatenate([fx["acc0"], fx["acc1"], fx["acc2"]]), ODT[dt])
    assert np.any(got != 0.0) and got.shape == exp.shape
    assert _ref_rel(got, exp) <= REF_TOL[dt]
    assert rel_err(got, exp) <= TOL[dt]                     # and this build's own, tighter bound


@pytest.mark.parametrize("dt", ["f32", "f16", "bf16"])
def test_batched_4_via_dispatch(ctx, dt):
    """test_batched_4_qgemv_fast (crates/metaltile-std/src/ffai/batched_4_qgemv.rs:421-472): four outputs a_out .. d_out."""
    from helpers import bytes_to_f32, dt_bytes
    fx = _batched_fixture(f"test_batched_4_qgemv_fast_{dt}.npz")
    in_dim, gs, outs = int(fx["meta"][0]), int(fx["meta"][1]), [int(v) for v in fx["meta"][2:]]
    esz = 4 if dt == "f32" else 2
    bufs, consts = {"x": dt_bytes(fx["x"], dt)}, {"in_dim": in_dim, "group_size": gs}
    for i, sfx in enumerate("abcd"):
        bufs[f"w_{sfx}"], bufs[f"scales_{sfx}"], bufs[f"biases_{sfx}"] = fx[f"w{i}"].tobytes(), dt_bytes(fx[f"scales{i}"], dt), dt_bytes(fx[f"biases{i}"], dt)
        bufs[f"{sfx}_out"] = bytes(outs[i] * esz)
        consts[f"out_{sfx}"] = outs[i]
    res = ctx.dispatch_with_grid("ffai_batched_4_qgemv_fast", bufs, consts, (2, 1, 4), (64, 1, 1), dtype=dt,
                                 outputs=("a_out", "b_out", "c_out", "d_out"))
    for i, sfx in enumerate("abcd"):
        got = bytes_to_f32(res.outputs[f"{sfx}_out"], dt)
        exp = oracle.round_through(fx[f"acc{i}"], ODT[dt])
        assert np.any(got != 0.0)
        assert _ref_rel(got, exp) <= 2e-1 and rel_err(got, exp) <= TOL[dt]     # the reference's tol = 2e-1; ours


def test_batched_dispatch_refuses_missing_pieces(ctx):
    from metaltile_b200 import MetalTileError
    fx = _batched_fixture("batched_qkv_k256_g64_q16_kv4_f32.npz")
    from helpers import dt_bytes
    bufs = {"x": dt_bytes(fx["x"], "f32"), "out": bytes(24 * 4)}
    for i, sfx in enumerate("qk"):                          # v is missing
        bufs[f"w_{sfx}"], bufs[f"scales_{sfx}"], bufs[f"biases_{sfx}"] = fx[f"w{i}"].tobytes(), dt_bytes(fx[f"scales{i}"], "f32"), dt_bytes(fx[f"biases{i}"], "f32")
    with pytest.raises(MetalTileError) as ei:
        ctx.dispatch_with_grid("ffai_batched_qkv_qgemv", bufs, {"out_q": 16, "out_k": 4, "out_v": 4, "in_dim": 256, "group_size": 64})
    assert ei.value.variant == "Buffer" and "w_v" in str(ei.value)
    bufs["w_v"], bufs["scales_v"], bufs["biases_v"] = bufs["w_k"], bufs["scales_k"], bufs["biases_k"]
    bufs["out"] = bytes(23 * 4)                             # one element short
    with pytest.raises(MetalTileError) as ei:
        ctx.dispatch_with_grid("ffai_batched_qkv_qgemv", bufs, {"out_q": 16, "out_k": 4, "out_v": 4, "in_dim": 256, "group_size": 64})
    assert ei.value.variant == "BufferSize"


def test_dispatch_chain_is_the_passes_in_order(ctx):
    """Context::dispatch_chain (crates/metaltile-runtime/src/context.rs:347-395): several passes, one commit.  No two
    registered kernels of this path share an output and an input name, so nothing links here: every pass's outputs come
    back, equal to the same passes dispatched one by one."""
    from helpers import bytes_to_f32, dt_bytes
    w, s, b, x = dense_case(1, 64, 512, 4, 64, "bf16", seed=7)
    p1 = ("mt_qmv", {"w": w.tobytes(), "scales": dt_bytes(s, "bf16"), "biases": dt_bytes(b, "bf16"), "x": dt_bytes(x, "bf16"),
                     "out": bytes(64 * 2)}, {"k": 512, "gs_per_row": 8}, "bf16", ("out",))
    g = np.linspace(-3, 3, 256, dtype=np.float32)
    p2 = ("mt_swiglu", {"gate": dt_bytes(g, "f32"), "up": dt_bytes(g[::-1].copy(), "f32"), "out": bytes(256 * 4)}, {}, "f32", ("out",))
    res = ctx.dispatch_chain([p1, p2])
    one = [ctx.dispatch_with_grid(k, bufs, consts, dtype=dt, outputs=outs) for (k, bufs, consts, dt, outs) in (p1, p2)]
    assert len(res) == 2 and res[1].elapsed_us > 0.0
    for r, o in zip(res, one):
        assert r.outputs["out"] == o.outputs["out"]
    assert rel_err(bytes_to_f32(res[0].outputs["out"], "bf16").reshape(1, 64), oracle.qmm(w, s, b, x, 1, 64, 512, 4, 64)) <= TOL["bf16"]
    from metaltile_b200 import MetalTileError
    with pytest.raises(MetalTileError) as ei:               # checked before anything runs: the second pass names no kernel
        ctx.dispatch_chain([p1, ("mt_nothing", {}, {}, "f32", ())])
    assert ei.value.variant == "FunctionNotFound"
