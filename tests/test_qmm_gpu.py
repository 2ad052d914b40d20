"""Parity of the tensor-core (tcgen05) prefill qmm with the CPU oracle, through the C ABI."""
import numpy as np
import pytest

import oracle
from helpers import TOL, dense_case, rel_err, to_dev

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    from metaltile_b200 import ops
    return ops.context(0)


def run_qmm(w, s, b, x, bits, gs, dt):
    import torch
    from metaltile_b200 import ops
    out = ops.qmm(to_dev(w), to_dev(s, dt), to_dev(b, dt), to_dev(x, dt), bits, gs)
    torch.cuda.synchronize()
    return out.float().cpu().numpy()


def test_routing_follows_m_and_dtype(ctx):
    """The selector (mt_qmm_for, crates/metaltile-std/src/mlx/quantized.rs:5040-5065,5127-5199) in this back end."""
    assert ctx.qmm_route(1, 4096, 4096, 4, 64, "bf16") == "qmv_stream"
    assert ctx.qmm_route(8, 4096, 4096, 4, 128, "f16") == "qmv_mma_sync"          # the streaming kernel takes M = 1 by default
    assert ctx.qmm_route(1, 4096, 4096, 4, 64, "f32") == "qmv_cuda_core"
    assert ctx.qmm_route(1, 4096, 4096, 3, 64, "bf16") == "qmv_cuda_core"
    assert ctx.qmm_route(16, 4096, 4096, 4, 64, "bf16") == "qmv_mma_sync"
    assert ctx.qmm_route(9, 4096, 4096, 4, 128, "f16") == "qmv_mma_sync"
    assert ctx.qmm_route(2, 4096, 4160, 4, 64, "f16") == "qmv_mma_sync"           # K % 256 != 0: not the streaming kernel
    # group < 64 or other widths: no warp-level kernel; 9..16 token rows (and 5..8 on large matrices) take the
    # tensor-memory kernel with K slices, fewer stay on CUDA cores
    assert ctx.qmm_route(16, 4096, 4096, 4, 32, "bf16") == "qmm_tcgen05"
    assert ctx.qmm_route(16, 4096, 4096, 8, 64, "bf16") == "qmm_tcgen05"
    assert ctx.qmm_route(8, 4096, 4096, 8, 64, "bf16") == "qmv_cuda_core"
    assert ctx.qmm_route(8, 8192, 8192, 3, 64, "f16") == "qmm_tcgen05"
    assert ctx.qmm_route(4, 8192, 8192, 8, 64, "bf16") == "qmv_cuda_core"
    assert ctx.qmm_route(16, 512, 512, 8, 64, "bf16") == "qmv_cuda_core"          # too small to pay three launches
    assert ctx.qmm_route(16, 4096, 4096, 4, 64, "f32") == "qmv_cuda_core"
    assert ctx.qmm_route(17, 4096, 4096, 4, 64, "bf16") == "qmv_mma_sync"      # few rows: 16-row chunks of the small-M kernel
    assert ctx.qmm_route(32, 4096, 4096, 4, 64, "bf16") == "qmv_mma_sync"
    assert ctx.qmm_route(64, 4096, 4096, 4, 64, "bf16") == "qmm_tcgen05"       # 32 weight tiles x 4 K slices fill the SMs
    assert ctx.qmm_route(64, 14336, 4096, 4, 64, "bf16") == "qmm_tcgen05"
    assert ctx.qmm_route(65, 4096, 4096, 4, 64, "bf16") == "qmm_tcgen05"
    assert ctx.qmm_route(17, 4096, 4096, 8, 64, "bf16") == "qmm_tcgen05"
    assert ctx.qmm_route(2048, 14336, 4096, 4, 64, "f16") == "qmm_tcgen05"
    assert ctx.qmm_route(2048, 14336, 4096, 4, 64, "f32") == "qmv_cuda_core"      # no f32 MMA: stays exact
    assert ctx.qmm_route(64, 256, 96, 4, 32, "bf16") == "qmv_cuda_core"           # K % 64 != 0
    assert ctx.qmm_route(64, 256, 512, 7, 64, "bf16") == "qmv_cuda_core"


@pytest.mark.parametrize("m,n,k,bits,gs,dt", [
    (32, 64, 512, 4, 64, "bf16"), (32, 64, 512, 4, 64, "f16"),      # registered mma shape
    (17, 8, 128, 4, 64, "bf16"),                                   # smallest: two k blocks, N < 128
    (128, 256, 512, 4, 64, "bf16"),
    (200, 304, 1024, 4, 64, "bf16"),                               # ragged M and N
    (257, 129, 256, 4, 32, "f16"),                                 # two token chunks, group 32
    (300, 512, 2048, 4, 128, "bf16"),                              # group 128
    (64, 96, 256, 8, 32, "f16"),
    (130, 288, 512, 2, 64, "bf16"), (130, 288, 512, 3, 64, "bf16"), (130, 288, 512, 5, 64, "f16"),
    (130, 288, 512, 6, 128, "bf16"), (130, 288, 512, 8, 64, "bf16"),
    (1000, 200, 4096, 4, 64, "bf16"),                              # long K: many ring wraps
])
def test_qmm_matches_oracle(ctx, m, n, k, bits, gs, dt):
    """Every shape on the tcgen05 kernel (the chunked small-M route of few-row shapes is switched off here and has
    its own test below)."""
    assert ctx.qmm_route(m, n, k, bits, gs, dt) in ("qmm_tcgen05", "qmv_mma_sync")
    w, s, b, x = dense_case(m, n, k, bits, gs, dt, seed=0, salt=m + n)
    ref = oracle.qmm(w, s, b, x, m, n, k, bits, gs)
    ctx.set_option("qmm_mma_chunks", 0)
    try:
        got = run_qmm(w, s, b, x, bits, gs, dt)
    finally:
        ctx.set_option("qmm_mma_chunks", 1)
    assert got.shape == (m, n)
    assert rel_err(got, ref) <= TOL[dt]
    assert ctx.status_word() == 0


@pytest.mark.parametrize("m,n,k,gs,dt", [(17, 4096, 4096, 64, "bf16"), (32, 1000, 512, 128, "f16"), (50, 2048, 2048, 64, "bf16"),
                                         (64, 272, 1024, 64, "f16")])
def test_few_rows_run_as_chunks_of_the_small_m_kernel(ctx, m, n, k, gs, dt):
    """17 <= M <= 32 (up to 64 when the tcgen05 kernel may not cut K into slices) on a matrix too small to fill the GPU
    with 128-row tiles: 16-row chunks of the tensor-core qmv; same oracle, and within round-off of the tcgen05 kernel."""
    assert ctx.qmm_route(m, n, k, 4, gs, dt) == ("qmv_mma_sync" if m <= 32 else "qmm_tcgen05")
    w, s, b, x = dense_case(m, n, k, 4, gs, dt, seed=16, salt=m)
    ref = oracle.qmm(w, s, b, x, m, n, k, 4, gs)
    ctx.set_option("qmm_ksplit", 1 if m <= 32 else 0)
    try:
        got = run_qmm(w, s, b, x, 4, gs, dt)
    finally:
        ctx.set_option("qmm_ksplit", 1)
    assert got.shape == (m, n)
    assert rel_err(got, ref) <= TOL[dt]
    ctx.set_option("qmm_mma_chunks", 0)
    try:
        tc = run_qmm(w, s, b, x, 4, gs, dt)
    finally:
        ctx.set_option("qmm_mma_chunks", 1)
    assert rel_err(got, tc) <= TOL[dt]


def test_exact_integer_case(ctx):
    """Scales 1, biases 0, one-hot activations: every output is one integer code, so the result is exact."""
    import torch
    from metaltile_b200 import ops, synth
    m, n, k, bits = 256, 384, 256, 4
    w = synth.words(n * k * bits // 32, seed=11).reshape(n, -1)
    codes = oracle.unpack_matrix(w, k, bits)
    x = np.zeros((m, k), np.float32)
    x[np.arange(m), (np.arange(m) * 7) % k] = 1.0
    ones, zeros = np.ones((n, k // 64), np.float32), np.zeros((n, k // 64), np.float32)
    out = ops.qmm(to_dev(w), to_dev(ones, "bf16"), to_dev(zeros, "bf16"), to_dev(x, "bf16"), bits, 64)
    torch.cuda.synchronize()
    assert np.array_equal(out.float().cpu().numpy(), codes[:, (np.arange(m) * 7) % k].T.astype(np.float32))


@pytest.mark.parametrize("n,k", [(14336, 4096), (4096, 14336)])
def test_prefill_2048_on_a_slice(ctx, n, k):
    """The prefill benchmark shapes; the oracle checks a slice of the weight rows (the CPU needs
    ~1 s per 64 rows at M = 2048), the rest is covered by the linearity property below."""
    m, bits, gs, dt = 2048, 4, 64, "bf16"
    w, s, b, x = dense_case(m, n, k, bits, gs, dt, seed=0, salt=3)
    got = run_qmm(w, s, b, x, bits, gs, dt)
    for rows in ((0, 128), (n // 2 - 64, n // 2 + 64), (n - 128, n)):          # first, middle and last weight-row tile
        ref = oracle.qmm(w, s, b, x, m, n, k, bits, gs, rows=rows)
        assert rel_err(got[:, rows[0]:rows[1]], ref[:, rows[0]:rows[1]]) <= TOL[dt], rows
    # 4096 random (token, weight row) points anywhere in the output
    rng = np.random.default_rng(n)
    worst = 0.0
    for mi, ni in zip(rng.integers(0, m, 4096), rng.integers(0, n, 4096)):
        ref1 = oracle.qmm(w[ni:ni + 1], s[ni:ni + 1], b[ni:ni + 1], x[mi:mi + 1], 1, 1, k, bits, gs)[0, 0]
        worst = max(worst, abs(float(got[mi, ni]) - float(ref1)) / max(abs(float(ref1)), 1.0))
    assert worst <= TOL[dt]
    assert np.all(np.isfinite(got))
    assert ctx.status_word() == 0


def test_linearity_and_row_independence_at_full_size(ctx):
    """Size-independent properties at M = 2048, N = 14336, K = 4096: rows of x do not interact, and the
    same row gives the same result wherever it sits in the batch (bit for bit)."""
    import torch
    from metaltile_b200 import ops
    m, n, k, bits, gs, dt = 2048, 14336, 4096, 4, 64, "bf16"
    w, s, b, x = dense_case(m, n, k, bits, gs, dt, seed=0, salt=5)
    wd, sd, bd = to_dev(w), to_dev(s, dt), to_dev(b, dt)
    full = ops.qmm(wd, sd, bd, to_dev(x, dt), bits, gs)
    perm = np.random.default_rng(0).permutation(m)
    shuf = ops.qmm(wd, sd, bd, to_dev(x[perm], dt), bits, gs)
    torch.cuda.synchronize()
    assert torch.equal(shuf, full[torch.from_numpy(perm).cuda()])
    # and the decode kernel agrees with the prefill kernel on a few rows
    few = ops.qmv(wd, sd, bd, to_dev(x[:4], dt), bits, gs)
    torch.cuda.synchronize()
    assert rel_err(full[:4].float().cpu().numpy(), few.float().cpu().numpy()) <= TOL[dt]


@pytest.mark.parametrize("bits,dt", [(4, "f16"), (8, "bf16")])
def test_tiny_and_mixed_scales(ctx, bits, dt):
    """4- and 8-bit codes are dequantised in packed-half arithmetic only when the scale is a normal f16 number;
    groups with scales below 2^-14 (here 1e-7 .. 1e-5, mixed with ordinary ones) take the f32 path."""
    m, n, k, gs = 96, 160, 512, 64
    w, s, b, x = dense_case(m, n, k, bits, gs, dt, seed=12, salt=bits)
    rng = np.random.default_rng(12)
    tiny = rng.random(s.shape) < 0.5
    s = np.where(tiny, (10.0 ** rng.uniform(-7, -5, s.shape)), s).astype(np.float32)
    s = oracle.round_through(s, oracle.BF16 if dt == "bf16" else oracle.F16)
    ref = oracle.qmm(w, s, b, x, m, n, k, bits, gs)
    got = run_qmm(w, s, b, x, bits, gs, dt)
    assert rel_err(got, ref) <= TOL[dt]
    assert ctx.status_word() == 0


@pytest.mark.parametrize("m,n,k,bits,gs", [(300, 304, 1024, 4, 64), (130, 288, 768, 3, 32), (64, 200, 512, 8, 128)])
def test_loader_and_wait_options_do_not_change_results(ctx, m, n, k, bits, gs):
    """The packed words reach the dequant warps through shared-memory staging buffers or straight from global
    memory, and the waits poll with or without a suspend-time hint: same arithmetic, bit-identical output."""
    import torch
    from metaltile_b200 import ops
    dt = "bf16"
    w, s, b, x = dense_case(m, n, k, bits, gs, dt, seed=13, salt=k)
    args = (to_dev(w), to_dev(s, dt), to_dev(b, dt), to_dev(x, dt), bits, gs)
    base = ops.qmm(*args)
    outs = []
    try:
        for name, value in (("qmm_raw", 0), ("qmm_wait_hint_ns", 0), ("qmm_max_stages", 2)):
            ctx.set_option(name, value)
            outs.append(ops.qmm(*args))
            ctx.set_option(name, {"qmm_raw": 1, "qmm_wait_hint_ns": 5000, "qmm_max_stages": 0}[name])
    finally:
        ctx.set_option("qmm_raw", 1)
        ctx.set_option("qmm_wait_hint_ns", 5000)
        ctx.set_option("qmm_max_stages", 0)
    torch.cuda.synchronize()
    for o in outs:
        assert torch.equal(o, base)
    ref = oracle.qmm(w, s, b, x, m, n, k, bits, gs)
    assert rel_err(base.float().cpu().numpy(), ref) <= TOL[dt]
    assert ctx.status_word() == 0


def test_k_not_a_multiple_of_256(ctx):
    """K = 320: no whole raw super-block, so the dequant warps load straight from global memory."""
    m, n, k, bits, gs, dt = 100, 136, 320, 4, 64, "f16"
    w, s, b, x = dense_case(m, n, k, bits, gs, dt, seed=14)
    ref = oracle.qmm(w, s, b, x, m, n, k, bits, gs)
    assert rel_err(run_qmm(w, s, b, x, bits, gs, dt), ref) <= TOL[dt]


@pytest.mark.parametrize("m,n,k,bits,gs,dt", [
    (257, 300, 512, 4, 64, "bf16"),        # second token chunk holds one row
    (512, 136, 768, 4, 64, "f16"),         # exactly two full chunks
    (700, 520, 512, 8, 128, "bf16"),       # a wide item and a 188-row single-chunk item per weight tile
    (1300, 129, 1024, 3, 32, "bf16"),      # three items per tile, ragged rows in the last chunk and in the last tile
    (512, 19200, 256, 4, 64, "bf16"),      # 150 wide units on 148 SMs: the two left over run as four single-chunk items
    (1024, 9600, 256, 4, 64, "f16"),       # the same with two units per weight tile
])
def test_wide_items_equal_single_chunk_items(ctx, m, n, k, bits, gs, dt):
    """"qmm_wide": a dense work item covers two 256-row token chunks that share every dequantised weight
    stage.  Every output is the same sum in the same order as with one chunk per item: bit-identical."""
    import torch
    from metaltile_b200 import ops
    w, s, b, x = dense_case(m, n, k, bits, gs, dt, seed=21, salt=m)
    args = (to_dev(w), to_dev(s, dt), to_dev(b, dt), to_dev(x, dt), bits, gs)
    ctx.set_option("qmm_wide", 2)              # whenever the shape allows (the default takes them only when they save rounds)
    try:
        wide = ops.qmm(*args)
        again = ops.qmm(*args)
        ctx.set_option("qmm_wide", 0)
        single = ops.qmm(*args)
        torch.cuda.synchronize()
    finally:
        ctx.set_option("qmm_wide", 1)
    assert ctx.status_word() == 0
    assert torch.equal(wide, single) and torch.equal(wide, again)
    for (r0, r1) in ((0, 64), (m - 40, m)):                  # the oracle on the first and the last rows
        ref = oracle.qmm(w, s, b, x[r0:r1], r1 - r0, n, k, bits, gs)
        assert rel_err(wide[r0:r1].float().cpu().numpy(), ref) <= TOL[dt]


def test_qmm_multi_writes_column_blocks_of_wider_matrices(ctx):
    """mtc_qmm_multi: the [M, N] result lands as a column block (row stride ld) in every destination - the form the
    sharded prefill uses to gather through peer stores.  Same values as mtc_qmm, nothing outside the block is touched."""
    import torch
    from metaltile_b200 import MetalTileError
    from metaltile_b200.ops import _TORCH_DT
    m, n, k, bits, gs, dt = 300, 200, 512, 4, 64, "bf16"
    w, s, b, x = dense_case(m, n, k, bits, gs, dt, seed=23)
    wd, sd, bd, xd = to_dev(w), to_dev(s, dt), to_dev(b, dt), to_dev(x, dt)
    from metaltile_b200 import ops
    ref = ops.qmm(wd, sd, bd, xd, bits, gs, ctx=ctx)
    ld, col0 = 520, 136
    dests = [torch.full((m, ld), 7.0, dtype=torch.bfloat16, device="cuda") for _ in range(3)]
    st = torch.cuda.current_stream().cuda_stream
    ctx.qmm_multi(wd.data_ptr(), sd.data_ptr(), bd.data_ptr(), xd.data_ptr(), [d.data_ptr() + col0 * 2 for d in dests], ld, m, n, k,
                  bits, gs, _TORCH_DT[xd.dtype], stream=st)
    torch.cuda.synchronize()
    assert ctx.status_word() == 0
    for d in dests:
        assert torch.equal(d[:, col0:col0 + n], ref)
        assert bool((d[:, :col0] == 7.0).all()) and bool((d[:, col0 + n:] == 7.0).all())
    with pytest.raises(MetalTileError) as ei:               # a row stride narrower than the block
        ctx.qmm_multi(wd.data_ptr(), sd.data_ptr(), bd.data_ptr(), xd.data_ptr(), [dests[0].data_ptr()], n - 1, m, n, k, bits, gs,
                      _TORCH_DT[xd.dtype], stream=st)
    assert ei.value.variant == "Invalid"
    with pytest.raises(MetalTileError) as ei:               # M <= 16 belongs to the decode kernels
        ctx.qmm_multi(wd.data_ptr(), sd.data_ptr(), bd.data_ptr(), xd.data_ptr(), [dests[0].data_ptr()], ld, 8, n, k, bits, gs,
                      _TORCH_DT[xd.dtype], stream=st)
    assert ei.value.variant == "Unsupported"


@pytest.mark.parametrize("m,n,k,bits,gs,dt", [
    (16, 4096, 4096, 8, 64, "bf16"), (9, 2048, 2048, 3, 32, "f16"), (12, 1024, 4096, 6, 128, "bf16"), (16, 2048, 2048, 2, 64, "bf16"),
    (40, 4096, 4096, 8, 64, "bf16"), (200, 1024, 8192, 5, 64, "f16"), (256, 640, 2048, 4, 32, "bf16"), (130, 288, 512, 6, 128, "bf16"),
    (24, 1000, 1344, 8, 64, "f16"),                                # 21 k blocks, K % 256 != 0: three slices of 7 on the direct loader
    (24, 1000, 1280, 8, 64, "f16"),                                # 20 k blocks: five slices of one super-block each
])
def test_k_slices_match_oracle_and_the_unsliced_kernel(ctx, m, n, k, bits, gs, dt):
    """Few weight-row tiles and one token chunk: K is cut into slices that run as work items of their own, f32 partial
    sums added in slice order by a second kernel.  Checked against the oracle and against the same kernel without slices
    (option `qmm_ksplit` 0); M <= 16 reaches the kernel through mtc_qmv (option `qmv_small_m_tc`)."""
    import torch
    from metaltile_b200 import ops
    w, s, b, x = dense_case(m, n, k, bits, gs, dt, seed=6, salt=m + n)
    band = (n // 2, min(n, n // 2 + 64))
    ref = oracle.qmm(w, s, b, x, m, n, k, bits, gs, rows=band)[:, band[0]:band[1]]
    dev = [to_dev(w), to_dev(s, dt), to_dev(b, dt), to_dev(x, dt)]
    outs = {}
    for ks in (1, 0):
        ctx.set_option("qmm_ksplit", ks)
        ctx.set_option("qmv_small_m_tc", 2)
        ctx.set_option("qmm_mma_chunks", 0)
        try:
            got = (ops.qmv if m <= 16 else ops.qmm)(*dev, bits, gs, ctx=ctx)
            torch.cuda.synchronize()
        finally:
            ctx.set_option("qmm_ksplit", 1)
            ctx.set_option("qmv_small_m_tc", 1)
            ctx.set_option("qmm_mma_chunks", 1)
        outs[ks] = got.float().cpu().numpy()
        assert ctx.status_word() == 0
        assert rel_err(outs[ks][:, band[0]:band[1]], ref) <= TOL[dt], ks
    # the same products, summed per slice first: equal up to the rounding of the output type
    assert rel_err(outs[1], outs[0]) <= (2.0 ** -7 if dt == "bf16" else 2.0 ** -10)


def test_small_m_default_route_is_within_tolerance(ctx):
    """M = 16, 8-bit: the default route (tensor-memory kernel) through mtc_qmv against the oracle."""
    import torch
    from metaltile_b200 import ops
    m, n, k = 16, 2048, 4096
    assert ctx.qmm_route(m, n, k, 8, 64, "bf16") == "qmm_tcgen05"
    w, s, b, x = dense_case(m, n, k, 8, 64, "bf16", seed=8)
    got = ops.qmv(to_dev(w), to_dev(s, "bf16"), to_dev(b, "bf16"), to_dev(x, "bf16"), 8, 64, ctx=ctx)
    torch.cuda.synchronize()
    ref = oracle.qmm(w, s, b, x, m, n, k, 8, 64, rows=(512, 576))[:, 512:576]
    assert rel_err(got.float().cpu().numpy()[:, 512:576], ref) <= TOL["bf16"] and ctx.status_word() == 0


def test_k_slices_replay_from_a_cuda_graph(ctx):
    """A launch that cuts K into slices (product kernel + sum kernel, linked by programmatic dependent launch) captured
    in a CUDA graph after one eager run: every replay gives the eager result."""
    import torch
    from metaltile_b200 import ops
    m, n, k, bits, gs, dt = 48, 1024, 4096, 8, 64, "bf16"
    w, s, b, x = dense_case(m, n, k, bits, gs, dt, seed=12)
    dev = [to_dev(w), to_dev(s, dt), to_dev(b, dt), to_dev(x, dt)]
    eager = ops.qmm(*dev, bits, gs, ctx=ctx).clone()
    torch.cuda.synchronize()
    out = torch.zeros_like(eager)
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            ops.qmm(*dev, bits, gs, out=out, ctx=ctx)
    for _ in range(3):
        out.zero_()
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(out, eager)
    assert ctx.status_word() == 0


def test_small_m_capture_without_a_first_run_falls_back_to_cuda_cores():
    """M = 16, 8-bit captured on a fresh context: the tensor-memory route would have to grow a scratch block during
    capture, so mtc_qmv takes the CUDA-core kernel for that call instead of failing; the replay matches the oracle."""
    import torch
    from metaltile_b200 import Context
    from metaltile_b200.ops import _TORCH_DT
    fresh = Context(0)
    m, n, k, bits, gs, dt = 16, 1024, 2048, 8, 64, "bf16"
    w, s, b, x = dense_case(m, n, k, bits, gs, dt, seed=13)
    wd, sd, bd, xd = to_dev(w), to_dev(s, dt), to_dev(b, dt), to_dev(x, dt)
    out = torch.zeros((m, n), dtype=torch.bfloat16, device="cuda")
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            fresh.qmv(wd.data_ptr(), sd.data_ptr(), bd.data_ptr(), xd.data_ptr(), out.data_ptr(), m, n, k, bits, gs,
                      _TORCH_DT[xd.dtype], stream=torch.cuda.current_stream().cuda_stream)
    graph.replay()
    torch.cuda.synchronize()
    ref = oracle.qmm(w, s, b, x, m, n, k, bits, gs)
    assert rel_err(out.float().cpu().numpy(), ref) <= TOL[dt] and fresh.status_word() == 0
