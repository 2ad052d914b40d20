"""Runtime behaviour of the C ABI on a GPU: a bounded device-side wait that really runs out and reaches the caller as
Timeout, the host deadline of mtc_sync_deadline, and one context per device in one process."""
import numpy as np
import pytest

import oracle
from helpers import ODT, TOL, dense_case, rel_err, to_dev

pytestmark = pytest.mark.gpu


def test_a_bounded_wait_expires_and_reaches_the_caller():
    """A peer barrier for two ranks whose second rank never arrives (its flag array is a local buffer nobody writes):
    with a poll limit of a few thousand the kernel gives up, records 0x601 + the missing rank and returns; the next
    synchronising call reports Timeout; after mtc_status_clear the context works as before.  Nothing faults or spins
    without a bound."""
    import torch
    from metaltile_b200 import MetalTileError, ops
    ctx = ops.context(0)
    assert ctx.status_word() == 0
    mine = torch.zeros(64, dtype=torch.int32, device="cuda")       # 8 flag words, the epoch counter at byte 128
    absent = torch.zeros(64, dtype=torch.int32, device="cuda")     # "rank 1": never written by anybody
    st = torch.cuda.current_stream().cuda_stream
    ctx.set_option("peer_poll_limit", 4000)
    try:
        ctx.peer_barrier([mine.data_ptr(), absent.data_ptr()], 0, mine.data_ptr(), mine.data_ptr() + 128, stream=st)
        with pytest.raises(MetalTileError) as ei:
            ctx.sync(st)
        assert ei.value.variant == "Timeout" and "0x602" in str(ei.value)
        assert ctx.status_word() == 0x602
        # the name-keyed dispatch reports it too, instead of returning whatever the buffers hold
        w, s, b, x = dense_case(1, 8, 64, 4, 64, "f32")
        bufs = {"w": w.tobytes(), "scales": s.tobytes(), "biases": b.tobytes(), "x": x.tobytes(), "out": bytes(32)}
        with pytest.raises(MetalTileError) as ei:
            ctx.dispatch_with_grid("mt_qmm", bufs, {"k": 64, "n": 8, "gs_per_row": 1})
        assert ei.value.variant == "Timeout"
    finally:
        ctx.set_option("peer_poll_limit", 1 << 22)
        ctx.status_clear()
    assert ctx.status_word() == 0
    ctx.sync(st)
    res = ctx.dispatch_with_grid("mt_qmm", bufs, {"k": 64, "n": 8, "gs_per_row": 1})
    ref = oracle.qmm(w, s, b, x, 1, 8, 64, 4, 64)
    assert rel_err(np.frombuffer(res.outputs["out"], dtype=np.float32).reshape(1, 8), ref) <= TOL["f32"]


def test_sync_deadline():
    """mtc_sync_deadline returns when the stream is done (well inside the deadline here); a deadline of 0 ms on a
    stream with queued work either finds it finished or reports Timeout while the work carries on."""
    import torch
    from metaltile_b200 import MetalTileError, ops
    ctx = ops.context(0)
    st = torch.cuda.current_stream().cuda_stream
    w, s, b, x = dense_case(1, 8192, 8192, 4, 64, "bf16", seed=1)
    args = (to_dev(w), to_dev(s, "bf16"), to_dev(b, "bf16"), to_dev(x, "bf16"), 4, 64)
    out = ops.qmv(*args, ctx=ctx)
    ctx.sync(st, timeout_ms=10000)
    for _ in range(200):
        out = ops.qmv(*args, out=out, ctx=ctx)
    try:
        ctx.sync(st, timeout_ms=0)
    except MetalTileError as e:
        assert e.variant == "Timeout" and "did not finish" in str(e)
    ctx.sync(st)
    assert ctx.status_word() == 0


def test_one_context_per_device():
    """Contexts on two devices in one process: qmv, qmm and gather_qmm on both (per-device kernel attributes, every
    entry makes its context's device current)."""
    import torch
    from metaltile_b200 import ops
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two devices")
    w, s, b, x = dense_case(40, 256, 512, 4, 64, "bf16", seed=3)
    ref = oracle.qmm(w, s, b, x, 40, 256, 512, 4, 64)
    off = np.array([0, 25, 40], dtype=np.uint32)
    gw, gs_, gb = (np.stack([a, a]) for a in (w, s, b))          # two experts with the same matrix
    for d in (1, 0, 1):
        dev = torch.device("cuda", d)
        ctx = ops.context(dev)
        with torch.cuda.device(dev):
            td = lambda a, dt=None: to_dev(a, dt).to(dev)
            one = ops.qmv(td(w), td(s, "bf16"), td(b, "bf16"), td(x[:1], "bf16"), 4, 64, ctx=ctx)
            full = ops.qmm(td(w), td(s, "bf16"), td(b, "bf16"), td(x, "bf16"), 4, 64, ctx=ctx)
            gat = ops.gather_qmm(td(x, "bf16"), td(gw), td(gs_, "bf16"), td(gb, "bf16"), 4, 64, expert_offsets=td(off), ctx=ctx)
            torch.cuda.synchronize(dev)
            assert rel_err(one.float().cpu().numpy(), ref[:1]) <= TOL["bf16"]
            assert rel_err(full.float().cpu().numpy(), ref) <= TOL["bf16"]
            assert rel_err(gat.float().cpu().numpy(), ref) <= TOL["bf16"]
            assert ctx.status_word() == 0


def _sync_case(n=1024, k=4096):
    from metaltile_b200 import synth
    x = oracle.round_through(synth.activations(1, k, seed=5), ODT["bf16"])
    w, s, b, _ = dense_case(1, n, k, 4, 64, "bf16", seed=5, salt=3)
    return w, s, b, x


def test_hand_off_inside_the_decode_kernel_single_rank():
    """mtc_qmv_batched_sync with one rank: every launch waits for the epoch its predecessor published (already there),
    publishes the next one and leaves the CTA ticket at zero; results are those of mtc_qmv_batched, in two destinations."""
    import torch
    from metaltile_b200 import ops
    ctx = ops.context(0)
    n, k = 1024, 4096
    w, s, b, x = _sync_case(n, k)
    wd, sd, bd, xd = to_dev(w), to_dev(s, "bf16"), to_dev(b, "bf16"), to_dev(x, "bf16")
    flags = torch.zeros(64, dtype=torch.int32, device="cuda")      # flag words, epoch at byte 128, ticket at byte 192
    outs = [torch.zeros((1, n), dtype=torch.bfloat16, device="cuda") for _ in range(2)]
    desc = dict(w=wd.data_ptr(), scales=sd.data_ptr(), biases=bd.data_ptr(), x=xd.data_ptr(), outs=[o.data_ptr() for o in outs],
                M=1, N=n, K=k, bits=4, group_size=64, dtype="bf16")
    st = torch.cuda.current_stream().cuda_stream
    f = flags.data_ptr()
    for _ in range(3):
        ctx.qmv_batched_sync([desc], [f], 0, f, f + 128, f + 192, stream=st)
    ctx.sync(st)
    assert ctx.status_word() == 0
    host = flags.cpu()
    assert host[0].item() == 3 and host[32].item() == 3 and host[48].item() == 0
    ref = ops.qmv(wd, sd, bd, xd, 4, 64, ctx=ctx)
    assert torch.equal(outs[0], ref) and torch.equal(outs[1], ref)
    assert rel_err(ref.float().cpu().numpy(), oracle.qmm(w, s, b, x, 1, n, k, 4, 64)) <= TOL["bf16"]


def test_hand_off_wait_for_an_absent_rank_expires():
    """Two ranks of which the second never publishes (its flag array is a local buffer nobody writes): the first launch
    passes (epoch 0), the second waits for epoch 1 of rank 1, gives up after the poll limit, records 0x602 and still
    finishes its own product; the caller gets Timeout."""
    import torch
    from metaltile_b200 import MetalTileError, ops
    ctx = ops.context(0)
    n, k = 1024, 4096
    w, s, b, x = _sync_case(n, k)
    wd, sd, bd, xd = to_dev(w), to_dev(s, "bf16"), to_dev(b, "bf16"), to_dev(x, "bf16")
    mine = torch.zeros(64, dtype=torch.int32, device="cuda")
    absent = torch.zeros(64, dtype=torch.int32, device="cuda")
    out = torch.zeros((1, n), dtype=torch.bfloat16, device="cuda")
    desc = dict(w=wd.data_ptr(), scales=sd.data_ptr(), biases=bd.data_ptr(), x=xd.data_ptr(), outs=[out.data_ptr()],
                M=1, N=n, K=k, bits=4, group_size=64, dtype="bf16")
    st = torch.cuda.current_stream().cuda_stream
    f = mine.data_ptr()
    ctx.set_option("peer_poll_limit", 2000)
    try:
        ctx.qmv_batched_sync([desc], [f, absent.data_ptr()], 0, f, f + 128, f + 192, stream=st)
        ctx.sync(st)                                   # epoch 0: nothing to wait for
        assert ctx.status_word() == 0
        ctx.qmv_batched_sync([desc], [f, absent.data_ptr()], 0, f, f + 128, f + 192, stream=st)
        with pytest.raises(MetalTileError) as ei:
            ctx.sync(st)
        assert ei.value.variant == "Timeout" and "0x602" in str(ei.value)
    finally:
        ctx.set_option("peer_poll_limit", 1 << 22)
        ctx.status_clear()
    assert torch.equal(out, ops.qmv(wd, sd, bd, xd, 4, 64, ctx=ctx))
    with pytest.raises(MetalTileError) as ei:          # a shape outside the streaming kernel's contract is refused
        bad = dict(desc, group_size=32)
        ctx.qmv_batched_sync([bad], [f], 0, f, f + 128, f + 192, stream=st)
    assert ei.value.variant in ("Unsupported", "Invalid")


# ---- mtc_measure: GpuRunner::measure / bench / bench_gbps (crates/metaltile-std/src/runner.rs:413-442,638-650) ----
def _measure_case(dt="bf16", n=2048, k=2048, gs=64):
    from helpers import dt_bytes
    w, s, b, x = dense_case(1, n, k, 4, gs, dt, seed=11)
    bufs = {"w": w.tobytes(), "scales": dt_bytes(s, dt), "biases": dt_bytes(b, dt), "x": dt_bytes(x, dt),
            "out": bytes(n * (4 if dt == "f32" else 2))}
    return bufs, {"k": k, "gs_per_row": k // gs}, (w, s, b, x)


@pytest.mark.parametrize("cold", [False, True])
def test_measure_matches_dispatch_and_summarises_like_the_reference(cold):
    from helpers import bytes_to_f32
    from metaltile_b200 import ops
    ctx = ops.context(0)
    bufs, consts, (w, s, b, x) = _measure_case()
    one = ctx.dispatch_with_grid("mt_qmv", bufs, consts, (256, 1, 1), (64, 1, 1), dtype="bf16")
    stats, samples, outs = ctx.bench("mt_qmv", bufs, consts, dtype="bf16", warmup=3, iters=21, cold_l2=cold)
    assert outs["out"] == one.outputs["out"]                       # the last timed launch computed the same bytes
    ref = oracle.qmm(w, s, b, x, 1, 2048, 2048, 4, 64)
    assert rel_err(bytes_to_f32(outs["out"], "bf16").reshape(1, -1), ref) <= TOL["bf16"]
    assert len(samples) == 21 and all(v > 0.0 for v in samples)
    srt = sorted(samples)                                          # BenchStats::from_samples, stats.rs:24-47
    mean = sum(srt) / 21
    std = (sum((v - mean) ** 2 for v in srt) / 21) ** 0.5
    assert stats.min_us == srt[0] and stats.median_us == srt[10] and stats.p95_us == srt[19] and stats.p99_us == srt[20]
    assert abs(stats.mean_us - mean) <= 1e-9 * mean and abs(stats.stddev_us - std) <= 1e-6 * max(std, 1e-9) + 1e-12
    assert abs(stats.cv_pct - std / mean * 100.0) <= 1e-6
    assert stats.is_valid() and ctx.status_word() == 0


def test_measure_gbps_and_errors():
    from metaltile_b200 import MetalTileError, ops
    ctx = ops.context(0)
    bufs, consts, _ = _measure_case("f32", n=1024, k=1024)
    nbytes = 1024 * 1024 // 2 + 2 * 1024 * 16 * 4 + 1024 * 4 + 1024 * 4
    gbps, stats = ctx.bench_gbps("mt_qmv", bufs, nbytes, fn_consts=consts, dtype="f32", warmup=2, iters=5)
    assert gbps is not None and gbps > 0.0 and abs(gbps - nbytes / (stats.min_us * 1e-6) / 1e9) <= 1e-6 * gbps
    with pytest.raises(MetalTileError) as ei:
        ctx.bench("mt_no_such_kernel", bufs, consts, dtype="f32", warmup=0, iters=1)
    assert ei.value.variant == "FunctionNotFound"
    with pytest.raises(MetalTileError) as ei:
        ctx.bench("mt_qmv", bufs, consts, dtype="f32", warmup=0, iters=0)
    assert ei.value.variant == "Invalid"
    short = dict(bufs, w=bufs["w"][:-4])
    with pytest.raises(MetalTileError) as ei:
        ctx.bench("mt_qmv", short, consts, dtype="f32", warmup=0, iters=1)
    assert ei.value.variant == "BufferSize"
    stats, samples, _ = ctx.bench("mt_qmv", bufs, consts, dtype="f32", warmup=0, iters=1, cold_l2=False)
    assert len(samples) == 1 and stats.min_us == stats.p99_us == samples[0]
