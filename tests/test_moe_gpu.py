"""Parity of the MoE kernels (router top-k, sort, permute, unpermute, SwiGLU, gather_qmm) with the CPU oracle."""
import os

import numpy as np
import pytest

import oracle
from helpers import DT_NAMES, ODT, TOL, bytes_to_f32, dt_bytes, rel_err, to_dev

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


@pytest.fixture(scope="module")
def ctx():
    from metaltile_b200 import ops
    return ops.context(0)


@pytest.fixture(scope="module")
def moe():
    return dict(np.load(os.path.join(GOLDEN, "moe_and_layout.npz")))


def _topk(logits, k, norm=1, dt="f32"):
    import torch
    from metaltile_b200 import ops
    idx, w = ops.moe_router_topk(to_dev(logits, dt), k, norm)
    torch.cuda.synchronize()
    return idx.cpu().numpy().astype(np.uint32), w.float().cpu().numpy()


def test_router_topk_reference_cases(moe):
    """crates/metaltile-std/tests/moe_gpu_correctness.rs:96-134,288-335,441-470: indices exact, weights 1e-5."""
    idx, w = _topk(moe["topk_base_logits"], 4)
    assert np.array_equal(idx, moe["topk_base_idx"])
    assert np.max(np.abs(w - moe["topk_base_w"])) < 1e-5
    idx, w = _topk(moe["topk_k1_logits"], 1)
    assert np.array_equal(idx, moe["topk_k1_idx"]) and np.all(np.abs(w - 1.0) < 1e-6)
    idx, _ = _topk(moe["topk_tie_logits"], 2)
    assert idx.tolist() == [[2, 5]]
    idx, w = _topk(moe["topk_next_logits"], 4, norm=0)
    assert np.array_equal(idx, moe["topk_next_idx"])
    assert np.max(np.abs(w - moe["topk_next_w"])) < 1e-5 and np.all(w.sum(axis=1) < 1.0)


def test_router_topk_nan_inf(moe):
    """moe_gpu_correctness.rs:524-597."""
    idx, _ = _topk(moe["topk_naninf_logits"], 4)
    assert np.array_equal(idx, moe["topk_naninf_idx"])
    for r in range(4):
        assert len(set(idx[r].tolist())) == 4
    assert idx[1, 0] == 7 and idx[3, 0] == 11
    assert 3 not in idx[2] and 5 not in idx[0] and 2 not in idx[3]


@pytest.mark.parametrize("dt", DT_NAMES)
def test_router_topk_config4(dt):
    """512 tokens, 128 experts, top-8; logits rounded through dt so ties do occur for 16-bit types."""
    from metaltile_b200 import synth
    logits = oracle.round_through(synth.router_logits(512, 128, seed=0), ODT[dt])
    ref_idx, ref_w = oracle.router_topk(logits, 128, 8)
    idx, w = _topk(logits, 8, dt=dt)
    assert np.array_equal(idx, ref_idx)
    assert np.max(np.abs(w - ref_w)) <= {"f32": 1e-5, "f16": 1e-3, "bf16": 8e-3}[dt]


@pytest.mark.parametrize("n_tokens,k,n_experts", [(512, 8, 128), (37, 4, 9), (4096, 8, 128), (1, 1, 1), (300, 2, 1000)])
def test_moe_sort_exact(n_tokens, k, n_experts):
    import torch
    from metaltile_b200 import ops
    rng = np.random.default_rng(n_tokens)
    topk = np.stack([rng.permutation(n_experts)[:k] for _ in range(n_tokens)]).astype(np.uint32)
    ref = oracle.moe_sort(topk, n_experts)
    got = ops.moe_sort(to_dev(topk), n_experts)
    torch.cuda.synchronize()
    for g, r, name in zip(got, ref, ("sort_token_idx", "inv_perm", "expert_offsets", "row_expert")):
        assert np.array_equal(g.cpu().numpy().astype(np.uint32).reshape(r.shape), r), name


@pytest.mark.parametrize("dt", DT_NAMES)
def test_permute_is_a_bit_exact_copy_and_unpermute_matches(dt):
    import torch
    from metaltile_b200 import ops, synth
    n_tokens, k, ne, hidden = 64, 4, 16, 256
    rng = np.random.default_rng(1)
    topk = np.stack([rng.permutation(ne)[:k] for _ in range(n_tokens)]).astype(np.uint32)
    sti, inv, off, rex = oracle.moe_sort(topk, ne)
    tok = oracle.round_through(synth.activations(n_tokens, hidden, seed=2), ODT[dt])
    perm = ops.moe_permute(to_dev(tok, dt), to_dev(sti))
    torch.cuda.synchronize()
    assert np.array_equal(perm.float().cpu().numpy(), tok[sti])          # moe_gpu_correctness.rs:627-672
    wts = oracle.round_through(rng.random((n_tokens, k)).astype(np.float32), ODT[dt])
    eo = oracle.round_through(synth.activations(n_tokens * k, hidden, seed=3), ODT[dt])
    ref = oracle.moe_unpermute(eo, inv, wts)
    got = ops.moe_unpermute(to_dev(eo, dt), to_dev(inv), to_dev(wts, dt))
    torch.cuda.synchronize()
    assert rel_err(got.float().cpu().numpy(), ref) <= TOL[dt]


def test_unpermute_and_swiglu_reference_cases(ctx, moe):
    """Through the name-keyed dispatch with host buffers (moe_gpu_correctness.rs:164-215, swiglu.rs:65-80)."""
    eo, w, inv = moe["unperm_eo"], moe["unperm_w"], moe["unperm_inv"]
    res = ctx.dispatch_with_grid("mt_moe_unpermute", {
        "expert_outputs": eo.tobytes(), "inv_perm": inv.tobytes(), "top_k_weights": w.tobytes(),
        "out": bytes(4 * 256 * 4)}, {"hidden": 256, "k": 4}, (4, 1, 1), (128, 1, 1))
    got = np.frombuffer(res.outputs["out"], np.float32).reshape(4, 256)
    assert np.max(np.abs(got - moe["unperm_out"])) < 1e-4
    g, u = moe["swiglu_gate"], moe["swiglu_up"]
    for dt, tol in (("f32", 1e-4), ("f16", 5e-3), ("bf16", 5e-2)):       # the reference's registered tolerances
        res = ctx.dispatch_with_grid("mt_swiglu", {"gate": dt_bytes(g, dt), "up": dt_bytes(u, dt),
                                                   "out": bytes(1024 * (4 if dt == "f32" else 2))}, {}, dtype=dt)
        gr, ur = oracle.round_through(g, ODT[dt]), oracle.round_through(u, ODT[dt])
        assert np.max(np.abs(bytes_to_f32(res.outputs["out"], dt) - oracle.swiglu(gr, ur))) <= tol
    res = ctx.dispatch_with_grid("mt_moe_router_topk", {
        "router_logits": moe["topk_tie_logits"].tobytes(), "indices_out": bytes(8), "weights_out": bytes(8)},
        {"n_experts": 8, "k": 2, "norm_topk_prob": 1}, outputs=("indices_out", "weights_out"))
    assert np.frombuffer(res.outputs["indices_out"], np.uint32).tolist() == [2, 5]


@pytest.mark.parametrize("dt", DT_NAMES)
@pytest.mark.parametrize("kernel", ["mt_moe_gather_qmm_int4", "mt_moe_gather_qmm_int4_m8"])
def test_registered_gather_case(ctx, kernel, dt):
    """test_moe_gather_qmm_int4 / _m8 (crates/metaltile-std/src/ffai/moe.rs:3627-3695): 3 experts, offsets [0,2,5,6]."""
    fx = dict(np.load(os.path.join(GOLDEN, f"test_moe_gather_qmm_int4_{dt}.npz")))
    t_rows, k_in, m_out, ne, bits, gs = (int(v) for v in fx["meta"])
    bufs = {"x": dt_bytes(fx["x"], dt), "weight_packed": fx["w"].tobytes(), "scales": dt_bytes(fx["scales"], dt),
            "biases": dt_bytes(fx["biases"], dt), "expert_offsets": fx["expert_offsets"].tobytes(),
            "out": bytes(t_rows * m_out * (4 if dt == "f32" else 2))}
    res = ctx.dispatch_with_grid(kernel, bufs, {"k_in": k_in, "m_out": m_out, "n_experts": ne, "group_size": gs},
                                 (m_out, t_rows, 1), (32, 1, 1), dtype=dt)
    got = bytes_to_f32(res.outputs["out"], dt).reshape(t_rows, m_out)
    assert rel_err(got, fx["expected"]) <= TOL[dt]


def _gather_case(n_experts, n_out, k_in, bits, gs, dt, counts, seed=0):
    from metaltile_b200 import synth
    w, s, b = synth.quantized_matrix(n_experts * n_out, k_in, bits, gs, seed=seed, salt=9)
    total = int(np.sum(counts))
    x = synth.activations(total, k_in, seed=seed, salt=9)
    s, b, x = (oracle.round_through(a, ODT[dt]) for a in (s, b, x))
    off = np.concatenate([[0], np.cumsum(counts)]).astype(np.uint32)
    idx = np.repeat(np.arange(n_experts), counts).astype(np.uint32)
    return (w.reshape(n_experts, n_out, -1), s.reshape(n_experts, n_out, -1), b.reshape(n_experts, n_out, -1), x, off, idx)


@pytest.mark.parametrize("n_experts,n_out,k_in,bits,gs,dt,counts", [
    (3, 8, 64, 4, 32, "bf16", [2, 3, 1]),
    (4, 256, 512, 4, 64, "bf16", [5, 0, 40, 3]),            # an empty expert, uneven sizes
    (8, 130, 256, 4, 64, "f16", [17, 1, 300, 0, 0, 33, 16, 2]),   # > 256 rows in one expert, ragged n_out
    (4, 64, 256, 8, 64, "bf16", [10, 20, 30, 40]),
    (4, 64, 256, 3, 64, "bf16", [10, 20, 30, 40]),
    (4, 64, 256, 6, 32, "f16", [10, 20, 30, 40]),
    (3, 16, 96, 4, 32, "f32", [4, 0, 7]),                   # f32 and K % 64 != 0: CUDA-core path
])
def test_gather_qmm_matches_oracle(ctx, n_experts, n_out, k_in, bits, gs, dt, counts):
    import torch
    from metaltile_b200 import ops
    w, s, b, x, off, idx = _gather_case(n_experts, n_out, k_in, bits, gs, dt, counts)
    total = x.shape[0]
    ref = oracle.gather_qmm(x, w, s, b, total, k_in, n_out, n_experts, bits, gs, expert_offsets=off)
    wd, sd, bd, xd = to_dev(w), to_dev(s, dt), to_dev(b, dt), to_dev(x, dt)
    got_stream = ops.gather_qmm(xd, wd, sd, bd, bits, gs, expert_offsets=to_dev(off))    # small groups may take the streaming kernel
    ctx.set_option("gather_stream", 0)
    try:
        got_csr = ops.gather_qmm(xd, wd, sd, bd, bits, gs, expert_offsets=to_dev(off))
        got_idx = ops.gather_qmm(xd, wd, sd, bd, bits, gs, indices=to_dev(idx))
    finally:
        ctx.set_option("gather_stream", 1)
    torch.cuda.synchronize()
    assert rel_err(got_stream.float().cpu().numpy(), ref) <= TOL[dt]
    assert rel_err(got_csr.float().cpu().numpy(), ref) <= TOL[dt]
    assert torch.equal(got_csr, got_idx)                     # CSR and per-row-index forms agree bit for bit
    assert ctx.status_word() == 0


@pytest.mark.parametrize("n_experts,n_out,k_in,gs,dt,counts", [
    (6, 768, 2048, 64, "bf16", [31, 32, 33, 0, 1, 65]),                 # one, two and three passes per expert; an empty one
    (5, 2048, 768, 64, "bf16", [8, 9, 40, 17, 24]),                     # K = 1.5 x 512: runs of 256 codes
    (4, 130, 512, 128, "f16", [3, 70, 0, 12]),                          # group 128, ragged n_out (last tile has 2 rows)
    (3, 96, 4096, 64, "bf16", [16, 17, 5]),                             # K = 4096: 16 rows per pass
    (2, 48, 8192, 128, "f16", [9, 2]),                                  # K = 8192: 8 rows per pass
    (40, 64, 256, 64, "bf16", [(7 * i) % 11 for i in range(40)]),       # many small experts, more experts than a scan round
    (1, 16, 256, 64, "f16", [1]),
])
def test_gather_stream_matches_oracle(ctx, n_experts, n_out, k_in, gs, dt, counts):
    """The weight-streaming grouped product (few rows per expert) against the oracle, and - where the tensor-memory kernel
    takes the shape too - against that kernel within rounding."""
    import torch
    from metaltile_b200 import ops
    w, s, b, x, off, _ = _gather_case(n_experts, n_out, k_in, 4, gs, dt, counts, seed=2)
    total = x.shape[0]
    ref = oracle.gather_qmm(x, w, s, b, total, k_in, n_out, n_experts, 4, gs, expert_offsets=off)
    wd, sd, bd, xd = to_dev(w), to_dev(s, dt), to_dev(b, dt), to_dev(x, dt)
    out = torch.full((total, n_out), float("nan"), dtype=xd.dtype, device="cuda")
    ops.gather_qmm(xd, wd, sd, bd, 4, gs, expert_offsets=to_dev(off), out=out)
    again = ops.gather_qmm(xd, wd, sd, bd, 4, gs, expert_offsets=to_dev(off))
    torch.cuda.synchronize()
    assert ctx.status_word() == 0
    assert not torch.isnan(out).any()                        # every element is written
    assert torch.equal(out, again)                           # and the same on every run
    assert rel_err(out.float().cpu().numpy(), ref) <= TOL[dt]
    ctx.set_option("gather_stream", 0)
    try:
        other = ops.gather_qmm(xd, wd, sd, bd, 4, gs, expert_offsets=to_dev(off))
    finally:
        ctx.set_option("gather_stream", 1)
    assert rel_err(out.float().cpu().numpy(), other.float().cpu().numpy()) <= 2 * TOL[dt]


@pytest.mark.parametrize("stream_kernel", [1, 0])
def test_gather_reports_bad_offsets(ctx, stream_kernel):
    """expert_offsets that run past m_total are clamped to it on both tensor-core paths (nothing outside x or out is
    touched: the rows that exist get their expert's product, the others do not exist) and reported: 0x901."""
    import torch
    from metaltile_b200 import MetalTileError, ops
    w, s, b, x, off, _ = _gather_case(3, 32, 256, 4, 64, "bf16", [4, 4, 4], seed=3)
    bad = off.copy()
    bad[2] = 1000                                            # beyond m_total = 12: expert 1 owns rows 4..11, expert 2 none
    wd, sd, bd, xd = to_dev(w), to_dev(s, "bf16"), to_dev(b, "bf16"), to_dev(x, "bf16")
    ctx.set_option("gather_stream", stream_kernel)
    try:
        got = ops.gather_qmm(xd, wd, sd, bd, 4, 64, expert_offsets=to_dev(bad))
        with pytest.raises(MetalTileError):
            ctx.sync(torch.cuda.current_stream().cuda_stream)
        assert ctx.status_word() == 0x901
    finally:
        ctx.set_option("gather_stream", 1)
        ctx.status_clear()
    clamped = np.array([0, 4, 12, 12], dtype=np.uint32)
    ref = oracle.gather_qmm(x, w, s, b, 12, 256, 32, 3, 4, 64, expert_offsets=clamped)
    assert rel_err(got.float().cpu().numpy(), ref) <= TOL["bf16"]


def test_moe_layer_config4(ctx):
    """512 tokens x hidden 2048, 128 experts (gate/up 2048->768, down 768->2048), top-8, 4-bit g64 bf16:
    the whole pipeline against the oracle on routing (exact) and on the outputs of a sample of experts."""
    import torch
    from metaltile_b200 import ops, synth
    T, H, I, E, K8, bits, gs, dt = 512, 2048, 768, 128, 8, 4, 64, "bf16"
    tok = oracle.round_through(synth.activations(T, H, seed=0), oracle.BF16)
    logits = oracle.round_through(synth.router_logits(T, E, seed=0), oracle.BF16)
    wg, sg, bg = synth.quantized_matrix(E * I, H, bits, gs, seed=0, salt=20)
    wu, su, bu = synth.quantized_matrix(E * I, H, bits, gs, seed=0, salt=21)
    wd, sd, bd = synth.quantized_matrix(E * H, I, bits, gs, seed=0, salt=22)
    rnd = lambda a: oracle.round_through(a, oracle.BF16)
    sg, bg, su, bu, sd, bd = (rnd(a) for a in (sg, bg, su, bu, sd, bd))
    dev3 = lambda w, s, b, n, k: (to_dev(w.reshape(E, n, -1)), to_dev(s.reshape(E, n, -1), dt), to_dev(b.reshape(E, n, -1), dt))

    idx, wts = ops.moe_router_topk(to_dev(logits, dt), K8)
    sti, inv, off, rex = ops.moe_sort(idx, E)
    xp = ops.moe_permute(to_dev(tok, dt), sti)
    g = ops.gather_qmm(xp, *dev3(wg, sg, bg, I, H), bits, gs, expert_offsets=off)
    u = ops.gather_qmm(xp, *dev3(wu, su, bu, I, H), bits, gs, expert_offsets=off)
    a = ops.swiglu(g, u)
    y = ops.gather_qmm(a, *dev3(wd, sd, bd, H, I), bits, gs, expert_offsets=off)
    out = ops.moe_unpermute(y, inv, wts)
    torch.cuda.synchronize()

    ref_idx, ref_w = oracle.router_topk(logits, E, K8)
    assert np.array_equal(idx.cpu().numpy().astype(np.uint32), ref_idx)            # routing indices exact
    r_sti, r_inv, r_off, r_rex = oracle.moe_sort(ref_idx, E)
    assert np.array_equal(sti.cpu().numpy().astype(np.uint32), r_sti)
    assert np.array_equal(off.cpu().numpy().astype(np.uint32), r_off)
    # expert outputs for a sample of experts, each stage fed with the device's own rounded input
    xp_h = xp.float().cpu().numpy()
    g_h, u_h, a_h, y_h = (t.float().cpu().numpy() for t in (g, u, a, y))
    for e in (0, 17, 127):
        r0, r1 = int(r_off[e]), int(r_off[e + 1])
        if r1 == r0:
            continue
        sl = slice(e * I, (e + 1) * I)
        ref_g = oracle.qmm(wg[sl], sg[sl], bg[sl], xp_h[r0:r1], r1 - r0, I, H, bits, gs)
        assert rel_err(g_h[r0:r1], ref_g) <= TOL[dt]
        ref_a = oracle.swiglu(g_h[r0:r1], u_h[r0:r1])
        assert rel_err(a_h[r0:r1], ref_a) <= TOL[dt]
        sl = slice(e * H, (e + 1) * H)
        ref_y = oracle.qmm(wd[sl], sd[sl], bd[sl], a_h[r0:r1], r1 - r0, H, I, bits, gs)
        assert rel_err(y_h[r0:r1], ref_y) <= TOL[dt]
    ref_out = oracle.moe_unpermute(y_h, r_inv, wts.float().cpu().numpy())
    assert rel_err(out.float().cpu().numpy(), ref_out) <= TOL[dt]
    assert ctx.status_word() == 0


@pytest.mark.parametrize("dt,hidden,inter,gs,bits,counts", [
    ("bf16", 512, 256, 64, 4, [9, 0, 33, 20, 2]),          # the streamed form (four launches)
    ("f16", 256, 512, 128, 4, [5, 17, 1]),
    ("bf16", 128, 64, 32, 4, [4, 6]),                      # outside the streaming kernel's contract: composed from the entries
    ("f32", 128, 64, 32, 8, [3, 0, 5]),
])
def test_moe_experts_equals_the_separate_entries(ctx, dt, hidden, inter, gs, bits, counts):
    """mtc_moe_experts == permute -> gather_qmm(gate), gather_qmm(up) -> swiglu -> gather_qmm(down), bit for bit, with and
    without the permutation folded in; and against the oracle for one expert."""
    import torch
    from metaltile_b200 import ops, synth
    E, total = len(counts), int(np.sum(counts))
    n_tok = max(4, total // 2)
    mk = lambda n, k, salt: synth.quantized_matrix(E * n, k, bits, gs, seed=4, salt=salt)
    mats_h = [mk(inter, hidden, 31), mk(inter, hidden, 32), mk(hidden, inter, 33)]
    dev3 = lambda m, n: (to_dev(m[0].reshape(E, n, -1)), to_dev(oracle.round_through(m[1], ODT[dt]).reshape(E, n, -1), dt),
                         to_dev(oracle.round_through(m[2], ODT[dt]).reshape(E, n, -1), dt))
    gate, up, down = dev3(mats_h[0], inter), dev3(mats_h[1], inter), dev3(mats_h[2], hidden)
    tok = to_dev(oracle.round_through(synth.activations(n_tok, hidden, seed=4), ODT[dt]), dt)
    rng = np.random.default_rng(4)
    sti = to_dev(rng.integers(0, n_tok, size=total).astype(np.uint32))
    off = to_dev(np.concatenate([[0], np.cumsum(counts)]).astype(np.uint32))

    xp = ops.moe_permute(tok, sti, ctx=ctx)
    g = ops.gather_qmm(xp, *gate, bits, gs, expert_offsets=off, ctx=ctx)
    u = ops.gather_qmm(xp, *up, bits, gs, expert_offsets=off, ctx=ctx)
    act = ops.swiglu(g, u, ctx=ctx)
    ref = ops.gather_qmm(act, *down, bits, gs, expert_offsets=off, ctx=ctx)
    got_perm = ops.moe_experts(tok, gate, up, down, bits, gs, off, sort_token_idx=sti, ctx=ctx)
    got_rows = ops.moe_experts(xp, gate, up, down, bits, gs, off, ctx=ctx)
    torch.cuda.synchronize()
    assert ctx.status_word() == 0
    assert torch.equal(got_perm, ref) and torch.equal(got_rows, ref)
    # one expert against the oracle, stage by stage on the device's own rounded inputs
    e = int(np.argmax(counts))
    r0, r1 = int(np.sum(counts[:e])), int(np.sum(counts[:e + 1]))
    rnd = lambda a: oracle.round_through(a, ODT[dt])
    sl = slice(e * inter, (e + 1) * inter)
    xh = xp.float().cpu().numpy()[r0:r1]
    gh = rnd(oracle.qmm(mats_h[0][0][sl], rnd(mats_h[0][1][sl]), rnd(mats_h[0][2][sl]), xh, r1 - r0, inter, hidden, bits, gs))
    uh = rnd(oracle.qmm(mats_h[1][0][sl], rnd(mats_h[1][1][sl]), rnd(mats_h[1][2][sl]), xh, r1 - r0, inter, hidden, bits, gs))
    assert rel_err(g.float().cpu().numpy()[r0:r1], gh) <= TOL[dt]
    ah = act.float().cpu().numpy()[r0:r1]
    sl = slice(e * hidden, (e + 1) * hidden)
    yh = oracle.qmm(mats_h[2][0][sl], rnd(mats_h[2][1][sl]), rnd(mats_h[2][2][sl]), ah, r1 - r0, hidden, inter, bits, gs)
    assert rel_err(got_perm.float().cpu().numpy()[r0:r1], yh) <= TOL[dt]


def test_moe_experts_reports_a_bad_row_index(ctx):
    """sort_token_idx naming a row that x does not have: row 0 is read instead (no out-of-range access), status 0x903."""
    import torch
    from metaltile_b200 import MetalTileError, ops, synth
    E, hidden, inter = 2, 256, 256
    mk = lambda n, k, salt: synth.quantized_matrix(E * n, k, 4, 64, seed=5, salt=salt)
    dev3 = lambda m, n: (to_dev(m[0].reshape(E, n, -1)), to_dev(m[1].reshape(E, n, -1), "bf16"), to_dev(m[2].reshape(E, n, -1), "bf16"))
    gate, up, down = dev3(mk(inter, hidden, 1), inter), dev3(mk(inter, hidden, 2), inter), dev3(mk(hidden, inter, 3), hidden)
    tok = to_dev(synth.activations(4, hidden, seed=5), "bf16")
    sti = to_dev(np.array([0, 3, 99, 1], dtype=np.uint32))
    off = to_dev(np.array([0, 2, 4], dtype=np.uint32))
    try:
        ops.moe_experts(tok, gate, up, down, 4, 64, off, sort_token_idx=sti, ctx=ctx)
        with pytest.raises(MetalTileError):
            ctx.sync(torch.cuda.current_stream().cuda_stream)
        assert ctx.status_word() == 0x903
    finally:
        ctx.status_clear()


@pytest.mark.parametrize("dt", DT_NAMES)
def test_reference_decode_tail_cases(ctx, dt):
    """test_dequant_gemv_int4_expert_indexed (ffai/dequant_gemv_expert_indexed.rs:129-208) and
    test_moe_down_swiglu_accum_int4_chain8 (ffai/moe_down_swiglu_accum.rs:405-487) under the reference's names, with its
    tolerances (5e-3 / 5e-2 / 2e-1) and this build's."""
    ref_tol = {"f32": 5e-3, "f16": 5e-2, "bf16": 2e-1}[dt]
    esz = 4 if dt == "f32" else 2
    fx = dict(np.load(os.path.join(GOLDEN, f"expert_indexed_gemv_{dt}.npz")))
    ne, od, idim, gs, e = (int(v) for v in fx["meta"])
    bufs = {"weights_stacked": fx["w"].tobytes(), "scales_stacked": dt_bytes(fx["scales"], dt), "biases_stacked": dt_bytes(fx["biases"], dt),
            "input": dt_bytes(fx["x"], dt), "expert_index": np.array([e], dtype=np.uint32).tobytes(), "output": bytes(od * esz)}
    res = ctx.dispatch_with_grid("dequant_gemv_int4_expert_indexed", bufs, {"in_dim": idim, "out_dim": od, "group_size": gs}, (od, 1, 1),
                                 (64, 1, 1), dtype=dt, outputs=("output",))
    got = bytes_to_f32(res.outputs["output"], dt)
    assert np.any(got != 0.0) and float(np.max(np.abs(got - fx["acc"]))) <= ref_tol
    assert rel_err(got.reshape(1, -1), fx["acc"].reshape(1, -1)) <= TOL[dt]
    fx = dict(np.load(os.path.join(GOLDEN, f"moe_down_swiglu_accum_{dt}.npz")))
    ne, idim, od, gs, ns = (int(v) for v in fx["meta"])
    bufs = {"weights_stacked": fx["w"].tobytes(), "scales_stacked": dt_bytes(fx["scales"], dt), "biases_stacked": dt_bytes(fx["biases"], dt),
            "expert_indices": fx["experts"].astype(np.uint32).tobytes(), "slot_weights": dt_bytes(fx["slot_weights"], dt), "output": bytes(od * esz)}
    for k in range(ns):
        bufs[f"gate_{k}"], bufs[f"up_{k}"] = dt_bytes(fx["gates"][k], dt), dt_bytes(fx["ups"][k], dt)
    res = ctx.dispatch_with_grid("ffai_moe_down_swiglu_accum_int4_chain8", bufs, {"in_dim": idim, "out_dim": od, "group_size": gs},
                                 (od, 1, 1), (64, 1, 1), dtype=dt, outputs=("output",))
    got = bytes_to_f32(res.outputs["output"], dt)
    assert np.any(got != 0.0) and float(np.max(np.abs(got - fx["acc"]))) <= ref_tol
    assert rel_err(got.reshape(1, -1), fx["acc"].reshape(1, -1)) <= TOL[dt]


@pytest.mark.parametrize("dt,n_slots,in_dim,out_dim,gs", [("bf16", 8, 768, 2048, 64), ("f16", 4, 512, 300, 128), ("f32", 8, 64, 40, 32),
                                                          ("bf16", 2, 2048, 72, 64)])      # the last: more than 4 words per lane
def test_moe_decode_tail_at_size(ctx, dt, n_slots, in_dim, out_dim, gs):
    """The fused M = 1 tail (SwiGLU, expert-indexed down projection, weighted sum over the routed slots) against the oracle,
    and against its unfused composition: mt_swiglu per slot, the expert-indexed product of all slots in one launch, the sum."""
    import torch
    from metaltile_b200 import ops, synth
    from metaltile_b200.ops import _TORCH_DT
    E = 16
    w, s, b = synth.quantized_matrix(E * out_dim, in_dim, 4, gs, seed=70)
    rt = lambda a: oracle.round_through(a, ODT[dt])
    s, b = rt(s), rt(b)
    gates, ups = rt(synth.activations(n_slots, in_dim, seed=71)), rt(synth.activations(n_slots, in_dim, seed=72))
    experts = np.array([(5 * k + 3) % E for k in range(n_slots)], dtype=np.uint32)
    sw = rt((0.05 + 0.03 * np.arange(n_slots)).astype(np.float32))
    wd, sd, bd = to_dev(w), to_dev(s, dt), to_dev(b, dt)
    gd, ud, ed, swd = to_dev(gates, dt), to_dev(ups, dt), to_dev(experts), to_dev(sw, dt)
    out = torch.zeros(out_dim, dtype=gd.dtype, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    esz = gd.element_size()
    ctx.moe_down_swiglu_accum([gd.data_ptr() + k * in_dim * esz for k in range(n_slots)], [ud.data_ptr() + k * in_dim * esz for k in range(n_slots)],
                              ed.data_ptr(), swd.data_ptr(), wd.data_ptr(), sd.data_ptr(), bd.data_ptr(), out.data_ptr(), in_dim, out_dim, E, gs,
                              _TORCH_DT[gd.dtype], stream=st)
    torch.cuda.synchronize()
    ref = oracle.moe_down_swiglu_accum(gates, ups, experts, sw, w, s, b, in_dim, out_dim, gs)
    assert ctx.status_word() == 0
    assert rel_err(out.float().cpu().numpy().reshape(1, -1), ref.reshape(1, -1)) <= TOL[dt]
    # unfused: swiglu (rounded to T, as the stand-alone kernel stores it), expert-indexed products, weighted sum on the host
    act = ops.swiglu(gd, ud, ctx=ctx)
    per = torch.zeros((n_slots, out_dim), dtype=gd.dtype, device="cuda")
    ctx.qmv_expert_indexed([act.data_ptr() + k * in_dim * esz for k in range(n_slots)], ed.data_ptr(), wd.data_ptr(), sd.data_ptr(), bd.data_ptr(),
                           per.data_ptr(), in_dim, out_dim, E, gs, _TORCH_DT[gd.dtype], stream=st)
    torch.cuda.synchronize()
    act_h = act.float().cpu().numpy()
    for k in (0, n_slots - 1):
        e = int(experts[k])
        sl = slice(e * out_dim, (e + 1) * out_dim)
        assert rel_err(per[k].float().cpu().numpy().reshape(1, -1), oracle.qmm(w[sl], s[sl], b[sl], act_h[k:k + 1], 1, out_dim, in_dim, 4, gs)) <= TOL[dt]
    comp = (per.float().cpu().numpy() * sw[:, None]).sum(axis=0)
    assert rel_err(out.float().cpu().numpy().reshape(1, -1), comp.reshape(1, -1)) <= 3 * TOL[dt]


def test_moe_decode_tail_reports_a_bad_expert(ctx):
    import torch
    from metaltile_b200 import MetalTileError, synth
    from metaltile_b200.ops import _TORCH_DT
    E, in_dim, out_dim = 4, 64, 16
    w, s, b = synth.quantized_matrix(E * out_dim, in_dim, 4, 32, seed=73)
    x = to_dev(synth.activations(1, in_dim, seed=74), "bf16")
    out = torch.zeros((1, out_dim), dtype=torch.bfloat16, device="cuda")
    bad = to_dev(np.array([77], dtype=np.uint32))
    try:
        ctx.qmv_expert_indexed([x.data_ptr()], bad.data_ptr(), to_dev(w).data_ptr(), to_dev(s, "bf16").data_ptr(), to_dev(b, "bf16").data_ptr(),
                               out.data_ptr(), in_dim, out_dim, E, 32, _TORCH_DT[x.dtype], stream=torch.cuda.current_stream().cuda_stream)
        with pytest.raises(MetalTileError):
            ctx.sync(torch.cuda.current_stream().cuda_stream)
        assert ctx.status_word() == 0x905
    finally:
        ctx.status_clear()
