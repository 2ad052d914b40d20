#!/usr/bin/env python
"""Benchmark of the quantized-matmul hot path on B200 (one JSON line on stdout).

    python bench.py --gpus N --steps K --warmup W [--impl reference] [--m 1]

Workload (``config.workload``): the Llama-3-8B-shaped decode projection set, 4-bit
codes, group 64, bf16 activations, M = 1: per layer q 4096->4096, k/v 4096->1024 (x2),
o 4096->4096, gate/up 4096->14336 (x2), down 14336->4096, over 32 layers of random
codes (3.9 GB of packed weights, scales and biases: far larger than L2, so every step
streams from HBM).  One "step" = one pass of qmv over all 224 matrices.  With N > 1
every matrix is N-split (row blocks of the weight) and the output slices are
all-gathered over NCCL, one collective per dependent phase of a layer (qkv | o |
gate,up | down).

metric = qmv HBM GB/s = algorithmic bytes of the whole job / step time, with
algorithmic bytes per matrix = N*K*bits/8 + 2*N*(K/G)*sz + M*K*sz + M*N*sz
(the reference's bytes_moved, crates/metaltile-std/src/mlx/quantized.rs:5804).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

LAYERS = 32
# (name, K, N, phase)
PROJ = [("q", 4096, 4096, 0), ("k", 4096, 1024, 0), ("v", 4096, 1024, 0), ("o", 4096, 4096, 1),
        ("gate", 4096, 14336, 2), ("up", 4096, 14336, 2), ("down", 14336, 4096, 3)]
BITS, GROUP = 4, 64
METRIC = "qmv HBM GB/s (% of peak) and qmm TFLOP/s at 1/2/4/8xB200 vs CPU oracle"


def alg_bytes(m, n, k, bits=BITS, g=GROUP, sz=2):
    return n * k * bits // 8 + 2 * n * (k // g) * sz + m * k * sz + m * n * sz


def step_bytes(m, layers=LAYERS):
    return layers * sum(alg_bytes(m, n, k) for _, k, n, _ in PROJ)


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d.get("hbm_gbs", 6650.0), d.get("bf16_tflops", 1590.0), d.get("bf16_tflops_sustained", 1400.0), "measured"
    return 6650.0, 1590.0, 1400.0, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML while the timed region runs."""

    def __init__(self, index):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thr = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            vis = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = int(vis.split(",")[index]) if vis and vis.split(",")[index].isdigit() else index
            self.h = pynvml.nvmlDeviceGetHandleByIndex(phys)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _loop(self):
        nv = self.nv
        names = {"hw_slowdown": 0x8, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20,
                 "sw_power_cap": 0x4, "hw_power_brake": 0x80}
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                r = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                for k, bit in names.items():
                    if r & bit:
                        self.reasons.add(k)
            except Exception:
                pass
            time.sleep(0.005)

    def start(self):
        if self.nv:
            self._thr = threading.Thread(target=self._loop, daemon=True)
            self._thr.start()

    def stop(self):
        if self._thr:
            self._stop.set()
            self._thr.join()
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None,
                "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(self.samples)}


# ------------------------------------------------------------------------------------------
def cpu_reference_arm(args):
    """The reference's own CPU implementation of the path (the scalar dequant-then-dot oracle,
    restated in C because no Rust toolchain exists here), all host threads, bounded sample."""
    import numpy as np
    import oracle
    from metaltile_b200 import synth
    # all host cores, whatever OMP_NUM_THREADS the launcher exported (torch.distributed.run sets it to 1)
    threads = os.cpu_count() or oracle.max_threads()
    layers = 1
    mats = []
    for li in range(layers):
        for pi, (_, k, n, _) in enumerate(PROJ):
            w, s, b = synth.quantized_matrix(n, k, BITS, GROUP, seed=0, salt=li * 8 + pi)
            x = synth.activations(args.m, k, seed=0, salt=li * 8 + pi)
            s, b, x = (oracle.round_through(a, oracle.BF16) for a in (s, b, x))
            mats.append((w, s, b, x, n, k))

    def one_step():
        for w, s, b, x, n, k in mats:
            oracle.qmm(w, s, b, x, args.m, n, k, BITS, GROUP, threads=threads)

    for _ in range(max(args.warmup, 1)):
        one_step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        one_step()
    dt = (time.perf_counter() - t0) / args.steps
    nbytes = step_bytes(args.m, layers)
    return nbytes / dt / 1e9, dt * 1e3, threads, f"{layers} of {LAYERS} layers ({len(mats)} matrices) per step"


def spot_check(layers, xs, tiles, out_local, out_full, M, world, phase_cols):
    """Untimed: 64 weight rows of the first and of the last projection of the step against the CPU oracle (rank 0's
    shard).  Returns True / False; the benchmark number is a claim only if the kernels computed the right thing."""
    import numpy as np
    import torch
    import oracle
    ok = True
    for li, pi in ((0, 0), (len(layers) - 1, len(PROJ) - 1)):
        w, sc, bi, k, nl, phase = layers[li][pi]
        rows = min(64, nl)
        x = xs[k].float().cpu().numpy()
        kl = x.shape[1]
        ref = oracle.qmm(w[:rows].cpu().numpy().view(np.uint32), sc[:rows].float().cpu().numpy(), bi[:rows].float().cpu().numpy(),
                         np.ascontiguousarray(x), M, rows, kl, BITS, GROUP)
        col = sum(n for (_, _, _, _, n, p) in layers[li][:pi] if p == phase)
        if M == 1 or world > 1:
            got = out_local[li][phase][:, col:col + rows]
            if out_full is not None:      # peer-store gather: this rank's slot of the gathered block
                got = out_full[li][phase].view(world, M, phase_cols[phase])[0][:, col:col + rows]
        else:
            got = tiles[li][pi][:, :rows]
        err = np.abs(got.float().cpu().numpy() - ref) / np.maximum(np.abs(ref), 1.0)
        ok = ok and bool(np.all(err <= 1e-2))
    return ok


def p2p_trial(ctx, dev, rank, world, stream_opt=1):
    """One small projection gathered through peer stores + barrier, compared with NCCL; every rank must agree."""
    import torch
    import torch.distributed as dist
    from metaltile_b200 import ops
    ok = 1
    try:
        from metaltile_b200.parallel import PeerGather
        nl, k = 256, 512
        gen = torch.Generator(device=dev)
        gen.manual_seed(99 + rank)
        w = torch.randint(-2 ** 31, 2 ** 31 - 1, (nl, k * BITS // 32), dtype=torch.int32, device=dev, generator=gen)
        sc = (0.002 + 0.018 * torch.rand((nl, k // GROUP), device=dev, generator=gen)).to(torch.bfloat16)
        bi = (-8.0 * sc.float()).to(torch.bfloat16)
        x = torch.randn((1, k), generator=torch.Generator().manual_seed(5)).to(torch.bfloat16).to(dev)
        peer = PeerGather(ctx, world * nl * 2)
        st = torch.cuda.current_stream().cuda_stream
        for _ in range(2):
            peer.qmv_into(w, sc, bi, x, BITS, GROUP, rank * nl * 2, st)
            peer.barrier(st)
        # the reference projection on the same kernel as the peer path (a single small projection would otherwise take
        # the CUDA-core kernel, whose results differ in the last bit of some outputs)
        ctx.set_option("qmv_stream", 2)
        try:
            loc = ops.qmv(w, sc, bi, x, BITS, GROUP, ctx=ctx)
        finally:
            ctx.set_option("qmv_stream", stream_opt)
        ref = torch.empty((world, nl), dtype=torch.bfloat16, device=dev)
        dist.all_gather_into_tensor(ref, loc)
        torch.cuda.synchronize()
        if not torch.equal(ref.reshape(-1), peer.tensor(torch.bfloat16)) or ctx.status_word() != 0:
            ok = 0
        dist.barrier()
        peer.close()
    except Exception as e:  # any failure of the peer path means the NCCL path is used
        print(f"[rank {rank}] p2p trial failed: {e!r}", file=sys.stderr, flush=True)
        ok = 0
    t = torch.tensor([ok], device=dev, dtype=torch.int32)
    dist.all_reduce(t, op=dist.ReduceOp.MIN)
    return bool(int(t.item()))


# dram__bytes_read.sum + dram__bytes_write.sum over algorithmic bytes for one launch of the step's kernel
# (qmv_stream_kernel on the 14336 x 4096 projection, ncu --set full, cold L2: 33.69 MB read, 0.8 KB written, 33.07 MB algorithmic)
NCU_TRAFFIC_RATIO = 1.019


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--m", type=int, default=1, help="activation rows per projection (1 or 8)")
    ap.add_argument("--layers", type=int, default=LAYERS)
    ap.add_argument("--tp", default="gather", choices=["gather", "megatron"],
                    help="N > 1: every projection N-split with an all-gather of the outputs per dependent phase (gather, "
                         "the configuration the metric is quoted on), or column-parallel q/k/v/gate/up + row-parallel "
                         "o/down with one all-reduce each (megatron)")
    ap.add_argument("--collective", default="auto", choices=["auto", "nccl", "p2p"],
                    help="N > 1, --tp gather, M = 1: all-gather with NCCL, or by the qmv kernels' own stores into every "
                         "rank's buffer (cudaIpc peer mappings) and a one-warp barrier kernel per phase; auto = p2p when "
                         "a small trial of it on every rank reproduces the NCCL all-gather, else nccl")
    ap.add_argument("--verify", action="store_true", help="N > 1: check the p2p gather against the NCCL all-gather once")
    ap.add_argument("--option", action="append", default=[], metavar="NAME=VALUE", help="mtc_set_option before running")
    ap.add_argument("--mode", default="batched", choices=["batched", "chain", "launches"],
                    help="one GPU: projections that share their activations fused (q/k/v and gate/up: mtc_qmv_batched, 4 launches "
                         "per layer), the whole step as one prepared chain (mtc_chain_run), or one mtc_qmv launch per projection")
    ap.add_argument("--streams", type=int, default=1, help="parallel streams for the independent projections of a phase")
    ap.add_argument("--no-extra", action="store_true", help="skip the secondary single-kernel measurements")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU-baseline leg")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    config = {"workload": f"llama3_8b_decode_projections_4bit_g64_bf16_m{args.m}", "layers": args.layers,
              "matrices_per_step": 7 * args.layers, "bits": BITS, "group_size": GROUP, "M": args.m,
              "sharding": "none" if world == 1 else (f"tp{world}_column_qkv_gate_up_row_o_down_2_allreduce_per_layer"
                                                    if args.tp == "megatron" else f"n_split_{world}_allgather_per_phase"),
              "l2": "working set 3.9 GB per step >> 126 MB L2"}

    if args.impl == "reference":
        if rank != 0:
            return
        val, ms, threads, sample = cpu_reference_arm(args)
        emit({
            "impl": "reference", "metric": METRIC, "value": val, "unit": "GB/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": config,
            "cpu_baseline": {"value": val, "unit": "GB/s", "cores": threads, "kind": "port", "sample": sample},
            "e2e": {"value": val, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0})
        return

    import torch
    import torch.distributed as dist
    from metaltile_b200 import ops

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (no CPU fallback)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    ctx = ops.context(dev)
    for item in args.option:
        name, value = item.split("=")
        ctx.set_option(name, int(value))
    M = args.m

    # ---- synthetic weights, sharded across ranks -------------------------------------------
    # megatron: phases 0 and 2 (q/k/v, gate/up) are N-split and their outputs stay on the rank that made them (the
    # attention heads and the SwiGLU that consume them are sharded the same way); phases 1 and 3 (o, down) are
    # K-split - each rank multiplies its slice of the activations - and summed with one all-reduce each.
    row_parallel = (lambda phase: world > 1 and args.tp == "megatron" and phase in (1, 3))
    gen = torch.Generator(device=dev)
    gen.manual_seed(1234 + rank)
    layers = []
    for _ in range(args.layers):
        mats = []
        for name, k, n, phase in PROJ:
            nl, kl = (n, k // world) if row_parallel(phase) else (n // world, k)
            w = torch.randint(-2 ** 31, 2 ** 31 - 1, (nl, kl * BITS // 32), dtype=torch.int32, device=dev, generator=gen)
            sc = (0.002 + 0.018 * torch.rand((nl, kl // GROUP), device=dev, generator=gen))
            bi = -8.0 * sc + 1e-3 * torch.randn((nl, kl // GROUP), device=dev, generator=gen)
            mats.append((w, sc.to(torch.bfloat16), bi.to(torch.bfloat16), (k, kl), nl, phase))
        layers.append(mats)
    # activations: one x per distinct K
    xs_host = {k: torch.randn((M, k), generator=torch.Generator().manual_seed(7)).to(torch.bfloat16).pin_memory()
               for k in (4096, 14336)}
    xs_full = {k: v.to(dev) for k, v in xs_host.items()}
    # (K, local K) -> the activations a projection reads: all of x, or this rank's K slice (a view for M = 1)
    xs = {}
    for k in (4096, 14336):
        xs[(k, k)] = xs_full[k]
        if world > 1:
            kl = k // world
            xs[(k, kl)] = xs_full[k][:, rank * kl:(rank + 1) * kl]
    # per layer, per phase: local output slab [M, sum(nl)] and the gathered buffer [world, M, sum(nl)];
    # all slabs are views of one allocation, so the end-to-end leg reads the step's results back in one copy
    phase_cols = [sum((n if row_parallel(p) else n // world) for _, _, n, p in PROJ if p == ph) for ph in range(4)]
    gather = world > 1 and args.tp == "gather"
    cols_per_layer = sum(phase_cols)
    local_all = torch.empty(args.layers * M * cols_per_layer, dtype=torch.bfloat16, device=dev)
    p2p = gather and args.collective in ("p2p", "auto") and M == 1
    if p2p and args.collective == "auto":
        p2p = p2p_trial(ctx, dev, rank, world,
                        next((int(o.split("=")[1]) for o in args.option if o.startswith("qmv_stream=")), 1))
    config_collective = "p2p" if p2p else "nccl"
    peer = None
    if p2p:
        from metaltile_b200.parallel import PeerGather
        peer = PeerGather(ctx, args.layers * world * M * cols_per_layer * 2)
        full_all = peer.tensor(torch.bfloat16)
    else:
        full_all = torch.empty(args.layers * world * M * cols_per_layer, dtype=torch.bfloat16, device=dev) if gather else None
    out_local, out_full = [], ([] if gather else None)
    full_off = []                                  # element offset of every (layer, phase) gathered block
    lo = fo = 0
    for _ in range(args.layers):
        ll, fl = [], []
        for c in phase_cols:
            ll.append(local_all[lo:lo + M * c].view(M, c))
            lo += M * c
            if gather:
                fl.append(full_all[fo:fo + world * M * c].view(world * M, c))
                full_off.append(fo)
                fo += world * M * c
        out_local.append(ll)
        if gather:
            out_full.append(fl)
    # each projection writes its own contiguous [M, nl] tile, then tiles are packed per phase
    tiles = [[torch.empty((M, nl), dtype=torch.bfloat16, device=dev) for (_, _, _, _, nl, _) in mats] for mats in layers]
    if world == 1 and M > 1:
        # nothing is exchanged on one GPU: the tiles themselves are the result, laid out one after the other in the
        # result allocation (same bytes as the per-phase slabs), and no packing copy is launched
        to = 0
        for li, mats in enumerate(layers):
            for pi, (_, _, _, _, nl, _) in enumerate(mats):
                tiles[li][pi] = local_all[to:to + M * nl].view(M, nl)
                to += M * nl

    # the projections of one phase (q/k/v; gate/up) read the same activations and are independent:
    # with --streams > 1 they are launched on parallel streams, joined before the phase's all-gather
    branches = [torch.cuda.Stream() for _ in range(max(0, args.streams - 1))]

    def step():
        main = torch.cuda.current_stream()
        for li, mats in enumerate(layers):
            for ph in range(4):
                col = 0
                used = []
                for pi, (w, sc, bi, k, nl, phase) in enumerate(mats):
                    if phase != ph:
                        continue
                    lane = len(used) % (len(branches) + 1)
                    st = main if lane == 0 else branches[lane - 1]
                    if st is not main and st not in used:
                        st.wait_stream(main)
                    used.append(st)
                    with torch.cuda.stream(st):
                        if p2p:      # this rank's slot of the gathered block, in every rank's buffer
                            c = phase_cols[ph]
                            off = (full_off[li * 4 + ph] + rank * M * c + col) * 2
                            peer.qmv_into(w, sc, bi, xs[k], BITS, GROUP, off, st.cuda_stream)
                        elif M == 1:   # a [1, nl] slice of the phase slab is contiguous: write in place
                            ops.qmv(w, sc, bi, xs[k], BITS, GROUP, out=out_local[li][ph][:, col:col + nl], ctx=ctx)
                        else:
                            xin = xs[k] if xs[k].is_contiguous() else xs[k].contiguous()
                            ops.qmv(w, sc, bi, xin, BITS, GROUP, out=tiles[li][pi], ctx=ctx)
                            if world > 1:
                                out_local[li][ph][:, col:col + nl].copy_(tiles[li][pi])
                    col += nl
                for st in set(used):
                    if st is not main:
                        main.wait_stream(st)
                if p2p:
                    peer.barrier(main.cuda_stream)
                elif gather:
                    dist.all_gather_into_tensor(out_full[li][ph], out_local[li][ph])
                elif row_parallel(ph):
                    dist.all_reduce(out_local[li][ph])

    launches_per_step = 7 * args.layers
    run_info = {"dispatch": "one launch per projection"}
    chain = None
    if world == 1 and args.mode in ("chain", "batched"):
        from metaltile_b200.ops import _projection

        def out_of(li, pi, phase, col, nl):
            return out_local[li][phase][:, col:col + nl] if M == 1 else tiles[li][pi]

        if args.mode == "chain":
            # one prepared chain for the whole step: a persistent grid walks the 224 projections, the four dependent
            # phases of every layer are device-side counters instead of launch boundaries
            projs = []
            for li, mats in enumerate(layers):
                col = [0, 0, 0, 0]
                for pi, (w, sc, bi, k, nl, phase) in enumerate(mats):
                    projs.append(_projection(w, sc, bi, xs[k], BITS, GROUP, [out_of(li, pi, phase, col[phase], nl)], phase=li * 4 + phase))
                    col[phase] += nl
            chain = ctx.chain_create(projs)
            if chain.fused:
                launches_per_step = 1

                def step():      # noqa: F811
                    chain.run(torch.cuda.current_stream().cuda_stream)
            run_info["dispatch"] = "one chain per step" if chain.fused else "one launch per projection"
        else:
            # projections of a phase read the same activations: one launch per phase (q/k/v, o, gate/up, down),
            # the counterpart of ffai_batched_qkv_qgemv (crates/metaltile-std/src/ffai/batched_qkv_qgemv.rs:1-35)
            groups = []
            for li, mats in enumerate(layers):
                col = [0, 0, 0, 0]
                per_phase = [[], [], [], []]
                for pi, (w, sc, bi, k, nl, phase) in enumerate(mats):
                    per_phase[phase].append(_projection(w, sc, bi, xs[k], BITS, GROUP, [out_of(li, pi, phase, col[phase], nl)]))
                    col[phase] += nl
                groups.extend(g for g in per_phase if g)
            launches_per_step = len(groups)

            def step():      # noqa: F811
                st = torch.cuda.current_stream().cuda_stream
                for g in groups:
                    ctx.qmv_batched(g, st)
            run_info["dispatch"] = "one launch per phase (projections that share x fused)"
    barrier_launches = 4 * args.layers if p2p else 0
    if p2p and args.mode == "batched":
        # sharded decode: one launch per phase whose kernel stores this rank's tiles into every rank's gathered block
        # and carries the hand-off itself (wait for the peers' previous launch, publish its own completion); one barrier
        # kernel at the end of the step, before anything outside the chain of launches reads the blocks
        pgroups = []
        for li, mats in enumerate(layers):
            for ph in range(4):
                col, g, offs, k0 = 0, [], [], None
                for (w, sc, bi, k, nl, phase) in mats:
                    if phase != ph:
                        continue
                    g.append((w, sc, bi))
                    offs.append((full_off[li * 4 + ph] + rank * M * phase_cols[ph] + col) * 2)
                    col += nl
                    k0 = k
                pgroups.append((g, xs[k0], offs))

        def step():      # noqa: F811
            st = torch.cuda.current_stream().cuda_stream
            for g, x, offs in pgroups:
                peer.batched_into(g, x, BITS, GROUP, offs, st)
            peer.barrier(st)
        launches_per_step, barrier_launches = len(pgroups), 1
        run_info["dispatch"] = "one launch per phase (projections that share x fused), hand-off between the GPUs inside the kernel"
    # capture the step in a CUDA graph: 224 launches of ~1-5 us each are otherwise host-bound
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(2):
            step()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    if p2p and args.verify:
        # the blocks the kernels' own stores assembled must equal an NCCL all-gather of the same projections
        dist.barrier()
        bad = 0
        stream_opt = next((int(o.split("=")[1]) for o in args.option if o.startswith("qmv_stream=")), 1)
        ctx.set_option("qmv_stream", 2)     # the reference shards on the kernel the peer path runs, whatever their size
        for li in (0, args.layers - 1):
            for ph in range(4):
                c, col = phase_cols[ph], 0
                loc = torch.empty((M, c), dtype=torch.bfloat16, device=dev)
                for (w, sc, bi, k, nl, phase) in layers[li]:
                    if phase == ph:
                        ops.qmv(w, sc, bi, xs[k], BITS, GROUP, out=loc[:, col:col + nl], ctx=ctx)
                        col += nl
                ref = torch.empty((world * M, c), dtype=torch.bfloat16, device=dev)
                dist.all_gather_into_tensor(ref, loc)
                bad += int(not torch.equal(ref, out_full[li][ph]))
        ctx.set_option("qmv_stream", stream_opt)
        torch.cuda.synchronize()
        print(f"[rank {rank}] p2p gather vs NCCL all-gather: {'identical' if bad == 0 else str(bad) + ' blocks differ'}; "
              f"status word {ctx.status_word():#x}", file=sys.stderr, flush=True)
        if bad or ctx.status_word():
            raise SystemExit("p2p gather failed verification")
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        step()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1) / steps
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    for _ in range(args.warmup):
        graph.replay()
    verified = None
    if rank == 0:
        if not (world > 1 and args.tp == "megatron"):      # row-parallel outputs are sums over ranks: nothing local to compare
            verified = spot_check(layers, xs, tiles, out_local, out_full if p2p else None, M, world, phase_cols)
    sampler = ClockSampler(local_rank)
    sampler.start()
    ms = timed(graph.replay, args.steps)
    clocks = sampler.stop()
    total_bytes = step_bytes(M, args.layers)       # whole job (all ranks together)
    value = total_bytes / (ms * 1e-3) / 1e9

    # ---- end to end: pinned host activations in, host results out, through the C ABI ---------
    result_dev = full_all if gather else local_all
    out_host = torch.empty(result_dev.numel(), dtype=torch.bfloat16).pin_memory()
    h2d = sum(v.numel() * 2 for v in xs_host.values())
    d2h = result_dev.numel() * 2
    stream = torch.cuda.current_stream().cuda_stream
    lib, h = ctx._lib, ctx._h

    def e2e_step():
        for k, v in xs_host.items():
            lib.mtc_upload(h, stream, xs_full[k].data_ptr(), v.data_ptr(), v.numel() * 2)
        graph.replay()
        lib.mtc_download(h, stream, out_host.data_ptr(), result_dev.data_ptr(), d2h)
        lib.mtc_sync(h, stream)

    for _ in range(3):
        e2e_step()
    e2e_steps = max(3, min(args.steps, 50))
    e2e_ms = timed(e2e_step, e2e_steps)
    e2e_value = total_bytes / (e2e_ms * 1e-3) / 1e9

    def finish():
        # NCCL communicators captured in a CUDA graph do not tear down reliably: leave without destroying them
        sys.stdout.flush()
        sys.stderr.flush()
        if world > 1:
            os._exit(0)

    multi = None
    if world > 1 and not args.no_extra:
        try:
            multi = multi_gpu_extras(ctx, dev, rank, world, timed, peer_ok=p2p)
        except Exception as e:  # all ranks take the same path: an exception here is raised on every rank or on none
            multi = {"error": repr(e)}
    if rank != 0:
        finish()
        return

    if world > 1:
        run_info["collective"] = config_collective
    hbm_peak, tf_burst, tf_sus, peak_kind = measured_peaks()
    per_launch_bytes = total_bytes / world / launches_per_step
    us_per_launch = ms * 1e3 / launches_per_step
    roofline = {"bound": "hbm", "achieved": value / world, "peak": hbm_peak, "unit": "GB/s",
                "frac": value / world / hbm_peak, "traffic": per_launch_bytes * NCU_TRAFFIC_RATIO, "peak_kind": peak_kind,
                "traffic_source": f"ncu dram bytes / algorithmic bytes = {NCU_TRAFFIC_RATIO} on the 14336x4096 launch of the streaming kernel, scaled to the average launch",
                "kernel": "qmv_stream_kernel<bf16, g64, M1>", "alg_bytes_per_launch": per_launch_bytes,
                "avg_us_per_launch": us_per_launch,
                "note": "per-GPU; launch-averaged over the 4 matrix shapes of the step (graph replay, events)"}
    line = {"metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": config, "run": run_info, "verified": verified,
            "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": e2e_ms},
            "gpu_launches": (launches_per_step + barrier_launches) * args.steps, "roofline": roofline}

    if not args.no_extra:
        try:
            line["extra"] = extra_measurements(ctx, dev, hbm_peak, tf_burst, local_rank, layers if world == 1 else None)
        except Exception as e:  # secondary numbers must never sink the headline line
            line["extra"] = {"error": repr(e)}
        if multi is not None:
            line["extra"].update(multi)
    if not args.no_cpu and world == 1:
        try:
            ns = argparse.Namespace(m=M, steps=3, warmup=1)
            val, cms, threads, sample = cpu_reference_arm(ns)
            line["cpu_baseline"] = {"value": val, "unit": "GB/s", "cores": threads, "kind": "port",
                                    "sample": sample, "ms_per_sample": cms}
        except Exception as e:
            line["cpu_baseline"] = {"error": repr(e)}
    emit(line)
    finish()


def multi_gpu_extras(ctx, dev, rank, world, timed, peer_ok=False):
    """The sharded forms of the prefill matmul (config 3: N-split + all-gather) and of the MoE layer (config 4: expert
    parallel, all-to-all dispatch and combine), run by every rank; rank 0 checks its result against the unsharded
    kernels on the same data (sharding changes no row's arithmetic, so the comparison is for equality)."""
    import torch
    import torch.distributed as dist
    from metaltile_b200 import ops
    from metaltile_b200.parallel import ColumnParallelLinear, ExpertParallelMoE, ExpertShard, CudaBackend, shard_rows
    out = {}
    be = CudaBackend(ctx)

    def same_on_all_ranks(seed):
        g = torch.Generator(device=dev)
        g.manual_seed(seed)          # same generator, same device type: every rank draws the same numbers
        return g

    # ---- config 3: x bf16 [2048, K], W K -> N, every rank owns N / world weight rows
    for name, (m, n, k) in {"c3_qmm_nsplit_4096to14336": (2048, 14336, 4096), "c3_qmm_nsplit_14336to4096": (2048, 4096, 14336)}.items():
        g = same_on_all_ranks(4242)
        w = torch.randint(-2 ** 31, 2 ** 31 - 1, (n, k * BITS // 32), dtype=torch.int32, device=dev, generator=g)
        sc = (0.002 + 0.018 * torch.rand((n, k // GROUP), device=dev, generator=g)).to(torch.bfloat16)
        bi = (-8.0 * sc.float()).to(torch.bfloat16)
        x = torch.randn((m, k), device=dev, generator=g).to(torch.bfloat16)
        r0, r1 = shard_rows(n, world, rank)
        lin = ColumnParallelLinear(w[r0:r1].contiguous(), sc[r0:r1].contiguous(), bi[r0:r1].contiguous(), BITS, GROUP, backend=be)
        got = lin.forward(x)
        torch.cuda.synchronize()
        verified = None
        if rank == 0:
            ref = ops.qmm(w, sc, bi, x, BITS, GROUP, ctx=ctx)
            torch.cuda.synchronize()
            verified = bool(torch.equal(ref, got))
        ms = timed(lambda: lin.forward(x), 5)
        tf = 2.0 * m * n * k / (ms * 1e-3) / 1e12
        out[name] = {"us": ms * 1e3, "TFLOP/s": tf, "ranks": world, "verified": verified,
                     "note": "aggregate over all ranks, NCCL all-gather of the [M, N / ranks] slices and the row-major interleave included"}
        # the same product with the all-gather fused into the kernel: every rank's epilogue stores its column block into
        # every rank's [M, N] buffer through peer mappings; one barrier kernel makes the blocks visible
        if peer_ok:
            try:
                from metaltile_b200.parallel import PeerGather
                pg = PeerGather(ctx, m * n * 2)
                wl, sl, bl = lin.w, lin.scales, lin.biases
                st = torch.cuda.current_stream().cuda_stream

                def fused():
                    pg.qmm_into(wl, sl, bl, x, BITS, GROUP, n, r0, torch.cuda.current_stream().cuda_stream)
                    pg.barrier(torch.cuda.current_stream().cuda_stream)

                fused()
                torch.cuda.synchronize()
                dist.barrier()
                v2 = None
                if rank == 0:
                    v2 = bool(torch.equal(ref.reshape(-1), pg.tensor(torch.bfloat16)[:m * n])) and ctx.status_word() == 0
                ms2 = timed(fused, 5)
                out[name + "_fused"] = {"us": ms2 * 1e3, "TFLOP/s": 2.0 * m * n * k / (ms2 * 1e-3) / 1e12, "ranks": world, "verified": v2,
                                        "note": "aggregate over all ranks; the kernel's epilogue stores each rank's column block into "
                                                "every rank's [M, N] buffer (peer stores), one barrier kernel; no NCCL call"}
                dist.barrier()
                pg.close()
            except Exception as e:   # the peer path is optional: the NCCL figure above stands
                print(f"[rank {rank}] fused qmm all-gather unavailable: {e!r}", file=sys.stderr, flush=True)
        del w, sc, bi, x, lin, got
    # ---- config 4: 512 tokens (data parallel), 128 experts split over the ranks, top-8
    T, H, I, E, K8 = 512, 2048, 768, 128, 8
    if E % world == 0 and T % world == 0:
        g = same_on_all_ranks(777)

        def experts(n, k):
            w = torch.randint(-2 ** 31, 2 ** 31 - 1, (E, n, k * BITS // 32), dtype=torch.int32, device=dev, generator=g)
            sc = (0.002 + 0.018 * torch.rand((E, n, k // GROUP), device=dev, generator=g)).to(torch.bfloat16)
            return w, sc, (-8.0 * sc.float()).to(torch.bfloat16)

        gate, up, down = experts(I, H), experts(I, H), experts(H, I)
        tok = torch.randn((T, H), device=dev, generator=g).to(torch.bfloat16)
        logits = torch.randn((T, E), device=dev, generator=g).to(torch.bfloat16)
        e0, e1 = rank * (E // world), (rank + 1) * (E // world)
        t0, t1 = rank * (T // world), (rank + 1) * (T // world)
        cut = lambda trip: tuple(a[e0:e1].contiguous() for a in trip)
        moe = ExpertParallelMoE(ExpertShard(cut(gate), cut(up), cut(down), BITS, GROUP), E, K8, 1, backend=be)
        tl, ll = tok[t0:t1].contiguous(), logits[t0:t1].contiguous()
        got = moe.forward(tl, ll)
        torch.cuda.synchronize()
        verified = None
        if rank == 0:
            one = ExpertParallelMoE(ExpertShard(gate, up, down, BITS, GROUP), E, K8, 1, backend=be, group=None)
            one.world, one.e_local = 1, E          # the unsharded layer on this rank's tokens
            ref = one.forward(tl, ll)
            torch.cuda.synchronize()
            verified = bool(torch.equal(ref, got))
            if not verified:
                verified = {"max_abs_diff": float((ref.float() - got.float()).abs().max())}
        ms = timed(lambda: moe.forward(tl, ll), 5)
        flops = 2.0 * T * K8 * 3 * H * I
        out["c4_moe_ep"] = {"us": ms * 1e3, "TFLOP/s": flops / (ms * 1e-3) / 1e12, "ranks": world, "verified": verified,
                            "tokens_per_rank": T // world, "experts_per_rank": E // world,
                            "note": "per layer, both all-to-alls (dispatch, combine) and the count exchange included"}
    return out


def extra_measurements(ctx, dev, hbm_peak, tf_peak, local_rank=0, layers=None):
    """Single-kernel numbers for the other configurations (cold L2: buffers rotate through > 126 MB).  Every entry
    carries the SM clock sampled while it ran."""
    import torch
    from metaltile_b200 import ops
    out = {}

    def with_clocks(fn):
        sampler = ClockSampler(local_rank)
        sampler.start()
        val = fn()
        c = sampler.stop()
        return val, {"sm_mhz": c["sm_mhz"], "reasons": c["reasons"]}
    gen = torch.Generator(device=dev)
    gen.manual_seed(99)

    def make(n, k, m, copies):
        sets = []
        for _ in range(copies):
            w = torch.randint(-2 ** 31, 2 ** 31 - 1, (n, k * BITS // 32), dtype=torch.int32, device=dev, generator=gen)
            sc = (0.002 + 0.018 * torch.rand((n, k // GROUP), device=dev, generator=gen)).to(torch.bfloat16)
            bi = (-8.0 * sc.float()).to(torch.bfloat16)
            sets.append((w, sc, bi))
        x = torch.randn((m, k), device=dev, generator=gen).to(torch.bfloat16)
        o = torch.empty((m, n), dtype=torch.bfloat16, device=dev)
        return sets, x, o

    def time_rot(fn_list, reps):
        g = torch.cuda.CUDAGraph()
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            for f in fn_list:
                f()
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize()
        with torch.cuda.graph(g):
            for f in fn_list:
                f()
        for _ in range(3):
            g.replay()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(reps):
            g.replay()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1e3 / (reps * len(fn_list))  # us per launch

    for name, (m, n, k) in {"c0_qmv_m1_4096x4096": (1, 4096, 4096), "qmv_m1_8192x8192": (1, 8192, 8192),
                            "qmv_m8_4096x4096": (8, 4096, 4096), "qmv_m16_4096x4096": (16, 4096, 4096)}.items():
        copies = max(2, int(300e6 // alg_bytes(m, n, k)) + 1)   # > 2x L2 in rotation
        sets, x, o = make(n, k, m, copies)
        fns = [(lambda w=w, sc=sc, bi=bi: ops.qmv(w, sc, bi, x, BITS, GROUP, out=o, ctx=ctx)) for (w, sc, bi) in sets]
        us, clk = with_clocks(lambda: time_rot(fns, 20))
        gbs = alg_bytes(m, n, k) / us / 1e3
        out[name] = {"us": us, "GB/s": gbs, "frac_of_hbm_peak": gbs / hbm_peak, "cold_l2_copies": copies, "clocks": clk}
        del sets, fns
    # ---- prefill qmm on the tensor cores (M = 2048), TFLOP/s = 2*M*N*K / time
    def time_calls(fn, reps=10):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1e3 / reps

    for name, (m, n, k) in {"c3_qmm_m2048_4096to14336": (2048, 14336, 4096), "c3_qmm_m2048_14336to4096": (2048, 4096, 14336)}.items():
        sets, x, o = make(n, k, m, 1)
        w, sc, bi = sets[0]
        us, clk = with_clocks(lambda: time_calls(lambda: ops.qmm(w, sc, bi, x, BITS, GROUP, out=o, ctx=ctx)))
        tf = 2.0 * m * n * k / us / 1e6
        out[name] = {"us": us, "TFLOP/s": tf, "frac_of_bf16_peak": tf / tf_peak, "route": ctx.qmm_route(m, n, k, BITS, GROUP, "bf16"),
                     "clocks": clk}
        del sets

    # ---- MoE layer: 512 tokens x hidden 2048, 128 experts (gate/up 2048->768, down 768->2048), top-8
    T, H, I, E, K8 = 512, 2048, 768, 128, 8

    def experts(n, k):
        w = torch.randint(-2 ** 31, 2 ** 31 - 1, (E, n, k * BITS // 32), dtype=torch.int32, device=dev, generator=gen)
        sc = (0.002 + 0.018 * torch.rand((E, n, k // GROUP), device=dev, generator=gen)).to(torch.bfloat16)
        return w, sc, (-8.0 * sc.float()).to(torch.bfloat16)

    # two layers with their own weights (2 x 340 MB), replayed from one CUDA graph: every layer finds its weights cold
    # in L2, and the figure is device time, not the host's launch time
    sets = [(experts(I, H), experts(I, H), experts(H, I)) for _ in range(2)]
    tok = torch.randn((T, H), device=dev, generator=gen).to(torch.bfloat16)
    logits = torch.randn((T, E), device=dev, generator=gen).to(torch.bfloat16)

    def moe_layer(gate, up, down):
        idx, wts = ops.moe_router_topk(logits, K8, 1, ctx=ctx)
        sti, inv, off, _ = ops.moe_sort(idx, E, ctx=ctx)
        y = ops.moe_experts(tok, gate, up, down, BITS, GROUP, off, sort_token_idx=sti, ctx=ctx)
        return ops.moe_unpermute(y, inv, wts, ctx=ctx)

    def two_layers():
        for gate, up, down in sets:
            moe_layer(gate, up, down)

    two_layers()                                   # scratch blocks of the context reach their size before the capture
    torch.cuda.synchronize()
    moe_graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(moe_graph):
        two_layers()
    us, clk = with_clocks(lambda: time_calls(moe_graph.replay))
    us /= 2
    flops = 2.0 * T * K8 * 3 * H * I
    wbytes = 3 * E * (H * I * BITS // 8 + 2 * (H * I // GROUP) * 2)
    out["c4_moe_layer_512tok_128e_top8"] = {"us": us, "TFLOP/s": flops / us / 1e6, "weight_GB/s": wbytes / us / 1e3,
                                            "frac_of_hbm_peak": wbytes / us / 1e3 / hbm_peak,
                                            "route": ctx.gather_qmm_route(T * K8, I, H, E, BITS, GROUP, "bf16"),
                                            "note": "HBM-bound: 340 MB of expert weights per layer; two layers with separate weights "
                                                    "replayed from one CUDA graph (cold L2, device time)", "clocks": clk}
    del sets, moe_graph
    # ---- the decode set at M = 8 (config 2 names M = 1 and 8): the step's own weights, 8 activation rows
    if layers is not None:
        from metaltile_b200.ops import _projection
        m8 = 8
        x8 = {k: torch.randn((m8, k), device=dev, generator=gen).to(torch.bfloat16) for k in (4096, 14336)}
        groups, keep = [], []
        for mats in layers:
            per_phase = [[], [], [], []]
            for (w, sc, bi, k, nl, phase) in mats:
                o = torch.empty((m8, nl), dtype=torch.bfloat16, device=dev)
                keep.append(o)
                per_phase[phase].append(_projection(w, sc, bi, x8[k[0]], BITS, GROUP, [o]))
            groups.extend(g for g in per_phase if g)

        def step8():
            st = torch.cuda.current_stream().cuda_stream
            for g in groups:
                ctx.qmv_batched(g, st)

        us, clk = with_clocks(lambda: time_rot([step8], 10))
        nbytes = step_bytes(m8, len(layers))
        out["c2_decode_set_m8"] = {"ms": us / 1e3, "GB/s": nbytes / us / 1e3, "frac_of_hbm_peak": nbytes / us / 1e3 / hbm_peak,
                                   "launches": len(groups) if ctx.qmm_route(m8, 4096, 4096, BITS, GROUP, "bf16") == "qmv_stream"
                                   else sum(len(g) for g in groups),
                                   "route": ctx.qmm_route(m8, 4096, 4096, BITS, GROUP, "bf16"), "clocks": clk}
    return out


def emit(line: dict):
    """The result line goes to the process's original stdout; everything else any library prints goes to stderr."""
    _RESULT_OUT.write(json.dumps(line) + "\n")
    _RESULT_OUT.flush()


if __name__ == "__main__":
    # libraries loaded later (NCCL prints its version line from C) write to file descriptor 1: keep a private copy of it
    # for the one JSON line and point descriptor 1 at stderr
    sys.stdout.flush()
    _RESULT_OUT = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)
    main()
