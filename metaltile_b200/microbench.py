"""One kernel family at one shape, timed with CUDA events: the command to put under a profiler.

    python -m metaltile_b200.microbench qmv --m 1 --n 14336 --k 4096 --bits 4 --copies 8
    python -m metaltile_b200.microbench qmm --m 2048 --n 2304 --k 4096 --dtype bf16
    python -m metaltile_b200.microbench qvm --m 1 --n 4096 --k 14336 --bits 4 --copies 8
    python -m metaltile_b200.microbench sweep --dtype bf16       # bits x group x M x K = N grid, one line per cell
    python -m metaltile_b200.microbench moe --tokens 512 --hidden 2048 --inter 768 --experts 128 --top-k 8

`qmv` and `qvm` cycle through `--copies` independent weight sets so that consecutive launches do not find
their weights in L2 (pick copies * bytes > 126 MB for DRAM figures); `qmm` and `moe` reuse one set,
as a prefill does.  Prints one line per repetition: microseconds per launch (qmv, qmm) or per
layer (moe).  Counterpart of the reference's `tile bench --kernel NAME` for a single shape
(crates/metaltile-std/src/run_kernel.rs:197).
"""
from __future__ import annotations

import argparse

import torch

from . import ops

_DT = {"bf16": torch.bfloat16, "f16": torch.float16, "f32": torch.float32}


def _weights(shape_prefix, n, k, bits, group, dt, dev):
    w = torch.randint(-2 ** 31, 2 ** 31 - 1, (*shape_prefix, n, k * bits // 32), dtype=torch.int32, device=dev)
    sc = (0.002 + 0.018 * torch.rand((*shape_prefix, n, k // group), device=dev)).to(dt)
    return w, sc, (-8.0 * sc.float()).to(dt)


def _timed(fn, reps, per):
    for _ in range(reps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        print(f"us {e0.elapsed_time(e1) * 1e3 / per:.2f}", flush=True)


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("family", choices=["qmv", "qvm", "qmm", "moe", "sweep"])
    ap.add_argument("--m", type=int, default=1)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--bits", type=int, default=4)
    ap.add_argument("--group", type=int, default=64)
    ap.add_argument("--dtype", choices=sorted(_DT), default="bf16")
    ap.add_argument("--copies", type=int, default=8)
    ap.add_argument("--reps", type=int, default=3)
    ap.add_argument("--tokens", type=int, default=512)
    ap.add_argument("--hidden", type=int, default=2048)
    ap.add_argument("--inter", type=int, default=768)
    ap.add_argument("--experts", type=int, default=128)
    ap.add_argument("--top-k", type=int, default=8)
    ap.add_argument("--option", action="append", default=[], metavar="NAME=VALUE", help="mtc_set_option before running")
    a = ap.parse_args(argv)

    dev = torch.device("cuda", 0)
    ctx = ops.context(0)
    for item in a.option:
        name, value = item.split("=")
        ctx.set_option(name, int(value))
    dt = _DT[a.dtype]

    if a.family == "sweep":
        # the sweep grid of the qmv family: every cell cycles enough weight copies to exceed L2 twice over
        hbm = 6552.3
        print("bits group M KN us GB/s frac_of_6552", flush=True)
        for kn in (2048, 4096, 8192):
            for bits in (2, 3, 4, 6, 8):
                for group in (32, 64, 128):
                    nbytes = kn * kn * bits // 8 + 2 * kn * (kn // group) * dt.itemsize
                    copies = max(2, min(256, -(-2 * 132_000_000 // nbytes)))
                    scale = 16.0 / 2 ** bits
                    sets = []
                    for _ in range(copies):
                        w = torch.randint(-2 ** 31, 2 ** 31 - 1, (kn, kn * bits // 32), dtype=torch.int32, device=dev)
                        sc = (scale * (0.002 + 0.018 * torch.rand((kn, kn // group), device=dev))).to(dt)
                        sets.append((w, sc, (-(2 ** (bits - 1)) * sc.float()).to(dt)))
                    for m in (1, 4, 8, 16):
                        x = torch.randn((m, kn), device=dev).to(dt)
                        out = torch.empty((m, kn), dtype=dt, device=dev)

                        def body():
                            for w, sc, bi in sets:
                                ops.qmv(w, sc, bi, x, bits, group, out=out, ctx=ctx)

                        body()
                        torch.cuda.synchronize()
                        graph = torch.cuda.CUDAGraph()
                        with torch.cuda.graph(graph):
                            body()
                        graph.replay()
                        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                        torch.cuda.synchronize()
                        e0.record()
                        for _ in range(a.reps):
                            graph.replay()
                        e1.record()
                        torch.cuda.synchronize()
                        us = e0.elapsed_time(e1) * 1e3 / (a.reps * copies)
                        tot = nbytes + 2 * m * kn * dt.itemsize
                        print(f"{bits} {group} {m} {kn} {us:.2f} {tot / us / 1e3:.0f} {tot / us / 1e3 / hbm:.3f}", flush=True)
                        del graph
                    del sets
                    torch.cuda.empty_cache()
    elif a.family in ("qmv", "qvm", "qmm"):
        copies = a.copies if a.family != "qmm" else 1
        if a.family == "qvm":                # transposed storage: w [K, N*bits/32], scales / biases [K/group, N]
            sets = []
            for _ in range(copies):
                w = torch.randint(-2 ** 31, 2 ** 31 - 1, (a.k, a.n * a.bits // 32), dtype=torch.int32, device=dev)
                sc = (0.002 + 0.018 * torch.rand((a.k // a.group, a.n), device=dev)).to(dt)
                sets.append((w, sc, (-8.0 * sc.float()).to(dt)))
        else:
            sets = [_weights((), a.n, a.k, a.bits, a.group, dt, dev) for _ in range(copies)]
        x = torch.randn((a.m, a.k), device=dev).to(dt)
        out = torch.empty((a.m, a.n), dtype=dt, device=dev)
        op = {"qmv": ops.qmv, "qvm": ops.qvm, "qmm": ops.qmm}[a.family]

        def body():
            for w, sc, bi in sets:
                op(w, sc, bi, x, a.bits, a.group, out=out, ctx=ctx)

        body()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()       # replay the launches from a graph: the figure is device time, not host launch time
        with torch.cuda.graph(graph):
            body()
        _timed(graph.replay, a.reps, copies)
    else:
        t, h, i, e = a.tokens, a.hidden, a.inter, a.experts
        gate, up, down = (_weights((e,), i, h, a.bits, a.group, dt, dev), _weights((e,), i, h, a.bits, a.group, dt, dev),
                          _weights((e,), h, i, a.bits, a.group, dt, dev))
        tok = torch.randn((t, h), device=dev).to(dt)
        logits = torch.randn((t, e), device=dev).to(dt)

        def layer():
            idx, wts = ops.moe_router_topk(logits, a.top_k, 1, ctx=ctx)
            sti, inv, off, _ = ops.moe_sort(idx, e, ctx=ctx)
            y = ops.moe_experts(tok, gate, up, down, a.bits, a.group, off, sort_token_idx=sti, ctx=ctx)
            return ops.moe_unpermute(y, inv, wts, ctx=ctx)

        layer()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()       # device time of the layer's launches, not the host's launch time
        with torch.cuda.graph(graph):
            layer()
        _timed(graph.replay, a.reps, 1)
    print("status_word", ctx.status_word())


if __name__ == "__main__":
    main()
