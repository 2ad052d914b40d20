"""Host-side mirror of the reference's runtime interface, over the C ABI.

``Context`` follows ``metaltile_runtime::Context``
(crates/metaltile-runtime/src/context.rs:160-399): ``dispatch_with_grid`` binds
host byte buffers and constexprs BY NAME, runs the kernel selected by its
reference name and returns the output buffers plus the kernel's device time.
``MetalTileError`` carries the same variants as crates/metaltile-runtime/src/error.rs:7-56.
The typed methods (``qmv``, ``qmm`` ...) take device pointers and are asynchronous;
they are what a resident-buffer caller (GpuRunner, crates/metaltile-std/src/runner.rs:413)
uses.
"""
from __future__ import annotations

import ctypes
import json
from dataclasses import dataclass, field
from typing import Dict, Mapping, Optional, Sequence

from . import _lib
from ._lib import BF16, F16, F32, BenchStatsC, DispatchSpec, NamedBuf, PeerSync, QMat, QmvDesc

DTYPES = {"f32": F32, "f16": F16, "bf16": BF16}


class MetalTileError(RuntimeError):
    """Error of a back-end call; ``variant`` is the reference's enum variant name."""

    def __init__(self, code: int, message: str):
        self.code = code
        self.variant = _lib.STATUS_NAMES.get(code, f"Unknown({code})")
        super().__init__(f"{self.variant}: {message}")


@dataclass
class DispatchResult:
    """crates/metaltile-runtime/src/context.rs:49-56."""
    outputs: Dict[str, bytes] = field(default_factory=dict)
    elapsed_us: float = 0.0


@dataclass
class BenchStats:
    """crates/metaltile-std/src/stats.rs:5-22: summary of a set of device timings, microseconds."""
    min_us: float
    mean_us: float
    median_us: float
    p95_us: float
    p99_us: float
    stddev_us: float
    cv_pct: float

    def is_valid(self) -> bool:
        return self.mean_us > 0.0


def _dt(dtype) -> int:
    if isinstance(dtype, int):
        return dtype
    return DTYPES[str(dtype).replace("torch.", "").replace("bfloat16", "bf16").replace("float16", "f16")
                  .replace("float32", "f32")]


class Context:
    """One per device; not thread-safe (the caller serialises, as the reference's tests do)."""

    def __init__(self, device: int = 0):
        self._lib = _lib.load()
        h = ctypes.c_void_p()
        rc = self._lib.mtc_init(int(device), ctypes.byref(h))
        if rc != 0:
            raise MetalTileError(rc, (self._lib.mtc_last_error(None) or b"").decode())
        self._h = h
        self.device = int(device)

    # ---- lifecycle ------------------------------------------------------------
    def close(self):
        if getattr(self, "_h", None):
            self._lib.mtc_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _check(self, rc: int):
        if rc != 0:
            raise MetalTileError(rc, (self._lib.mtc_last_error(self._h) or b"").decode())

    def device_info(self) -> dict:
        buf = ctypes.create_string_buffer(1024)
        self._check(self._lib.mtc_device_info(self._h, buf, len(buf)))
        return json.loads(buf.value.decode())

    def status_word(self) -> int:
        w = ctypes.c_uint32()
        self._check(self._lib.mtc_status_word(self._h, ctypes.byref(w)))
        return int(w.value)

    def status_clear(self):
        self._check(self._lib.mtc_status_clear(self._h))

    def sync(self, stream: int = 0, timeout_ms: Optional[int] = None):
        """Wait for ``stream``; raises ``Timeout`` if a kernel gave up on a bounded wait, or (with ``timeout_ms``)
        if the stream is still running after that many milliseconds."""
        if timeout_ms is None:
            self._check(self._lib.mtc_sync(self._h, ctypes.c_void_p(stream)))
        else:
            self._check(self._lib.mtc_sync_deadline(self._h, ctypes.c_void_p(stream), int(timeout_ms)))

    # ---- name-keyed host-buffer dispatch ----------------------------------------
    def dispatch_with_grid(self, kernel: str, buffers: Mapping[str, bytes],
                           fn_consts: Optional[Mapping[str, int]] = None,
                           grid_groups: Sequence[int] = (1, 1, 1),
                           threads_per_group: Sequence[int] = (1, 1, 1),
                           dtype="f32", outputs: Sequence[str] = ("out",)) -> DispatchResult:
        """``Context::dispatch_with_grid`` (context.rs:269-284).

        ``buffers`` maps parameter names to host bytes; constexprs may be given either
        as 4-byte little-endian entries of ``buffers`` (as the reference's test runner
        does, run_kernel.rs:56-65) or through ``fn_consts``.  ``grid_groups`` /
        ``threads_per_group`` are accepted and ignored.
        """
        items = dict(buffers)
        for k, v in (fn_consts or {}).items():
            items[k] = int(v).to_bytes(4, "little")
        keep = []
        arr = (NamedBuf * len(items))()
        for i, (name, data) in enumerate(items.items()):
            raw = ctypes.create_string_buffer(bytes(data), len(data))
            keep.append(raw)
            arr[i].name = name.encode()
            arr[i].data = ctypes.cast(raw, ctypes.c_void_p)
            arr[i].bytes = len(data)
            arr[i].is_output = 1 if name in outputs else 0
        g = (ctypes.c_uint32 * 3)(*[int(v) for v in grid_groups])
        t = (ctypes.c_uint32 * 3)(*[int(v) for v in threads_per_group])
        us = ctypes.c_float(0.0)
        self._check(self._lib.mtc_dispatch(self._h, kernel.encode(), _dt(dtype), arr, len(items), g, t,
                                           ctypes.byref(us)))
        res = DispatchResult(elapsed_us=float(us.value))
        for i, name in enumerate(items):
            if arr[i].is_output:
                res.outputs[name] = keep[i].raw
        return res

    def bench(self, kernel: str, buffers: Mapping[str, bytes], fn_consts: Optional[Mapping[str, int]] = None,
              dtype="f32", outputs: Sequence[str] = ("out",), warmup: int = 15, iters: int = 10, cold_l2: bool = True):
        """``GpuRunner::bench`` (crates/metaltile-std/src/runner.rs:432-442) with the reference's defaults of 15 warm-up and
        10 timed launches (runner.rs:635-636): the buffers are staged once, every timed launch sits between its own pair
        of events, ``cold_l2`` rewrites a block larger than L2 before every launch (``flush_slc``, runner.rs:444-458).
        Returns ``(BenchStats, samples_us, outputs)``; the outputs are the last launch's."""
        items = dict(buffers)
        for k, v in (fn_consts or {}).items():
            items[k] = int(v).to_bytes(4, "little")
        keep = []
        arr = (NamedBuf * len(items))()
        for i, (name, data) in enumerate(items.items()):
            raw = ctypes.create_string_buffer(bytes(data), len(data))
            keep.append(raw)
            arr[i].name = name.encode()
            arr[i].data = ctypes.cast(raw, ctypes.c_void_p)
            arr[i].bytes = len(data)
            arr[i].is_output = 1 if name in outputs else 0
        samples = (ctypes.c_double * int(iters))()
        st = BenchStatsC()
        self._check(self._lib.mtc_measure(self._h, kernel.encode(), _dt(dtype), arr, len(items), int(warmup), int(iters),
                                          1 if cold_l2 else 0, samples, ctypes.byref(st)))
        stats = BenchStats(**{n: getattr(st, n) for n in ("min_us", "mean_us", "median_us", "p95_us", "p99_us", "stddev_us", "cv_pct")})
        outs = {name: keep[i].raw for i, name in enumerate(items) if arr[i].is_output}
        return stats, list(samples), outs

    def bench_gbps(self, kernel: str, buffers: Mapping[str, bytes], nbytes: float, **kw):
        """``bench_gbps`` (crates/metaltile-std/src/runner.rs:638-650): GB/s of ``nbytes`` over the minimum sample."""
        stats, _, _ = self.bench(kernel, buffers, **kw)
        return (nbytes / (stats.min_us * 1e-6) / 1e9 if stats.is_valid() else None), stats

    def dispatch_chain(self, passes) -> list:
        """``Context::dispatch_chain`` (context.rs:347-395): ``passes`` is a list of
        ``(kernel, buffers, fn_consts, dtype, outputs)``; a buffer that one pass outputs and a later pass binds under the
        same name stays on the device.  Returns one ``DispatchResult`` per pass; outputs consumed by a later pass are
        not read back (their entry is absent), ``elapsed_us`` of the last result is the device time of the chain."""
        specs = (DispatchSpec * len(passes))()
        keep, per_pass = [], []
        for si, (kernel, buffers, fn_consts, dtype, outputs) in enumerate(passes):
            items = dict(buffers)
            for k, v in (fn_consts or {}).items():
                items[k] = int(v).to_bytes(4, "little")
            arr = (NamedBuf * len(items))()
            raws = []
            for i, (name, data) in enumerate(items.items()):
                raw = ctypes.create_string_buffer(bytes(data), len(data))
                raws.append(raw)
                arr[i].name = name.encode()
                arr[i].data = ctypes.cast(raw, ctypes.c_void_p)
                arr[i].bytes = len(data)
                arr[i].is_output = 1 if name in outputs else 0
            keep.append((arr, raws))
            per_pass.append((list(items), set(outputs)))
            specs[si].kernel_name = kernel.encode()
            specs[si].dtype = _dt(dtype)
            specs[si].bufs = ctypes.cast(arr, ctypes.c_void_p)
            specs[si].n_bufs = len(items)
        us = ctypes.c_float(0.0)
        self._check(self._lib.mtc_dispatch_chain(self._h, specs, len(passes), ctypes.byref(us)))
        results = []
        for si, (names, outs) in enumerate(per_pass):
            later = set()
            for names2, outs2 in per_pass[si + 1:]:
                later |= {n for n in names2 if n not in outs2}
            res = DispatchResult(elapsed_us=float(us.value) if si == len(per_pass) - 1 else 0.0)
            for i, name in enumerate(names):
                if name in outs and name not in later:
                    res.outputs[name] = keep[si][1][i].raw
            results.append(res)
        return results

    def kernel_names(self):
        return [self._lib.mtc_kernel_name(i).decode() for i in range(self._lib.mtc_kernel_count())]

    # ---- typed, device-pointer ops (asynchronous on `stream`) ---------------------
    def qmv(self, w, scales, biases, x, out, M, N, K, bits, group_size, dtype, stream: int = 0):
        self._check(self._lib.mtc_qmv(self._h, stream, w, scales, biases, x, out, M, N, K, bits, group_size,
                                      _dt(dtype)))

    def qmv_multi(self, w, scales, biases, x, outs, M, N, K, bits, group_size, dtype, stream: int = 0):
        """qmv whose output tile is stored to every pointer of ``outs`` (1 to 8)."""
        arr = (ctypes.c_void_p * len(outs))(*[int(o) for o in outs])
        self._check(self._lib.mtc_qmv_multi(self._h, stream, w, scales, biases, x, arr, len(outs), M, N, K, bits,
                                            group_size, _dt(dtype)))

    def affine_quantize(self, w, out, scales, biases, n_elem, bits, group_size, dtype, stream: int = 0):
        self._check(self._lib.mtc_affine_quantize(self._h, stream, w, out, scales, biases, n_elem, bits, group_size, _dt(dtype)))

    def affine_dequantize(self, w, scales, biases, out, n_elem, bits, group_size, dtype, stream: int = 0):
        self._check(self._lib.mtc_affine_dequantize(self._h, stream, w, scales, biases, out, n_elem, bits, group_size, _dt(dtype)))

    def moe_down_swiglu_accum(self, gates, ups, expert_indices, slot_weights, w, scales, biases, out, in_dim, out_dim, n_experts,
                              group_size, dtype, stream: int = 0):
        ga = (ctypes.c_void_p * len(gates))(*[int(p) for p in gates])
        ua = (ctypes.c_void_p * len(ups))(*[int(p) for p in ups])
        self._check(self._lib.mtc_moe_down_swiglu_accum(self._h, stream, ga, ua, len(gates), expert_indices, slot_weights, w, scales,
                                                        biases, out, in_dim, out_dim, n_experts, group_size, _dt(dtype)))

    def qmv_expert_indexed(self, xs, expert_indices, w, scales, biases, out, in_dim, out_dim, n_experts, group_size, dtype, stream: int = 0):
        xa = (ctypes.c_void_p * len(xs))(*[int(p) for p in xs])
        self._check(self._lib.mtc_qmv_expert_indexed(self._h, stream, xa, len(xs), expert_indices, w, scales, biases, out, in_dim, out_dim,
                                                     n_experts, group_size, _dt(dtype)))

    def qvm(self, w, scales, biases, x, out, M, N, K, bits, group_size, dtype, stream: int = 0):
        self._check(self._lib.mtc_qvm(self._h, stream, w, scales, biases, x, out, M, N, K, bits, group_size, _dt(dtype)))

    def dequant_gather(self, weight, scales, biases, indices, out, n_tokens, hidden, vocab, bits, group_size, dtype, stream: int = 0):
        self._check(self._lib.mtc_dequant_gather(self._h, stream, weight, scales, biases, indices, out, n_tokens, hidden, vocab, bits,
                                                 group_size, _dt(dtype)))

    def rms_norm_qmv(self, x, norm_weight, eps, w, scales, biases, out, N, K, bits, group_size, dtype, stream: int = 0):
        self._check(self._lib.mtc_rms_norm_qmv(self._h, stream, x, norm_weight, float(eps), w, scales, biases, out, N, K, bits,
                                               group_size, _dt(dtype)))

    def qmm_multi(self, w, scales, biases, x, outs, ld, M, N, K, bits, group_size, dtype, stream: int = 0):
        """qmm whose [M, N] result is a column block (row stride ``ld`` elements) of every destination in ``outs``."""
        arr = (ctypes.c_void_p * len(outs))(*[int(o) for o in outs])
        self._check(self._lib.mtc_qmm_multi(self._h, stream, w, scales, biases, x, arr, len(outs), int(ld), M, N, K, bits,
                                            group_size, _dt(dtype)))

    # ---- fused and chained decode projections ---------------------------------------
    @staticmethod
    def _descs(projections):
        """``projections``: dicts with w, scales, biases, x, outs (list of device pointers), M, N, K, bits,
        group_size, dtype and optionally phase -> a ctypes array of ``mtc_qmv_desc``."""
        arr = (QmvDesc * len(projections))()
        for d, p in zip(arr, projections):
            d.w, d.scales, d.biases, d.x = int(p["w"]), int(p["scales"]), int(p["biases"]), int(p["x"])
            outs = list(p["outs"])
            for i, o in enumerate(outs):
                d.outs[i] = int(o)
            d.n_outs = len(outs)
            d.M, d.N, d.K = int(p["M"]), int(p["N"]), int(p["K"])
            d.bits, d.group_size, d.dtype = int(p["bits"]), int(p["group_size"]), _dt(p["dtype"])
            d.phase = int(p.get("phase", 0))
        return arr

    def qmv_batched(self, projections, stream: int = 0):
        """1 to 4 projections that read the same activations, one launch (``mtc_qmv_batched``)."""
        arr = self._descs(projections)
        self._check(self._lib.mtc_qmv_batched(self._h, stream, arr, len(projections)))

    def qmv_batched_sync(self, projections, peer_flags, rank: int, local_flags: int, epoch: int, ticket: int, stream: int = 0):
        """``qmv_batched`` whose launch also hands over to the other ranks (``mtc_qmv_batched_sync``)."""
        arr = self._descs(projections)
        ps = PeerSync()
        for i, p in enumerate(peer_flags):
            ps.peer_flags[i] = int(p)
        ps.local_flags, ps.epoch, ps.ticket = int(local_flags), int(epoch), int(ticket)
        ps.n_peers, ps.rank = len(peer_flags), int(rank)
        self._check(self._lib.mtc_qmv_batched_sync(self._h, stream, arr, len(projections), ctypes.byref(ps)))

    def chain_create(self, projections) -> "Chain":
        """A prepared list of projections walked by one persistent grid (``mtc_chain_create``)."""
        arr = self._descs(projections)
        h = ctypes.c_void_p()
        self._check(self._lib.mtc_chain_create(self._h, arr, len(projections), ctypes.byref(h)))
        return Chain(self, h)

    # ---- buffers shared between the rank processes of one node --------------------
    def alloc(self, nbytes: int) -> int:
        p = ctypes.c_void_p()
        self._check(self._lib.mtc_alloc(self._h, nbytes, ctypes.byref(p)))
        return int(p.value)

    def free(self, ptr: int):
        self._check(self._lib.mtc_free(self._h, ptr))

    def memset(self, ptr: int, value: int, nbytes: int, stream: int = 0):
        self._check(self._lib.mtc_memset(self._h, stream, ptr, value, nbytes))

    def ipc_export(self, ptr: int) -> bytes:
        h = ctypes.create_string_buffer(64)
        self._check(self._lib.mtc_ipc_export(self._h, ptr, h))
        return h.raw

    def ipc_open(self, handle: bytes) -> int:
        p = ctypes.c_void_p()
        self._check(self._lib.mtc_ipc_open(self._h, ctypes.create_string_buffer(handle, 64), ctypes.byref(p)))
        return int(p.value)

    def ipc_close(self, ptr: int):
        self._check(self._lib.mtc_ipc_close(self._h, ptr))

    def peer_barrier(self, peer_flags, rank: int, local_flags: int, epoch: int, stream: int = 0):
        arr = (ctypes.c_void_p * len(peer_flags))(*[int(p) for p in peer_flags])
        self._check(self._lib.mtc_peer_barrier(self._h, stream, arr, len(peer_flags), rank, local_flags, epoch))

    def qmm(self, w, scales, biases, x, out, M, N, K, bits, group_size, dtype, stream: int = 0):
        self._check(self._lib.mtc_qmm(self._h, stream, w, scales, biases, x, out, M, N, K, bits, group_size,
                                      _dt(dtype)))

    def qmm_route(self, M, N, K, bits, group_size, dtype) -> str:
        return self._lib.mtc_qmm_route(M, N, K, bits, group_size, _dt(dtype)).decode()

    def gather_qmm(self, x, w, scales, biases, out, m_total, n_out, k_in, n_experts, bits, group_size, dtype,
                   expert_offsets=None, indices=None, stream: int = 0):
        self._check(self._lib.mtc_gather_qmm(self._h, stream, x, w, scales, biases, expert_offsets, indices, out,
                                             m_total, n_out, k_in, n_experts, bits, group_size, _dt(dtype)))

    def gather_qmm_static(self, x, w, scales, biases, out, m_total, n_out, k_in, n_experts, bits, group_size, dtype,
                          expert_offsets=None, indices=None, stream: int = 0):
        """``gather_qmm`` with its scratch in a fixed array of the library: allocates nothing (see mtcuda.h)."""
        self._check(self._lib.mtc_gather_qmm_static(self._h, stream, x, w, scales, biases, expert_offsets, indices,
                                                    out, m_total, n_out, k_in, n_experts, bits, group_size, _dt(dtype)))

    def moe_experts(self, x, sort_token_idx, n_tokens, gate, up, down, expert_offsets, y, m_total, hidden, inter, n_experts,
                    bits, group_size, dtype, stream: int = 0):
        """``mtc_moe_experts``; gate / up / down are (w, scales, biases) device pointers."""
        mats = [QMat(int(m[0]), int(m[1]), int(m[2])) for m in (gate, up, down)]
        self._check(self._lib.mtc_moe_experts(self._h, stream, x, sort_token_idx, n_tokens, ctypes.byref(mats[0]),
                                              ctypes.byref(mats[1]), ctypes.byref(mats[2]), expert_offsets, y, m_total, hidden,
                                              inter, n_experts, bits, group_size, _dt(dtype)))

    def gather_qmm_route(self, m_total, n_out, k_in, n_experts, bits, group_size, dtype) -> str:
        return self._lib.mtc_gather_qmm_route(m_total, n_out, k_in, n_experts, bits, group_size, _dt(dtype)).decode()

    def moe_router_topk(self, logits, indices_out, weights_out, n_rows, n_experts, k, norm_topk_prob, dtype,
                        stream: int = 0):
        self._check(self._lib.mtc_moe_router_topk(self._h, stream, logits, indices_out, weights_out, n_rows,
                                                  n_experts, k, norm_topk_prob, _dt(dtype)))

    def moe_sort(self, topk_idx, n_tokens, k, n_experts, sort_token_idx, inv_perm, expert_offsets, row_expert=None,
                 stream: int = 0):
        self._check(self._lib.mtc_moe_sort(self._h, stream, topk_idx, n_tokens, k, n_experts, sort_token_idx,
                                           inv_perm, expert_offsets, row_expert))

    def moe_permute(self, tokens, sort_token_idx, permuted, n_rows, hidden, dtype, stream: int = 0):
        self._check(self._lib.mtc_moe_permute(self._h, stream, tokens, sort_token_idx, permuted, n_rows, hidden,
                                              _dt(dtype)))

    def moe_unpermute(self, expert_outputs, inv_perm, weights, out, n_tokens, hidden, k, dtype, stream: int = 0):
        self._check(self._lib.mtc_moe_unpermute(self._h, stream, expert_outputs, inv_perm, weights, out, n_tokens,
                                                hidden, k, _dt(dtype)))

    def swiglu(self, gate, up, out, n, dtype, stream: int = 0):
        self._check(self._lib.mtc_swiglu(self._h, stream, gate, up, out, n, _dt(dtype)))

    def set_option(self, name: str, value: int):
        self._check(self._lib.mtc_set_option(self._h, name.encode(), int(value)))

    def unpack_codes(self, w, codes, N, K, bits, stream: int = 0):
        self._check(self._lib.mtc_unpack_codes(self._h, stream, w, codes, N, K, bits))


class Chain:
    """Handle of ``mtc_chain``: ``run(stream)`` enqueues every projection of the list, ``close()`` frees it.
    Mirrors the passes handed to ``Context::dispatch_chain`` (crates/metaltile-runtime/src/context.rs:363-395)."""

    def __init__(self, ctx: Context, handle):
        self._ctx, self._h = ctx, handle

    @property
    def fused(self) -> bool:
        return bool(self._ctx._lib.mtc_chain_is_fused(self._h))

    def run(self, stream: int = 0):
        self._ctx._check(self._ctx._lib.mtc_chain_run(self._ctx._h, stream, self._h))

    def close(self):
        if self._h:
            self._ctx._lib.mtc_chain_destroy(self._ctx._h, self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
