"""Sharding of the quantized matmuls over the GPUs of one node (one process per GPU).

Three natural splits, each with at most one exchange step:

* dense projections — N-split (column parallel): rank g owns the contiguous weight rows
  ``[g*N/G, (g+1)*N/G)`` of ``w``, ``scales`` and ``biases`` (all three are row-of-N major, so no
  repacking), computes ``out[:, slice]``; the slices are all-gathered, or stay where they are when the
  consumer is sharded the same way (attention heads, SwiGLU);
* dense projections — K-split (row parallel): rank g owns the columns ``[g*K/G, (g+1)*K/G)`` of every row
  (a contiguous range of packed words and of groups per row, copied out once at load time), multiplies its
  slice of the activations and the partial outputs are summed with one all-reduce.  A transformer layer then
  needs two exchanges (after o and after down) instead of one per projection;
* MoE — expert parallel: rank g owns experts ``[g*E/G, (g+1)*E/G)``; tokens are data parallel; routed
  rows travel to the owner of their expert with an all-to-all, come back with a second one.

The reference is a single-device library (its tests serialise GPU access with one mutex,
crates/metaltile-std/tests/common/mod.rs:11-27), so none of this has a counterpart there.

``torch.distributed`` carries the collectives (NCCL on GPUs).  The compute steps go through a backend
object; the default backend calls the CUDA kernels, and the CPU tests of the exchange logic pass their
own backend (gloo ranks have no GPU).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.distributed as dist


def shard_rows(n: int, world: int, rank: int):
    """Row range of rank ``rank`` in an even N-split; N must divide evenly (every layer shape here does)."""
    if n % world != 0:
        raise ValueError(f"N = {n} does not split evenly over {world} ranks")
    per = n // world
    return rank * per, (rank + 1) * per


class CudaBackend:
    """Compute steps on the local GPU through the C ABI."""

    def __init__(self, ctx=None):
        from . import ops
        self.ops = ops
        self.ctx = ctx

    def qmv(self, w, s, b, x, bits, gs, out=None):
        return self.ops.qmm(w, s, b, x, bits, gs, out=out, ctx=self.ctx)

    def router_topk(self, logits, k, norm):
        return self.ops.moe_router_topk(logits, k, norm, ctx=self.ctx)

    def moe_sort(self, idx, n_experts):
        return self.ops.moe_sort(idx, n_experts, ctx=self.ctx)

    def permute(self, tokens, sti):
        return self.ops.moe_permute(tokens, sti, ctx=self.ctx)

    def unpermute(self, eo, inv, wts):
        return self.ops.moe_unpermute(eo, inv, wts, ctx=self.ctx)

    def swiglu(self, g, u):
        return self.ops.swiglu(g, u, ctx=self.ctx)

    def gather_qmm(self, x, w, s, b, bits, gs, offsets):
        return self.ops.gather_qmm(x, w, s, b, bits, gs, expert_offsets=offsets, ctx=self.ctx)

    def experts(self, x, gate, up, down, bits, gs, offsets):
        """gate, up, SwiGLU and down of rows sorted by expert as one call (same results as the separate steps)."""
        return self.ops.moe_experts(x, gate, up, down, bits, gs, offsets, ctx=self.ctx)


class ColumnParallelLinear:
    """One N-split quantized projection: local ``w[N/G, K*bits/32]``, ``scales``/``biases[N/G, K/g]``."""

    def __init__(self, w, scales, biases, bits: int, group_size: int, backend=None, group=None):
        self.w, self.scales, self.biases = w, scales, biases
        self.bits, self.group_size = bits, group_size
        self.backend = backend or CudaBackend()
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1

    def forward(self, x):
        """x [M, K] replicated on every rank -> out [M, N] replicated."""
        local = self.backend.qmv(self.w, self.scales, self.biases, x, self.bits, self.group_size)
        if self.world == 1:
            return local
        m, nl = local.shape
        flat = torch.empty((self.world * m, nl), dtype=local.dtype, device=local.device)
        dist.all_gather_into_tensor(flat, local.contiguous(), group=self.group)
        gathered = flat.view(self.world, m, nl)
        # all-gather yields [G][M][N/G]; row-major [M][N] needs the rank axis next to the columns
        return gathered.permute(1, 0, 2).reshape(m, self.world * nl) if m > 1 else gathered.reshape(1, -1)


def shard_cols(w, scales, biases, bits: int, group_size: int, world: int, rank: int):
    """The K-slice of rank ``rank``: packed words, scales and biases of columns [rank*K/G, (rank+1)*K/G).
    K/G must be a multiple of the group size and of 32 codes, so that the slice is whole words and groups."""
    k = w.shape[-1] * 32 // bits
    if k % world != 0 or (k // world) % group_size != 0 or ((k // world) * bits) % 32 != 0:
        raise ValueError(f"K = {k} does not split into {world} slices of whole groups and words")
    kw, kg = (k // world) * bits // 32, (k // world) // group_size
    return (w[..., rank * kw:(rank + 1) * kw].contiguous(), scales[..., rank * kg:(rank + 1) * kg].contiguous(),
            biases[..., rank * kg:(rank + 1) * kg].contiguous())


class RowParallelLinear:
    """One K-split quantized projection: local ``w[N, (K/G)*bits/32]``, ``scales``/``biases[N, (K/G)/g]``."""

    def __init__(self, w, scales, biases, bits: int, group_size: int, backend=None, group=None):
        self.w, self.scales, self.biases = w, scales, biases
        self.bits, self.group_size = bits, group_size
        self.backend = backend or CudaBackend()
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1

    def forward(self, x_local, out=None):
        """x_local [M, K/G]: this rank's slice of the activations -> out [M, N], summed over the ranks."""
        y = self.backend.qmv(self.w, self.scales, self.biases, x_local, self.bits, self.group_size, out=out)
        if self.world > 1:
            dist.all_reduce(y, group=self.group)
        return y


class _RawCuda:
    """Adapter that lets torch wrap memory the library allocated (``__cuda_array_interface__``)."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


class PeerGather:
    """A gathered-output buffer that every rank's kernels store into directly (one process per GPU).

    Each rank allocates ``nbytes`` plus a flag block with the library (plain device memory), the ranks exchange
    cudaIpc handles over ``torch.distributed`` and map each other's blocks.  ``qmv_into`` then runs a projection whose
    output tile lands in every rank's buffer at the same byte offset, and ``barrier`` enqueues the one-warp kernel that
    makes a phase's tiles visible everywhere - the N-split all-gather without a collective launch.  ``batched_into`` runs
    up to four projections that share x as one launch which also carries the hand-off (no barrier launch between
    phases; one ``barrier`` before the host reads the buffer).  A region of the buffer may be rewritten only by a launch
    that comes after every rank's readers of it - with ``batched_into`` at least one launch later, which a decode step
    that writes each region once satisfies.  The waits inside are bounded; ``ctx.status_word()`` reports a rank that
    never arrived (0x601 + rank)."""

    def __init__(self, ctx, nbytes: int, group=None):
        self.ctx, self.group, self.nbytes = ctx, group, nbytes
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        if self.world > 8:
            raise ValueError("at most 8 ranks")
        # every step that can fail locally is followed by an exchange of its outcome, so that either all ranks get a
        # working object or all ranks raise: no rank is left waiting in a collective for one that gave up
        self.buf = self.flags = None
        self.peer_bufs, self.peer_flags = [], []
        mine = None
        try:
            self.buf = ctx.alloc(nbytes)
            # two flag blocks of 256 bytes: [0] for the barrier kernel, [1] for the hand-off inside the decode kernels;
            # each: 8 flag words, at +128 the epoch counter, at +192 the launch's CTA ticket
            self.flags = ctx.alloc(512)
            ctx.memset(self.buf, 0, nbytes)
            ctx.memset(self.flags, 0, 512)
            ctx.sync()
            mine = (ctx.ipc_export(self.buf), ctx.ipc_export(self.flags))
        except Exception as e:  # reported through the exchange below
            mine = None
            self._why = repr(e)
        handles = [None] * self.world
        dist.all_gather_object(handles, mine, group=group)
        opened = all(h is not None for h in handles)
        if opened:
            try:
                for r, (hb, hf) in enumerate(handles):
                    self.peer_bufs.append(self.buf if r == self.rank else ctx.ipc_open(hb))
                    self.peer_flags.append(self.flags if r == self.rank else ctx.ipc_open(hf))
            except Exception as e:
                opened = False
                self._why = repr(e)
        oks = [None] * self.world
        dist.all_gather_object(oks, bool(opened), group=group)
        if not all(oks):
            self._release()
            raise RuntimeError(f"peer buffers could not be shared between the ranks ({getattr(self, '_why', 'another rank failed')})")

    def _release(self):
        for r, (pb, pf) in enumerate(zip(self.peer_bufs, self.peer_flags)):
            if r != self.rank:
                self.ctx.ipc_close(pb)
                self.ctx.ipc_close(pf)
        self.peer_bufs, self.peer_flags = [], []
        if self.buf:
            self.ctx.free(self.buf)
        if self.flags:
            self.ctx.free(self.flags)
        self.buf = self.flags = None

    def tensor(self, dtype=torch.bfloat16):
        """The local buffer as a flat tensor of ``dtype``."""
        return torch.as_tensor(_RawCuda(self.buf, self.nbytes), device="cuda").view(dtype)

    def qmv_into(self, w, scales, biases, x, bits, group_size, byte_offset: int, stream: int):
        """out tile [M, N_local] of this rank -> every rank's buffer at ``byte_offset``."""
        from .ops import _TORCH_DT
        m, k = x.shape
        n = w.shape[0]
        outs = [self.peer_bufs[self.rank] + byte_offset] + [p + byte_offset for r, p in enumerate(self.peer_bufs) if r != self.rank]
        self.ctx.qmv_multi(w.data_ptr(), scales.data_ptr(), biases.data_ptr(), x.data_ptr(), outs, m, n, k, bits,
                           group_size, _TORCH_DT[x.dtype], stream=stream)

    def batched_into(self, mats, x, bits, group_size, byte_offsets, stream: int):
        """Up to four projections ``(w, scales, biases)`` of one x -> every rank's buffer at ``byte_offsets[i]``, as one
        launch that waits for the peers' previous launch and publishes its own completion."""
        from .ops import _TORCH_DT
        m, k = x.shape
        descs = []
        for (w, sc, bi), off in zip(mats, byte_offsets):
            outs = [self.peer_bufs[self.rank] + off] + [p + off for r, p in enumerate(self.peer_bufs) if r != self.rank]
            descs.append(dict(w=w.data_ptr(), scales=sc.data_ptr(), biases=bi.data_ptr(), x=x.data_ptr(), outs=outs, M=m,
                              N=w.shape[0], K=k, bits=bits, group_size=group_size, dtype=_TORCH_DT[x.dtype]))
        f = self.flags + 256
        self.ctx.qmv_batched_sync(descs, [p + 256 for p in self.peer_flags], self.rank, f, f + 128, f + 192, stream=stream)

    def qmm_into(self, w, scales, biases, x, bits, group_size, n_total: int, col0: int, stream: int):
        """Prefill product of this rank's weight rows, stored by the kernel's epilogue as columns ``[col0, col0 + N_local)``
        of the row-major ``[M, n_total]`` matrix at the start of every rank's buffer (the N-split all-gather without a
        collective, overlapped with the product)."""
        from .ops import _TORCH_DT
        m, k = x.shape
        esz = x.element_size()
        if m * n_total * esz > self.nbytes:
            raise ValueError("the gathered matrix does not fit in the shared buffer")
        outs = [self.peer_bufs[self.rank] + col0 * esz] + [p + col0 * esz for r, p in enumerate(self.peer_bufs) if r != self.rank]
        self.ctx.qmm_multi(w.data_ptr(), scales.data_ptr(), biases.data_ptr(), x.data_ptr(), outs, n_total, m, w.shape[0], k,
                           bits, group_size, _TORCH_DT[x.dtype], stream=stream)

    def barrier(self, stream: int):
        self.ctx.peer_barrier(self.peer_flags, self.rank, self.flags, self.flags + 128, stream=stream)

    def close(self):
        """Unmap the peers' blocks and free the own ones; every rank calls it after a ``dist.barrier``."""
        self._release()


@dataclass
class ExpertShard:
    """The experts a rank owns: gate / up [E_l, I, H*bits/32], down [E_l, H, I*bits/32] (+ scales, biases)."""
    gate: tuple
    up: tuple
    down: tuple
    bits: int
    group_size: int


class ExpertParallelMoE:
    """router -> sort -> permute -> all-to-all -> gather_qmm(gate, up) -> SwiGLU -> gather_qmm(down)
    -> all-to-all -> unpermute, with ``n_experts`` split evenly over the ranks of ``group``."""

    def __init__(self, shard: ExpertShard, n_experts: int, top_k: int, norm_topk_prob: int = 1, backend=None,
                 group=None):
        self.shard, self.n_experts, self.top_k, self.norm = shard, n_experts, top_k, norm_topk_prob
        self.backend = backend or CudaBackend()
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        if n_experts % self.world != 0:
            raise ValueError("n_experts must split evenly over the ranks")
        self.e_local = n_experts // self.world

    def _experts(self, x_sorted, offsets):
        be, sh = self.backend, self.shard
        if hasattr(be, "experts"):
            return be.experts(x_sorted, sh.gate, sh.up, sh.down, sh.bits, sh.group_size, offsets)
        g = be.gather_qmm(x_sorted, *sh.gate, sh.bits, sh.group_size, offsets)
        u = be.gather_qmm(x_sorted, *sh.up, sh.bits, sh.group_size, offsets)
        a = be.swiglu(g, u)
        return be.gather_qmm(a, *sh.down, sh.bits, sh.group_size, offsets)

    def forward(self, tokens, logits):
        """tokens [T_local, H], logits [T_local, E] -> [T_local, H]."""
        be, world, e_l = self.backend, self.world, self.e_local
        idx, wts = be.router_topk(logits, self.top_k, self.norm)
        sti, inv, off, _ = be.moe_sort(idx, self.n_experts)
        xp = be.permute(tokens, sti)                      # rows sorted by global expert id = by owner rank
        if world == 1:
            y = self._experts(xp, off)
            return be.unpermute(y, inv, wts)

        off64 = off.to(torch.int64)
        counts = (off64[1:] - off64[:-1]).reshape(world, e_l)          # rows I send, per (owner, its expert)
        recv_counts = torch.empty_like(counts)
        dist.all_to_all_single(recv_counts, counts, group=self.group)  # rows I receive, per (source, my expert)
        send_splits = counts.sum(dim=1).tolist()                       # host sync: split sizes are Python ints
        recv_splits = recv_counts.sum(dim=1).tolist()
        n_recv = int(sum(recv_splits))
        recv = torch.empty((n_recv, tokens.shape[1]), dtype=tokens.dtype, device=tokens.device)
        dist.all_to_all_single(recv, xp, recv_splits, send_splits, group=self.group)

        # received rows are source-major, expert-minor; the experts want expert-major order
        order = expert_major_order(recv_counts)
        x_sorted = recv.index_select(0, order)
        local_off = torch.zeros(e_l + 1, dtype=torch.int32, device=tokens.device)
        local_off[1:] = recv_counts.sum(dim=0).cumsum(0).to(torch.int32)
        y_sorted = self._experts(x_sorted, local_off)

        y_recv = torch.empty_like(y_sorted)
        y_recv.index_copy_(0, order, y_sorted)            # back to source-major order
        y = torch.empty((xp.shape[0], y_recv.shape[1]), dtype=y_recv.dtype, device=y_recv.device)
        dist.all_to_all_single(y, y_recv, send_splits, recv_splits, group=self.group)
        return be.unpermute(y, inv, wts)


def expert_major_order(recv_counts: torch.Tensor) -> torch.Tensor:
    """Gather index turning a source-major / expert-minor row list into expert-major / source-minor.

    ``recv_counts[s, e]`` = rows received from source ``s`` for local expert ``e``; rows arrive as
    ``for s: for e: rows``.  The result lists, for e ascending and s ascending, the positions of those rows.
    """
    world, e_l = recv_counts.shape
    flat = recv_counts.reshape(-1).to(torch.int64)                      # index s*e_l + e
    start = torch.cumsum(flat, 0) - flat                                # first row of block (s, e) on arrival
    blocks = torch.arange(world * e_l, device=recv_counts.device).reshape(world, e_l).t().reshape(-1)  # (e, s) order
    lens = flat[blocks]
    total = int(lens.sum())
    if total == 0:
        return torch.zeros(0, dtype=torch.int64, device=recv_counts.device)
    block_of_row = torch.repeat_interleave(torch.arange(blocks.numel(), device=lens.device), lens)
    first_out = torch.cumsum(lens, 0) - lens
    within = torch.arange(total, device=lens.device) - first_out[block_of_row]
    return start[blocks][block_of_row] + within
