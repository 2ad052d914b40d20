"""Typed ops on tensors that already live on the GPU (thin wrappers over the C ABI).

PyTorch is used only as the owner of device memory and streams: every function
passes raw device pointers and the current CUDA stream to ``libmtcuda.so``.
"""
from __future__ import annotations

import torch

from ._lib import BF16, F16, F32
from .context import Context

_TORCH_DT = {torch.float32: F32, torch.float16: F16, torch.bfloat16: BF16}

_ctx_cache = {}


def context(device=None) -> Context:
    """The process-wide Context of a device (created on first use)."""
    idx = torch.cuda.current_device() if device is None else torch.device(device).index or 0
    if idx not in _ctx_cache:
        _ctx_cache[idx] = Context(idx)
    return _ctx_cache[idx]


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _check_dense(w, scales, biases, x, bits, group_size):
    if not (w.is_cuda and scales.is_cuda and biases.is_cuda and x.is_cuda):
        raise ValueError("all operands must be CUDA tensors")
    if w.dtype not in (torch.int32, torch.uint32):
        raise TypeError("w must hold packed 32-bit words (torch.int32 / torch.uint32)")
    if x.dtype not in _TORCH_DT or scales.dtype != x.dtype or biases.dtype != x.dtype:
        raise TypeError("x, scales and biases must share one dtype in {f32, f16, bf16}")
    x2 = x.reshape(-1, x.shape[-1])
    M, K = x2.shape
    N = w.shape[0]
    if w.shape[1] * 32 != K * bits:
        raise ValueError(f"w has {w.shape[1]} words per row, expected K*bits/32 = {K * bits / 32}")
    if scales.shape != (N, K // group_size) or biases.shape != scales.shape:
        raise ValueError("scales/biases must be [N, K/group_size]")
    for t in (w, scales, biases, x2):
        if not t.is_contiguous():
            raise ValueError("operands must be contiguous")
    return x2, M, N, K


def _check_out(out, M, N, like):
    """A caller-supplied output must be the dense row-major [M, N] block the kernels write."""
    if out.device != like.device or out.dtype != like.dtype:
        raise TypeError("out must live on the same device and have the dtype of x")
    if out.numel() != M * N or not out.is_contiguous():
        raise ValueError(f"out must be a contiguous block of M*N = {M * N} elements "
                         "(a column slice of a wider tensor with M > 1 is not)")


def qmv(w, scales, biases, x, bits: int, group_size: int, out=None, ctx: Context = None):
    """out[M, N] = x[M, K] @ dequant(w)[N, K]^T on the CUDA-core path (decode, M <= 16 tuned)."""
    x2, M, N, K = _check_dense(w, scales, biases, x, bits, group_size)
    if out is None:
        out = torch.empty((M, N), dtype=x.dtype, device=x.device)
    else:
        _check_out(out, M, N, x)
    ctx = ctx or context(x.device)
    ctx.qmv(w.data_ptr(), scales.data_ptr(), biases.data_ptr(), x2.data_ptr(), out.data_ptr(), M, N, K, bits,
            group_size, _TORCH_DT[x.dtype], _stream())
    return out


def qmm(w, scales, biases, x, bits: int, group_size: int, out=None, ctx: Context = None):
    """Like ``qmv`` but routed by M as the reference's ``mt_qmm_for`` does (prefill -> tensor cores)."""
    x2, M, N, K = _check_dense(w, scales, biases, x, bits, group_size)
    if out is None:
        out = torch.empty((M, N), dtype=x.dtype, device=x.device)
    else:
        _check_out(out, M, N, x)
    ctx = ctx or context(x.device)
    ctx.qmm(w.data_ptr(), scales.data_ptr(), biases.data_ptr(), x2.data_ptr(), out.data_ptr(), M, N, K, bits,
            group_size, _TORCH_DT[x.dtype], _stream())
    return out


def _projection(w, scales, biases, x, bits, group_size, outs, phase=0):
    x2, M, N, K = _check_dense(w, scales, biases, x, bits, group_size)
    for o in outs:
        _check_out(o, M, N, x)
    return {"w": w.data_ptr(), "scales": scales.data_ptr(), "biases": biases.data_ptr(), "x": x2.data_ptr(),
            "outs": [o.data_ptr() for o in outs], "M": M, "N": N, "K": K, "bits": bits, "group_size": group_size,
            "dtype": _TORCH_DT[x.dtype], "phase": phase}


def qmv_batched(mats, x, bits: int, group_size: int, out=None, ctx: Context = None):
    """Several projections of the same activations in one launch: ``mats`` = [(w, scales, biases), ...] (1 to 4).

    Returns ``out[M, sum(N_i)]`` with the results side by side - for M = 1 the concatenated vector of
    ``ffai_batched_qkv_qgemv`` (crates/metaltile-std/src/ffai/batched_qkv_qgemv.rs:1-35).  For M > 1 every
    projection writes its own contiguous [M, N_i] tile and the tiles are returned as a list instead."""
    x2 = x.reshape(-1, x.shape[-1])
    M = x2.shape[0]
    ns = [w.shape[0] for (w, _, _) in mats]
    ctx = ctx or context(x.device)
    if M == 1:
        if out is None:
            out = torch.empty((1, sum(ns)), dtype=x.dtype, device=x.device)
        col, tiles = 0, []
        for n in ns:
            tiles.append(out[:, col:col + n])
            col += n
    else:
        tiles = [torch.empty((M, n), dtype=x.dtype, device=x.device) for n in ns]
    projs = [_projection(w, s, b, x2, bits, group_size, [t]) for (w, s, b), t in zip(mats, tiles)]
    ctx.qmv_batched(projs, _stream())
    return out if M == 1 else tiles


def unpack_codes(w, K: int, bits: int, ctx: Context = None):
    """u8[N, K] integer codes of a packed matrix (for bit-exact checks)."""
    N = w.shape[0]
    codes = torch.empty((N, K), dtype=torch.uint8, device=w.device)
    ctx = ctx or context(w.device)
    ctx.unpack_codes(w.data_ptr(), codes.data_ptr(), N, K, bits, _stream())
    return codes


# ---- MoE -----------------------------------------------------------------------------------------
def moe_router_topk(logits, k: int, norm_topk_prob: int = 1, ctx: Context = None):
    """(indices int32[rows, k], weights T[rows, k]) of ``mt_moe_router_topk``."""
    rows, n_experts = logits.shape
    idx = torch.empty((rows, k), dtype=torch.int32, device=logits.device)
    wts = torch.empty((rows, k), dtype=logits.dtype, device=logits.device)
    ctx = ctx or context(logits.device)
    ctx.moe_router_topk(logits.data_ptr(), idx.data_ptr(), wts.data_ptr(), rows, n_experts, k, norm_topk_prob,
                        _TORCH_DT[logits.dtype], _stream())
    return idx, wts


def moe_sort(topk_idx, n_experts: int, ctx: Context = None):
    """Stable expert sort: (sort_token_idx[T*k], inv_perm[T, k], expert_offsets[E+1], row_expert[T*k]), int32."""
    n_tokens, k = topk_idx.shape
    dev = topk_idx.device
    sti = torch.empty(n_tokens * k, dtype=torch.int32, device=dev)
    inv = torch.empty((n_tokens, k), dtype=torch.int32, device=dev)
    off = torch.empty(n_experts + 1, dtype=torch.int32, device=dev)
    rex = torch.empty(n_tokens * k, dtype=torch.int32, device=dev)
    ctx = ctx or context(dev)
    ctx.moe_sort(topk_idx.data_ptr(), n_tokens, k, n_experts, sti.data_ptr(), inv.data_ptr(), off.data_ptr(),
                 rex.data_ptr(), _stream())
    return sti, inv, off, rex


def moe_permute(tokens, sort_token_idx, out=None, ctx: Context = None):
    rows, hidden = sort_token_idx.numel(), tokens.shape[1]
    if out is None:
        out = torch.empty((rows, hidden), dtype=tokens.dtype, device=tokens.device)
    ctx = ctx or context(tokens.device)
    ctx.moe_permute(tokens.data_ptr(), sort_token_idx.data_ptr(), out.data_ptr(), rows, hidden,
                    _TORCH_DT[tokens.dtype], _stream())
    return out


def moe_unpermute(expert_outputs, inv_perm, weights, out=None, ctx: Context = None):
    n_tokens, k = inv_perm.shape
    hidden = expert_outputs.shape[1]
    if out is None:
        out = torch.empty((n_tokens, hidden), dtype=expert_outputs.dtype, device=expert_outputs.device)
    ctx = ctx or context(expert_outputs.device)
    ctx.moe_unpermute(expert_outputs.data_ptr(), inv_perm.data_ptr(), weights.data_ptr(), out.data_ptr(), n_tokens,
                      hidden, k, _TORCH_DT[expert_outputs.dtype], _stream())
    return out


def swiglu(gate, up, out=None, ctx: Context = None):
    if out is None:
        out = torch.empty_like(gate)
    ctx = ctx or context(gate.device)
    ctx.swiglu(gate.data_ptr(), up.data_ptr(), out.data_ptr(), gate.numel(), _TORCH_DT[gate.dtype], _stream())
    return out


def gather_qmm(x, w, scales, biases, bits: int, group_size: int, expert_offsets=None, indices=None, out=None,
               ctx: Context = None):
    """out[t, n] = sum_k x[t, k] * dequant(w[E(t)])[n, k]; x rows sorted by expert; w [E, n_out, k*bits/32]."""
    if (expert_offsets is None) == (indices is None):
        raise ValueError("give exactly one of expert_offsets and indices")
    m_total, k_in = x.shape
    n_experts, n_out = w.shape[0], w.shape[1]
    if w.shape[2] * 32 != k_in * bits:
        raise ValueError("w must be [E, n_out, k_in*bits/32]")
    if scales.shape != (n_experts, n_out, k_in // group_size) or biases.shape != scales.shape:
        raise ValueError("scales/biases must be [E, n_out, k_in/group_size]")
    for t in (x, w, scales, biases):
        if not t.is_contiguous():
            raise ValueError("operands must be contiguous")
    if out is None:
        out = torch.empty((m_total, n_out), dtype=x.dtype, device=x.device)
    else:
        _check_out(out, m_total, n_out, x)
    ctx = ctx or context(x.device)
    ctx.gather_qmm(x.data_ptr(), w.data_ptr(), scales.data_ptr(), biases.data_ptr(), out.data_ptr(), m_total, n_out,
                   k_in, n_experts, bits, group_size, _TORCH_DT[x.dtype],
                   expert_offsets=None if expert_offsets is None else expert_offsets.data_ptr(),
                   indices=None if indices is None else indices.data_ptr(), stream=_stream())
    return out


def moe_experts(x, gate, up, down, bits: int, group_size: int, expert_offsets, sort_token_idx=None, out=None, ctx: Context = None):
    """y[r] = down_e(silu(gate_e(x_r)) * up_e(x_r)) for rows sorted by expert; gate / up / down are (w, scales, biases)
    with w [E, inter, hidden*bits/32] (gate, up) and [E, hidden, inter*bits/32] (down).  ``sort_token_idx`` folds the
    permutation in: row r reads ``x[sort_token_idx[r]]``."""
    n_experts, inter = gate[0].shape[0], gate[0].shape[1]
    hidden = down[0].shape[1]
    m_total = x.shape[0] if sort_token_idx is None else sort_token_idx.numel()
    if x.shape[1] != hidden or gate[0].shape[2] * 32 != hidden * bits or down[0].shape[2] * 32 != inter * bits:
        raise ValueError("gate / up must be [E, inter, hidden*bits/32] and down [E, hidden, inter*bits/32] for x [rows, hidden]")
    for t in (x, *gate, *up, *down):
        if not t.is_contiguous():
            raise ValueError("operands must be contiguous")
    if out is None:
        out = torch.empty((m_total, hidden), dtype=x.dtype, device=x.device)
    else:
        _check_out(out, m_total, hidden, x)
    ctx = ctx or context(x.device)
    ptr = lambda m: tuple(t.data_ptr() for t in m)
    ctx.moe_experts(x.data_ptr(), None if sort_token_idx is None else sort_token_idx.data_ptr(), x.shape[0], ptr(gate), ptr(up),
                    ptr(down), expert_offsets.data_ptr(), out.data_ptr(), m_total, hidden, inter, n_experts, bits, group_size,
                    _TORCH_DT[x.dtype], stream=_stream())
    return out


def rms_norm_qmv(w, scales, biases, x, norm_weight, eps: float, bits: int, group_size: int, out=None, ctx: Context = None):
    """``qmv(rms_norm(x) * norm_weight)`` in one launch (``ffai_rms_norm_qgemv``,
    crates/metaltile-std/src/ffai/rms_norm_qgemv.rs:51-107): x and norm_weight are vectors of length K, out [1, N]."""
    k = x.numel()
    n = w.shape[0]
    if norm_weight.numel() != k or w.shape[1] * 32 != k * bits:
        raise ValueError("x and norm_weight must have K elements and w must be [N, K*bits/32]")
    if out is None:
        out = torch.empty((1, n), dtype=x.dtype, device=x.device)
    else:
        _check_out(out, 1, n, x)
    ctx = ctx or context(x.device)
    ctx.rms_norm_qmv(x.data_ptr(), norm_weight.data_ptr(), eps, w.data_ptr(), scales.data_ptr(), biases.data_ptr(), out.data_ptr(),
                     n, k, bits, group_size, _TORCH_DT[x.dtype], stream=_stream())
    return out


def affine_quantize(w, bits: int, group_size: int, ctx: Context = None):
    """Float tensor ``w [..., K]`` (K a multiple of the group size) -> (packed int32 ``[..., K*bits/32]``, scales, biases
    ``[..., K/group_size]``) in the layout the quantized matmuls read (``mt_affine_quantize_int*``,
    crates/metaltile-std/src/mlx/quantized.rs:3629-3667)."""
    if not w.is_contiguous():
        raise ValueError("w must be contiguous")
    k = w.shape[-1]
    if k % group_size or (group_size * bits) % 32:
        raise ValueError("the last dimension must hold whole groups and group_size * bits must be a multiple of 32")
    lead = tuple(w.shape[:-1])
    out = torch.empty(lead + (k * bits // 32,), dtype=torch.int32, device=w.device)
    scales = torch.empty(lead + (k // group_size,), dtype=w.dtype, device=w.device)
    biases = torch.empty_like(scales)
    ctx = ctx or context(w.device)
    ctx.affine_quantize(w.data_ptr(), out.data_ptr(), scales.data_ptr(), biases.data_ptr(), w.numel(), bits, group_size,
                        _TORCH_DT[w.dtype], stream=_stream())
    return out, scales, biases


def affine_dequantize(w, scales, biases, bits: int, group_size: int, ctx: Context = None):
    """The inverse of ``affine_quantize``: ``scale * q + bias`` in the type of ``scales`` (``mt_affine_dequantize_int*``)."""
    for t in (w, scales, biases):
        if not t.is_contiguous():
            raise ValueError("operands must be contiguous")
    k = w.shape[-1] * 32 // bits
    out = torch.empty(tuple(w.shape[:-1]) + (k,), dtype=scales.dtype, device=w.device)
    ctx = ctx or context(w.device)
    ctx.affine_dequantize(w.data_ptr(), scales.data_ptr(), biases.data_ptr(), out.data_ptr(), out.numel(), bits, group_size,
                          _TORCH_DT[scales.dtype], stream=_stream())
    return out


def dequant_gather(weight, scales, biases, indices, bits: int, group_size: int, ctx: Context = None):
    """Rows ``indices`` (int32) of a quantized table ``weight [vocab, hidden*bits/32]`` dequantized: ``[n_tokens, hidden]``
    in the type of ``scales`` (``dequant_gather_int*``, crates/metaltile-std/src/ffai/dequant_gather.rs:44-101)."""
    for t in (weight, scales, biases, indices):
        if not t.is_contiguous():
            raise ValueError("operands must be contiguous")
    vocab, hidden = weight.shape[0], weight.shape[1] * 32 // bits
    n_tokens = indices.numel()
    out = torch.empty((n_tokens, hidden), dtype=scales.dtype, device=weight.device)
    ctx = ctx or context(weight.device)
    ctx.dequant_gather(weight.data_ptr(), scales.data_ptr(), biases.data_ptr(), indices.data_ptr(), out.data_ptr(), n_tokens, hidden,
                       vocab, bits, group_size, _TORCH_DT[scales.dtype], stream=_stream())
    return out


def qvm(w, scales, biases, x, bits: int, group_size: int, out=None, ctx: Context = None):
    """``x @ W`` with W stored transposed and quantized along K: w [K, N*bits/32], scales / biases [K/group_size, N],
    x [M, K] -> out [M, N] (``mt_qvm_*``, crates/metaltile-std/src/mlx/quantized.rs:4397-4530)."""
    for t in (w, scales, biases, x):
        if not t.is_contiguous():
            raise ValueError("operands must be contiguous")
    x2 = x.reshape(-1, x.shape[-1])
    m, k = x2.shape
    n = w.shape[1] * 32 // bits
    if w.shape[0] != k or scales.shape != (k // group_size, n) or biases.shape != scales.shape:
        raise ValueError("w must be [K, N*bits/32] and scales / biases [K/group_size, N]")
    if out is None:
        out = torch.empty((m, n), dtype=x.dtype, device=x.device)
    else:
        _check_out(out, m, n, x)
    ctx = ctx or context(x.device)
    ctx.qvm(w.data_ptr(), scales.data_ptr(), biases.data_ptr(), x2.data_ptr(), out.data_ptr(), m, n, k, bits, group_size,
            _TORCH_DT[x.dtype], stream=_stream())
    return out
