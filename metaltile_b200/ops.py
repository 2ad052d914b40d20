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


def qmv(w, scales, biases, x, bits: int, group_size: int, out=None, ctx: Context = None):
    """out[M, N] = x[M, K] @ dequant(w)[N, K]^T on the CUDA-core path (decode, M <= 16 tuned)."""
    x2, M, N, K = _check_dense(w, scales, biases, x, bits, group_size)
    if out is None:
        out = torch.empty((M, N), dtype=x.dtype, device=x.device)
    ctx = ctx or context(x.device)
    ctx.qmv(w.data_ptr(), scales.data_ptr(), biases.data_ptr(), x2.data_ptr(), out.data_ptr(), M, N, K, bits,
            group_size, _TORCH_DT[x.dtype], _stream())
    return out


def qmm(w, scales, biases, x, bits: int, group_size: int, out=None, ctx: Context = None):
    """Like ``qmv`` but routed by M as the reference's ``mt_qmm_for`` does (prefill -> tensor cores)."""
    x2, M, N, K = _check_dense(w, scales, biases, x, bits, group_size)
    if out is None:
        out = torch.empty((M, N), dtype=x.dtype, device=x.device)
    ctx = ctx or context(x.device)
    ctx.qmm(w.data_ptr(), scales.data_ptr(), biases.data_ptr(), x2.data_ptr(), out.data_ptr(), M, N, K, bits,
            group_size, _TORCH_DT[x.dtype], _stream())
    return out


def unpack_codes(w, K: int, bits: int, ctx: Context = None):
    """u8[N, K] integer codes of a packed matrix (for bit-exact checks)."""
    N = w.shape[0]
    codes = torch.empty((N, K), dtype=torch.uint8, device=w.device)
    ctx = ctx or context(w.device)
    ctx.unpack_codes(w.data_ptr(), codes.data_ptr(), N, K, bits, _stream())
    return codes
