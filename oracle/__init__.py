"""CPU oracle for the affine group-quantized matmul family (TEST INFRASTRUCTURE).

ctypes front end of ``mt_oracle.c``, the C restatement of metaltile's scalar
reference (``qmm_oracle`` at crates/metaltile-std/src/mlx/quantized.rs:5374-5404,
``cpu_gather_qmm_int4`` at crates/metaltile-std/src/ffai/moe.rs:3577-3622,
``cpu_topk_reference`` at crates/metaltile-std/tests/moe_gpu_correctness.rs:55-93).

Only the test-suite, the smoke check and the CPU-baseline leg of the benchmark
may import this package: it is the checker, never the product.  The product
library (``metaltile_b200``) does not depend on it and has no CPU fallback.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libmt_oracle.so")

F32, F16, BF16 = 0, 1, 2
DT_CODES = {"f32": F32, "f16": F16, "bf16": BF16}


def build(force: bool = False) -> str:
    """Compile ``mt_oracle.c`` with gcc (see ``Makefile``) and return the .so path."""
    src = os.path.join(_HERE, "mt_oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-B", "libmt_oracle.so"], stdout=subprocess.DEVNULL)
    return _LIB_PATH


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        try:
            build()
        except Exception:
            if not os.path.exists(_LIB_PATH):
                raise
        _lib = ctypes.CDLL(_LIB_PATH)
    return _lib


def _p(a: np.ndarray):
    return a.ctypes.data_as(ctypes.c_void_p)


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def _u32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.uint32)


_sz = ctypes.c_size_t


def round_through(a, dt: int) -> np.ndarray:
    """``unpack_f32(pack_f32(a, dt), dt)`` of crates/metaltile-std/src/utils.rs:26-66."""
    a = _f32(a)
    out = np.empty_like(a)
    lib().mto_round_through(_p(a), _p(out), _sz(a.size), ctypes.c_int(dt))
    return out


def to_bits16(a, dt: int) -> np.ndarray:
    a = _f32(a)
    out = np.empty(a.shape, dtype=np.uint16)
    lib().mto_f32_to_bits16(_p(a), _p(out), _sz(a.size), ctypes.c_int(dt))
    return out


def from_bits16(a, dt: int) -> np.ndarray:
    a = np.ascontiguousarray(a, dtype=np.uint16)
    out = np.empty(a.shape, dtype=np.float32)
    lib().mto_bits16_to_f32(_p(a), _p(out), _sz(a.size), ctypes.c_int(dt))
    return out


def pack_matrix(codes, bits: int) -> np.ndarray:
    """[rows, k] codes -> [rows, k*bits/32] u32 words (LSB-first row bit-stream)."""
    codes = _u32(codes)
    rows, k = codes.shape
    assert (k * bits) % 32 == 0
    words = np.zeros((rows, k * bits // 32), dtype=np.uint32)
    lib().mto_pack_matrix(_p(codes), _sz(rows), _sz(k), ctypes.c_uint32(bits), _p(words))
    return words


def unpack_matrix(words, k: int, bits: int) -> np.ndarray:
    words = _u32(words)
    rows = words.reshape(-1, k * bits // 32).shape[0]
    codes = np.empty((rows, k), dtype=np.uint8)
    lib().mto_unpack_matrix(_p(words), _sz(rows), _sz(k), ctypes.c_uint32(bits), _p(codes))
    return codes


def qmm(w, scales, biases, x, m, n, k, bits, group_size, threads=0, rows=None) -> np.ndarray:
    """f32 accumulators [m, n]; inputs must already be rounded through the dtype.

    ``rows=(n0, n1)`` computes only those weight rows (other outputs stay 0).
    """
    w, scales, biases, x = _u32(w), _f32(scales), _f32(biases), _f32(x)
    assert w.size == n * k * bits // 32 and scales.size == n * (k // group_size) and x.size == m * k
    out = np.zeros((m, n), dtype=np.float32)
    n0, n1 = rows if rows is not None else (0, n)
    lib().mto_qmm_rows(_p(w), _p(scales), _p(biases), _p(x), _p(out), _sz(m), _sz(n), _sz(k),
                       ctypes.c_uint32(bits), _sz(group_size), _sz(n0), _sz(n1), ctypes.c_int(threads))
    return out


def dequant(w, scales, biases, n, k, bits, group_size) -> np.ndarray:
    w, scales, biases = _u32(w), _f32(scales), _f32(biases)
    out = np.empty((n, k), dtype=np.float32)
    lib().mto_dequant(_p(w), _p(scales), _p(biases), _p(out), _sz(n), _sz(k), ctypes.c_uint32(bits),
                      _sz(group_size))
    return out


def gather_qmm(x, w, scales, biases, t_rows, k_in, n_out, n_experts, bits, group_size,
               expert_offsets=None, indices=None, threads=0) -> np.ndarray:
    x, w, scales, biases = _f32(x), _u32(w), _f32(scales), _f32(biases)
    assert (expert_offsets is None) != (indices is None)
    eo = _u32(expert_offsets) if expert_offsets is not None else None
    ix = _u32(indices) if indices is not None else None
    out = np.zeros((t_rows, n_out), dtype=np.float32)
    lib().mto_gather_qmm(_p(x), _p(w), _p(scales), _p(biases),
                         _p(eo) if eo is not None else None, _p(ix) if ix is not None else None,
                         _p(out), _sz(t_rows), _sz(k_in), _sz(n_out), _sz(n_experts),
                         ctypes.c_uint32(bits), _sz(group_size), ctypes.c_int(threads))
    return out


def router_topk(logits, n_experts: int, k: int, norm_topk_prob: int = 1):
    logits = _f32(logits).reshape(-1, n_experts)
    rows = logits.shape[0]
    idx = np.empty((rows, k), dtype=np.uint32)
    wts = np.empty((rows, k), dtype=np.float32)
    lib().mto_router_topk(_p(logits), _p(idx), _p(wts), _sz(rows), _sz(n_experts), _sz(k),
                          ctypes.c_int(norm_topk_prob))
    return idx, wts


def moe_sort(topk_idx, n_experts: int):
    topk_idx = _u32(topk_idx)
    n_tokens, k = topk_idx.shape
    sti = np.empty(n_tokens * k, dtype=np.uint32)
    inv = np.empty((n_tokens, k), dtype=np.uint32)
    off = np.empty(n_experts + 1, dtype=np.uint32)
    rex = np.empty(n_tokens * k, dtype=np.uint32)
    lib().mto_moe_sort(_p(topk_idx), _sz(n_tokens), _sz(k), _sz(n_experts), _p(sti), _p(inv), _p(off),
                       _p(rex))
    return sti, inv, off, rex


def moe_permute(tokens, sort_token_idx) -> np.ndarray:
    tokens, sti = _f32(tokens), _u32(sort_token_idx)
    hidden = tokens.shape[1]
    out = np.empty((sti.size, hidden), dtype=np.float32)
    lib().mto_moe_permute(_p(tokens), _p(sti), _p(out), _sz(sti.size), _sz(hidden))
    return out


def moe_unpermute(expert_out, inv_perm, weights) -> np.ndarray:
    eo, inv, wts = _f32(expert_out), _u32(inv_perm), _f32(weights)
    n_tokens, k = inv.shape
    hidden = eo.shape[1]
    out = np.empty((n_tokens, hidden), dtype=np.float32)
    lib().mto_moe_unpermute(_p(eo), _p(inv), _p(wts), _p(out), _sz(n_tokens), _sz(hidden), _sz(k))
    return out


def swiglu(gate, up) -> np.ndarray:
    g, u = _f32(gate), _f32(up)
    out = np.empty_like(g)
    lib().mto_swiglu(_p(g), _p(u), _p(out), _sz(g.size))
    return out


def rms_normed(x, norm_weight, eps: float) -> np.ndarray:
    """``x * norm_weight * inv_rms`` in f32 (crates/metaltile-std/tests/rms_norm_qgemv_gpu_correctness.rs:59-72)."""
    xv, nw = _f32(x).reshape(-1), _f32(norm_weight).reshape(-1)
    out = np.empty_like(xv)
    lib().mto_rms_normed(_p(xv), _p(nw), _p(out), _sz(xv.size), ctypes.c_float(eps))
    return out


def rms_norm_qmv(w, scales, biases, x, norm_weight, eps, n, k, bits, group_size) -> np.ndarray:
    """ffai_rms_norm_qgemv: the quantized product of the normalised activation, f32 accumulator [1, n]."""
    return qmm(w, scales, biases, rms_normed(x, norm_weight, eps).reshape(1, k), 1, n, k, bits, group_size)


def affine_quantize(w, bits: int, group_size: int):
    """(packed u32 [n_groups * group_size * bits / 32], scales f32 [n_groups], biases f32 [n_groups]) of
    ``mt_affine_quantize_int*`` (crates/metaltile-std/src/mlx/quantized.rs:3629-3667)."""
    v = _f32(w).reshape(-1)
    if v.size % group_size or (group_size * bits) % 32:
        raise ValueError("whole groups of whole words only")
    ng = v.size // group_size
    out = np.zeros(ng * group_size * bits // 32, dtype=np.uint32)
    sc, bi = np.empty(ng, dtype=np.float32), np.empty(ng, dtype=np.float32)
    lib().mto_affine_quantize(_p(v), _p(out), _p(sc), _p(bi), _sz(ng), _sz(group_size), ctypes.c_uint32(bits))
    return out, sc, bi


def affine_dequantize(w, scales, biases, n_elem: int, bits: int, group_size: int) -> np.ndarray:
    """f32 [n_elem] of ``mt_affine_dequantize_int*`` (quantized.rs:3575-3604); scales / biases already rounded through T."""
    ww, sc, bi = _u32(w).reshape(-1), _f32(scales).reshape(-1), _f32(biases).reshape(-1)
    out = np.empty(n_elem, dtype=np.float32)
    lib().mto_affine_dequantize(_p(ww), _p(sc), _p(bi), _p(out), _sz(n_elem), _sz(group_size), ctypes.c_uint32(bits))
    return out


def dequant_gather(weight, scales, biases, indices, hidden: int, bits: int, group_size: int) -> np.ndarray:
    """f32 [n_tokens, hidden] of ``dequant_gather_int*`` (crates/metaltile-std/src/ffai/dequant_gather.rs:44-94)."""
    ww, sc, bi, ix = _u32(weight).reshape(-1), _f32(scales).reshape(-1), _f32(biases).reshape(-1), _u32(indices).reshape(-1)
    out = np.empty((ix.size, hidden), dtype=np.float32)
    lib().mto_dequant_gather(_p(ww), _p(sc), _p(bi), _p(ix), _p(out), _sz(ix.size), _sz(hidden), _sz(group_size), ctypes.c_uint32(bits))
    return out


def qvm(w, scales, biases, x, m: int, n: int, k: int, bits: int, group_size: int) -> np.ndarray:
    """f32 accumulator [m, n] of ``mt_qvm_*``: w [k, n*bits/32], scales / biases [k/group_size, n], x [m, k]
    (crates/metaltile-std/src/mlx/quantized.rs:5613-5635)."""
    ww, sc, bi, xv = _u32(w).reshape(-1), _f32(scales).reshape(-1), _f32(biases).reshape(-1), _f32(x).reshape(-1)
    out = np.empty((m, n), dtype=np.float32)
    lib().mto_qvm(_p(ww), _p(sc), _p(bi), _p(xv), _p(out), _sz(m), _sz(n), _sz(k), ctypes.c_uint32(bits), _sz(group_size))
    return out


def moe_down_swiglu_accum(gates, ups, experts, slot_weights, w, scales, biases, in_dim: int, out_dim: int, group_size: int) -> np.ndarray:
    """f32 [out_dim] of ``ffai_moe_down_swiglu_accum_int4_chain8`` (crates/metaltile-std/src/ffai/moe_down_swiglu_accum.rs:
    355-402): gates / ups [n_slots, in_dim], stacked int4 weights [E, out_dim, in_dim/8], scales / biases [E, out_dim, in_dim/G]."""
    g, u = _f32(gates).reshape(-1), _f32(ups).reshape(-1)
    ex, sw = _u32(experts).reshape(-1), _f32(slot_weights).reshape(-1)
    ww, sc, bi = _u32(w).reshape(-1), _f32(scales).reshape(-1), _f32(biases).reshape(-1)
    out = np.empty(out_dim, dtype=np.float32)
    lib().mto_moe_down_swiglu_accum(_p(g), _p(u), _p(ex), _p(sw), _p(ww), _p(sc), _p(bi), _p(out), _sz(ex.size), _sz(in_dim), _sz(out_dim),
                                    _sz(group_size))
    return out


def max_threads() -> int:
    return int(lib().mto_max_threads())
