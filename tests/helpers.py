"""Shared helpers for the parity tests (CUDA path vs CPU oracle)."""
from __future__ import annotations

import numpy as np

import oracle
from metaltile_b200 import synth

DT_NAMES = ("f32", "f16", "bf16")
ODT = {"f32": oracle.F32, "f16": oracle.F16, "bf16": oracle.BF16}
# Pass criterion |got - oracle| / max(|oracle|, 1) <= tol — the reference's combined abs/rel form
# (crates/metaltile-std/tests/qmm_gpu_correctness.rs:2085-2106) with the tolerances the benchmark
# definition states: 1e-2 for f16/bf16 activations, 1e-4 for f32.
TOL = {"f32": 1e-4, "f16": 1e-2, "bf16": 1e-2}


def torch_dtype(name):
    import torch
    return {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}[name]


def rel_err(got: np.ndarray, ref: np.ndarray) -> float:
    got = np.asarray(got, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    if got.size == 0:
        return 0.0
    return float(np.max(np.abs(got - ref) / np.maximum(np.abs(ref), 1.0)))


def dense_case(m, n, k, bits, gs, dt, seed=0, salt=0):
    """Synthetic case; returns numpy inputs already rounded through dt plus raw words."""
    w, s, b = synth.quantized_matrix(n, k, bits, gs, seed, salt)
    x = synth.activations(m, k, seed, salt)
    s, b, x = (oracle.round_through(a, ODT[dt]) for a in (s, b, x))
    return w, s, b, x


def to_dev(arr, dt=None):
    import torch
    t = torch.from_numpy(np.ascontiguousarray(arr))
    if arr.dtype == np.uint32:
        t = torch.from_numpy(np.ascontiguousarray(arr).view(np.int32))
    t = t.cuda()
    if dt is not None:
        t = t.to(torch_dtype(dt))
    return t


def dt_bytes(arr_f32: np.ndarray, dt: str) -> bytes:
    """pack_f32 (crates/metaltile-std/src/utils.rs:26-37): f32 values -> little-endian dt bytes."""
    a = np.ascontiguousarray(arr_f32, dtype=np.float32)
    if dt == "f32":
        return a.tobytes()
    return oracle.to_bits16(a, ODT[dt]).tobytes()


def bytes_to_f32(raw: bytes, dt: str) -> np.ndarray:
    if dt == "f32":
        return np.frombuffer(raw, dtype=np.float32).copy()
    return oracle.from_bits16(np.frombuffer(raw, dtype=np.uint16), ODT[dt])
