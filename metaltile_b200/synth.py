"""Deterministic synthetic inputs for the quantized-matmul benchmarks and tests.

A SplitMix64 counter stream (seed * 0x9E3779B97F4A7C15 + stream id) gives u32 words,
24-bit uniforms and Box-Muller normals, vectorised in numpy so the same numbers can
be regenerated anywhere.  Value distributions follow the benchmark definition:
codes uniform in [0, 2^bits) (every field of a random word is uniform, also for the
3/5/6-bit streams), scale ~ U(0.002, 0.02) * 16 / 2^bits,
bias = -2^(bits-1) * scale + N(0, 1e-3), activations ~ N(0, 1).
"""
from __future__ import annotations

import numpy as np

GAMMA = np.uint64(0x9E3779B97F4A7C15)
STREAM_W, STREAM_SCALE, STREAM_BIAS, STREAM_X, STREAM_LOGITS = 1, 2, 3, 4, 5


def _splitmix(n: int, seed: int, stream: int) -> np.ndarray:
    with np.errstate(over="ignore"):
        base = np.uint64(seed) * GAMMA + np.uint64(stream)
        z = base + (np.arange(1, n + 1, dtype=np.uint64)) * GAMMA
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        return z ^ (z >> np.uint64(31))


def words(n: int, seed: int = 0, stream: int = STREAM_W) -> np.ndarray:
    return (_splitmix(n, seed, stream) >> np.uint64(32)).astype(np.uint32)


def uniform(n: int, seed: int = 0, stream: int = STREAM_SCALE) -> np.ndarray:
    return ((_splitmix(n, seed, stream) >> np.uint64(40)).astype(np.float32) * np.float32(2.0 ** -24))


def normal(n: int, seed: int = 0, stream: int = STREAM_X) -> np.ndarray:
    u = uniform(2 * n, seed, stream).astype(np.float64)
    u1 = np.maximum(u[:n], 2.0 ** -25)
    return (np.sqrt(-2.0 * np.log(u1)) * np.cos(2.0 * np.pi * u[n:])).astype(np.float32)


def quantized_matrix(n: int, k: int, bits: int, group_size: int, seed: int = 0, salt: int = 0):
    """(w u32[n, k*bits/32], scales f32[n, k/g], biases f32[n, k/g]) — not yet dtype-rounded."""
    assert (k * bits) % 32 == 0 and k % group_size == 0
    w = words(n * k * bits // 32, seed, STREAM_W + 16 * salt).reshape(n, k * bits // 32)
    g = n * (k // group_size)
    lo, hi = 0.002 * 16.0 / 2 ** bits, 0.02 * 16.0 / 2 ** bits
    scales = (np.float32(lo) + uniform(g, seed, STREAM_SCALE + 16 * salt) * np.float32(hi - lo)).astype(np.float32)
    biases = (-np.float32(2 ** (bits - 1)) * scales
              + normal(g, seed, STREAM_BIAS + 16 * salt) * np.float32(1e-3)).astype(np.float32)
    return w, scales.reshape(n, -1), biases.reshape(n, -1)


def activations(m: int, k: int, seed: int = 0, salt: int = 0) -> np.ndarray:
    return normal(m * k, seed, STREAM_X + 16 * salt).reshape(m, k)


def router_logits(rows: int, n_experts: int, seed: int = 0) -> np.ndarray:
    return normal(rows * n_experts, seed, STREAM_LOGITS).reshape(rows, n_experts)
