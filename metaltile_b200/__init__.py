"""metaltile_b200 — B200 (sm_100a) back end for metaltile's affine group-quantized
matmul family (qmv / qmm / MoE gather_qmm), behind the C ABI of ``include/mtcuda.h``.

``Context`` mirrors the reference runtime's interface; ``ops`` wraps the typed entry
points for tensors already resident on the GPU.  Nothing here falls back to the CPU.
"""
from .context import BenchStats, Context, DispatchResult, MetalTileError  # noqa: F401
from ._lib import BF16, F16, F32  # noqa: F401

__all__ = ["Context", "DispatchResult", "BenchStats", "MetalTileError", "F32", "F16", "BF16"]
