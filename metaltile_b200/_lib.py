"""ctypes loader for ``libmtcuda.so`` (the C ABI declared in ``include/mtcuda.h``).

There is no fallback: if the shared library is missing or a symbol is absent the
import of the op raises, and without a CUDA device ``mtc_init`` reports
``NoDevice``.
"""
from __future__ import annotations

import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libmtcuda.so")

F32, F16, BF16 = 0, 1, 2

STATUS_NAMES = {
    0: "Ok", -1: "NoDevice", -2: "Buffer", -3: "BufferSize", -4: "Dispatch",
    -5: "FunctionNotFound", -6: "Unsupported", -7: "Timeout", -8: "Invalid",
}


class QmvDesc(ctypes.Structure):
    """mtc_qmv_desc: one projection of a fused launch or of a chain."""
    _fields_ = [("w", ctypes.c_void_p), ("scales", ctypes.c_void_p), ("biases", ctypes.c_void_p), ("x", ctypes.c_void_p),
                ("outs", ctypes.c_void_p * 8), ("n_outs", ctypes.c_int), ("M", ctypes.c_int), ("N", ctypes.c_int),
                ("K", ctypes.c_int), ("bits", ctypes.c_int), ("group_size", ctypes.c_int), ("dtype", ctypes.c_int),
                ("phase", ctypes.c_int)]


class PeerSync(ctypes.Structure):
    """mtc_peer_sync: flag arrays and counters of the in-kernel hand-off between the GPUs of a node."""
    _fields_ = [("peer_flags", ctypes.c_void_p * 8), ("local_flags", ctypes.c_void_p), ("epoch", ctypes.c_void_p),
                ("ticket", ctypes.c_void_p), ("n_peers", ctypes.c_int), ("rank", ctypes.c_int)]


class DispatchSpec(ctypes.Structure):
    """mtc_dispatch_spec: one pass of mtc_dispatch_chain."""
    _fields_ = [("kernel_name", ctypes.c_char_p), ("dtype", ctypes.c_int), ("bufs", ctypes.c_void_p), ("n_bufs", ctypes.c_int)]


class BenchStatsC(ctypes.Structure):
    """mtc_bench_stats: the summary mtc_measure fills."""
    _fields_ = [(n, ctypes.c_double) for n in ("min_us", "mean_us", "median_us", "p95_us", "p99_us", "stddev_us", "cv_pct")] + \
               [("iters", ctypes.c_int)]


class QMat(ctypes.Structure):
    """mtc_qmat: packed words, scales and biases of one stacked expert matrix."""
    _fields_ = [("w", ctypes.c_void_p), ("scales", ctypes.c_void_p), ("biases", ctypes.c_void_p)]


class NamedBuf(ctypes.Structure):
    _fields_ = [("name", ctypes.c_char_p), ("data", ctypes.c_void_p), ("bytes", ctypes.c_size_t),
                ("is_output", ctypes.c_int)]


_vp, _i, _sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t
_DENSE = [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i]

# name -> (restype, argtypes); every symbol include/mtcuda.h declares
SIGNATURES = {
    "mtc_init": (_i, [_i, ctypes.POINTER(_vp)]),
    "mtc_destroy": (_i, [_vp]),
    "mtc_last_error": (ctypes.c_char_p, [_vp]),
    "mtc_device_info": (_i, [_vp, ctypes.c_char_p, _sz]),
    "mtc_alloc": (_i, [_vp, _sz, ctypes.POINTER(_vp)]),
    "mtc_free": (_i, [_vp, _vp]),
    "mtc_upload": (_i, [_vp, _vp, _vp, _vp, _sz]),
    "mtc_download": (_i, [_vp, _vp, _vp, _vp, _sz]),
    "mtc_memset": (_i, [_vp, _vp, _vp, _i, _sz]),
    "mtc_sync": (_i, [_vp, _vp]),
    "mtc_sync_deadline": (_i, [_vp, _vp, _i]),
    "mtc_status_word": (_i, [_vp, ctypes.POINTER(ctypes.c_uint32)]),
    "mtc_status_clear": (_i, [_vp]),
    "mtc_qmv": (_i, _DENSE),
    "mtc_qmm": (_i, _DENSE),
    "mtc_qmm_route": (ctypes.c_char_p, [_i, _i, _i, _i, _i, _i]),
    "mtc_qmv_multi": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, ctypes.POINTER(_vp), _i, _i, _i, _i, _i, _i, _i]),
    "mtc_affine_quantize": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, ctypes.c_size_t, _i, _i, _i]),
    "mtc_affine_dequantize": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, ctypes.c_size_t, _i, _i, _i]),
    "mtc_moe_down_swiglu_accum": (_i, [_vp, _vp, ctypes.POINTER(_vp), ctypes.POINTER(_vp), _i, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i]),
    "mtc_qmv_expert_indexed": (_i, [_vp, _vp, ctypes.POINTER(_vp), _i, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i]),
    "mtc_qvm": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i]),
    "mtc_dequant_gather": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, ctypes.c_size_t, _i, _i, _i, _i, _i]),
    "mtc_rms_norm_qmv": (_i, [_vp, _vp, _vp, _vp, ctypes.c_float, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i]),
    "mtc_qmm_multi": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, ctypes.POINTER(_vp), _i, ctypes.c_longlong, _i, _i, _i, _i, _i, _i]),
    "mtc_qmv_batched": (_i, [_vp, _vp, ctypes.POINTER(QmvDesc), _i]),
    "mtc_qmv_batched_sync": (_i, [_vp, _vp, ctypes.POINTER(QmvDesc), _i, ctypes.POINTER(PeerSync)]),
    "mtc_chain_create": (_i, [_vp, ctypes.POINTER(QmvDesc), _i, ctypes.POINTER(_vp)]),
    "mtc_chain_run": (_i, [_vp, _vp, _vp]),
    "mtc_chain_destroy": (_i, [_vp, _vp]),
    "mtc_chain_is_fused": (_i, [_vp]),
    "mtc_ipc_export": (_i, [_vp, _vp, _vp]),
    "mtc_ipc_open": (_i, [_vp, _vp, ctypes.POINTER(_vp)]),
    "mtc_ipc_close": (_i, [_vp, _vp]),
    "mtc_peer_barrier": (_i, [_vp, _vp, ctypes.POINTER(_vp), _i, _i, _vp, _vp]),
    "mtc_gather_qmm": (_i, [_vp] * 9 + [_i] * 7),
    "mtc_gather_qmm_static": (_i, [_vp] * 9 + [_i] * 7),
    "mtc_dispatch_chain": (_i, [_vp, ctypes.POINTER(DispatchSpec), _i, ctypes.POINTER(ctypes.c_float)]),
    "mtc_moe_experts": (_i, [_vp, _vp, _vp, _vp, _i, ctypes.POINTER(QMat), ctypes.POINTER(QMat), ctypes.POINTER(QMat), _vp, _vp,
                            _i, _i, _i, _i, _i, _i, _i]),
    "mtc_gather_qmm_route": (ctypes.c_char_p, [_i] * 7),
    "mtc_moe_router_topk": (_i, [_vp] * 5 + [_i] * 5),
    "mtc_moe_sort": (_i, [_vp, _vp, _vp, _i, _i, _i, _vp, _vp, _vp, _vp]),
    "mtc_moe_permute": (_i, [_vp] * 5 + [_i] * 3),
    "mtc_moe_unpermute": (_i, [_vp] * 6 + [_i] * 4),
    "mtc_swiglu": (_i, [_vp] * 5 + [_sz, _i]),
    "mtc_set_option": (_i, [_vp, ctypes.c_char_p, _i]),
    "mtc_unpack_codes": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i]),
    "mtc_measure": (_i, [_vp, ctypes.c_char_p, _i, ctypes.POINTER(NamedBuf), _i, _i, _i, _i, ctypes.POINTER(ctypes.c_double),
                         ctypes.POINTER(BenchStatsC)]),
    "mtc_dispatch": (_i, [_vp, ctypes.c_char_p, _i, ctypes.POINTER(NamedBuf), _i,
                          ctypes.POINTER(ctypes.c_uint32), ctypes.POINTER(ctypes.c_uint32),
                          ctypes.POINTER(ctypes.c_float)]),
    "mtc_kernel_count": (_i, []),
    "mtc_kernel_name": (ctypes.c_char_p, [_i]),
}

_lib = None


def load() -> ctypes.CDLL:
    """Load the library and bind every declared symbol; raises if anything is missing."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} not found: build it with `python -m metaltile_b200.build` "
            "(there is no CPU or PyTorch fallback for these ops)")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the export is missing
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib
