"""CPU-side checks of the boundary: the shared library loads, exports every symbol the
header declares, and refuses to run without a device (no CPU fallback)."""
import os
import re

import pytest

from metaltile_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    names = set()
    inc = os.path.join(ROOT, "include")
    for fn in os.listdir(inc):
        if fn.endswith(".h"):
            text = open(os.path.join(inc, fn)).read()
            text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
            names.update(re.findall(r"\b(mtc_[a-z0-9_]+)\s*\(", text))
    return names


def test_library_exports_every_declared_symbol():
    lib = _lib.load()
    declared = _declared_symbols()
    assert declared, "no declarations found in include/*.h"
    for name in sorted(declared):
        assert hasattr(lib, name), f"{name} declared in include/ but not exported by libmtcuda.so"
    # and the ctypes table covers exactly the declared set
    assert set(_lib.SIGNATURES) == declared


def test_registry_holds_reference_kernel_names():
    lib = _lib.load()
    names = {lib.mtc_kernel_name(i).decode() for i in range(lib.mtc_kernel_count())}
    for n in ("mt_qmv", "mt_qmv_int8_fast", "mt_qmm", "mt_qmm_bm2", "mt_qmm_bm4", "mt_qmm_mma", "mt_qmm_mma_m16",
              "mt_qmm_mma_int8", "mt_qmm_mma_int2", "mt_qmm_mma_b3", "mt_qmv_b3", "mt_qmv_b6", "mt_qmm_b5"):
        assert n in names
    assert lib.mtc_kernel_name(-1) is None and lib.mtc_kernel_name(10_000) is None


def test_no_device_is_an_error_not_a_fallback():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    from metaltile_b200 import Context, MetalTileError
    with pytest.raises(MetalTileError) as ei:
        Context(0)
    assert ei.value.variant == "NoDevice"


def test_product_does_not_import_the_oracle():
    pkg = os.path.join(ROOT, "metaltile_b200")
    for dirpath, _, files in os.walk(pkg):
        for fn in files:
            if fn.endswith((".py", ".cu", ".cuh", ".cpp", ".h")):
                text = open(os.path.join(dirpath, fn)).read()
                assert "import oracle" not in text and "from oracle" not in text and "mt_oracle" not in text, fn
