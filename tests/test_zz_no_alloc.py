"""The allocation-free gather_qmm entry point against the regular one.

Some callers of the library cannot allocate device memory at the point where they run a MoE layer
(their own allocator owns all device memory, or the loop is latency-critical and must not take the
allocator's lock), so
``mtc_gather_qmm_static`` keeps its scratch in a fixed array of the library image.  It must give exactly
the results of ``mtc_gather_qmm``, also when it is called twice in a row on different inputs (the
array keeps the previous call's contents).  This file is collected last on purpose.
"""
import numpy as np
import pytest

import oracle
from helpers import ODT, TOL, rel_err, to_dev

pytestmark = pytest.mark.gpu


def _case(n_experts, n_out, k_in, bits, gs, dt, counts, seed):
    from metaltile_b200 import synth
    w, s, b = synth.quantized_matrix(n_experts * n_out, k_in, bits, gs, seed=seed, salt=31)
    total = int(np.sum(counts))
    x = synth.activations(total, k_in, seed=seed, salt=31)
    s, b, x = (oracle.round_through(a, ODT[dt]) for a in (s, b, x))
    off = np.concatenate([[0], np.cumsum(counts)]).astype(np.uint32)
    return (w.reshape(n_experts, n_out, -1), s.reshape(n_experts, n_out, -1), b.reshape(n_experts, n_out, -1), x, off)


def _run_both(ctx, w, s, b, x, off, bits, gs, dt):
    import torch
    from metaltile_b200 import ops
    from metaltile_b200.ops import _TORCH_DT
    wd, sd, bd, xd, od = to_dev(w), to_dev(s, dt), to_dev(b, dt), to_dev(x, dt), to_dev(off)
    ctx.set_option("gather_stream", 0)      # the static entry is the tensor-memory kernel: compare with that kernel's regular entry
    try:
        ref = ops.gather_qmm(xd, wd, sd, bd, bits, gs, expert_offsets=od, ctx=ctx)
    finally:
        ctx.set_option("gather_stream", 1)
    out = torch.zeros_like(ref)
    e, n_out, _ = w.shape
    ctx.gather_qmm_static(xd.data_ptr(), wd.data_ptr(), sd.data_ptr(), bd.data_ptr(), out.data_ptr(), x.shape[0], n_out,
                          x.shape[1], e, bits, gs, _TORCH_DT[xd.dtype], expert_offsets=od.data_ptr(),
                          stream=torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    return ref, out


def test_static_scratch_matches_regular_entry_twice_in_a_row():
    import torch
    from metaltile_b200 import MetalTileError, ops
    ctx = ops.context(0)
    # call 1: bf16 (uses the work list and the f16 staging area), 40 rows over 4 experts
    c1 = _case(4, 256, 512, 4, 64, "bf16", [5, 0, 32, 3], seed=1)
    ref1, out1 = _run_both(ctx, *c1, 4, 64, "bf16")
    assert torch.equal(ref1, out1)
    oracle_ref = oracle.gather_qmm(c1[3], c1[0], c1[1], c1[2], c1[3].shape[0], 512, 256, 4, 4, 64, expert_offsets=c1[4])
    assert rel_err(out1.float().cpu().numpy(), oracle_ref) <= TOL["bf16"]
    # call 2 right after: other shapes and fewer items, so stale list entries of call 1 lie behind the new count
    c2 = _case(3, 128, 256, 8, 32, "f16", [7, 9, 1], seed=2)
    ref2, out2 = _run_both(ctx, *c2, 8, 32, "f16")
    assert torch.equal(ref2, out2)
    # and call 1's inputs again: same answer as the first time
    ref3, out3 = _run_both(ctx, *c1, 4, 64, "bf16")
    assert torch.equal(out3, out1)
    assert ctx.status_word() == 0
    # sizes beyond the fixed array are refused with a clear error, nothing is launched
    xd = torch.empty((4097, 2048), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(MetalTileError) as ei:
        ctx.gather_qmm_static(xd.data_ptr(), 256, 256, 256, 256, 4097, 256, 2048, 4, 4, 64, "bf16", expert_offsets=256)
    assert ei.value.variant == "BufferSize" and "8388608" in str(ei.value)
    with pytest.raises(MetalTileError) as ei:
        ctx.gather_qmm_static(xd.data_ptr(), 256, 256, 256, 256, 16, 256, 96, 4, 4, 32, "bf16", expert_offsets=256)
    assert ei.value.variant == "Unsupported"


def test_static_scratch_refuses_what_does_not_fit():
    """The other two limits of the fixed array: more than 16384 work items, and more than 65536 bf16 rows.  Both are
    refused before anything is launched (the pointers below are never dereferenced)."""
    import torch
    from metaltile_b200 import MetalTileError, ops
    ctx = ops.context(0)
    dummy = 256
    with pytest.raises(MetalTileError) as ei:      # 5 row tiles x (1 + 4096 experts) items
        ctx.gather_qmm_static(dummy, dummy, dummy, dummy, dummy, 16, 640, 64, 4096, 4, 64, "f16", expert_offsets=dummy)
    assert ei.value.variant == "BufferSize" and "16384 work items" in str(ei.value)
    with pytest.raises(MetalTileError) as ei:      # 65537 rows of 64 elements: within the element limit, over the row limit
        ctx.gather_qmm_static(dummy, dummy, dummy, dummy, dummy, 65537, 128, 64, 4, 4, 64, "bf16", expert_offsets=dummy)
    assert ei.value.variant == "BufferSize" and "65536" in str(ei.value)
    torch.cuda.synchronize()
    assert ctx.status_word() == 0
