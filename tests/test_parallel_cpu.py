"""World-size-2 gloo runs of the N-split and expert-parallel exchange logic on CPU.  The compute steps are
played by the CPU oracle through the backend interface of metaltile_b200.parallel (gloo ranks have no GPU);
what is under test is the sharding arithmetic, the all-gather layout and the two all-to-all exchanges."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from metaltile_b200 import parallel, synth

BITS, GS = 4, 32


class OracleBackend:
    """f32 CPU tensors in, f32 CPU tensors out; every step is the reference's scalar semantics."""

    def qmv(self, w, s, b, x, bits, gs, out=None):
        n, k = w.shape[0], x.shape[1]
        return torch.from_numpy(oracle.qmm(w.numpy().view(np.uint32), s.numpy(), b.numpy(), x.numpy(), x.shape[0], n, k, bits, gs))

    def router_topk(self, logits, k, norm):
        idx, w = oracle.router_topk(logits.numpy(), logits.shape[1], k, norm)
        return torch.from_numpy(idx.view(np.int32)), torch.from_numpy(w)

    def moe_sort(self, idx, n_experts):
        return tuple(torch.from_numpy(a.view(np.int32)) for a in oracle.moe_sort(idx.numpy().view(np.uint32), n_experts))

    def permute(self, tokens, sti):
        return torch.from_numpy(oracle.moe_permute(tokens.numpy(), sti.numpy().view(np.uint32)))

    def unpermute(self, eo, inv, wts):
        return torch.from_numpy(oracle.moe_unpermute(eo.numpy(), inv.numpy().view(np.uint32), wts.numpy()))

    def swiglu(self, g, u):
        return torch.from_numpy(oracle.swiglu(g.numpy(), u.numpy()))

    def gather_qmm(self, x, w, s, b, bits, gs, offsets):
        e, n, _ = w.shape
        k = x.shape[1]
        return torch.from_numpy(oracle.gather_qmm(x.numpy(), w.numpy().view(np.uint32), s.numpy(), b.numpy(), x.shape[0], k, n, e,
                                                  bits, gs, expert_offsets=offsets.numpy().view(np.uint32)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _moe_weights(E, H, I):
    mk = lambda n, k, salt: synth.quantized_matrix(E * n, k, BITS, GS, seed=0, salt=salt)
    t3 = lambda w, s, b, n: (torch.from_numpy(w.view(np.int32).reshape(E, n, -1)), torch.from_numpy(s.reshape(E, n, -1)),
                             torch.from_numpy(b.reshape(E, n, -1)))
    return t3(*mk(I, H, 1), I), t3(*mk(I, H, 2), I), t3(*mk(H, I, 3), H)


def _worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        be = OracleBackend()
        # ---- N-split + all-gather
        n, k, m = 48, 64, 3
        w, s, b = synth.quantized_matrix(n, k, BITS, GS, seed=1)
        x = synth.activations(m, k, seed=1)
        r0, r1 = parallel.shard_rows(n, world, rank)
        lin = parallel.ColumnParallelLinear(torch.from_numpy(w[r0:r1].view(np.int32)), torch.from_numpy(s[r0:r1]),
                                            torch.from_numpy(b[r0:r1]), BITS, GS, backend=be)
        got = lin.forward(torch.from_numpy(x)).numpy()
        ref = oracle.qmm(w, s, b, x, m, n, k, BITS, GS)
        assert got.shape == (m, n) and np.array_equal(got, ref), "column-parallel result differs"
        one = lin.forward(torch.from_numpy(x[:1])).numpy()
        assert np.array_equal(one, ref[:1])

        # ---- K-split + all-reduce: each rank multiplies its slice of the columns, partial sums are added
        n, k, m = 24, 128, 2                       # K / world = 64 = two groups of 32
        w, s, b = synth.quantized_matrix(n, k, BITS, GS, seed=3)
        x = synth.activations(m, k, seed=3)
        wl, sl_, bl = parallel.shard_cols(torch.from_numpy(w.view(np.int32)), torch.from_numpy(s), torch.from_numpy(b),
                                          BITS, GS, world, rank)
        row = parallel.RowParallelLinear(wl, sl_, bl, BITS, GS, backend=be)
        kl = k // world
        got = row.forward(torch.from_numpy(x[:, rank * kl:(rank + 1) * kl].copy())).numpy()
        ref = oracle.qmm(w, s, b, x, m, n, k, BITS, GS)
        # the split changes the order of the f32 additions only: one extra rounding per rank
        assert got.shape == (m, n) and np.max(np.abs(got - ref) / np.maximum(np.abs(ref), 1.0)) <= 1e-5, "row-parallel result differs"

        # ---- peer-buffer setup: a rank whose allocation fails must make every rank raise, none may be left waiting
        class FakeCtx:
            def __init__(self, fail):
                self.fail, self.freed, self.closed, self.n = fail, [], [], 0
            def alloc(self, nbytes):
                if self.fail:
                    raise RuntimeError("out of memory (injected)")
                self.n += 1
                return 0x1000 * self.n
            def memset(self, *a): pass
            def sync(self): pass
            def ipc_export(self, ptr): return ptr.to_bytes(8, "little") * 8
            def ipc_open(self, h): return int.from_bytes(h[:8], "little") + 0x100000
            def ipc_close(self, ptr): self.closed.append(ptr)
            def free(self, ptr): self.freed.append(ptr)
        fake = FakeCtx(fail=(rank == 1))
        try:
            parallel.PeerGather(fake, 64)
            raise AssertionError("peer-buffer setup should have failed on every rank")
        except RuntimeError as e:
            assert "could not be shared" in str(e)
        assert fake.closed == [] and (fake.freed == [0x1000, 0x2000] if rank == 0 else fake.freed == [])
        good = FakeCtx(fail=False)
        pg = parallel.PeerGather(good, 64)
        assert pg.peer_bufs[rank] == 0x1000 and pg.peer_bufs[1 - rank] == 0x1000 + 0x100000
        assert pg.peer_flags[1 - rank] == 0x2000 + 0x100000
        pg.close()
        assert sorted(good.closed) == [0x101000, 0x102000] and good.freed == [0x1000, 0x2000]

        # ---- expert parallel: 8 experts over 2 ranks, 10 tokens per rank, top-2
        E, H, I, T, K2 = 8, 64, 32, 10, 2
        gate, up, down = _moe_weights(E, H, I)
        el = E // world
        sl = slice(rank * el, (rank + 1) * el)
        shard = parallel.ExpertShard(tuple(t[sl].contiguous() for t in gate), tuple(t[sl].contiguous() for t in up),
                                     tuple(t[sl].contiguous() for t in down), BITS, GS)
        tok_all = synth.activations(T * world, H, seed=2)
        log_all = synth.router_logits(T * world, E, seed=2)
        mine = slice(rank * T, (rank + 1) * T)
        layer = parallel.ExpertParallelMoE(shard, E, K2, backend=be)
        got = layer.forward(torch.from_numpy(tok_all[mine].copy()), torch.from_numpy(log_all[mine].copy())).numpy()
        # unsharded reference: the same layer with every expert local, world size 1 semantics
        full = parallel.ExpertParallelMoE.__new__(parallel.ExpertParallelMoE)
        full.shard = parallel.ExpertShard(gate, up, down, BITS, GS)
        full.n_experts, full.top_k, full.norm, full.backend, full.group, full.world, full.e_local = E, K2, 1, be, None, 1, E
        ref = full.forward(torch.from_numpy(tok_all[mine].copy()), torch.from_numpy(log_all[mine].copy())).numpy()
        # the experts see the same rows in a different order, so every row's arithmetic is identical
        assert np.array_equal(got, ref), f"expert-parallel result differs on rank {rank}"
        q.put((rank, "ok"))
    except Exception as e:  # pragma: no cover - reported to the parent
        q.put((rank, repr(e)))
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(180)
def test_two_rank_gloo_exchange():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=150) for _ in procs]
    for p in procs:
        p.join(timeout=30)
    assert sorted(results) == [(0, "ok"), (1, "ok")], results


def test_shard_cols():
    w, s, b = synth.quantized_matrix(6, 256, BITS, GS, seed=4)
    wt, st, bt = torch.from_numpy(w.view(np.int32)), torch.from_numpy(s), torch.from_numpy(b)
    parts = [parallel.shard_cols(wt, st, bt, BITS, GS, 4, r) for r in range(4)]
    assert torch.equal(torch.cat([p_[0] for p_ in parts], dim=1), wt)
    assert torch.equal(torch.cat([p_[1] for p_ in parts], dim=1), st)
    assert parts[0][0].shape == (6, 256 // 4 * BITS // 32) and parts[0][1].shape == (6, 2)
    # the codes of a slice are the slice of the codes
    full = oracle.unpack_matrix(w, 256, BITS)
    part = oracle.unpack_matrix(parts[2][0].numpy().view(np.uint32), 64, BITS)
    assert np.array_equal(part, full[:, 128:192])
    with pytest.raises(ValueError):
        parallel.shard_cols(wt, st, bt, BITS, GS, 16, 0)      # 16 columns per rank: less than a group


def test_shard_rows_and_order():
    assert parallel.shard_rows(14336, 8, 3) == (5376, 7168)
    with pytest.raises(ValueError):
        parallel.shard_rows(10, 4, 0)
    rc = torch.tensor([[2, 0, 1], [1, 3, 0]])        # 2 sources x 3 local experts
    order = parallel.expert_major_order(rc).tolist()
    # arrival: s0:[e0,e0,e2] s1:[e0,e1,e1,e1] -> expert-major: e0:(s0:0,1)(s1:3) e1:(s1:4,5,6) e2:(s0:2)
    assert order == [0, 1, 3, 4, 5, 6, 2]
    assert parallel.expert_major_order(torch.zeros((2, 3), dtype=torch.int64)).numel() == 0
