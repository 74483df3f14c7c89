"""Multi-rank host logic on CPU (gloo, world_size 2): the K-shard bookkeeping of the row-parallel
linears with an all-reduce, and the expert-parallel dispatch/combine with two all-to-alls.  The
arithmetic inside is done by the CPU oracle, so these tests need no GPU."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from arcquant_b200 import tp
from arcquant_b200.moe_block import ExpertParallelDispatcher, route_top_k


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _init(rank, world, port):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)


def test_shard_bookkeeping():
    idx = torch.randperm(1024, generator=torch.Generator().manual_seed(0)).to(torch.int16)
    seen = []
    for r in range(4):
        a, b = tp.shard_range(1024, 4, r)
        loc = tp.local_reorder_index(idx, a, b)
        assert sorted(loc.tolist()) == list(range(256))                  # a permutation of the slice
        glob = [int(v) for v in idx.tolist() if a <= v < b]
        assert [v + a for v in loc.tolist()] == glob                     # global importance order kept
        seen += [v + a for v in loc.tolist()]
    assert sorted(seen) == list(range(1024))
    assert tp.shard_select_num(128, 1, 4096) == 128
    assert [tp.shard_select_num(128, t, 4096 // t) for t in (2, 4, 8)] == [64, 64, 64]
    assert tp.shard_select_num(0, 4, 1024) == 0
    assert (14336 // 8 + tp.shard_select_num(128, 8, 14336 // 8)) % 64 == 0
    with pytest.raises(ValueError):
        tp.shard_range(10, 4, 0)


def _row_parallel_worker(rank, world, port, q):
    from oracle import oracle as O

    _init(rank, world, port)
    try:
        g = torch.Generator().manual_seed(0)                             # same tensors on every rank
        K, N, M, KE = 512, 64, 24, 128
        x = (torch.randn(M, K, generator=g) * 3).to(torch.bfloat16)
        w = (torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16)
        idx = torch.randperm(K, generator=g).to(torch.int16)
        a, b = tp.shard_range(K, world, rank)
        loc = tp.local_reorder_index(idx, a, b).numpy()
        ke = tp.shard_select_num(KE, world, b - a)
        qa, sfa = O.quantize_x(x[:, a:b].contiguous(), loc, ke)
        qb, sfb = O.quantize_w(w[:, a:b].contiguous(), loc, ke)
        part = torch.from_numpy(O.gemm_fast(qa, sfa, qb, sfb, 1.0))
        total = tp.all_reduce_sum(part.clone())
        # every rank can recompute all shards locally: the collective must equal their sum
        ref = torch.zeros(M, N)
        for r in range(world):
            a2, b2 = tp.shard_range(K, world, r)
            l2 = tp.local_reorder_index(idx, a2, b2).numpy()
            k2 = tp.shard_select_num(KE, world, b2 - a2)
            q1, s1 = O.quantize_x(x[:, a2:b2].contiguous(), l2, k2)
            q2, s2 = O.quantize_w(w[:, a2:b2].contiguous(), l2, k2)
            ref += torch.from_numpy(O.gemm_fast(q1, s1, q2, s2, 1.0))
        full = x.float() @ w.float().T
        ok = torch.allclose(total, ref, rtol=1e-6, atol=1e-6) and \
            float((total - full).norm() / full.norm()) < 0.2
        q.put((rank, bool(ok)))
    finally:
        dist.destroy_process_group()


def _moe_worker(rank, world, port, q):
    _init(rank, world, port)
    try:
        E, H, T, k = 8, 32, 50 + 7 * rank, 2                              # ragged token counts per rank
        g = torch.Generator().manual_seed(100 + rank)
        x = torch.randn(T, H, generator=g)
        router = torch.randn(E, H, generator=torch.Generator().manual_seed(1))
        ids, w = route_top_k(x, router, k)
        d = ExpertParallelDispatcher(E, rank, world)
        batch = d.dispatch(x, ids)
        rows, owner = batch.rows(), batch.row_expert()
        assert rows.shape[0] == batch.rows_bound and batch.rows_bound % 256 == 0
        assert int((owner >= 0).sum()) == int(batch.groups[d.e_local:].sum())
        # fake expert e: y = x * (e + 1); padding rows get a value that must never reach a token
        y = torch.where(owner[:, None] >= 0, rows * (rank * d.e_local + owner[:, None] + 1).to(rows.dtype),
                        torch.full_like(rows, float("nan")))
        state = batch
        out = d.combine(y, w, state)
        ref = torch.zeros_like(x)
        for t in range(T):
            for j in range(k):
                ref[t] += x[t] * (int(ids[t, j]) + 1) * w[t, j]
        q.put((rank, bool(torch.allclose(out, ref, rtol=1e-5, atol=1e-5))))
    finally:
        dist.destroy_process_group()


def _moe_overflow_worker(rank, world, port, q):
    """Blocks of limited capacity: every copy is routed to rank 0's first expert, more than a block holds.
    The copies that fit are exact, the dropped ones contribute zero, and the dispatcher says so."""
    _init(rank, world, port)
    try:
        E, H, T, k = 4, 16, 200, 2
        x = torch.randn(T, H, generator=torch.Generator().manual_seed(7 + rank))
        ids = torch.zeros(T, k, dtype=torch.int64)
        w = torch.full((T, k), 0.5)
        d = ExpertParallelDispatcher(E, rank, world, capacity_factor=1.0)
        batch = d.dispatch(x, ids)
        assert d.capacity == 256                                           # even share 200, rounded up to 128s
        rows, owner = batch.rows(), batch.row_expert()
        y = torch.where(owner[:, None] >= 0, rows * 3.0, torch.full_like(rows, float("nan")))
        out = d.combine(y, w, batch)
        kept = torch.arange(T * k).reshape(T, k) < 256                     # copies in token order fill the block
        ref = (x[:, None, :] * 3.0 * 0.5 * kept[:, :, None]).sum(1)
        ok = torch.allclose(out, ref, rtol=1e-5, atol=1e-5) and d.overflowed()
        exact = ExpertParallelDispatcher(E, rank, world)                   # worst-case capacity: nothing dropped
        b2 = exact.dispatch(x, ids)
        r2, o2 = b2.rows(), b2.row_expert()
        out2 = exact.combine(torch.where(o2[:, None] >= 0, r2 * 3.0, torch.full_like(r2, float("nan"))), w, b2)
        ok = ok and torch.allclose(out2, x * 3.0, rtol=1e-5, atol=1e-5) and not exact.overflowed()
        q.put((rank, bool(ok)))
    finally:
        dist.destroy_process_group()


def _peer_block_failure_worker(rank, world, port, q):
    """Setting up peer memory when one rank cannot: the device steps are replaced by fakes (an allocation that
    fails on rank 1; a mapping that fails on rank 0), everything else - the exchanges through the process
    group - is the real code.  Every rank must come back with the same error instead of waiting for the other
    in a collective, and a set-up in which nothing fails must work with the same fakes."""
    _init(rank, world, port)
    try:
        from arcquant_b200.peer import PeerBlock

        class Fake(PeerBlock):
            fail_alloc_on = fail_open_on = None

            def _make_own(self):
                if self.rank == self.fail_alloc_on:
                    raise RuntimeError("out of memory (fake)")
                self._own.value = 0x1000 * (self.rank + 1)
                return bytes([self.rank]) * 64

            def _open(self, handle, owner):
                if self.rank == self.fail_open_on:
                    raise RuntimeError("cannot map (fake)")
                return 0x100000 + handle[0]

        ok = True
        good = Fake(1024, rank, world, None, "cpu")
        ok = ok and good.base == [0x1000 if rank == 0 else 0x100000, 0x100001 if rank == 0 else 0x2000]
        for attr, who, text in (("fail_alloc_on", 1, "out of memory"), ("fail_open_on", 0, "cannot map")):
            setattr(Fake, attr, who)
            try:
                Fake(1024, rank, world, None, "cpu")
                ok = False
            except RuntimeError as exc:
                ok = ok and "peer memory unavailable" in str(exc) and f"rank {who}" in str(exc) and text in str(exc)
            setattr(Fake, attr, None)
        q.put((rank, bool(ok)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("worker", [_row_parallel_worker, _moe_worker, _moe_overflow_worker, _peer_block_failure_worker])
def test_two_rank_gloo(worker):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=180) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert sorted(results) == [(0, True), (1, True)]


def test_single_rank_dispatch_matches_dense():
    E, H, T, k = 4, 16, 33, 2
    g = torch.Generator().manual_seed(0)
    x = torch.randn(T, H, generator=g)
    router = torch.randn(E, H, generator=g)
    ids, w = route_top_k(x, router, k)
    assert torch.allclose(w.sum(1), torch.ones(T))
    d = ExpertParallelDispatcher(E)
    batch = d.dispatch(x, ids)
    rows, owner = batch.rows(), batch.row_expert()
    # every run starts on a 256-row tile and holds exactly the copies routed to its expert, in token order
    g = batch.groups.tolist()
    for e in range(E):
        assert g[e] % 256 == 0 and g[E + e] == int((ids == e).sum())
        assert bool((owner[g[e]:g[e] + g[E + e]] == e).all())
        tok = torch.where(ids == e)[0]
        assert torch.equal(rows[g[e]:g[e] + g[E + e]], x[tok])
        assert set(batch.tile_group[g[e] // 256:(g[e] + g[E + e] + 255) // 256].tolist()) <= {e}
    assert int((batch.tile_group >= 0).sum()) == sum((g[E + e] + 255) // 256 for e in range(E))
    y = torch.where(owner[:, None] >= 0, rows * (owner[:, None] + 1).to(rows.dtype), torch.full_like(rows, float("nan")))
    state = batch
    out = d.combine(y, w, state)
    ref = sum(x * (ids[:, j:j + 1] + 1) * w[:, j:j + 1] for j in range(k))
    assert torch.allclose(out, ref, rtol=1e-5, atol=1e-5)
