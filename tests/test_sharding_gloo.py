"""Host logic of the column-parallel / expert-parallel split, two gloo ranks on CPU.
The compute callable is a plain fp32 stand-in: these tests check partition arithmetic, shard
placement and the all-gather layout, not the kernels."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from dsl_tool_b200.sharding import (ColumnParallelLinear, ExpertParallelGroupedLinear, column_ranges,
                                    expert_ranges, local_rows, shard_weight_columns, shard_weight_experts)


def test_column_ranges():
    assert column_ranges(14336, 8) == [(i * 1792, (i + 1) * 1792) for i in range(8)]
    assert column_ranges(28672, 4)[3] == (21504, 28672)
    r = column_ranges(1000, 3)          # 8 aligned blocks -> 3, 3, 2; last one ragged
    assert r == [(0, 384), (384, 768), (768, 1000)]
    assert column_ranges(100, 4) == [(0, 100), (100, 100), (100, 100), (100, 100)]
    for n, w in [(8192, 8), (3072, 2), (777, 5)]:
        rr = column_ranges(n, w)
        assert rr[0][0] == 0 and rr[-1][1] == n and all(a[1] == b[0] for a, b in zip(rr, rr[1:]))
        assert all(s % 128 == 0 for s, _ in rr if s < n)


def test_expert_ranges_and_local_rows():
    assert expert_ranges(64, 8) == [(8 * i, 8 * i + 8) for i in range(8)]
    assert expert_ranges(5, 2) == [(0, 3), (3, 5)]
    offs = [0, 4, 4, 10, 17, 20]
    assert local_rows(offs, 0, 3) == (0, 10, [0, 4, 4, 10])
    assert local_rows(offs, 3, 5) == (10, 20, [0, 7, 10])


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _fake_linear(x, w, expert_offsets=None, **kw):
    if expert_offsets is None:
        return x.float() @ w.float().t()
    out = torch.zeros(x.shape[0], w.shape[1])
    for g in range(w.shape[0]):
        a, b = int(expert_offsets[g]), int(expert_offsets[g + 1])
        out[a:b] = x[a:b].float() @ w[g].float().t()
    return out


def _worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(0)                      # identical tensors on every rank
        x = torch.randn(37, 64, generator=g)
        w = torch.randn(1000, 64, generator=g)                    # ragged split: 512 + 488 columns
        full = x @ w.t()
        lin = ColumnParallelLinear(shard_weight_columns(w, rank, world), 1000, _fake_linear)
        y = lin.forward(x)
        s, e = column_ranges(1000, world)[rank]
        ok = torch.allclose(y, full[:, s:e], atol=1e-5)
        ok &= torch.allclose(lin.forward(x, gather=True), full, atol=1e-5)
        w2 = torch.randn(1024, 64, generator=g)                   # even split -> all_gather_into_tensor path
        lin2 = ColumnParallelLinear(shard_weight_columns(w2, rank, world), 1024, _fake_linear)
        ok &= torch.allclose(lin2.forward(x, gather=True), x @ w2.t(), atol=1e-5)
        G = 5
        wg = torch.randn(G, 48, 64, generator=g)
        offs = [0, 4, 4, 10, 30, 37]                              # an empty expert, uneven expert split (3 + 2)
        want = _fake_linear(x, wg, offs)
        ep = ExpertParallelGroupedLinear(shard_weight_experts(wg, rank, world), G, _fake_linear)
        r0, r1, _ = local_rows(offs, ep.first, ep.last)
        ok &= torch.allclose(ep.forward_from_global(x, offs), want[r0:r1], atol=1e-5)
        ok &= torch.allclose(ep.forward_from_global(x, offs, gather=True), want, atol=1e-5)
        results[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


def test_two_rank_split_and_gather():
    world = 2
    ctx = mp.get_context("spawn")
    results = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, results)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert dict(results) == {0: True, 1: True}


# ---- token all-to-all (host side) and what happens when a rank stops taking part -------------------------------

def _exchange_worker(rank, world, port, results):
    from dsl_tool_b200.sharding import arrival_expert_ids, exchange_rows, return_rows
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        E = 5                                                     # experts 0-2 on rank 0, 3-4 on rank 1
        counts = torch.tensor([[3, 0, 2, 4, 1], [0, 0, 5, 0, 2]][rank], dtype=torch.int32)   # expert 1 gets nothing at all
        n = int(counts.sum())
        expert_of = torch.repeat_interleave(torch.arange(E), counts.long())
        # a record says who sent it, for which expert, and its position in the sender's sorted order
        records = torch.stack([torch.full((n,), rank), expert_of, torch.arange(n)], dim=1).to(torch.int32)
        ex = exchange_rows(records, counts, E, None)
        first = [0, 3][rank]
        ids = arrival_expert_ids(ex, "cpu")
        ok = bool((ex.received[:, 1] - first == ids).all())       # every arrived record belongs to the expert the counts say
        ok &= ex.recv_rows == [int(((ex.received[:, 0] == s)).sum()) for s in range(world)]
        ok &= sorted(ex.received[ex.received[:, 0] == 0][:, 2].tolist()) == ex.received[ex.received[:, 0] == 0][:, 2].tolist()
        back = return_rows(ex.received * 10, ex, None)            # "compute" = times ten, then the way back
        ok &= bool(torch.equal(back, records * 10))
        results[rank] = ok
    finally:
        dist.destroy_process_group()


def test_token_exchange_round_trip():
    port = _free_port()
    mgr = mp.Manager()
    results = mgr.dict()
    mp.spawn(_exchange_worker, args=(2, port, results), nprocs=2, join=True)
    assert results[0] and results[1]


def _leaving_worker(rank, world, port, results, what):
    import datetime
    import time
    from dsl_tool_b200.sharding import all_gather_columns, column_ranges, exchange_rows
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=4))
    store = dist.distributed_c10d._get_default_store()

    def step():
        if what == "gather":
            return all_gather_columns(torch.full((3, 128), float(rank)), column_ranges(256, world), None)
        counts = torch.tensor([2, 1], dtype=torch.int32)
        return exchange_rows(torch.arange(6, dtype=torch.int32).reshape(3, 2), counts, 2, None)

    step()                                                        # step 1: everybody takes part
    if rank == 1:
        # leaves BETWEEN two steps (nothing of its own is in flight) and stays away until rank 0 has seen the failure
        store.wait(["rank0_saw_it"], datetime.timedelta(seconds=60))
        results[rank] = "left"
        return                                                    # no destroy_process_group: the group is broken by design
    t0 = time.monotonic()
    try:
        step()                                                    # step 2: the peer never joins
        results[rank] = "no error"
    except Exception as exc:                                      # the group's time limit (or the transport) ends the wait
        results[rank] = f"raised after {time.monotonic() - t0:.1f}s: {type(exc).__name__}"
    store.set("rank0_saw_it", "1")


@pytest.mark.parametrize("what", ["gather", "exchange"])
def test_a_rank_that_stops_taking_part_ends_the_collective_with_an_error(what):
    """The all-gather of the column shards and the token exchange are host-launched collectives: when a rank does not
    join, the others must come back with an exception within the process group's time limit instead of hanging."""
    port = _free_port()
    mgr = mp.Manager()
    results = mgr.dict()
    mp.spawn(_leaving_worker, args=(2, port, results, what), nprocs=2, join=True)
    assert results[1] == "left"
    assert results[0].startswith("raised after"), results[0]
    assert float(results[0].split()[2].rstrip("s:")) < 30.0
