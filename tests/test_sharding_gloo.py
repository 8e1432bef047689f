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
