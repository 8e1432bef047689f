"""Single-box partitioning of the quantised GEMMs: column-parallel weights for the dense
GEMMs and expert-parallel weights for grouped GEMM, one process per GPU.

The reference has no multi-device code at all (its dispatcher reports a single device,
dispatcher/dispatcher.py:338-344); this module is the layer above `linear` that the north-star
configs ask for.  The GEMM step itself needs no collective: output columns / experts are
independent, so every rank runs the ordinary kernels on its shard.  Only when the caller wants
the full output on every rank is an NCCL all-gather issued (over NVLink / NVSwitch), on the
stream the GEMM ran on.

Host logic (partition arithmetic, gather layout) is kept free of CUDA so it can be exercised
with the gloo backend on CPU; the compute callable is injected (`linear_fn`).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

COLUMN_ALIGN = 128   # scale-factor tiles and 128x128 weight blocks must stay whole inside a shard


def column_ranges(n: int, world: int, align: int = COLUMN_ALIGN) -> List[Tuple[int, int]]:
    """Contiguous column ranges [start, end) per rank, every boundary a multiple of `align`
    (except the end of the matrix); ranks differ by at most one aligned block."""
    if n <= 0 or world <= 0:
        raise ValueError("n and world must be positive")
    blocks = (n + align - 1) // align
    base, extra = divmod(blocks, world)
    out, start = [], 0
    for r in range(world):
        nb = base + (1 if r < extra else 0)
        end = min(n, start + nb * align)
        out.append((start, end))
        start = end
    return out


def expert_ranges(groups: int, world: int) -> List[Tuple[int, int]]:
    """Contiguous expert ranges [first, last) per rank, sizes differing by at most one."""
    if groups < 0 or world <= 0:
        raise ValueError("bad arguments")
    base, extra = divmod(groups, world)
    out, start = [], 0
    for r in range(world):
        n = base + (1 if r < extra else 0)
        out.append((start, start + n))
        start += n
    return out


def local_rows(expert_offsets: Sequence[int], first: int, last: int) -> Tuple[int, int, List[int]]:
    """Rows of the expert-sorted activation matrix that belong to experts [first, last):
    (row_start, row_end, local offsets rebased to 0)."""
    r0, r1 = int(expert_offsets[first]), int(expert_offsets[last])
    return r0, r1, [int(expert_offsets[g]) - r0 for g in range(first, last + 1)]


def _world(group) -> Tuple[int, int]:
    if dist.is_available() and dist.is_initialized():
        return dist.get_rank(group), dist.get_world_size(group)
    return 0, 1


@dataclass
class ColumnParallelLinear:
    """y[:, shard] = linear(x, W[shard, :]) on every rank; `gather=True` returns the full y.

    `weight_shard` is whatever `linear_fn` accepts as its second argument (a PackedWeight for
    the CUDA path); `n_total` is the unsharded output width.
    """
    weight_shard: object
    n_total: int
    linear_fn: Callable[..., torch.Tensor]
    group: Optional[object] = None

    def __post_init__(self):
        self.rank, self.world = _world(self.group)
        self.ranges = column_ranges(self.n_total, self.world)
        self.start, self.end = self.ranges[self.rank]

    def forward(self, x: torch.Tensor, gather: bool = False, **kw) -> torch.Tensor:
        y = self.linear_fn(x, self.weight_shard, **kw)
        if y.shape[1] != self.end - self.start:
            raise ValueError(f"shard produced {y.shape[1]} columns, expected {self.end - self.start}")
        if not gather or self.world == 1:
            return y
        return all_gather_columns(y, self.ranges, self.group)


def all_gather_columns(y: torch.Tensor, ranges: Sequence[Tuple[int, int]], group=None) -> torch.Tensor:
    """All-gather column shards [M, n_r] into [M, sum n_r] on every rank."""
    world = len(ranges)
    widths = [e - s for s, e in ranges]
    m = y.shape[0]
    y = y.contiguous()
    if len(set(widths)) == 1:
        buf = torch.empty((world * m, widths[0]), dtype=y.dtype, device=y.device)
        dist.all_gather_into_tensor(buf, y, group=group)
        return buf.view(world, m, widths[0]).permute(1, 0, 2).reshape(m, world * widths[0])
    # uneven shards: pad to the widest, gather once, drop the padding
    wmax = max(widths)
    padded = y if y.shape[1] == wmax else torch.nn.functional.pad(y, (0, wmax - y.shape[1]))
    buf = torch.empty((world * m, wmax), dtype=y.dtype, device=y.device)
    dist.all_gather_into_tensor(buf, padded.contiguous(), group=group)
    buf = buf.view(world, m, wmax)
    return torch.cat([buf[r, :, :w] for r, w in enumerate(widths)], dim=1)


@dataclass
class ExpertParallelGroupedLinear:
    """Grouped GEMM with the experts split across ranks: rank r owns experts
    `expert_ranges(G, world)[r]` and multiplies only the rows routed to them.

    `forward` takes the rows of this rank's experts (already expert-sorted) with their local
    offsets.  `forward_from_global` slices them out of a replicated expert-sorted matrix and,
    with `gather=True`, all-gathers the ragged row blocks back into the global order.
    """
    weight_local: object
    groups_total: int
    linear_fn: Callable[..., torch.Tensor]
    group: Optional[object] = None

    def __post_init__(self):
        self.rank, self.world = _world(self.group)
        self.ranges = expert_ranges(self.groups_total, self.world)
        self.first, self.last = self.ranges[self.rank]

    def forward(self, x_local: torch.Tensor, local_offsets: torch.Tensor, **kw) -> torch.Tensor:
        return self.linear_fn(x_local, self.weight_local, expert_offsets=local_offsets, **kw)

    def forward_from_global(self, x_sorted: torch.Tensor, expert_offsets: Sequence[int], gather: bool = False,
                            **kw) -> torch.Tensor:
        r0, r1, offs = local_rows(expert_offsets, self.first, self.last)
        local = torch.tensor(offs, dtype=torch.int32, device=x_sorted.device)
        y = self.forward(x_sorted[r0:r1], local, **kw)
        if not gather or self.world == 1:
            return y
        rows = [int(expert_offsets[l]) - int(expert_offsets[f]) for f, l in self.ranges]
        rmax = max(rows)
        padded = y if y.shape[0] == rmax else torch.nn.functional.pad(y, (0, 0, 0, rmax - y.shape[0]))
        buf = torch.empty((self.world * rmax, y.shape[1]), dtype=y.dtype, device=y.device)
        dist.all_gather_into_tensor(buf, padded.contiguous(), group=self.group)
        buf = buf.view(self.world, rmax, y.shape[1])
        return torch.cat([buf[r, :n] for r, n in enumerate(rows)], dim=0)


# ---- token all-to-all of an expert-parallel layer (host side; kernel-free so that gloo ranks on CPU can run it) ----

@dataclass
class RowExchange:
    """What one rank knows after the count exchange of `exchange_rows`."""
    send_rows: List[int]            # records this rank sends to each rank (its entries for that rank's experts)
    recv_rows: List[int]            # records it receives from each rank
    counts_in: torch.Tensor         # [world, local experts] int32 (CPU): rows from source s for local expert e
    received: torch.Tensor          # [sum(recv_rows), record width]: source-major, expert-sorted within a source


def exchange_rows(records: torch.Tensor, counts_per_expert: torch.Tensor, experts: int, group=None) -> RowExchange:
    """Sends every expert-sorted record to the rank that owns its expert.

    records [entries, width] are this rank's routed rows in expert-sorted order (all `experts` global experts);
    counts_per_expert [experts] int32 says how many belong to each.  Two collectives: the per-expert counts
    (all-to-all of a few integers, then ONE read-back to the host, which sizes the receive buffer) and the
    records themselves.  Both honour the process group's time limit: a rank that never joins makes them raise
    on the others instead of hanging them.
    """
    rank, world = _world(group)
    ranges = expert_ranges(experts, world)
    first, last = ranges[rank]
    local = last - first
    counts_per_expert = counts_per_expert.to(torch.int32).contiguous()
    if world == 1:
        counts_in = counts_per_expert.cpu().view(1, local)
        n = int(counts_in.sum())
        return RowExchange([n], [n], counts_in, records[:n])
    counts_in_dev = torch.empty(world * local, dtype=torch.int32, device=records.device)
    dist.all_to_all_single(counts_in_dev, counts_per_expert, [local] * world, [l - f for f, l in ranges], group=group)
    both = torch.cat([counts_per_expert, counts_in_dev]).cpu()          # the layer's one read-back
    counts_host, counts_in = both[:experts], both[experts:].view(world, local)
    send_rows = [int(counts_host[f:l].sum()) for f, l in ranges]
    recv_rows = [int(v) for v in counts_in.sum(dim=1)]
    received = torch.empty((sum(recv_rows),) + tuple(records.shape[1:]), dtype=records.dtype, device=records.device)
    dist.all_to_all_single(received, records[:sum(send_rows)].contiguous(), recv_rows, send_rows, group=group)
    return RowExchange(send_rows, recv_rows, counts_in, received)


def return_rows(results: torch.Tensor, ex: RowExchange, group=None) -> torch.Tensor:
    """The way back: `results` [received rows, width] in arrival order -> this rank's own entries, in the
    expert-sorted order it sent them in."""
    _, world = _world(group)
    if world == 1:
        return results
    back = torch.empty((sum(ex.send_rows),) + tuple(results.shape[1:]), dtype=results.dtype, device=results.device)
    dist.all_to_all_single(back, results.contiguous(), ex.send_rows, ex.recv_rows, group=group)
    return back


def arrival_expert_ids(ex: RowExchange, device) -> torch.Tensor:
    """Local expert index of every received record (int32 [received rows]): records arrive source by source,
    expert-sorted inside a source.  Built on `device` (the counts travel there once; the output size is already known
    on the host, so nothing is read back)."""
    world, local = ex.counts_in.shape
    experts = torch.arange(local, dtype=torch.int32, device=device).repeat(world)
    counts = ex.counts_in.reshape(-1).to(device=device, dtype=torch.int64, non_blocking=True)
    return torch.repeat_interleave(experts, counts, output_size=int(sum(ex.recv_rows)))


def shard_weight_columns(w_nk: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """Rows [start, end) of a K-major weight [N, K] for `rank` (a view)."""
    s, e = column_ranges(w_nk.shape[0], world)[rank]
    return w_nk[s:e]


def shard_weight_experts(w_gnk: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    f, l = expert_ranges(w_gnk.shape[0], world)[rank]
    return w_gnk[f:l]


# ---- sum of the ranks' partial results over peer memory (own kernel, plain loads over NVLink) ----

class PeerReducer:
    """The ranks' partial results [rows, cols] summed by reading the peers' buffers directly, every rank keeping its
    rows [rank * rows / world, (rank + 1) * rows / world): the reduce-scatter of an expert-parallel layer without a
    collective library moving the data.

    Each rank writes its partial result into `buffer()` (symmetric memory: the same allocation on every rank, mapped into
    every peer).  `reduce()` first runs a one-element NCCL all-reduce on the stream - a barrier that tells every rank that
    all buffers are complete, and that honours the process group's time limit if a rank is missing - and then launches
    `dsl_moe_reduce_pull`, which loads the rank's own rows from all `world` buffers and adds them in rank order in fp32.
    Two buffers alternate, so a rank can start writing the next step's partial result while its peers still read this
    step's; by the time it comes back to a buffer, every rank has passed another barrier and is done reading it.
    Nothing is written to a peer and no TMA or multicast instruction touches peer memory; the multicast binding of the
    symmetric allocation is switched off (TORCH_SYMM_MEM_DISABLE_MULTICAST), the loads are plain ones."""

    def __init__(self, rows: int, cols: int, dtype: torch.dtype, device, group=None):
        import ctypes
        import os
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm_mem
        if dtype not in (torch.float32, torch.bfloat16):
            raise TypeError("partial results travel as float32 or bfloat16")
        self.group = group if group is not None else dist.group.WORLD
        self.rank, self.world = dist.get_rank(self.group), dist.get_world_size(self.group)
        if rows % self.world:
            raise ValueError(f"the row count ({rows}) must be a multiple of the group size ({self.world})")
        if (cols * torch.empty((), dtype=dtype).element_size()) % 16:
            raise ValueError("a row must be a whole number of 16-byte vectors")
        self.rows, self.cols, self.dtype, self.device = rows, cols, dtype, torch.device(device)
        self._bufs, self._handles, self._ptrs = [], [], []
        for _ in range(2):
            t = symm_mem.empty((rows, cols), dtype=dtype, device=self.device)
            h = symm_mem.rendezvous(t, self.group)
            ptrs = [int(p) for p in h.buffer_ptrs]
            if len(ptrs) != self.world or any(p == 0 or p % 16 for p in ptrs) or ptrs[self.rank] != t.data_ptr():
                raise RuntimeError("symmetric memory did not map every rank's buffer")
            self._bufs.append(t)
            self._handles.append(h)
            self._ptrs.append((ctypes.c_void_p * self.world)(*ptrs))
        self._flag = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._step = 0

    def buffer(self) -> torch.Tensor:
        """Where this rank writes its partial result of the current step ([rows, cols], local memory)."""
        return self._bufs[self._step & 1]

    def reduce(self, out_dtype=None) -> torch.Tensor:
        """This rank's rows of the sum over the ranks' `buffer()`s, [rows / world, cols]; advances to the other buffer."""
        from . import _lib
        out_dtype = out_dtype or self.dtype
        dist.all_reduce(self._flag, group=self.group)          # every rank's buffer is complete from here on
        per = self.rows // self.world
        out = torch.empty((per, self.cols), dtype=out_dtype, device=self.device)
        with torch.cuda.device(self.device):
            rc = _lib.lib().dsl_moe_reduce_pull(self._ptrs[self._step & 1], self.world, self.rank * per, per, self.cols,
                                                _lib.dtype_code(self.dtype), out.data_ptr(), _lib.dtype_code(out_dtype),
                                                _lib.stream_ptr())
        _lib.check(rc, "dsl_moe_reduce_pull")
        self._step += 1
        return out


_PEER_REDUCERS = {}


def peer_reducer(rows: int, cols: int, dtype: torch.dtype, device, group=None) -> PeerReducer:
    """The PeerReducer of this shape on this group (created, i.e. allocated and exchanged among the ranks, on first use:
    every rank must ask for it at the same point)."""
    g = group if group is not None else dist.group.WORLD
    key = (id(g), rows, cols, dtype, torch.device(device))
    red = _PEER_REDUCERS.get(key)
    if red is None:
        red = _PEER_REDUCERS[key] = PeerReducer(rows, cols, dtype, device, g)
    return red
