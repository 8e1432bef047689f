"""Steps whose input and result live in pinned host memory, with the copies hidden behind the compute.

The reference dispatcher receives tensors from the host and hands results back to it on every call
(dispatcher/dispatcher.py:57-131: deserialise -> kernel -> serialise), one after the other.  On a
B200 the GEMM itself takes a few hundred microseconds while the PCIe copies of its operands take
milliseconds, so a caller that works from host buffers is bound by how well those copies overlap.

`HostPipeline` runs a device function over batches in pinned host memory on three streams:

    copy-in stream   host batch i+1  -> device staging buffer (two of them, used alternately)
    compute stream   fn(staging buffer of batch i)            (the library launches on torch's current stream)
    copy-out stream  result of batch i-1 -> host

Events order the three per buffer; nothing blocks the host until `join()` / `synchronize()`.  A batch
can also be cut into row chunks (`rows_per_chunk`), which lets the copy-out of the first rows start
while later rows are still being computed.  Chunking is only bit-identical to the unchunked call when
the step treats rows independently: FP8 with 1x128 activation scales, MXFP4, or NVFP4 / per-tensor
FP8 with a fixed (calibrated) global scale.  A dynamic whole-tensor amax is NOT row-local; leave
`rows_per_chunk` unset for those.
"""
from __future__ import annotations

from typing import Callable, List, Optional

import torch


class _Slot:
    def __init__(self) -> None:
        self.dev_in: Optional[torch.Tensor] = None
        self.in_done = torch.cuda.Event()
        self.compute_done = torch.cuda.Event()
        self.used = False


class HostPipeline:
    """`submit(host_in, host_out)` enqueues copy-in, `fn`, copy-out and returns at once.

    fn        callable(device_tensor) -> device tensor with the rows of `host_out` (same dtype)
    device    CUDA device the staging buffers live on
    depth     number of staging buffers (2 = copy-in of the next batch overlaps this batch's compute)
    """

    def __init__(self, fn: Callable[[torch.Tensor], torch.Tensor], device, depth: int = 2) -> None:
        if not torch.cuda.is_available():
            raise RuntimeError("HostPipeline needs a CUDA device; there is no CPU path")
        if depth < 1:
            raise ValueError("depth must be >= 1")
        self.fn = fn
        self.device = torch.device(device)
        with torch.cuda.device(self.device):
            self.copy_in = torch.cuda.Stream()
            self.compute = torch.cuda.Stream()
            self.copy_out = torch.cuda.Stream()
            self._slots: List[_Slot] = [_Slot() for _ in range(depth)]
        self._n = 0
        self._started = False

    def _start(self) -> None:
        # work already queued on the caller's stream (weights being packed, say) comes first
        if not self._started:
            cur = torch.cuda.current_stream(self.device)
            for s in (self.copy_in, self.compute, self.copy_out):
                s.wait_stream(cur)
            self._started = True

    def _one(self, host_in: torch.Tensor, host_out: torch.Tensor) -> None:
        slot = self._slots[self._n % len(self._slots)]
        self._n += 1
        rows = host_in.shape[0]
        if (slot.dev_in is None or slot.dev_in.shape[1:] != host_in.shape[1:] or slot.dev_in.dtype != host_in.dtype
                or slot.dev_in.shape[0] < rows):
            if slot.used:                                   # the old buffer may still be read by a running step
                slot.compute_done.synchronize()
            slot.dev_in = torch.empty(host_in.shape, dtype=host_in.dtype, device=self.device)
            self.copy_in.wait_stream(torch.cuda.current_stream(self.device))
        dev_in = slot.dev_in[:rows]                         # a short last chunk uses the head of the buffer
        with torch.cuda.stream(self.copy_in):
            if slot.used:
                self.copy_in.wait_event(slot.compute_done)  # the step that read this buffer has finished
            dev_in.copy_(host_in, non_blocking=True)
            slot.in_done.record()
        with torch.cuda.stream(self.compute):
            self.compute.wait_event(slot.in_done)
            out = self.fn(dev_in)
            slot.compute_done.record()
        if out.shape != host_out.shape or out.dtype != host_out.dtype:
            raise ValueError(f"step returned {tuple(out.shape)} {out.dtype}, host_out is {tuple(host_out.shape)} {host_out.dtype}")
        with torch.cuda.stream(self.copy_out):
            self.copy_out.wait_event(slot.compute_done)
            host_out.copy_(out, non_blocking=True)
            out.record_stream(self.copy_out)                # keeps the allocator from reusing it before the copy ran
        slot.used = True

    def submit(self, host_in: torch.Tensor, host_out: torch.Tensor, rows_per_chunk: Optional[int] = None) -> None:
        """Enqueue one batch.  Both tensors must be pinned host memory; rows are dimension 0 of each."""
        if host_in.device.type != "cpu" or host_out.device.type != "cpu":
            raise ValueError("HostPipeline.submit takes host tensors")
        if not (host_in.is_pinned() and host_out.is_pinned()):
            raise ValueError("host tensors must be pinned (tensor.pin_memory()): pageable copies do not overlap")
        if not (host_in.is_contiguous() and host_out.is_contiguous()):
            raise ValueError("host tensors must be contiguous")
        self._start()
        rows = host_in.shape[0]
        if rows_per_chunk is None or rows_per_chunk >= rows:
            self._one(host_in, host_out)
            return
        if rows_per_chunk < 1 or host_out.shape[0] != rows:
            raise ValueError("rows_per_chunk needs a step that maps row i of the input to row i of the result")
        for r0, r1 in chunk_bounds(rows, rows_per_chunk):
            self._one(host_in[r0:r1], host_out[r0:r1])

    def join(self) -> None:
        """Make torch's current stream wait for everything submitted so far (no host block)."""
        cur = torch.cuda.current_stream(self.device)
        for s in (self.copy_in, self.compute, self.copy_out):
            cur.wait_stream(s)

    def synchronize(self) -> None:
        """Block the host until every submitted batch is back in host memory."""
        for s in (self.copy_in, self.compute, self.copy_out):
            s.synchronize()


def chunk_bounds(rows: int, rows_per_chunk: int) -> List[tuple]:
    """[(r0, r1), ...] covering `rows` in order; the last chunk may be short."""
    if rows < 0 or rows_per_chunk < 1:
        raise ValueError("rows >= 0 and rows_per_chunk >= 1")
    return [(r0, min(rows, r0 + rows_per_chunk)) for r0 in range(0, rows, rows_per_chunk)]
