"""Packed weights kept for reuse: an in-memory cache keyed by tensor identity and an on-disk format.

Weights are static, activations are not.  The reference requantises both on every call
(cuda/gemm/fp8_gemm.cu:119-144, cuda/gemm/fp4_gemm.cu:184-185); here a weight is quantised,
made K-major and laid out in scale tiles once (`pack_weight`) and then either

* looked up again by identity - `cached_pack(w, format)` returns the same `PackedWeight` as long
  as `w` is the same storage, shape, strides and in-place version, on the same device - or
* written to a file (`save_packed`) and read back (`load_packed`) by a later process, which is
  also how a `run_from_spec` caller names a weight without shipping or requantising it:
  the tensor spec `{"packed_file": "<path>"}` deserialises to the `PackedWeight`.

File layout (little endian), the widely used "8-byte header length + JSON header + raw tensor
bytes" container, so generic tools can list the tensors:
    u64 n | n bytes of JSON | data
    JSON: {"__metadata__": {"producer": "dsl_tool_b200", "format": ..., "groups": ..., "n": ...,
           "k": ...}, "<name>": {"dtype": "U8"|"F32"|"BF16", "shape": [...],
           "data_offsets": [begin, end]}, ...}           (offsets relative to the start of data)
    tensors: "q" (packed bytes / bf16 values), "scale" and "global_scale" when the format has them.
"""
from __future__ import annotations

import json
import os
import struct
import threading
from collections import OrderedDict
from typing import Dict, Optional, Tuple, Union

import numpy as np
import torch

from .quantize import PackedWeight, pack_weight

_DT_TO_NAME = {torch.uint8: "U8", torch.float32: "F32", torch.bfloat16: "BF16"}
_NAME_TO_DT = {v: k for k, v in _DT_TO_NAME.items()}
_FORMATS = ("fp8", "fp8_block128", "nvfp4", "mxfp4", "bf16")
_MAX_HEADER = 1 << 20


def _tensor_bytes(t: torch.Tensor) -> bytes:
    host = t.detach().contiguous().cpu()
    if host.dtype == torch.bfloat16:
        host = host.view(torch.int16)
    return host.numpy().tobytes()


def save_packed(path: Union[str, os.PathLike], w: PackedWeight) -> None:
    """Write a PackedWeight to `path` (atomically: a temporary file is renamed into place)."""
    if w.format not in _FORMATS:
        raise ValueError(f"unknown packed-weight format {w.format!r}")
    header: Dict[str, object] = {"__metadata__": {"producer": "dsl_tool_b200", "format": w.format, "groups": str(w.groups),
                                                  "n": str(w.n), "k": str(w.k),
                                                  "gate_up_interleaved": "1" if w.gate_up_interleaved else "0"}}
    blobs = []
    pos = 0
    for name, t in (("q", w.q), ("scale", w.scale), ("global_scale", w.global_scale)):
        if t is None:
            continue
        if t.dtype not in _DT_TO_NAME:
            raise TypeError(f"tensor {name!r} has dtype {t.dtype}, which the container does not hold")
        raw = _tensor_bytes(t)
        header[name] = {"dtype": _DT_TO_NAME[t.dtype], "shape": list(t.shape), "data_offsets": [pos, pos + len(raw)]}
        blobs.append(raw)
        pos += len(raw)
    hdr = json.dumps(header, separators=(",", ":")).encode()
    hdr += b" " * (-len(hdr) % 8)                     # data starts 8-byte aligned
    tmp = f"{os.fspath(path)}.tmp.{os.getpid()}"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(hdr)))
        f.write(hdr)
        for raw in blobs:
            f.write(raw)
    os.replace(tmp, path)


def load_packed(path: Union[str, os.PathLike], device: Union[str, torch.device] = "cuda") -> PackedWeight:
    """Read a file written by `save_packed`.  Raises ValueError on a malformed or foreign file."""
    size = os.path.getsize(path)
    with open(path, "rb") as f:
        head = f.read(8)
        if len(head) != 8:
            raise ValueError(f"{path}: too short for a packed-weight file")
        (n,) = struct.unpack("<Q", head)
        if n < 2 or n > _MAX_HEADER or 8 + n > size:
            raise ValueError(f"{path}: implausible header length {n}")
        try:
            header = json.loads(f.read(n).decode())
        except (UnicodeDecodeError, json.JSONDecodeError) as exc:
            raise ValueError(f"{path}: header is not JSON ({exc})") from None
        data = f.read()
    meta = header.get("__metadata__") if isinstance(header, dict) else None
    if not isinstance(meta, dict) or meta.get("producer") != "dsl_tool_b200" or meta.get("format") not in _FORMATS:
        raise ValueError(f"{path}: not a packed-weight file of this library")
    tensors: Dict[str, Optional[torch.Tensor]] = {"q": None, "scale": None, "global_scale": None}
    for name in tensors:
        ent = header.get(name)
        if ent is None:
            continue
        dt = _NAME_TO_DT.get(ent.get("dtype"))
        shape = tuple(int(x) for x in ent.get("shape", ()))
        b, e = (int(x) for x in ent.get("data_offsets", (0, -1)))
        if dt is None or b < 0 or e < b or e > len(data):
            raise ValueError(f"{path}: bad entry for tensor {name!r}")
        item = 2 if dt == torch.bfloat16 else torch.empty(0, dtype=dt).element_size()
        if int(np.prod(shape, dtype=np.int64)) * item != e - b:
            raise ValueError(f"{path}: tensor {name!r}: shape {shape} does not match {e - b} bytes")
        np_dt = {torch.uint8: np.uint8, torch.float32: np.float32, torch.bfloat16: np.int16}[dt]
        arr = np.frombuffer(data, dtype=np_dt, count=(e - b) // item, offset=b).reshape(shape).copy()
        t = torch.from_numpy(arr)
        if dt == torch.bfloat16:
            t = t.view(torch.bfloat16)
        tensors[name] = t.to(device)
    if tensors["q"] is None:
        raise ValueError(f"{path}: no tensor 'q'")
    return PackedWeight(meta["format"], tensors["q"], tensors["scale"], tensors["global_scale"], int(meta["groups"]),
                        int(meta["n"]), int(meta["k"]), meta.get("gate_up_interleaved", "0") == "1")


# ---- identity cache -----------------------------------------------------------------------

def _identity(w: torch.Tensor) -> Tuple:
    return (w.device.type, w.device.index, w.data_ptr(), w.storage_offset(), tuple(w.shape), tuple(w.stride()), w.dtype,
            w._version)


def packed_nbytes(p: PackedWeight) -> int:
    return sum(t.numel() * t.element_size() for t in (p.q, p.scale, p.global_scale) if t is not None)


class WeightCache:
    """LRU cache of PackedWeight objects, bounded by the bytes they hold on the device.

    The key is the tensor's identity (device, address, shape, strides, dtype, in-place version
    counter), the format and the layout: an in-place update or a different view misses; a new
    tensor that happens to reuse a freed address with the same geometry would hit, so the cache
    keeps a reference to the source tensor, which keeps its address from being reused.
    """

    def __init__(self, max_bytes: int = 8 << 30) -> None:
        self.max_bytes = int(max_bytes)
        self._lock = threading.Lock()
        self._items: "OrderedDict[Tuple, Tuple[torch.Tensor, PackedWeight, int]]" = OrderedDict()
        self._bytes = 0
        self.hits = 0
        self.misses = 0

    def get(self, w: torch.Tensor, format: str, layout: str = "nk", packer=pack_weight, **pack_kwargs) -> PackedWeight:
        key = _identity(w) + (format, layout) + tuple(sorted(pack_kwargs.items()))
        with self._lock:
            hit = self._items.get(key)
            if hit is not None:
                self._items.move_to_end(key)
                self.hits += 1
                return hit[1]
        packed = packer(w, format, layout, **pack_kwargs)
        size = packed_nbytes(packed)
        with self._lock:
            self.misses += 1
            if size <= self.max_bytes and key not in self._items:
                self._items[key] = (w, packed, size)
                self._bytes += size
                while self._bytes > self.max_bytes and self._items:
                    _, (_, _, old) = self._items.popitem(last=False)
                    self._bytes -= old
        return packed

    def clear(self) -> None:
        with self._lock:
            self._items.clear()
            self._bytes = 0

    def __len__(self) -> int:
        return len(self._items)

    @property
    def nbytes(self) -> int:
        return self._bytes


_default_cache = WeightCache()
_file_cache: Dict[Tuple[str, str], Tuple[float, int, PackedWeight]] = {}
_file_lock = threading.Lock()


def cached_pack(w: torch.Tensor, format: str, layout: str = "nk", **pack_kwargs) -> PackedWeight:
    """`pack_weight` through the process-wide identity cache."""
    return _default_cache.get(w, format, layout, **pack_kwargs)


def default_cache() -> WeightCache:
    return _default_cache


def load_packed_cached(path: Union[str, os.PathLike], device: Union[str, torch.device] = "cuda") -> PackedWeight:
    """`load_packed`, remembered per (path, device) until the file's mtime or size changes."""
    p = os.path.abspath(os.fspath(path))
    st = os.stat(p)
    key = (p, str(device))
    with _file_lock:
        hit = _file_cache.get(key)
        if hit is not None and hit[0] == st.st_mtime and hit[1] == st.st_size:
            return hit[2]
    packed = load_packed(p, device)
    with _file_lock:
        _file_cache[key] = (st.st_mtime, st.st_size, packed)
    return packed
