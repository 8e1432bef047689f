"""`KernelDispatcher` with the reference's call surface and wire format
(dispatcher/dispatcher.py:75-145 tensor (de)serialisation, :152-185 `DispatchResult`,
:192-344 `KernelDispatcher`).

Tensor wire format: {"shape": [...], "dtype": "...", "data": "<base64 little-endian bytes>"} or
{"shape", "dtype", "fill": "zeros" | "ones" | "random" | <number>}.  bfloat16 travels as fp32
bytes in both directions (a quirk of the reference kept on purpose, dispatcher.py:88-95,120-128).
Beyond the reference's dtype names, "uint8", "float8_e8m0fnu" ("e8m0") and "float4_e2m1fn_x2"
("fp4x2") are accepted so packed FP4 values and scale bytes can be sent (one byte per element on the
wire), and a spec {"packed_file": "<path>"} stands for a weight written by `save_packed`: it
deserialises to the PackedWeight (read once per process and device), so repeated calls neither ship
nor requantise the weight.
"""
from __future__ import annotations

import base64
import logging
import time
from typing import Any, Dict, List, Optional

import numpy as np
import torch

from .registry import KernelEntry, get_registry

logger = logging.getLogger(__name__)

_DTYPES: Dict[str, torch.dtype] = {
    "float32": torch.float32, "fp32": torch.float32,
    "float16": torch.float16, "fp16": torch.float16,
    "bfloat16": torch.bfloat16, "bf16": torch.bfloat16,
    "float8_e4m3fn": torch.float8_e4m3fn, "fp8": torch.float8_e4m3fn,
    "int8": torch.int8, "uint8": torch.uint8, "int32": torch.int32, "int64": torch.int64,
    "float8_e8m0fnu": torch.float8_e8m0fnu, "e8m0": torch.float8_e8m0fnu,
    "float4_e2m1fn_x2": torch.float4_e2m1fn_x2, "fp4x2": torch.float4_e2m1fn_x2,
}
_BYTE_VIEW = (torch.float8_e4m3fn, torch.float8_e8m0fnu, torch.float4_e2m1fn_x2)     # travel as their raw bytes
# numpy view used for the raw bytes of each dtype on the wire
_WIRE_NP = {torch.float32: np.float32, torch.float16: np.float16, torch.bfloat16: np.float32,
            torch.int8: np.int8, torch.uint8: np.uint8, torch.int32: np.int32, torch.int64: np.int64,
            torch.float8_e4m3fn: np.uint8, torch.float8_e8m0fnu: np.uint8, torch.float4_e2m1fn_x2: np.uint8}


def _resolve_dtype(name: str) -> torch.dtype:
    try:
        return _DTYPES[name.lower()]
    except KeyError:
        raise ValueError(f"Unknown dtype '{name}'. Supported: {list(_DTYPES)}") from None


def deserialize_tensor(spec: Dict[str, Any], device: str = "cuda"):
    if "packed_file" in spec:
        from ..weight_store import load_packed_cached
        return load_packed_cached(spec["packed_file"], device)
    shape = tuple(spec["shape"])
    dtype = _resolve_dtype(spec.get("dtype", "bfloat16"))
    if "data" in spec:
        raw = base64.b64decode(spec["data"])
        arr = np.frombuffer(raw, dtype=_WIRE_NP[dtype]).reshape(shape).copy()
        t = torch.from_numpy(arr)
        if dtype == torch.bfloat16:
            t = t.to(torch.bfloat16)
        elif dtype in _BYTE_VIEW:
            t = t.view(dtype)
        return t.to(device)
    fill = spec.get("fill", "random")
    if dtype in _BYTE_VIEW and dtype != torch.float8_e4m3fn:      # packed / exponent-only bytes: only byte fills make sense
        if fill == "zeros":
            return torch.zeros(shape, dtype=torch.uint8, device=device).view(dtype)
        if fill == "random":
            return torch.randint(0, 127, shape, dtype=torch.uint8, device=device).view(dtype)
        raise ValueError(f"fill {fill!r} is not defined for {dtype}; send data, or fill 'zeros' / 'random'")
    if fill == "zeros":
        return torch.zeros(shape, dtype=dtype, device=device)
    if fill == "ones":
        return torch.ones(shape, dtype=dtype, device=device)
    if fill == "random":
        if dtype.is_floating_point and dtype != torch.float8_e4m3fn:
            return torch.randn(shape, dtype=dtype, device=device)
        if dtype == torch.float8_e4m3fn:
            return torch.randn(shape, dtype=torch.float32, device=device).to(dtype)
        return torch.randint(0, 127, shape, dtype=dtype, device=device)
    return torch.full(shape, float(fill), dtype=dtype, device=device)


def serialize_tensor(t: torch.Tensor) -> Dict[str, Any]:
    host = t.detach().cpu()
    if host.dtype == torch.bfloat16:
        host = host.to(torch.float32)
    elif host.dtype in _BYTE_VIEW:
        host = host.view(torch.uint8)
    payload = base64.b64encode(host.contiguous().numpy().tobytes()).decode()
    return {"shape": list(t.shape), "dtype": str(t.dtype).replace("torch.", ""), "data": payload}


def summarize_tensor(t: torch.Tensor) -> Dict[str, Any]:
    f = t.detach().cpu().float()
    return {"shape": list(t.shape), "dtype": str(t.dtype).replace("torch.", ""), "numel": t.numel(),
            "min": round(f.min().item(), 6), "max": round(f.max().item(), 6),
            "mean": round(f.mean().item(), 6), "std": round(f.std().item(), 6)}


class DispatchResult:
    def __init__(self, output: Any, kernel_name: str, backend: str, elapsed_ms: float, device_info: str) -> None:
        self.output = output
        self.kernel_name = kernel_name
        self.backend = backend
        self.elapsed_ms = elapsed_ms
        self.device_info = device_info

    def to_dict(self) -> dict:
        out = self.output
        if isinstance(out, torch.Tensor):
            out = serialize_tensor(out)
        elif isinstance(out, (list, tuple)):
            out = [serialize_tensor(o) if isinstance(o, torch.Tensor) else o for o in out]
        return {"kernel_name": self.kernel_name, "backend": self.backend, "elapsed_ms": round(self.elapsed_ms, 4),
                "device_info": self.device_info, "output": out}


class KernelDispatcher:
    """Programmatic API: `run` with real tensors, `run_from_spec` with JSON-safe tensor specs.

    As in the reference, `elapsed_ms` is the host wall-clock of the call (the kernels are
    asynchronous; it is not a device time), an exception inside the kernel callable is
    re-raised as RuntimeError("Kernel '<name>' [<backend>] raised: ..."), and an unknown
    kernel or backend raises KeyError.  Without a CUDA device tensors are built on the CPU and
    the "cuda" backend's callables then raise: there is no CPU path.
    """

    def __init__(self, device: str = "cuda") -> None:
        self.device = device if torch.cuda.is_available() else "cpu"
        self._registry = get_registry(auto_load=True)
        if self.device == "cpu":
            logger.warning("CUDA not available - the cuda backend's kernels will refuse to run")

    def run(self, kernel_name: str, backend: str, args: Optional[List[Any]] = None,
            kwargs: Optional[Dict[str, Any]] = None) -> DispatchResult:
        entry = self._resolve(kernel_name, backend)
        info = self._device_info()
        t0 = time.perf_counter()
        try:
            output = entry.fn(*(args or []), **(kwargs or {}))
        except Exception as exc:
            raise RuntimeError(f"Kernel '{kernel_name}' [{backend}] raised: {exc}") from exc
        elapsed_ms = (time.perf_counter() - t0) * 1000.0
        return DispatchResult(output, entry.kernel_name, entry.backend, elapsed_ms, info)

    def run_from_spec(self, kernel_name: str, backend: str, tensor_specs: Optional[List[Dict[str, Any]]] = None,
                      scalar_params: Optional[Dict[str, Any]] = None) -> DispatchResult:
        tensors = [deserialize_tensor(s, device=self.device) for s in (tensor_specs or [])]
        return self.run(kernel_name, backend, args=tensors, kwargs=scalar_params or {})

    def list_kernels(self) -> List[dict]:
        return self._registry.list_kernels()

    def list_backends(self, kernel_name: str) -> List[str]:
        return self._registry.list_backends_for(kernel_name)

    def kernel_info(self, kernel_name: str, backend: str) -> dict:
        e = self._resolve(kernel_name, backend)
        return {"kernel_name": e.kernel_name, "backend": e.backend, "description": e.description,
                "input_schema": e.input_schema, "output_schema": e.output_schema}

    def _resolve(self, kernel_name: str, backend: str) -> KernelEntry:
        entry = self._registry.get(kernel_name, backend)
        if entry is not None:
            return entry
        available = self._registry.list_backends_for(kernel_name)
        if available:
            raise KeyError(f"Backend '{backend}' not available for kernel '{kernel_name}'. "
                           f"Available backends: {available}")
        raise KeyError(f"Unknown kernel '{kernel_name}'. Run list_kernels() to see all registered kernels.")

    def _device_info(self) -> str:
        if not torch.cuda.is_available():
            return "cpu"
        idx = torch.cuda.current_device()
        props = torch.cuda.get_device_properties(idx)
        return f"{props.name} ({props.total_memory // (1024 ** 2)} MB) [device:{idx}]"
