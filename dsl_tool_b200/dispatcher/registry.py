"""(kernel name, backend) -> callable table with the reference registry's surface
(dispatcher/registry.py:26-122, 326-336): `KernelEntry`, `KernelRegistry.register / get /
list_kernels / list_backends_for / load_all`, and the `get_registry()` singleton.

`load_all` registers ONE backend, "cuda" (a name the reference's REST schema already accepts,
dispatcher/schemas.py:77-83, but never registered), for the quantised-GEMM kernel names.
"""
from __future__ import annotations

import logging
import threading
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Tuple

logger = logging.getLogger(__name__)

BACKEND = "cuda"


@dataclass
class KernelEntry:
    """What is known about one (kernel, backend) pair."""
    kernel_name: str
    backend: str
    fn: Callable
    description: str = ""
    input_schema: dict = field(default_factory=dict)
    output_schema: dict = field(default_factory=dict)


def _gemm_input_schema(kernel_name: str) -> dict:
    """Documentation dict returned by `kernel_info`; same keys as dispatcher/registry.py:274-283,
    plus the optional keyword arguments of the "cuda" backend."""
    schema = {"A": "Tensor[M, K] bf16", "B": "Tensor[K, N] bf16"}
    if "fp8" in kernel_name:
        schema["scale_a"] = "float"
        schema["scale_b"] = "float"
        schema["mode"] = "str: per_tensor | groupwise | block128 (default per_tensor)"
        schema["group_size"] = "int: K elements per scale, a multiple of 128 (default 128; other sizes only with already-quantised operands)"
    if "fp4" in kernel_name:
        schema["scale_a"] = "Tensor uint8 (tiled block scales; packed operands only)"
        schema["scale_b"] = "Tensor uint8 (tiled block scales; packed operands only)"
        schema["use_mxfp4"] = "bool (default false)"
        schema["format"] = "str: nvfp4 | mxfp4 | ref32 (the reference container: fp32 scale per 32)"
    if "grouped" in kernel_name:
        schema["num_groups"] = "int"
        schema["expert_offsets"] = "Tensor[G+1] int32 (ragged groups; optional)"
        schema["format"] = "str: bf16 | fp8 | fp8_groupwise | nvfp4 | mxfp4 (default bf16)"
    if "bf16" not in kernel_name:
        schema["b_layout"] = "str: kn | nk (default kn)"
        schema["out_dtype"] = "str: float32 | bfloat16"
        schema["B (alternative)"] = '{"packed_file": path}: a weight written by save_packed, used in place of the tensor spec of B'
        schema["cache_weights"] = "bool (default false): keep B's quantised form, keyed by tensor identity"
    return schema


class KernelRegistry:
    """Name/backend keys are lower-cased on the way in, as in the reference (registry.py:63)."""

    def __init__(self) -> None:
        self._store: Dict[Tuple[str, str], KernelEntry] = {}
        self._mutex = threading.Lock()

    def register(self, kernel_name: str, backend: str, fn: Callable, description: str = "",
                 input_schema: Optional[dict] = None, output_schema: Optional[dict] = None) -> None:
        name, be = kernel_name.lower(), backend.lower()
        entry = KernelEntry(name, be, fn, description, dict(input_schema or {}), dict(output_schema or {}))
        with self._mutex:
            self._store[(name, be)] = entry
        logger.debug("Registered kernel %s [%s]", kernel_name, backend)

    def get(self, kernel_name: str, backend: str) -> Optional[KernelEntry]:
        return self._store.get((kernel_name.lower(), backend.lower()))

    def list_kernels(self) -> List[dict]:
        rows = [{"kernel_name": e.kernel_name, "backend": e.backend, "description": e.description}
                for e in list(self._store.values())]
        rows.sort(key=lambda r: (r["kernel_name"], r["backend"]))
        return rows

    def list_backends_for(self, kernel_name: str) -> List[str]:
        wanted = kernel_name.lower()
        return sorted({be for (name, be) in list(self._store) if name == wanted})

    def load_all(self, transformer_root: Optional[str] = None) -> None:
        """Register the "cuda" backend.  `transformer_root` is accepted for signature
        compatibility (registry.py:113) and unused: nothing is discovered from files."""
        del transformer_root
        try:
            from .. import gemm_kernels as k
        except Exception as exc:   # a broken install must be visible, not a silently empty registry
            logger.warning("cuda backend could not be imported: %s", exc)
            return
        table = [
            ("gemm.fp8_gemm", k.fp8_gemm, "FP8 E4M3 GEMM with per-tensor or 128-group scaling (tcgen05, sm_100a)"),
            ("gemm.fp4_gemm", k.fp4_gemm, "Block-scaled FP4 GEMM: NVFP4 / MXFP4 (tcgen05, sm_100a)"),
            ("gemm.grouped_gemm", k.grouped_gemm, "Grouped / batched GEMM for MoE / LoRA, fixed or ragged groups"),
            ("gemm.bf16_gemm", k.bf16_gemm, "BF16 GEMM (A[M,K] @ B[K,N]), fp32 accumulate"),
        ]
        for name, fn, desc in table:
            self.register(name, BACKEND, fn, desc, input_schema=_gemm_input_schema(name),
                          output_schema={"C": "Tensor[M, N]"})


_registry: Optional[KernelRegistry] = None
_registry_lock = threading.Lock()


def get_registry(auto_load: bool = True) -> KernelRegistry:
    """Process-wide registry, filled on first use when `auto_load` is true."""
    global _registry
    with _registry_lock:
        if _registry is None:
            _registry = KernelRegistry()
            if auto_load:
                _registry.load_all()
        return _registry
