"""Kernel dispatch layer with the reference's public surface (dispatcher/__init__.py:1-11):
`KernelDispatcher` for programmatic dispatch and `get_registry` to inspect what is registered."""
from .dispatcher import DispatchResult, KernelDispatcher, deserialize_tensor, serialize_tensor, summarize_tensor
from .registry import KernelEntry, KernelRegistry, get_registry

__all__ = ["KernelDispatcher", "get_registry", "DispatchResult", "KernelEntry", "KernelRegistry",
           "deserialize_tensor", "serialize_tensor", "summarize_tensor"]
