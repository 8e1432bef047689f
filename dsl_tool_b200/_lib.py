"""ctypes binding of libdslgemm.so (the C ABI declared in include/dslgemm.h).

There is no fallback of any kind: if the library is missing or a CUDA device is absent,
the operators raise.
"""
from __future__ import annotations

import ctypes
import os
import threading
from typing import Dict, Optional

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("DSLGEMM_LIBRARY", os.path.join(_HERE, "libdslgemm.so"))

# enums of include/dslgemm.h
F32, BF16, F16 = 0, 1, 2
FP8_PER_TENSOR, FP8_GROUP_1X128, FP8_BLOCK_128X128 = 0, 1, 2
FP4_NV, FP4_MX = 0, 1
OP_GEMM_FP8, OP_GEMM_BF16, OP_GEMM_FP4_NV, OP_GEMM_FP4_MX, OP_GEMM_FP8_GROUPWISE = 0, 1, 2, 3, 4
ACT_NONE, ACT_SWIGLU, ACT_GEGLU = 0, 1, 2
OUT_NVFP4 = 3
MAX_GROUPS = 1024
STATIC_SCRATCH_BYTES = 4 << 20
WS_HEADER_BYTES = 64 << 10
PER_TOKEN_MAX_COLS = 32768

_ERR_NAMES = {
    -1: "a required pointer is NULL",
    -2: "bad shape (negative, too large, or not a multiple the format needs)",
    -3: "pointer or leading dimension not 16-byte aligned",
    -4: "unknown dtype / mode / format",
    -5: "the CUDA driver's tensor-map encoder is unavailable or refused the descriptor",
    -6: "beyond a fixed capacity of the library",
}
_STATUS_NAMES = {1: "TMA producer wait timed out", 2: "MMA issuer wait timed out",
                 4: "epilogue wait timed out", 8: "self-test wait timed out"}


class Epilogue(ctypes.Structure):
    _fields_ = [
        ("scale_a_host", ctypes.c_float),
        ("scale_b_host", ctypes.c_float),
        ("scale_a_dev", ctypes.c_void_p),
        ("scale_b_dev", ctypes.c_void_p),
        ("row_scale", ctypes.c_void_p),
        ("col_scale", ctypes.c_void_p),
        ("out_dtype", ctypes.c_int),
        ("workspace", ctypes.c_void_p),
        ("workspace_bytes", ctypes.c_size_t),
        ("b_is_static", ctypes.c_int),
        ("activation", ctypes.c_int),
        ("out_sf", ctypes.c_void_p),
        ("out_gs_host", ctypes.c_float),
        ("out_gs_dev", ctypes.c_void_p),
        ("act_scale_per_token", ctypes.c_int),
    ]


class Weight(ctypes.Structure):
    """dsl_weight of include/dslgemm.h."""
    _fields_ = [
        ("format", ctypes.c_int),
        ("groups", ctypes.c_int),
        ("n", ctypes.c_int),
        ("k", ctypes.c_int),
        ("q", ctypes.c_void_p),
        ("scale", ctypes.c_void_p),
        ("global_scale", ctypes.c_void_p),
    ]


W_FP8, W_FP8_BLOCK128, W_NVFP4, W_MXFP4, W_BF16 = 0, 1, 2, 3, 4

_lib: Optional[ctypes.CDLL] = None
_lock = threading.Lock()

_vp, _i, _ll, _f = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
_SIGNATURES = {
    "dsl_version": (ctypes.c_char_p, []),
    "dsl_sf_bytes": (ctypes.c_size_t, [_ll, _ll]),
    "dsl_sf_bytes_grouped": (ctypes.c_size_t, [_ll, _ll, _i]),
    "dsl_quant_fp8": (_i, [_vp, _i, _ll, _ll, _i, _vp, _i, _vp, _vp, _vp]),
    "dsl_quant_fp4": (_i, [_vp, _i, _ll, _ll, _i, _vp, _i, _vp, _vp, _vp, _i, _vp, _vp]),
    "dsl_quant_fp4_per_token": (_i, [_vp, _i, _ll, _ll, _vp, _vp, _vp, _vp, _i, _vp]),
    "dsl_transpose_u8": (_i, [_vp, _vp, _i, _i, _vp]),
    "dsl_gemm_fp8": (_i, [_vp, _vp, _vp, _ll, _ll, _i, _i, _vp, _i, ctypes.POINTER(Epilogue), _vp, _vp]),
    "dsl_gemm_fp8_groupwise": (_i, [_vp, _vp, _vp, _vp, _i, _vp, _ll, _ll, _i, _i, _vp, _i,
                                    ctypes.POINTER(Epilogue), _vp, _vp]),
    "dsl_gemm_fp4": (_i, [_vp, _vp, _vp, _vp, _i, _vp, _ll, _ll, _i, _i, _vp, _i,
                          ctypes.POINTER(Epilogue), _vp, _vp]),
    "dsl_gemm_fp4_static_scratch": (_i, [_vp, _vp, _vp, _vp, _i, _vp, _ll, _ll, _i, _i,
                                         ctypes.POINTER(Epilogue), _vp, _vp]),
    "dsl_workspace_bytes": (ctypes.c_size_t, [_i, _ll, _i, _i, _i]),
    "dsl_linear_scratch_bytes": (ctypes.c_size_t, [_i, _ll, _i, _i]),
    "dsl_linear": (_i, [_vp, _i, _ll, ctypes.POINTER(Weight), _vp, _vp, ctypes.c_size_t, _vp, _ll,
                        ctypes.POINTER(Epilogue), _vp, _vp]),
    "dsl_quant_fp4_ref32": (_i, [_vp, _i, _ll, _vp, _vp, _vp]),
    "dsl_gemm_fp4_ref32": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp]),
    "dsl_moe_route": (_i, [_vp, _i, _i, _i, _i, _i, _vp, _vp, _vp]),
    "dsl_moe_plan_scratch_bytes": (ctypes.c_size_t, [_i, _i]),
    "dsl_moe_plan": (_i, [_vp, _i, _i, _vp, _vp, _vp, _vp, _vp]),
    "dsl_moe_dispatch_fp4": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp, _vp, _vp]),
    "dsl_moe_dispatch_rows": (_i, [_vp, _vp, _vp, _vp, _i, _i, _ll, _i, _i, _vp, _vp]),
    "dsl_moe_combine": (_i, [_vp, _i, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp, _i, _vp]),
    "dsl_moe_wire_bytes": (ctypes.c_size_t, [_i, _i]),
    "dsl_moe_reduce_pull": (_i, [ctypes.POINTER(ctypes.c_void_p), _i, _ll, _ll, _i, _i, _vp, _i, _vp]),
    "dsl_moe_pack_wire_fp4": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _vp, _vp]),
    "dsl_moe_unpack_wire_fp4": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp, _vp, _vp]),
    "dsl_gemm_bf16": (_i, [_vp, _vp, _vp, _ll, _ll, _i, _i, _vp, _i, ctypes.POINTER(Epilogue), _vp, _vp]),
    "dsl_selftest_static_scratch_copy": (_i, [_vp, ctypes.c_size_t, ctypes.c_size_t, _i, _vp]),
    "dsl_selftest_bounded_wait": (_i, [_vp, ctypes.c_uint, _vp]),
    "dsl_selftest_groupwise_schedule": (_i, [_vp, _i, _ll, _i, _i, _i, _i, _vp, _i]),
}


def lib() -> ctypes.CDLL:
    """The loaded library; raises if it has not been built."""
    global _lib
    if _lib is None:
        with _lock:
            if _lib is None:
                if not os.path.exists(LIB_PATH):
                    raise RuntimeError(
                        f"{LIB_PATH} not found: build it with `python -m dsl_tool_b200.build` "
                        "(there is no fallback path)")
                cdll = ctypes.CDLL(LIB_PATH)
                for name, (res, args) in _SIGNATURES.items():
                    fn = getattr(cdll, name)
                    fn.restype = res
                    fn.argtypes = args
                _lib = cdll
    return _lib


def check(rc: int, what: str) -> None:
    if rc == 0:
        return
    if rc < 0:
        raise ValueError(f"{what}: {_ERR_NAMES.get(rc, 'invalid argument')} (code {rc})")
    raise RuntimeError(f"{what}: CUDA error {rc}")


def require_cuda(*tensors: torch.Tensor) -> torch.device:
    if not torch.cuda.is_available():
        raise RuntimeError("the 'cuda' backend needs a CUDA device (sm_100a); there is no CPU fallback")
    dev = None
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise RuntimeError("all tensors must live on a CUDA device; there is no CPU fallback")
        if dev is not None and t.device != dev:
            raise ValueError("tensors live on different devices")
        dev = t.device
    return dev


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def dtype_code(dt: torch.dtype) -> int:
    try:
        return {torch.float32: F32, torch.bfloat16: BF16, torch.float16: F16}[dt]
    except KeyError:
        raise TypeError(f"unsupported input dtype {dt}; use float32, bfloat16 or float16") from None


_status: Dict[int, torch.Tensor] = {}
_scratch: Dict[int, torch.Tensor] = {}


def status_word(device: torch.device) -> torch.Tensor:
    """Per-device status word the kernels OR their give-up bits into."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    t = _status.get(idx)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=device)
        _status[idx] = t
    return t


def scratch_word(device: torch.device) -> torch.Tensor:
    """Per-device 16-byte scratch (tensor amax cell)."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    t = _scratch.get(idx)
    if t is None:
        t = torch.zeros(4, dtype=torch.int32, device=device)
        _scratch[idx] = t
    return t


_workspace: Dict[tuple, torch.Tensor] = {}
WORKSPACE_BYTES = 16 << 20


def workspace(device: torch.device, need: int = WORKSPACE_BYTES) -> Optional[torch.Tensor]:
    """Scratch for partial sums along K, one buffer per (device, stream): launches on one stream use
    it in order, launches on different streams never share it.  `need` is what dsl_workspace_bytes()
    reports for the problem: 0 gives None (the kernels serving it use no scratch), anything else a
    buffer of at least that size (it only ever grows)."""
    if need <= 0:
        return None
    idx = device.index if device.index is not None else torch.cuda.current_device()
    key = (idx, torch.cuda.current_stream(device).cuda_stream)
    t = _workspace.get(key)
    if t is None or t.numel() < need:
        t = torch.empty(max(int(need), WORKSPACE_BYTES), dtype=torch.uint8, device=device)
        _workspace[key] = t
    return t


class ActArena:
    """Scratch for the quantised activations of `dsl_linear`, one per (device, stream).  The GEMM of a call
    consumes what the quantiser of the same call wrote, so calls issued in order on one stream share it; the
    lock keeps two host threads that launch on the same stream from interleaving their two launches."""

    def __init__(self) -> None:
        self.buf: Optional[torch.Tensor] = None
        self.lock = threading.Lock()
        self.retired: list = []      # outgrown buffers stay alive: a captured CUDA graph may still point at them

    def get(self, device: torch.device, need: int) -> torch.Tensor:
        buf = self.buf
        if buf is None or buf.numel() < need:
            if torch.cuda.is_current_stream_capturing():
                # memory allocated under capture belongs to that graph's pool: use it for this call only
                return torch.empty(need, dtype=torch.uint8, device=device)
            if buf is not None:
                self.retired.append(buf)
            buf = torch.empty(max(int(need * 1.25), 1 << 20), dtype=torch.uint8, device=device)
            self.buf = buf
        return buf


_arenas: Dict[tuple, ActArena] = {}


def act_arena(device: torch.device, stream: int) -> ActArena:
    key = (device.index, stream)
    a = _arenas.get(key)
    if a is None:
        with _lock:
            a = _arenas.setdefault(key, ActArena())
    return a


def check_status(device: Optional[torch.device] = None) -> None:
    """Synchronise and raise if any kernel since the last check gave up on a wait."""
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device())
    word = status_word(device)
    torch.cuda.synchronize(device)
    v = int(word.item())
    if v != 0:
        word.zero_()
        what = ", ".join(n for b, n in _STATUS_NAMES.items() if v & b)
        raise RuntimeError(f"a GEMM kernel gave up on a barrier wait ({what}; status {v})")
