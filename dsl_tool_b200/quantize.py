"""Host wrappers of the quantise / scale-pack kernels.

Replace, on the GPU, `quantize_to_fp8_kernel` (cuda/gemm/fp8_gemm.cu:119-144) and
`quantize_fp32_to_nvfp4` (cuda/gemm/fp4_gemm.cu:50-90) of the reference, for FP8 per-tensor /
1x128 / 128x128 scaling and for the NVFP4 and MXFP4 block formats.  All work happens in
libdslgemm.so; torch only owns the memory.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple, Union

import torch

from . import _lib

FP8_MODES = {"per_tensor": _lib.FP8_PER_TENSOR, "groupwise": _lib.FP8_GROUP_1X128, "block128": _lib.FP8_BLOCK_128X128}
FP4_FORMATS = {"nvfp4": _lib.FP4_NV, "mxfp4": _lib.FP4_MX}


def _as_2d(x: torch.Tensor) -> torch.Tensor:
    if x.dim() == 1:
        x = x.unsqueeze(0)
    if x.dim() != 2:
        x = x.reshape(-1, x.shape[-1])
    return x.contiguous()


def quantize_fp8(x: torch.Tensor, mode: str = "per_tensor",
                 scale: Union[None, float, torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """x [rows, cols] (float32 / bfloat16 / float16, CUDA) -> (E4M3 bytes [rows, cols] uint8, scales fp32).

    mode "per_tensor": scales has 1 element, computed as max(amax/448, 1e-12) unless `scale`
    is given (then it is used as is); "groupwise": 1x128 groups along the last axis, scales
    [rows, ceil(cols/128)]; "block128": 128x128 blocks, scales [ceil(rows/128), ceil(cols/128)].
    """
    if mode not in FP8_MODES:
        raise ValueError(f"mode must be one of {sorted(FP8_MODES)}, got {mode!r}")
    dev = _lib.require_cuda(x)
    x = _as_2d(x)
    rows, cols = x.shape
    q = torch.empty((rows, cols), dtype=torch.uint8, device=dev)
    given = 0
    if mode == "per_tensor":
        if scale is None:
            s = torch.empty(1, dtype=torch.float32, device=dev)
        else:
            s = (scale.detach().to(device=dev, dtype=torch.float32).reshape(1).clone()
                 if isinstance(scale, torch.Tensor) else torch.full((1,), float(scale), dtype=torch.float32, device=dev))
            given = 1
    elif mode == "groupwise":
        s = torch.empty((rows, (cols + 127) // 128), dtype=torch.float32, device=dev)
    else:
        s = torch.empty(((rows + 127) // 128, (cols + 127) // 128), dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        rc = _lib.lib().dsl_quant_fp8(x.data_ptr(), _lib.dtype_code(x.dtype), rows, cols, FP8_MODES[mode],
                                      s.data_ptr(), given, q.data_ptr(), _lib.scratch_word(dev).data_ptr(),
                                      _lib.stream_ptr())
    _lib.check(rc, "dsl_quant_fp8")
    return q, s


def sf_bytes(rows: int, nblk: int, groups: Optional[int] = None) -> int:
    if groups is None:
        return int(_lib.lib().dsl_sf_bytes(rows, nblk))
    return int(_lib.lib().dsl_sf_bytes_grouped(rows, nblk, groups))


def quantize_fp4(x: torch.Tensor, format: str = "nvfp4",
                 global_scale: Union[None, float, torch.Tensor] = None,
                 group_offsets: Optional[torch.Tensor] = None
                 ) -> Tuple[torch.Tensor, torch.Tensor, Optional[torch.Tensor]]:
    """x [rows, K] -> (packed e2m1 [rows, K/2] uint8, tiled scale bytes uint8 1-D, global scale or None).

    "nvfp4": unsigned-E4M3 scale per 16 + fp32 global scale (amax/2688 unless given);
    "mxfp4": E8M0 scale per 32.  With `group_offsets` (int32 [G+1], CUDA) rows form ragged
    groups and each group's scales start a fresh 128-row tile.
    global_scale="per_token" (NVFP4): one global scale per row, amax_row / 2688, returned as an fp32 tensor [rows];
    the quantiser is then a single pass over x (a tensor-wide dynamic scale needs an amax pass first).  Feed it to
    the GEMM as `token_scale`.
    """
    if format not in FP4_FORMATS:
        raise ValueError(f"format must be one of {sorted(FP4_FORMATS)}, got {format!r}")
    dev = _lib.require_cuda(x, group_offsets)
    x = _as_2d(x)
    rows, cols = x.shape
    if cols % 32 != 0:
        raise ValueError(f"K must be a multiple of 32 for {format}, got {cols}")
    nblk = cols // 16 if format == "nvfp4" else cols // 32
    groups = 0
    if group_offsets is not None:
        if group_offsets.dtype != torch.int32 or group_offsets.dim() != 1:
            raise TypeError("group_offsets must be a 1-D int32 tensor")
        groups = group_offsets.numel() - 1
    q = torch.empty((rows, cols // 2), dtype=torch.uint8, device=dev)
    sf = torch.empty(sf_bytes(rows, nblk, groups if group_offsets is not None else None),
                     dtype=torch.uint8, device=dev)
    if isinstance(global_scale, str):
        if global_scale != "per_token" or format != "nvfp4":
            raise ValueError("global_scale must be None, a number, a tensor, or 'per_token' (NVFP4 only)")
        if cols > _lib.PER_TOKEN_MAX_COLS:
            raise ValueError(f"per-token scales need rows of at most {_lib.PER_TOKEN_MAX_COLS} elements, got {cols}")
        gs = torch.empty(rows, dtype=torch.float32, device=dev)
        with torch.cuda.device(dev):
            rc = _lib.lib().dsl_quant_fp4_per_token(x.data_ptr(), _lib.dtype_code(x.dtype), rows, cols, gs.data_ptr(),
                                                    q.data_ptr(), sf.data_ptr(), _lib.ptr(group_offsets), groups,
                                                    _lib.stream_ptr())
        _lib.check(rc, "dsl_quant_fp4_per_token")
        return q, sf, gs
    gs = None
    given = 0
    if format == "nvfp4":
        if global_scale is None:
            gs = torch.empty(1, dtype=torch.float32, device=dev)
        else:
            gs = (global_scale.detach().to(device=dev, dtype=torch.float32).reshape(1).clone()
                  if isinstance(global_scale, torch.Tensor)
                  else torch.full((1,), float(global_scale), dtype=torch.float32, device=dev))
            given = 1
    with torch.cuda.device(dev):
        rc = _lib.lib().dsl_quant_fp4(x.data_ptr(), _lib.dtype_code(x.dtype), rows, cols, FP4_FORMATS[format],
                                      _lib.ptr(gs), given, q.data_ptr(), sf.data_ptr(),
                                      _lib.ptr(group_offsets), groups, _lib.scratch_word(dev).data_ptr(),
                                      _lib.stream_ptr())
    _lib.check(rc, "dsl_quant_fp4")
    return q, sf, gs


def quantize_fp4_ref32(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """The reference's FP4 quantiser (`quantize_fp32_to_nvfp4`, cuda/gemm/fp4_gemm.cu:50-90) over the flat
    buffer: (packed nibbles uint8 [ceil(n/2)], fp32 scale per 32 elements [ceil(n/32)])."""
    dev = _lib.require_cuda(x)
    x = x.contiguous()
    n = x.numel()
    q = torch.empty((n + 1) // 2, dtype=torch.uint8, device=dev)
    s = torch.empty((n + 31) // 32, dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        rc = _lib.lib().dsl_quant_fp4_ref32(x.data_ptr(), _lib.dtype_code(x.dtype), n, q.data_ptr(), s.data_ptr(),
                                            _lib.stream_ptr())
    _lib.check(rc, "dsl_quant_fp4_ref32")
    return q, s


def transpose_bytes(x: torch.Tensor) -> torch.Tensor:
    """[R, C] one-byte elements -> [C, R] (same dtype)."""
    dev = _lib.require_cuda(x)
    if x.dim() != 2 or x.element_size() != 1:
        raise TypeError("transpose_bytes takes a 2-D tensor of one-byte elements")
    x = x.contiguous()
    out = torch.empty((x.shape[1], x.shape[0]), dtype=x.dtype, device=dev)
    with torch.cuda.device(dev):
        rc = _lib.lib().dsl_transpose_u8(x.data_ptr(), out.data_ptr(), x.shape[0], x.shape[1], _lib.stream_ptr())
    _lib.check(rc, "dsl_transpose_u8")
    return out


@dataclass
class PackedWeight:
    """A weight quantised once and kept K-major ([N, K] or [G, N, K]) for repeated GEMMs."""
    format: str                      # "fp8" | "fp8_block128" | "nvfp4" | "mxfp4" | "bf16"
    q: torch.Tensor                  # bytes [G*N, K or K/2] (bf16: [G*N, K] bfloat16)
    scale: Optional[torch.Tensor]    # fp8: [1]; fp8_block128: [G, N/128, K/128]; fp4: tiled scale bytes
    global_scale: Optional[torch.Tensor]
    groups: int
    n: int
    k: int
    gate_up_interleaved: bool = False   # rows reordered to (gate_0, up_0, gate_1, up_1, ...) for the fused SwiGLU epilogue


def _pack_weight_impl(w: torch.Tensor, format: str, layout: str = "nk",
                global_scale: Union[None, float, torch.Tensor] = None, gate_up_interleave: bool = False) -> PackedWeight:
    """Quantise a weight for the GEMM entry points.

    w is [N, K] / [G, N, K] (layout "nk") or the reference's [K, N] / [G, K, N] (layout "kn",
    cuda/gemm/fp8_gemm.cu:29-35); it is made K-major first.  `global_scale` (NVFP4: the fp32 global scale;
    per-tensor FP8: the scale) fixes that value instead of deriving it from this tensor's amax - pass the unsharded tensor's
    amax/2688 when packing a column or expert shard so that every shard quantises exactly as the
    whole weight would.  `gate_up_interleave`: the N = 2H output rows are a fused gate/up projection
    ([gate; up], the input layout of the reference's swiglu, cuda/activations/fused_gated_activations.cu:75-90);
    they are reordered to gate_0, up_0, gate_1, up_1, ... so that `linear(..., activation="swiglu")` can fold
    each pair in the GEMM epilogue.
    """
    dev = _lib.require_cuda(w)
    if layout not in ("nk", "kn"):
        raise ValueError("layout must be 'nk' or 'kn'")
    if w.dim() == 2:
        w = w.unsqueeze(0)
    if w.dim() != 3:
        raise ValueError("weight must be 2-D or 3-D")
    if layout == "kn":
        w = w.transpose(1, 2)
    if gate_up_interleave:
        if w.shape[1] % 2:
            raise ValueError("gate_up_interleave needs an even number of output rows")
        h = w.shape[1] // 2
        w = torch.stack((w[:, :h], w[:, h:]), dim=2).reshape(w.shape[0], 2 * h, w.shape[2])
    w = w.contiguous()
    G, N, K = w.shape
    flat = w.reshape(G * N, K)
    if format == "bf16":
        return PackedWeight("bf16", flat.to(torch.bfloat16).contiguous(), None, None, G, N, K)
    if format == "fp8":
        q, s = quantize_fp8(flat, "per_tensor", scale=global_scale)
        return PackedWeight("fp8", q, s, None, G, N, K)
    if format == "fp8_block128":
        if G == 1 or N % 128 == 0:
            q, s = quantize_fp8(flat, "block128")
            s = s.reshape(G, (N + 127) // 128, (K + 127) // 128)
        else:   # blocks must not straddle two experts
            parts = [quantize_fp8(w[g], "block128") for g in range(G)]
            q = torch.cat([p[0] for p in parts])
            s = torch.stack([p[1] for p in parts])
        return PackedWeight("fp8_block128", q, s.contiguous(), None, G, N, K)
    if format in ("nvfp4", "mxfp4"):
        if G == 1 or N % 128 == 0:
            q, sf, gs = quantize_fp4(flat, format, global_scale=global_scale if format == "nvfp4" else None)
        else:   # every expert's scales start a fresh 128-row tile
            offs = torch.arange(G + 1, dtype=torch.int32, device=dev) * N
            gs_val = None
            if format == "nvfp4" and global_scale is not None:
                gs_val = global_scale
            elif format == "nvfp4":
                gs_val = (flat.abs().amax().float() / 2688.0)
                gs_val = torch.where(gs_val == 0, torch.ones_like(gs_val), gs_val)
            # the grouped layout packs groups back to back in whole tiles, i.e. exactly
            # ceil(N/128) tiles per expert, which is what the GEMM indexes
            q, sf, gs = quantize_fp4(flat, format, global_scale=gs_val, group_offsets=offs)
        return PackedWeight(format, q, sf, gs, G, N, K)
    raise ValueError(f"unknown weight format {format!r}")


def pack_weight(w: torch.Tensor, format: str, layout: str = "nk",
                global_scale: Union[None, float, torch.Tensor] = None, gate_up_interleave: bool = False) -> PackedWeight:
    packed = _pack_weight_impl(w, format, layout, global_scale, gate_up_interleave)
    packed.gate_up_interleaved = bool(gate_up_interleave)
    return packed


pack_weight.__doc__ = _pack_weight_impl.__doc__
