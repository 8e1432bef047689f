"""The "cuda" backend's GEMM callables: `fp8_gemm`, `fp4_gemm`, `grouped_gemm` (+ `bf16_gemm`).

Drop-in for the callables the reference registers under the same kernel names
(triton/gemm/gemm_kernels.py:104-122 `fp8_gemm`, :164-182 `grouped_gemm`;
tilelang/gemm/gemm_kernels.py:96-133) and for the host wrapper `fp4_gemm` of
cuda/gemm/fp4_gemm.cu:140-146, which the reference never registered.  Positional
arguments and defaults follow the reference (A [M,K], B [K,N], fp32 result); everything
else is an optional JSON-scalar keyword so it travels through `scalar_params`.

All compute runs in libdslgemm.so (hand-written sm_100a kernels).  No CPU path exists.
"""
from __future__ import annotations

import ctypes
from typing import Optional, Tuple, Union

import torch

from . import _lib
from .quantize import PackedWeight, pack_weight, quantize_fp4, quantize_fp8, transpose_bytes
from .weight_store import cached_pack

_FLOAT_DTYPES = (torch.float32, torch.bfloat16, torch.float16)
_BYTE_DTYPES = (torch.uint8, torch.int8, torch.float8_e4m3fn, torch.float8_e8m0fnu, torch.float4_e2m1fn_x2)
_OUT_DTYPES = {"float32": torch.float32, "fp32": torch.float32, "bfloat16": torch.bfloat16, "bf16": torch.bfloat16}

Scalar = Union[None, float, torch.Tensor]


def _out_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        name = str(name).replace("torch.", "")
    try:
        return _OUT_DTYPES[str(name).lower()]
    except KeyError:
        raise ValueError(f"out_dtype must be float32 or bfloat16, got {name!r}") from None


def _activation_code(activation: Optional[str]) -> int:
    if activation is None or activation == "none":
        return _lib.ACT_NONE
    if activation == "swiglu":
        return _lib.ACT_SWIGLU
    if activation == "geglu":
        return _lib.ACT_GEGLU
    raise ValueError(f"activation must be None, 'swiglu' or 'geglu', got {activation!r}")


def _out_cols(n: int, activation: Optional[str]) -> int:
    """Columns of the result: n, or n/2 when (gate, up) column pairs are folded by the epilogue."""
    if _activation_code(activation) != _lib.ACT_NONE:
        if n % 2:
            raise ValueError("a gated activation needs an even number of GEMM columns")
        return n // 2
    return n


def _is_nvfp4_out(out_dtype) -> bool:
    return isinstance(out_dtype, str) and out_dtype.lower() == "nvfp4"


def _make_output(dev, M: int, nc: int, out_dtype, out_global_scale: Scalar, offs, groups: int, ep: "_lib.Epilogue", keep: list):
    """Allocates the result and completes the epilogue description.  Returns (tensor handed to the kernel,
    leading dimension in elements, value to return to the caller).  out_dtype "nvfp4": the result is quantised
    in the GEMM epilogue with `out_global_scale`; the caller gets (packed bytes [M, nc/2], scale tiles, global
    scale [1]) - exactly what quantize_fp4(result, "nvfp4", global_scale=...) would give - ready to be the A
    operand of the next FP4 GEMM."""
    if not _is_nvfp4_out(out_dtype):
        out = torch.empty((M, nc), dtype=_out_dtype(out_dtype), device=dev)
        ep.out_dtype = _lib.F32 if out.dtype == torch.float32 else _lib.BF16
        return out, nc, out
    if out_global_scale is None:
        raise ValueError("out_dtype 'nvfp4' needs out_global_scale (the fp32 global scale of the quantised result)")
    if nc % 16:
        raise ValueError(f"out_dtype 'nvfp4' needs a multiple of 16 output columns, got {nc}")
    out = torch.empty((M, nc // 2), dtype=torch.uint8, device=dev)
    nblk = nc // 16
    nbytes = _lib.lib().dsl_sf_bytes(M, nblk) if offs is None else _lib.lib().dsl_sf_bytes_grouped(M, nblk, groups)
    sf = torch.zeros(int(nbytes), dtype=torch.uint8, device=dev)
    if isinstance(out_global_scale, torch.Tensor):
        gs = out_global_scale.detach().to(device=dev, dtype=torch.float32).reshape(1)
    else:
        gs = torch.full((1,), float(out_global_scale), dtype=torch.float32, device=dev)
    keep.extend((sf, gs))
    ep.out_dtype = _lib.OUT_NVFP4
    ep.out_sf = sf.data_ptr()
    ep.out_gs_host = 1.0
    ep.out_gs_dev = gs.data_ptr()
    return out, nc, (out, sf, gs)


def _epilogue(dev, scale_a: Scalar, scale_b: Scalar, out: torch.dtype,
              row_scale: Optional[torch.Tensor], col_scale: Optional[torch.Tensor], keep: list,
              b_static: bool = False, activation: Optional[str] = None, problem: Optional[tuple] = None) -> _lib.Epilogue:
    """`problem` = (DSL_OP_* code, M, N, K, groups): the scratch the kernels can use for it is asked
    from the library (dsl_workspace_bytes) and attached; without it no scratch is passed."""
    ep = _lib.Epilogue()
    ep.b_is_static = 1 if b_static else 0
    ep.activation = _activation_code(activation)
    for name, s in (("a", scale_a), ("b", scale_b)):
        host, devp = 1.0, None
        if isinstance(s, torch.Tensor):
            t = s.detach().to(device=dev, dtype=torch.float32).reshape(-1)
            if t.numel() != 1:
                raise ValueError(f"scale_{name} must be a scalar")
            keep.append(t)
            devp = t.data_ptr()
        elif s is not None:
            host = float(s)
        setattr(ep, f"scale_{name}_host", host)
        setattr(ep, f"scale_{name}_dev", devp)
    for name, t in (("row_scale", row_scale), ("col_scale", col_scale)):
        if t is not None:
            t = t.detach().to(device=dev, dtype=torch.float32).contiguous()
            keep.append(t)
            setattr(ep, name, t.data_ptr())
    ep.out_dtype = _lib.F32 if out in (None, torch.float32) else _lib.BF16
    if problem is not None:
        with torch.cuda.device(dev):
            ws = _lib.workspace(dev, int(_lib.lib().dsl_workspace_bytes(*problem)))
        if ws is not None:
            ep.workspace = ws.data_ptr()
            ep.workspace_bytes = ws.numel()
    return ep


def _bytes2d(t: torch.Tensor) -> torch.Tensor:
    t = t.contiguous()
    return t.view(torch.uint8) if t.dtype != torch.uint8 else t


def _offsets_arg(offsets: Optional[torch.Tensor], dev) -> Tuple[Optional[torch.Tensor], int]:
    if offsets is None:
        return None, 1
    if offsets.dtype != torch.int32 or offsets.dim() != 1 or offsets.numel() < 2:
        raise TypeError("expert_offsets must be a 1-D int32 tensor of length groups+1")
    offsets = offsets.to(dev).contiguous()
    groups = offsets.numel() - 1
    if groups > _lib.MAX_GROUPS:
        raise ValueError(f"at most {_lib.MAX_GROUPS} groups are supported, got {groups}")
    return offsets, groups


# --------------------------------------------------------------------------------------
# low-level launches on already-quantised operands
# --------------------------------------------------------------------------------------

def gemm_fp8_quantized(qa: torch.Tensor, qb_nk: torch.Tensor, scale_a: Scalar, scale_b: Scalar, *, n: int,
                       out_dtype=torch.float32, expert_offsets: Optional[torch.Tensor] = None,
                       row_scale=None, col_scale=None, b_static: bool = False, activation: Optional[str] = None,
                       out_global_scale: Scalar = None):
    """C = (qa @ qb^T) * scale_a * scale_b on E4M3 bytes; qa [M, K], qb_nk [G*N, K].
    `b_static`: the weight was complete before the previous kernel on this stream was launched
    (lets the decode kernel stream it while the activation quantiser still runs)."""
    dev = _lib.require_cuda(qa, qb_nk)
    qa, qb_nk = _bytes2d(qa), _bytes2d(qb_nk)
    M, K = qa.shape
    offs, groups = _offsets_arg(expert_offsets, dev)
    if qb_nk.shape != (groups * n, K):
        raise ValueError(f"weight must be [{groups}*{n}, {K}] K-major bytes, got {tuple(qb_nk.shape)}")
    nc = _out_cols(n, activation)
    keep: list = []
    ep = _epilogue(dev, scale_a, scale_b, None, row_scale, col_scale, keep, b_static, activation,
                   (_lib.OP_GEMM_FP8, M, n, K, groups))
    out, ldc, ret = _make_output(dev, M, nc, out_dtype, out_global_scale, offs, groups, ep, keep)
    with torch.cuda.device(dev):
        rc = _lib.lib().dsl_gemm_fp8(qa.data_ptr(), qb_nk.data_ptr(), out.data_ptr(), ldc, M, n, K, _lib.ptr(offs),
                                     groups, ctypes.byref(ep), _lib.status_word(dev).data_ptr(), _lib.stream_ptr())
    _lib.check(rc, "dsl_gemm_fp8")
    return ret


def gemm_fp8_groupwise_quantized(qa: torch.Tensor, qb_nk: torch.Tensor, sa: torch.Tensor, sb: torch.Tensor, *,
                                 n: int, sb_block: bool, out_dtype=torch.float32,
                                 expert_offsets: Optional[torch.Tensor] = None,
                                 row_scale=None, col_scale=None, activation: Optional[str] = None) -> torch.Tensor:
    """C = sum_g (qa_g @ qb_g^T) * sa[:, g] * sb[g]; sa [M, K/128]; sb [G, K/128, N] per-column
    (sb_block False, the layout of cuda/gemm/fp8_gemm.cu:75) or [G, ceil(N/128), K/128] blocks."""
    dev = _lib.require_cuda(qa, qb_nk, sa, sb)
    qa, qb_nk = _bytes2d(qa), _bytes2d(qb_nk)
    M, K = qa.shape
    if K % 128 != 0:
        raise ValueError(f"K must be a multiple of 128 for group-scaled FP8, got {K}")
    offs, groups = _offsets_arg(expert_offsets, dev)
    if qb_nk.shape != (groups * n, K):
        raise ValueError(f"weight must be [{groups}*{n}, {K}] K-major bytes, got {tuple(qb_nk.shape)}")
    sa = sa.to(torch.float32).contiguous()
    sb = sb.to(torch.float32).contiguous()
    if sa.numel() != M * (K // 128):
        raise ValueError(f"scale_a must have {M}x{K // 128} elements, got {tuple(sa.shape)}")
    want_sb = groups * ((n + 127) // 128) * (K // 128) if sb_block else groups * (K // 128) * n
    if sb.numel() != want_sb:
        raise ValueError(f"scale_b must have {want_sb} elements, got {tuple(sb.shape)}")
    if _is_nvfp4_out(out_dtype):
        raise ValueError("a quantised result is not available from the group-scaled FP8 GEMM")
    nc = _out_cols(n, activation)
    out = torch.empty((M, nc), dtype=_out_dtype(out_dtype), device=dev)
    keep: list = []
    ep = _epilogue(dev, None, None, out.dtype, row_scale, col_scale, keep, False, activation)
    with torch.cuda.device(dev):
        rc = _lib.lib().dsl_gemm_fp8_groupwise(qa.data_ptr(), qb_nk.data_ptr(), sa.data_ptr(), sb.data_ptr(),
                                               1 if sb_block else 0, out.data_ptr(), nc, M, n, K, _lib.ptr(offs),
                                               groups, ctypes.byref(ep), _lib.status_word(dev).data_ptr(),
                                               _lib.stream_ptr())
    _lib.check(rc, "dsl_gemm_fp8_groupwise")
    return out


def gemm_fp4_quantized(pa: torch.Tensor, pb_nk: torch.Tensor, sfa: torch.Tensor, sfb: torch.Tensor, *,
                       format: str, n: int, global_scale_a: Scalar = None, global_scale_b: Scalar = None,
                       out_dtype=torch.float32, expert_offsets: Optional[torch.Tensor] = None,
                       row_scale=None, col_scale=None, b_static: bool = False, activation: Optional[str] = None,
                       out_global_scale: Scalar = None, token_scale: Optional[torch.Tensor] = None):
    """Block-scaled FP4 GEMM on packed e2m1 operands pa [M, K/2], pb_nk [G*N, K/2] with tiled
    scale bytes; for NVFP4 the result is multiplied once by global_scale_a * global_scale_b.
    `b_static` as in gemm_fp8_quantized.  `token_scale` [M] fp32: the per-token global scales of activations quantised
    with global_scale="per_token" (then leave global_scale_a unset); they take the epilogue's per-token slot, so
    `row_scale` cannot be given as well."""
    dev = _lib.require_cuda(pa, pb_nk, sfa, sfb)
    pa, pb_nk = _bytes2d(pa), _bytes2d(pb_nk)
    M, kb2 = pa.shape
    K = kb2 * 2
    offs, groups = _offsets_arg(expert_offsets, dev)
    if pb_nk.shape != (groups * n, kb2):
        raise ValueError(f"weight must be [{groups}*{n}, {kb2}] packed bytes, got {tuple(pb_nk.shape)}")
    fmt = {"nvfp4": _lib.FP4_NV, "mxfp4": _lib.FP4_MX}.get(format)
    if fmt is None:
        raise ValueError(f"format must be 'nvfp4' or 'mxfp4', got {format!r}")
    nblk = K // 16 if format == "nvfp4" else K // 32
    katoms = (nblk + 3) // 4
    need_a = (((M + 127) // 128) if offs is None else 0) * katoms * 512
    if sfa.numel() < need_a or sfb.numel() < groups * ((n + 127) // 128) * katoms * 512:
        raise ValueError("scale buffers are smaller than the tiled layout needs")
    nc = _out_cols(n, activation)
    keep: list = []
    if token_scale is not None:
        if row_scale is not None or global_scale_a is not None:
            raise ValueError("token_scale replaces global_scale_a and occupies the row_scale slot")
        if token_scale.numel() != M:
            raise ValueError(f"token_scale must have {M} elements, got {token_scale.numel()}")
        row_scale = token_scale
    ep = _epilogue(dev, global_scale_a, global_scale_b, None, row_scale, col_scale, keep, b_static, activation,
                   (_lib.OP_GEMM_FP4_NV if fmt == _lib.FP4_NV else _lib.OP_GEMM_FP4_MX, M, n, K, groups))
    out, ldc, ret = _make_output(dev, M, nc, out_dtype, out_global_scale, offs, groups, ep, keep)
    with torch.cuda.device(dev):
        rc = _lib.lib().dsl_gemm_fp4(pa.data_ptr(), pb_nk.data_ptr(), _bytes2d(sfa).data_ptr(),
                                     _bytes2d(sfb).data_ptr(), fmt, out.data_ptr(), ldc, M, n, K, _lib.ptr(offs),
                                     groups, ctypes.byref(ep), _lib.status_word(dev).data_ptr(), _lib.stream_ptr())
    _lib.check(rc, "dsl_gemm_fp4")
    return ret


def gemm_bf16_raw(a: torch.Tensor, b_nk: torch.Tensor, *, n: int, out_dtype=torch.float32,
                  expert_offsets: Optional[torch.Tensor] = None, scale_a: Scalar = None,
                  scale_b: Scalar = None, activation: Optional[str] = None, out_global_scale: Scalar = None):
    dev = _lib.require_cuda(a, b_nk)
    a = a.to(torch.bfloat16).contiguous()
    b_nk = b_nk.to(torch.bfloat16).contiguous()
    M, K = a.shape
    offs, groups = _offsets_arg(expert_offsets, dev)
    if b_nk.shape != (groups * n, K):
        raise ValueError(f"weight must be [{groups}*{n}, {K}] K-major, got {tuple(b_nk.shape)}")
    nc = _out_cols(n, activation)
    keep: list = []
    ep = _epilogue(dev, scale_a, scale_b, None, None, None, keep, False, activation, (_lib.OP_GEMM_BF16, M, n, K, groups))
    out, ldc, ret = _make_output(dev, M, nc, out_dtype, out_global_scale, offs, groups, ep, keep)
    with torch.cuda.device(dev):
        rc = _lib.lib().dsl_gemm_bf16(a.data_ptr(), b_nk.data_ptr(), out.data_ptr(), ldc, M, n, K, _lib.ptr(offs),
                                      groups, ctypes.byref(ep), _lib.status_word(dev).data_ptr(), _lib.stream_ptr())
    _lib.check(rc, "dsl_gemm_bf16")
    return ret


# --------------------------------------------------------------------------------------
# quantise-and-multiply on one packed weight (shared by the public callables)
# --------------------------------------------------------------------------------------

_W_CODES = {"fp8": _lib.W_FP8, "fp8_block128": _lib.W_FP8_BLOCK128, "nvfp4": _lib.W_NVFP4, "mxfp4": _lib.W_MXFP4, "bf16": _lib.W_BF16}
_OP_OF_FORMAT = {"fp8": _lib.OP_GEMM_FP8, "fp8_block128": _lib.OP_GEMM_FP8_GROUPWISE, "nvfp4": _lib.OP_GEMM_FP4_NV,
                 "mxfp4": _lib.OP_GEMM_FP4_MX, "bf16": _lib.OP_GEMM_BF16}


def _weight_desc(w: PackedWeight) -> "_lib.Weight":
    """The weight's dsl_weight struct, built once and kept on the PackedWeight (rebuilt if its tensors were swapped)."""
    d = getattr(w, "_cdesc", None)
    if d is None or d.q != w.q.data_ptr():
        d = _lib.Weight()
        d.format, d.groups, d.n, d.k = _W_CODES[w.format], w.groups, w.n, w.k
        d.q = w.q.data_ptr()
        d.scale = None if w.scale is None else w.scale.data_ptr()
        d.global_scale = None if w.global_scale is None else w.global_scale.data_ptr()
        w._cdesc = d
        w._scratch_need = {}
    return d


def _linear_one_call(a: torch.Tensor, w: PackedWeight, out_dtype, offs: Optional[torch.Tensor], row_scale, col_scale,
                     activation: Optional[str], out_global_scale: Scalar, act_global_scale: Scalar = None):
    per_token = isinstance(act_global_scale, str)
    if per_token:
        if act_global_scale != "per_token" or w.format != "nvfp4":
            raise ValueError("act_global_scale must be a number, a tensor, or 'per_token' (NVFP4 weights)")
        if row_scale is not None:
            raise ValueError("per-token activation scales occupy the row_scale slot")
        if w.k > _lib.PER_TOKEN_MAX_COLS:
            raise ValueError(f"per-token scales need K <= {_lib.PER_TOKEN_MAX_COLS}")
        act_global_scale = None
    """Quantise + GEMM through the single C entry point `dsl_linear`: one call into the library, the quantised
    activations in a per-stream arena instead of fresh allocations."""
    dev = a.device
    lib = _lib.lib()
    M = a.shape[0]
    desc = _weight_desc(w)
    groups = w.groups
    nc = _out_cols(w.n, activation)
    keep: list = []
    ep = _lib.Epilogue()
    ep.scale_a_host = ep.scale_b_host = 1.0
    ep.activation = _activation_code(activation)
    ep.act_scale_per_token = 1 if per_token else 0
    if row_scale is not None:
        row_scale = row_scale.detach().to(device=dev, dtype=torch.float32).contiguous()
        ep.row_scale = row_scale.data_ptr()
    if col_scale is not None:
        col_scale = col_scale.detach().to(device=dev, dtype=torch.float32).contiguous()
        ep.col_scale = col_scale.data_ptr()
    if act_global_scale is not None:
        if w.format != "nvfp4":
            raise ValueError("act_global_scale applies to NVFP4 weights")
        ags = (act_global_scale.detach().to(device=dev, dtype=torch.float32).reshape(1) if isinstance(act_global_scale, torch.Tensor)
               else torch.full((1,), float(act_global_scale), dtype=torch.float32, device=dev))
        keep.append(ags)
        ep.scale_a_dev = ags.data_ptr()
    switch = torch.cuda.current_device() != dev.index
    if switch:
        prev = torch.cuda.current_device()
        torch.cuda.set_device(dev)
    try:
        if groups == 1:                    # row groups never use scratch; the library says what a dense problem can use
            ws = _lib.workspace(dev, int(lib.dsl_workspace_bytes(_OP_OF_FORMAT[w.format], M, w.n, w.k, 1)))
            if ws is not None:
                ep.workspace = ws.data_ptr()
                ep.workspace_bytes = ws.numel()
        out, ldc, ret = _make_output(dev, M, nc, out_dtype, out_global_scale, offs, groups, ep, keep)
        need = w._scratch_need.get(M)
        if need is None:
            need = int(lib.dsl_linear_scratch_bytes(desc.format, M, w.k, groups))
            if len(w._scratch_need) < 64:
                w._scratch_need[M] = need
        stream = torch.cuda.current_stream(dev).cuda_stream
        arena = _lib.act_arena(dev, stream)
        with arena.lock:
            buf = arena.get(dev, need) if need else None
            rc = lib.dsl_linear(a.data_ptr(), _lib.dtype_code(a.dtype), M, ctypes.byref(desc), _lib.ptr(offs),
                                _lib.ptr(buf), 0 if buf is None else buf.numel(), out.data_ptr(), ldc, ctypes.byref(ep),
                                _lib.status_word(dev).data_ptr(), stream)
    finally:
        if switch:
            torch.cuda.set_device(prev)
    _lib.check(rc, "dsl_linear")
    return ret


def linear(a: torch.Tensor, w: PackedWeight, *, out_dtype=torch.float32,
           expert_offsets: Optional[torch.Tensor] = None, row_scale=None, col_scale=None,
           activation: Optional[str] = None, out_global_scale: Scalar = None, act_global_scale: Scalar = None):
    """a [M, K] high-precision activations x packed weight -> [M, N]: quantise the activations
    in the weight's format (one pass on the GPU) and run the matching GEMM.  The packed weight is
    treated as complete (the activation quantiser always sits between its producer and the GEMM).
    activation "swiglu" / "geglu": the weight is a fused gate/up projection packed with `gate_up_interleave=True`;
    the result is [M, N/2] = silu(gate) * up (gelu(gate) * up, tanh form), computed in the GEMM epilogue
    (cuda/activations/fused_gated_activations.cu:75-90 without the [M, N] round trip through memory).
    out_dtype "nvfp4" (with `out_global_scale`): the result is quantised in the same epilogue and returned as
    (packed bytes, scale tiles, global scale), the A operand of a following `gemm_fp4_quantized`.
    `act_global_scale` (NVFP4 weights): the fp32 global scale of the activations, a float or a device scalar - a
    calibrated value instead of amax(a) / 2688 - or "per_token": one dynamic global scale per row (amax_row / 2688).
    Either way the quantiser reads `a` once instead of twice (no tensor-wide amax pass)."""
    if _activation_code(activation) != _lib.ACT_NONE and not w.gate_up_interleaved:
        raise ValueError("a gated activation needs a weight packed with gate_up_interleave=True")
    if a.dim() != 2 or a.shape[1] != w.k:
        raise ValueError(f"activations must be [M, {w.k}], got {tuple(a.shape)}")
    if w.groups > 1 and expert_offsets is None:
        raise ValueError("a multi-group weight needs expert_offsets")
    if _is_nvfp4_out(out_dtype) and w.format == "fp8_block128":
        raise ValueError("a quantised result is not available from the group-scaled FP8 GEMM")
    if (a.is_cuda and a.is_contiguous() and w.q.device == a.device and (w.groups > 1) == (expert_offsets is not None)
            and (a.dtype == torch.bfloat16 if w.format == "bf16" else a.dtype in _FLOAT_DTYPES)):
        offs = None
        if expert_offsets is not None:
            offs, groups = _offsets_arg(expert_offsets, a.device)
            if groups != w.groups:
                raise ValueError(f"expert_offsets describes {groups} groups, the weight holds {w.groups}")
        return _linear_one_call(a, w, out_dtype, offs, row_scale, col_scale, activation, out_global_scale, act_global_scale)
    if act_global_scale is not None and w.format != "nvfp4":
        raise ValueError("act_global_scale applies to NVFP4 weights")
    common = dict(n=w.n, out_dtype=out_dtype, expert_offsets=expert_offsets, activation=activation)
    if _is_nvfp4_out(out_dtype):
        common["out_global_scale"] = out_global_scale
    if w.format == "bf16":
        return gemm_bf16_raw(a, w.q, **common)
    if w.format == "fp8":
        qa, sa = quantize_fp8(a, "per_tensor")
        return gemm_fp8_quantized(qa, w.q, sa, w.scale, row_scale=row_scale, col_scale=col_scale, b_static=True, **common)
    if w.format == "fp8_block128":
        qa, sa = quantize_fp8(a, "groupwise")
        return gemm_fp8_groupwise_quantized(qa, w.q, sa, w.scale, sb_block=True, row_scale=row_scale,
                                            col_scale=col_scale, **common)
    if w.format in ("nvfp4", "mxfp4"):
        pa, sfa, gsa = quantize_fp4(a, w.format, global_scale=act_global_scale if w.format == "nvfp4" else None,
                                    group_offsets=expert_offsets)
        if isinstance(act_global_scale, str):
            return gemm_fp4_quantized(pa, w.q, sfa, w.scale, format=w.format, token_scale=gsa, global_scale_b=w.global_scale,
                                      col_scale=col_scale, b_static=True, **common)
        return gemm_fp4_quantized(pa, w.q, sfa, w.scale, format=w.format, global_scale_a=gsa,
                                  global_scale_b=w.global_scale, row_scale=row_scale, col_scale=col_scale, b_static=True,
                                  **common)
    raise ValueError(f"unknown packed-weight format {w.format!r}")


# --------------------------------------------------------------------------------------
# public callables (the registry entries)
# --------------------------------------------------------------------------------------

def fp8_gemm(A: torch.Tensor, B, scale_a: Scalar = None, scale_b: Scalar = None, *, mode: str = "per_tensor",
             group_size: int = 128, b_layout: str = "kn", out_dtype="float32",
             row_scale: Optional[torch.Tensor] = None, col_scale: Optional[torch.Tensor] = None,
             cache_weights: bool = False) -> torch.Tensor:
    """FP8 E4M3 GEMM, C[M,N] = A[M,K] @ B[K,N] (triton/gemm/gemm_kernels.py:104-122).

    * A and B already E4M3 (float8_e4m3fn / uint8 / int8 bytes): `scale_a`, `scale_b` are the
      dequantisation scales - floats for mode "per_tensor" (result (A@B)*scale_a*scale_b, fp32,
      as the reference), or fp32 tensors for mode "groupwise" (scale_a [M, K/128], scale_b
      [K/128, N], layout of cuda/gemm/fp8_gemm.cu:74-75) or "block128" (scale_b [N/128, K/128]).
    * A and B high-precision (float32 / bfloat16 / float16): they are quantised on the GPU
      first - per tensor with scale amax/448 (cuda/gemm/fp8_gemm.cu:119-144; a given scale_a /
      scale_b is used instead of the amax-derived one), or, for "groupwise"/"block128", with
      1x128 activation groups and 128x128 weight blocks.
    b_layout "kn" is the reference's B[K,N]; "nk" is a K-major weight [N,K] (no transpose
    needed).  B may also be a PackedWeight.  `cache_weights=True` keeps the quantised form of a
    high-precision B in the process-wide identity cache (weight_store.cached_pack), so the next call
    with the same, unmodified tensor skips its quantisation.
    """
    if mode not in ("per_tensor", "groupwise", "block128"):
        raise ValueError(f"mode must be per_tensor, groupwise or block128, got {mode!r}")
    group_size = int(group_size)
    if mode != "per_tensor" and (group_size < 128 or group_size % 128):
        # the tensor cores accumulate one 128-byte stage of K before a partial product can be rescaled
        raise ValueError(f"group_size must be a multiple of 128 (one K stage of the kernel), got {group_size}")
    if b_layout not in ("kn", "nk"):
        raise ValueError("b_layout must be 'kn' or 'nk'")
    dev = _lib.require_cuda(A, B if isinstance(B, torch.Tensor) else None)
    if A.dim() != 2:
        raise ValueError(f"A must be [M, K], got {tuple(A.shape)}")
    M, K = A.shape
    if isinstance(B, PackedWeight):
        want = "fp8" if mode == "per_tensor" else "fp8_block128"
        if B.format != want or B.groups != 1 or B.k != K:
            raise ValueError(f"packed weight is {B.format} [{B.n},{B.k}], need {want} with K={K}")
        return linear(A, B, out_dtype=out_dtype, row_scale=row_scale, col_scale=col_scale)
    if B.dim() != 2:
        raise ValueError(f"B must be 2-D, got {tuple(B.shape)}")
    if (B.shape[0] if b_layout == "kn" else B.shape[1]) != K:
        raise ValueError(f"inner dimensions differ: A {tuple(A.shape)} vs B {tuple(B.shape)} ({b_layout})")
    N = B.shape[1] if b_layout == "kn" else B.shape[0]
    a_q, b_q = A.dtype in _BYTE_DTYPES, B.dtype in _BYTE_DTYPES
    if a_q != b_q:
        raise TypeError("A and B must both be E4M3 bytes or both be high-precision")
    if a_q:
        qb = _bytes2d(B)
        if b_layout == "kn":
            qb = transpose_bytes(qb)
        if mode == "per_tensor":
            if scale_a is None or scale_b is None:
                raise ValueError("scale_a and scale_b are required for already-quantised operands")
            return gemm_fp8_quantized(A, qb, scale_a, scale_b, n=N, out_dtype=out_dtype, row_scale=row_scale,
                                      col_scale=col_scale)
        if not isinstance(scale_a, torch.Tensor) or not isinstance(scale_b, torch.Tensor):
            raise TypeError("group-scaled FP8 needs scale_a and scale_b tensors")
        if group_size != 128:
            # scales per `group_size` K-elements (cuda/gemm/fp8_gemm.cu:110-116 takes any size): each one is repeated
            # for the 128-element groups it covers, i.e. the same products are summed in 128-element partial sums
            rep = group_size // 128
            ng = -(-K // group_size)
            kg = K // 128
            if K % 128 or scale_a.shape != (M, ng):
                raise ValueError(f"scale_a must be [{M}, {ng}] for group_size={group_size} and K a multiple of 128")
            scale_a = scale_a.repeat_interleave(rep, dim=1)[:, :kg].contiguous()
            scale_b = (scale_b.repeat_interleave(rep, dim=1)[:, :kg] if mode == "block128"
                       else scale_b.repeat_interleave(rep, dim=0)[:kg]).contiguous()
        return gemm_fp8_groupwise_quantized(A, qb, scale_a, scale_b, n=N, sb_block=(mode == "block128"),
                                            out_dtype=out_dtype, row_scale=row_scale, col_scale=col_scale)
    if A.dtype not in _FLOAT_DTYPES or B.dtype not in _FLOAT_DTYPES:
        raise TypeError(f"unsupported dtypes {A.dtype}, {B.dtype}")
    if mode != "per_tensor" and group_size != 128:
        raise ValueError("high-precision inputs are quantised with 1x128 groups and 128x128 blocks: pass group_size=128, "
                         "or already-quantised operands with their own scales for a multiple of 128")
    if cache_weights and scale_b is None:
        w = cached_pack(B, "fp8" if mode == "per_tensor" else "fp8_block128", b_layout)
        if mode == "per_tensor" and scale_a is not None:
            qa, sa = quantize_fp8(A, "per_tensor", scale=scale_a)
            return gemm_fp8_quantized(qa, w.q, sa, w.scale, n=N, out_dtype=out_dtype, row_scale=row_scale,
                                      col_scale=col_scale, b_static=True)
        return linear(A, w, out_dtype=out_dtype, row_scale=row_scale, col_scale=col_scale)
    Bnk = B.t().contiguous() if b_layout == "kn" else B.contiguous()
    if mode == "per_tensor":
        qa, sa = quantize_fp8(A, "per_tensor", scale=scale_a)
        qb, sb = quantize_fp8(Bnk, "per_tensor", scale=scale_b)
        return gemm_fp8_quantized(qa, qb, sa, sb, n=N, out_dtype=out_dtype, row_scale=row_scale, col_scale=col_scale)
    qa, sa = quantize_fp8(A, "groupwise")
    qb, sb = quantize_fp8(Bnk, "block128")
    return gemm_fp8_groupwise_quantized(qa, qb, sa, sb, n=N, sb_block=True, out_dtype=out_dtype,
                                        row_scale=row_scale, col_scale=col_scale)


def fp4_gemm(A: torch.Tensor, B, scale_a: Optional[torch.Tensor] = None, scale_b: Optional[torch.Tensor] = None,
             use_mxfp4: bool = False, *, format: Optional[str] = None, b_layout: str = "kn",
             global_scale_a: Scalar = None, global_scale_b: Scalar = None, out_dtype="float32",
             row_scale: Optional[torch.Tensor] = None, col_scale: Optional[torch.Tensor] = None,
             cache_weights: bool = False) -> torch.Tensor:
    """Block-scaled FP4 GEMM; argument order of the reference host wrapper
    `fp4_gemm(A, B, C, scale_a, scale_b, M, N, K, use_mxfp4)` (cuda/gemm/fp4_gemm.cu:140-146), with
    M, N, K read from the tensors and C returned.

    format "nvfp4" (default; e2m1 + unsigned-E4M3 scale per 16 + fp32 global scale), "mxfp4"
    (`use_mxfp4=True`; e2m1 + E8M0 scale per 32), or "ref32" - the reference's own container (fp32 scale
    per 32, B packed [K, N/2]), computed bit-identically to its kernel.
    * High-precision A [M,K] and B ([K,N] for b_layout "kn", [N,K] for "nk"): quantised on the GPU.
    * Packed operands (uint8/int8, two e2m1 per byte, low nibble first): A [M,K/2], B K-major
      [N,K/2] (b_layout must be "nk"), `scale_a` / `scale_b` the tiled scale bytes, and for
      NVFP4 `global_scale_a` / `global_scale_b`.
    `cache_weights` as in fp8_gemm.
    """
    fmt = format if format is not None else ("mxfp4" if use_mxfp4 else "nvfp4")
    if fmt == "ref32":
        return _fp4_gemm_ref32(A, B, scale_a, scale_b)
    if fmt not in ("nvfp4", "mxfp4"):
        raise ValueError(f"format must be 'nvfp4', 'mxfp4' or 'ref32', got {fmt!r}")
    if b_layout not in ("kn", "nk"):
        raise ValueError("b_layout must be 'kn' or 'nk'")
    _lib.require_cuda(A, B if isinstance(B, torch.Tensor) else None)
    if A.dim() != 2:
        raise ValueError(f"A must be 2-D, got {tuple(A.shape)}")
    if isinstance(B, PackedWeight):
        if B.format != fmt or B.groups != 1:
            raise ValueError(f"packed weight is {B.format}, need single-group {fmt}")
        return linear(A, B, out_dtype=out_dtype, row_scale=row_scale, col_scale=col_scale)
    if A.dtype in _BYTE_DTYPES:
        if b_layout != "nk":
            raise ValueError("packed FP4 weights must be K-major: pass b_layout='nk' with B [N, K/2]")
        if scale_a is None or scale_b is None:
            raise ValueError("packed operands need scale_a and scale_b (tiled scale bytes)")
        return gemm_fp4_quantized(A, B, scale_a, scale_b, format=fmt, n=B.shape[0], global_scale_a=global_scale_a,
                                  global_scale_b=global_scale_b, out_dtype=out_dtype, row_scale=row_scale,
                                  col_scale=col_scale)
    if A.dtype not in _FLOAT_DTYPES or B.dtype not in _FLOAT_DTYPES:
        raise TypeError(f"unsupported dtypes {A.dtype}, {B.dtype}")
    if (B.shape[0] if b_layout == "kn" else B.shape[1]) != A.shape[1]:
        raise ValueError(f"inner dimensions differ: A {tuple(A.shape)} vs B {tuple(B.shape)} ({b_layout})")
    w = cached_pack(B, fmt, b_layout) if cache_weights else pack_weight(B, fmt, layout=b_layout)
    return linear(A, w, out_dtype=out_dtype, row_scale=row_scale, col_scale=col_scale)


def _fp4_gemm_ref32(A: torch.Tensor, B: torch.Tensor, scale_a: torch.Tensor, scale_b: torch.Tensor) -> torch.Tensor:
    """The reference's own container and arithmetic (cuda/gemm/fp4_gemm.cu:95-146): A packed [M, K/2], B packed
    [K, N/2] (pairs along N), scale_a [M, K/32] fp32, scale_b [K/32, N] fp32 -> fp32 [M, N], bit-identical to
    the reference kernel.  `use_mxfp4` has no numeric effect there (its two tables are equal, fp4_gemm.cu:30-39)."""
    dev = _lib.require_cuda(A, B, scale_a, scale_b)
    if scale_a is None or scale_b is None:
        raise ValueError("format 'ref32' takes packed operands with scale_a [M, K/32] and scale_b [K/32, N]")
    if A.dtype not in _BYTE_DTYPES or B.dtype not in _BYTE_DTYPES or A.dim() != 2 or B.dim() != 2:
        raise TypeError("format 'ref32' takes packed uint8 operands A [M, K/2] and B [K, N/2]")
    M, K = A.shape[0], A.shape[1] * 2
    N = B.shape[1] * 2
    if B.shape[0] != K:
        raise ValueError(f"inner dimensions differ: A {tuple(A.shape)} vs B {tuple(B.shape)}")
    if K % 32 or N % 8:
        raise ValueError("format 'ref32' needs K % 32 == 0 and N % 8 == 0")
    sa = scale_a.to(torch.float32).contiguous()
    sb = scale_b.to(torch.float32).contiguous()
    if sa.numel() != M * (K // 32) or sb.numel() != (K // 32) * N:
        raise ValueError("scale_a must hold M*K/32 and scale_b K/32*N fp32 values")
    out = torch.empty((M, N), dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        rc = _lib.lib().dsl_gemm_fp4_ref32(_bytes2d(A).data_ptr(), _bytes2d(B).data_ptr(), out.data_ptr(), sa.data_ptr(),
                                           sb.data_ptr(), M, N, K, _lib.stream_ptr())
    _lib.check(rc, "dsl_gemm_fp4_ref32")
    return out


def grouped_gemm(A: torch.Tensor, B, num_groups: Optional[int] = None, expert_offsets: Optional[torch.Tensor] = None,
                 *, format: str = "bf16", b_layout: str = "kn", out_dtype=None, cache_weights: bool = False,
                 activation: Optional[str] = None) -> torch.Tensor:
    """Grouped GEMM for MoE / LoRA (triton/gemm/gemm_kernels.py:164-182, tilelang/gemm/gemm_kernels.py:116-133).

    Fixed-size groups: A [G,M,K], B [G,K,N] -> [G,M,N] (the reference's form; `num_groups`
    optional, checked against A when given).  Ragged groups (cuda/gemm/grouped_gemm.cu:79-104):
    A [sum M_g, K] with `expert_offsets` int32 [G+1] on the device -> [sum M_g, N]; groups may
    be empty and their sizes never leave the GPU.
    format "bf16" multiplies unquantised (result in A.dtype, as the Triton reference); "fp8",
    "fp8_groupwise", "nvfp4", "mxfp4" quantise A and B on the GPU first (result fp32 unless
    out_dtype says otherwise).  B may be a PackedWeight.  b_layout "kn": B [G,K,N]; "nk": [G,N,K].
    `cache_weights` as in fp8_gemm.  activation "swiglu": B is a fused gate/up projection (N = 2H, gate rows
    first, the input layout of the reference's swiglu); the result has H columns, silu(gate) * up, computed
    in the GEMM epilogue.  A PackedWeight passed as B must have been packed with `gate_up_interleave=True`.
    """
    glu = _activation_code(activation) != _lib.ACT_NONE
    formats = {"bf16": "bf16", "fp8": "fp8", "fp8_groupwise": "fp8_block128", "nvfp4": "nvfp4", "mxfp4": "mxfp4"}
    if format not in formats:
        raise ValueError(f"format must be one of {sorted(formats)}, got {format!r}")
    dev = _lib.require_cuda(A, B if isinstance(B, torch.Tensor) else None, expert_offsets)
    fixed = A.dim() == 3
    if not fixed and (A.dim() != 2 or expert_offsets is None):
        raise ValueError("A must be [G,M,K], or [sum M, K] together with expert_offsets")
    if isinstance(B, PackedWeight):
        w = B
        if w.format != formats[format]:
            raise ValueError(f"packed weight is {w.format}, need {formats[format]}")
    else:
        if B.dim() != 3:
            raise ValueError(f"B must be 3-D, got {tuple(B.shape)}")
        w = (cached_pack(B, formats[format], b_layout, gate_up_interleave=glu) if cache_weights
             else pack_weight(B, formats[format], layout=b_layout, gate_up_interleave=glu))
    G = w.groups
    if num_groups is not None and int(num_groups) != G:
        raise ValueError(f"num_groups={num_groups} but B holds {G} groups")
    if fixed:
        if A.shape[0] != G:
            raise ValueError(f"A holds {A.shape[0]} groups but B holds {G}")
        Mg = A.shape[1]
        a2 = A.reshape(G * Mg, A.shape[2])
        offs = torch.arange(G + 1, dtype=torch.int32, device=dev) * Mg
    else:
        a2 = A
        offs = expert_offsets
        if offs.numel() != G + 1:
            raise ValueError(f"expert_offsets must have {G + 1} entries, got {offs.numel()}")
    if out_dtype is None:
        out_dtype = A.dtype if (format == "bf16" and A.dtype in (torch.float32, torch.bfloat16)) else torch.float32
    if G == 1:
        offs = None
    out = linear(a2.contiguous(), w, out_dtype=out_dtype, expert_offsets=offs, activation=activation)
    return out.reshape(G, Mg, out.shape[1]) if fixed else out


def bf16_gemm(A: torch.Tensor, B: torch.Tensor, *, b_layout: str = "kn", out_dtype="float32") -> torch.Tensor:
    """BF16 GEMM with fp32 accumulation, C = A[M,K] @ B[K,N] -> fp32 (triton/gemm/gemm_kernels.py:49-65)."""
    w = pack_weight(B, "bf16", layout=b_layout)
    return linear(A, w, out_dtype=out_dtype)
