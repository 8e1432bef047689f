"""Mixture-of-experts layer around the grouped GEMM: router top-k, expert-sorted dispatch, the two
expert projections and the weighted combine, single GPU or expert-parallel.

The reference has the grouped GEMM only (cuda/gemm/grouped_gemm.cu:79-104, registered
triton/gemm/gemm_kernels.py:164-182); a layer that uses it needs the steps on either side, which
live here.  Data flow of `moe_forward` (NVFP4 weights):

    logits --route--> ids, weights --plan--> offsets, tile0, dest          (all on the GPU, no host sync)
    x --quantise ONCE per token--> packed rows + scale tiles --dispatch--> expert-sorted packed rows
      --grouped GEMM (gate/up, fused SwiGLU, result quantised in the epilogue)--> --grouped GEMM (down)-->
      --combine (weights, slot order)--> out [tokens, d_model]

Expert parallelism, two ways (`moe_forward(..., dispatch=...)`):
  "replicated"  every rank sees all tokens and the full routing (the router is cheap), dispatches and computes only
                its contiguous range of experts (`sharding.expert_ranges`), and the per-rank partial results are
                summed with one all-reduce or reduce-scatter - no token exchange and no host-side knowledge of the
                row counts.  Buffers for the routed rows are sized for the worst case, tokens * k rows.  Everything
                outside the GEMMs is repeated on every rank, so it suits few tokens.
  "all_to_all"  every rank owns a share of the tokens: it routes and quantises only those, sends each routed row
                (packed e2m1 bytes + scale bytes, `dsl_moe_pack_wire_fp4`) to the rank that owns its expert with one
                NCCL all-to-all over NVLink, multiplies what arrived, and a second all-to-all carries the results
                back to the token's owner, which combines them.  One read-back of the per-expert row counts to the
                host sizes the receive buffers.  Results are bit-identical to the single-GPU layer.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch

from . import _lib
from .gemm_kernels import gemm_fp4_quantized, gemm_fp8_groupwise_quantized, gemm_fp8_quantized, linear
from .quantize import PackedWeight, pack_weight, quantize_fp4, quantize_fp8
from .sharding import arrival_expert_ids, exchange_rows, expert_ranges, return_rows


@dataclass
class MoEPlan:
    ids: torch.Tensor        # [tokens, k] int32: chosen experts
    weights: torch.Tensor    # [tokens, k] fp32
    offsets: torch.Tensor    # [experts + 1] int32: rows per expert, prefix sums
    tile0: torch.Tensor      # [experts + 1] int32: prefix sums of ceil(rows / 128)
    dest: torch.Tensor       # [tokens * k] int32: expert-sorted row of entry token * k + slot
    experts: int


def route(logits: torch.Tensor, k: int, renormalize: bool = True) -> Tuple[torch.Tensor, torch.Tensor]:
    """Softmax over the experts and top-k: (ids [T, k] int32, weights [T, k] fp32); ties go to the lower index."""
    dev = _lib.require_cuda(logits)
    if logits.dim() != 2 or logits.dtype not in (torch.float32, torch.bfloat16):
        raise TypeError("logits must be [tokens, experts] float32 or bfloat16")
    logits = logits.contiguous()
    T, E = logits.shape
    ids = torch.empty((T, k), dtype=torch.int32, device=dev)
    w = torch.empty((T, k), dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        rc = _lib.lib().dsl_moe_route(logits.data_ptr(), _lib.dtype_code(logits.dtype), T, E, k, 1 if renormalize else 0,
                                      ids.data_ptr(), w.data_ptr(), _lib.stream_ptr())
    _lib.check(rc, "dsl_moe_route")
    return ids, w


def plan(ids: torch.Tensor, weights: torch.Tensor, experts: int) -> MoEPlan:
    """Expert-sorted row plan of the routing (stable: within an expert, rows keep token / slot order)."""
    dev = _lib.require_cuda(ids, weights)
    if ids.dtype != torch.int32 or ids.dim() != 2:
        raise TypeError("ids must be [tokens, k] int32")
    ids = ids.contiguous()
    n = ids.numel()
    counts = torch.empty(int(_lib.lib().dsl_moe_plan_scratch_bytes(n, experts)) // 4, dtype=torch.int32, device=dev)
    offsets = torch.empty(experts + 1, dtype=torch.int32, device=dev)
    tile0 = torch.empty(experts + 1, dtype=torch.int32, device=dev)
    dest = torch.empty(n, dtype=torch.int32, device=dev)
    with torch.cuda.device(dev):
        rc = _lib.lib().dsl_moe_plan(ids.data_ptr(), n, experts, counts.data_ptr(), offsets.data_ptr(), tile0.data_ptr(),
                                     dest.data_ptr(), _lib.stream_ptr())
    _lib.check(rc, "dsl_moe_plan")
    return MoEPlan(ids, weights.contiguous(), offsets, tile0, dest, experts)


def _pad_cols(t: torch.Tensor, multiple: int) -> torch.Tensor:
    """Pads the last dimension with zeros to a multiple (rows of fp32 scales must be multiples of 16 bytes to be dispatched)."""
    extra = -t.shape[1] % multiple
    return t if extra == 0 else torch.nn.functional.pad(t, (0, extra))


def _local_offsets(p: MoEPlan, first: int, last: int) -> torch.Tensor:
    return (p.offsets[first:last + 1] - p.offsets[first]).contiguous()


def dispatch_fp4(p: MoEPlan, packed: torch.Tensor, sf: torch.Tensor, K: int, format: str, first: int, last: int):
    """Packed rows / scale tiles of tokens quantised once -> (expert-sorted packed rows [T*k, K/2], scale tiles in
    the ragged-group layout) for the experts [first, last).  Rows beyond the local total stay unwritten."""
    dev = _lib.require_cuda(packed, sf)
    T, k = p.ids.shape
    rows = T * k
    nblk = K // 16 if format == "nvfp4" else K // 32
    q_out = torch.empty((rows, K // 2), dtype=torch.uint8, device=dev)
    sf_out = torch.zeros(int(_lib.lib().dsl_sf_bytes_grouped(rows, nblk, last - first)), dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        rc = _lib.lib().dsl_moe_dispatch_fp4(packed.data_ptr(), sf.data_ptr(), p.ids.data_ptr(), p.dest.data_ptr(),
                                             p.offsets.data_ptr(), p.tile0.data_ptr(), T, k, K,
                                             _lib.FP4_NV if format == "nvfp4" else _lib.FP4_MX, first, last,
                                             q_out.data_ptr(), sf_out.data_ptr(), _lib.stream_ptr())
    _lib.check(rc, "dsl_moe_dispatch_fp4")
    return q_out, sf_out


def dispatch_rows(p: MoEPlan, x: torch.Tensor, first: int, last: int) -> torch.Tensor:
    """x [tokens, K] (any dtype whose row is a multiple of 16 bytes) -> expert-sorted rows [T*k, K]."""
    dev = _lib.require_cuda(x)
    x = x.contiguous()
    T, k = p.ids.shape
    out = torch.empty((T * k, x.shape[1]), dtype=x.dtype, device=dev)
    with torch.cuda.device(dev):
        rc = _lib.lib().dsl_moe_dispatch_rows(x.data_ptr(), p.ids.data_ptr(), p.dest.data_ptr(), p.offsets.data_ptr(), T, k,
                                              x.shape[1] * x.element_size(), first, last, out.data_ptr(), _lib.stream_ptr())
    _lib.check(rc, "dsl_moe_dispatch_rows")
    return out


def combine(p: MoEPlan, y: torch.Tensor, first: int, last: int, out_dtype=torch.float32, out=None) -> torch.Tensor:
    """y [rows, D] (expert-sorted results of the local experts) -> [tokens, D]: weighted sum over each token's
    local slots, in slot order.  `out` (contiguous [tokens, D], float32 or bfloat16) receives the result when given."""
    dev = _lib.require_cuda(y)
    if y.dtype not in (torch.float32, torch.bfloat16):
        raise TypeError("y must be float32 or bfloat16")
    y = y.contiguous()
    T, k = p.ids.shape
    if out is None:
        out = torch.empty((T, y.shape[1]), dtype=out_dtype, device=dev)
    elif out.shape != (T, y.shape[1]) or not out.is_contiguous() or out.device != y.device or \
            out.dtype not in (torch.float32, torch.bfloat16):
        raise ValueError("out must be a contiguous [tokens, D] float32 / bfloat16 tensor on the device of y")
    out_dtype = out.dtype
    with torch.cuda.device(dev):
        rc = _lib.lib().dsl_moe_combine(y.data_ptr(), _lib.dtype_code(y.dtype), p.ids.data_ptr(), p.dest.data_ptr(),
                                        p.offsets.data_ptr(), p.weights.data_ptr(), T, k, y.shape[1], first, last,
                                        out.data_ptr(), _lib.dtype_code(out_dtype), _lib.stream_ptr())
    _lib.check(rc, "dsl_moe_combine")
    return out


@dataclass
class MoEWeights:
    """One rank's experts: gate/up projection [E_local, 2H, K] packed with the rows interleaved for the fused
    SwiGLU, down projection [E_local, D, H]; `first` .. `last` is the rank's range of global expert indices."""
    gate_up: PackedWeight
    down: PackedWeight
    first: int
    last: int
    experts: int              # global number of experts
    hidden_global_scale: Optional[float] = None   # NVFP4: calibrated global scale of the hidden activation

    @staticmethod
    def pack(w_gate_up: torch.Tensor, w_down: torch.Tensor, format: str = "nvfp4", rank: int = 0, world: int = 1,
             hidden_global_scale: Optional[float] = None) -> "MoEWeights":
        """w_gate_up [E, 2H, K] ([gate; up] rows), w_down [E, D, H]: keeps and packs this rank's expert range.
        NVFP4 global scales and per-tensor FP8 scales are those of the whole tensors, so every sharding quantises
        identically."""
        E = w_gate_up.shape[0]
        first, last = expert_ranges(E, world)[rank]
        gs1 = gs2 = None
        if format in ("nvfp4", "fp8"):      # per-tensor quantities come from the WHOLE tensors
            div = 2688.0 if format == "nvfp4" else 448.0
            gs1 = w_gate_up.abs().amax().float() / div
            gs2 = w_down.abs().amax().float() / div
        gu = pack_weight(w_gate_up[first:last], format, global_scale=gs1, gate_up_interleave=True)
        dn = pack_weight(w_down[first:last], format, global_scale=gs2)
        return MoEWeights(gu, dn, first, last, E, hidden_global_scale)


def _experts_fp4(p: MoEPlan, packed: torch.Tensor, sf: torch.Tensor, gs, w: MoEWeights, K: int) -> torch.Tensor:
    """Tokens quantised once (packed rows + scale tiles, NVFP4 / MXFP4) -> the local experts' results, expert-sorted
    bf16 rows [tokens * k, D] (rows beyond the local total unwritten): dispatch, gate/up GEMM with SwiGLU, down GEMM."""
    fmt = w.gate_up.format
    offs = _local_offsets(p, w.first, w.last)
    q_rows, sf_rows = dispatch_fp4(p, packed, sf, K, fmt, w.first, w.last)
    common = dict(format=fmt, expert_offsets=offs, b_static=True)
    if fmt == "nvfp4" and w.hidden_global_scale is not None:
        hq, hsf, hgs = gemm_fp4_quantized(q_rows, w.gate_up.q, sf_rows, w.gate_up.scale, n=w.gate_up.n, global_scale_a=gs,
                                          global_scale_b=w.gate_up.global_scale, activation="swiglu", out_dtype="nvfp4",
                                          out_global_scale=w.hidden_global_scale, **common)
    else:
        h = gemm_fp4_quantized(q_rows, w.gate_up.q, sf_rows, w.gate_up.scale, n=w.gate_up.n, global_scale_a=gs,
                               global_scale_b=w.gate_up.global_scale, activation="swiglu", out_dtype=torch.bfloat16, **common)
        n_local = h.shape[0] if (w.last - w.first) == w.experts else int(offs[-1].item())
        hq, hsf, hgs = quantize_fp4(h[:n_local], fmt, group_offsets=offs)
    return gemm_fp4_quantized(hq, w.down.q, hsf, w.down.scale, n=w.down.n, global_scale_a=hgs,
                              global_scale_b=w.down.global_scale, out_dtype=torch.bfloat16, **common)


def moe_partial(x: torch.Tensor, logits: torch.Tensor, w: MoEWeights, k: int, *, renormalize: bool = True,
                out_dtype=torch.float32, act_global_scale=None, out=None) -> torch.Tensor:
    """This rank's share of the layer's result, [tokens, D] (fp32, or bf16 = the fp32 sum rounded once, which saves
    a conversion pass when the shares travel in bf16): the sum over the slots routed to its experts.
    NVFP4 / MXFP4 weights take the quantise-once path; with `hidden_global_scale` set (NVFP4) the hidden
    activation is quantised in the epilogue of the gate/up GEMM, otherwise it is written in bf16 and quantised
    by a separate pass (which, when the rank holds only part of the experts, reads the local row count back to
    the host once).  `act_global_scale` (NVFP4: a number or a one-element tensor) is a calibrated global scale of x;
    the quantiser then makes ONE pass over x instead of an amax pass and a quantise pass."""
    fmt = w.gate_up.format
    ids, wts = route(logits, k, renormalize)
    p = plan(ids, wts, w.experts)
    offs = _local_offsets(p, w.first, w.last)
    K = x.shape[1]
    if fmt in ("nvfp4", "mxfp4"):
        packed, sf, gs = quantize_fp4(x, fmt, global_scale=act_global_scale if fmt == "nvfp4" else None)
        y = _experts_fp4(p, packed, sf, gs, w, K)
    elif fmt == "fp8":
        # per-tensor scale: taken over the tokens, so that it does not depend on which experts are local;
        # the E4M3 bytes are dispatched.  The hidden activation's scale is this rank's (valid rows only).
        qa, sa = quantize_fp8(x, "per_tensor")
        rows = dispatch_rows(p, qa, w.first, w.last)
        h = gemm_fp8_quantized(rows, w.gate_up.q, sa, w.gate_up.scale, n=w.gate_up.n, expert_offsets=offs, activation="swiglu",
                               out_dtype=torch.bfloat16, b_static=True)
        n_local = h.shape[0] if (w.last - w.first) == w.experts else int(offs[-1].item())
        qh, sh = quantize_fp8(h[:n_local], "per_tensor")
        y = gemm_fp8_quantized(qh, w.down.q, sh, w.down.scale, n=w.down.n, expert_offsets=offs, out_dtype=torch.bfloat16,
                               b_static=True)
    elif fmt == "fp8_block128":
        # 1x128 activation groups: quantised once per token; the E4M3 rows and their scale rows are dispatched
        qa, sa = quantize_fp8(x, "groupwise")
        rows = dispatch_rows(p, qa, w.first, w.last)
        sa_rows = dispatch_rows(p, _pad_cols(sa, 4), w.first, w.last)[:, :sa.shape[1]].contiguous()
        h = gemm_fp8_groupwise_quantized(rows, w.gate_up.q, sa_rows, w.gate_up.scale, n=w.gate_up.n, sb_block=True,
                                         expert_offsets=offs, activation="swiglu", out_dtype=torch.bfloat16)
        y = linear(h, w.down, expert_offsets=offs, out_dtype=torch.bfloat16)     # rows are independent: unwritten ones harm nobody
    else:
        rows = dispatch_rows(p, x.to(torch.bfloat16), w.first, w.last)
        h = linear(rows, w.gate_up, expert_offsets=offs, activation="swiglu", out_dtype=torch.bfloat16)
        y = linear(h, w.down, expert_offsets=offs, out_dtype=torch.bfloat16)
    return combine(p, y, w.first, w.last, out_dtype=out_dtype, out=out)


def pack_wire(p: MoEPlan, packed: torch.Tensor, sf: torch.Tensor, K: int, format: str) -> torch.Tensor:
    """Rows quantised once per token -> one record per routed row ([tokens*k, wire bytes] uint8), expert-sorted."""
    dev = _lib.require_cuda(packed, sf)
    T, k = p.ids.shape
    fmt = _lib.FP4_NV if format == "nvfp4" else _lib.FP4_MX
    wb = int(_lib.lib().dsl_moe_wire_bytes(K, fmt))
    wire = torch.empty((T * k, wb), dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        rc = _lib.lib().dsl_moe_pack_wire_fp4(packed.data_ptr(), sf.data_ptr(), p.dest.data_ptr(), T, k, K, fmt, wire.data_ptr(),
                                              _lib.stream_ptr())
    _lib.check(rc, "dsl_moe_pack_wire_fp4")
    return wire


def unpack_wire(p: MoEPlan, wire: torch.Tensor, K: int, format: str):
    """Records in arrival order (planned by `p`: one slot per record, local expert ids) -> (packed rows [rows, K/2],
    scale tiles in the ragged-group layout): the A operand of the grouped GEMM."""
    dev = _lib.require_cuda(wire)
    rows = wire.shape[0]
    fmt = _lib.FP4_NV if format == "nvfp4" else _lib.FP4_MX
    nblk = K // 16 if format == "nvfp4" else K // 32
    q = torch.empty((rows, K // 2), dtype=torch.uint8, device=dev)
    sf = torch.zeros(int(_lib.lib().dsl_sf_bytes_grouped(rows, nblk, p.experts)), dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        rc = _lib.lib().dsl_moe_unpack_wire_fp4(wire.data_ptr(), p.ids.data_ptr(), p.dest.data_ptr(), p.offsets.data_ptr(),
                                                p.tile0.data_ptr(), rows, K, fmt, q.data_ptr(), sf.data_ptr(), _lib.stream_ptr())
    _lib.check(rc, "dsl_moe_unpack_wire_fp4")
    return q, sf


def _global_scale_of(amax: torch.Tensor) -> torch.Tensor:
    """amax / 2688 as the quantiser computes it (one IEEE division; an all-zero tensor gets 1).  Tensor by tensor:
    dividing by a Python number may be turned into a multiplication by its reciprocal, which rounds differently."""
    gs = torch.div(amax, torch.full_like(amax, 2688.0))
    return torch.where(amax == 0, torch.ones_like(amax), gs)


def moe_forward_all_to_all(x: torch.Tensor, logits: torch.Tensor, w: MoEWeights, k: int, *, renormalize: bool = True,
                           out_dtype=torch.float32, group=None, act_global_scale=None) -> torch.Tensor:
    """The layer for a rank that owns the token rows x [tokens_local, K] and the experts w.first .. w.last: returns
    its own tokens' results [tokens_local, D].  NVFP4 / MXFP4 weights.  The NVFP4 global scale of the activations
    is that of ALL ranks' tokens (one all-reduce of a float), so the layer computes exactly what one GPU holding
    every token would; a calibrated `act_global_scale` (number or one-element tensor) replaces it and saves that
    collective and the amax pass."""
    import torch.distributed as dist
    fmt = w.gate_up.format
    if fmt not in ("nvfp4", "mxfp4"):
        raise ValueError("the all-to-all layer serves NVFP4 and MXFP4 weights")
    dev = _lib.require_cuda(x, logits)
    world = dist.get_world_size(group) if dist.is_available() and dist.is_initialized() else 1
    if (w.last - w.first) < w.experts and world == 1:
        raise RuntimeError("these weights cover only part of the experts: initialise torch.distributed")
    K = x.shape[1]
    local_experts = w.last - w.first
    ids, wts = route(logits, k, renormalize)
    p = plan(ids, wts, w.experts)
    gs_in = act_global_scale if fmt == "nvfp4" else None
    if fmt == "nvfp4" and world > 1 and gs_in is None:
        amax = torch.linalg.vector_norm(x, ord=float("inf")).float().reshape(1)       # max |x| in one pass
        dist.all_reduce(amax, op=dist.ReduceOp.MAX, group=group)
        gs_in = _global_scale_of(amax)
    packed, sf, gs = quantize_fp4(x, fmt, global_scale=gs_in)
    wire = pack_wire(p, packed, sf, K, fmt)
    counts = p.offsets[1:] - p.offsets[:-1]
    ex = exchange_rows(wire, counts, w.experts, group)
    R = ex.received.shape[0]
    D = w.down.n
    fused_hidden = fmt == "nvfp4" and w.hidden_global_scale is not None
    h = hq = hsf = hgs = p2 = None
    common = {}
    if R > 0:
        ids_in = arrival_expert_ids(ex, dev).reshape(R, 1)
        p2 = plan(ids_in, torch.ones((R, 1), dtype=torch.float32, device=dev), local_experts)
        q_rows, sf_rows = unpack_wire(p2, ex.received, K, fmt)
        common = dict(format=fmt, expert_offsets=p2.offsets, b_static=True)
        if fused_hidden:
            hq, hsf, hgs = gemm_fp4_quantized(q_rows, w.gate_up.q, sf_rows, w.gate_up.scale, n=w.gate_up.n, global_scale_a=gs,
                                              global_scale_b=w.gate_up.global_scale, activation="swiglu", out_dtype="nvfp4",
                                              out_global_scale=w.hidden_global_scale, **common)
        else:
            h = gemm_fp4_quantized(q_rows, w.gate_up.q, sf_rows, w.gate_up.scale, n=w.gate_up.n, global_scale_a=gs,
                                   global_scale_b=w.gate_up.global_scale, activation="swiglu", out_dtype=torch.bfloat16, **common)
    if not fused_hidden:
        # the hidden activation's global scale is that of ALL ranks' rows (every rank joins, also one without rows)
        hgs_in = None
        if fmt == "nvfp4" and world > 1:
            amax_h = (torch.linalg.vector_norm(h, ord=float("inf")).float().reshape(1) if R > 0
                      else torch.zeros(1, dtype=torch.float32, device=dev))
            dist.all_reduce(amax_h, op=dist.ReduceOp.MAX, group=group)
            hgs_in = _global_scale_of(amax_h)
        if R > 0:
            hq, hsf, hgs = quantize_fp4(h, fmt, global_scale=hgs_in, group_offsets=p2.offsets)
    if R > 0:
        y = gemm_fp4_quantized(hq, w.down.q, hsf, w.down.scale, n=w.down.n, global_scale_a=hgs,
                               global_scale_b=w.down.global_scale, out_dtype=torch.bfloat16, **common)
        y_arrival = combine(p2, y, 0, local_experts, out_dtype=torch.bfloat16)      # back to arrival order (one slot, weight 1)
    else:
        y_arrival = torch.empty((0, D), dtype=torch.bfloat16, device=dev)
    back = return_rows(y_arrival, ex, group)
    return combine(p, back, 0, w.experts, out_dtype=out_dtype)


def _moe_forward_chunked(x, logits, w: MoEWeights, k: int, renormalize: bool, group, reduce: str, exchange_dtype,
                         chunks: int, act_global_scale=None) -> torch.Tensor:
    """Expert-parallel layer (replicated routing, NVFP4 / MXFP4) in `chunks` pipelined pieces: routing and the activation
    quantiser run once over all tokens (so the NVFP4 global scale is the whole tensor's, as without chunks), then every
    piece is dispatched, multiplied and combined on the compute stream while the previous piece's partial results
    are summed over the ranks by an asynchronous collective on NCCL's stream.  Returns the summed result in the exchange
    dtype: all tokens (all_reduce) or this rank's token rows (reduce_scatter)."""
    import torch.distributed as dist
    fmt = w.gate_up.format
    world = dist.get_world_size(group)
    T, K = x.shape
    D = w.down.n
    dt = exchange_dtype if exchange_dtype is not None else torch.float32
    if dt not in (torch.float32, torch.bfloat16):
        raise ValueError("chunks > 1: the exchange dtype must be float32 or bfloat16")
    scatter = reduce == "reduce_scatter"
    piece = T // (world * chunks) if scatter else T // chunks        # token rows of one piece (per rank when scattering)
    if piece * chunks * (world if scatter else 1) != T or piece % 128:
        raise ValueError(f"chunks={chunks}: every piece must be a multiple of 128 token rows "
                         f"(tokens {T}, ranks {world if scatter else 1})")
    ids, wts = route(logits, k, renormalize)
    packed, sf, gs = quantize_fp4(x, fmt, global_scale=act_global_scale if fmt == "nvfp4" else None)
    nblk = K // 16 if fmt == "nvfp4" else K // 32
    tile_bytes = ((nblk + 3) // 4) * 512                              # one 128-row scale tile row of the plain layout
    outer = world if scatter else 1
    # piece c = rows [c * piece, (c + 1) * piece) of every rank's token range: after the reduce-scatter rank r holds
    # rows [c * piece, (c + 1) * piece) of ITS range, i.e. the pieces land side by side in the rank's result
    packed_v = packed.view(outer, chunks, piece, K // 2)
    sf_v = sf[:(T // 128) * tile_bytes].view(outer, chunks, piece // 128, tile_bytes)
    ids_v = ids.view(outer, chunks, piece, k)
    wts_v = wts.view(outer, chunks, piece, k)
    out = torch.empty((piece * chunks, D), dtype=dt, device=x.device)
    works, keep = [], []
    for c in range(chunks):
        p = plan(ids_v[:, c].reshape(outer * piece, k), wts_v[:, c].reshape(outer * piece, k), w.experts)
        y = _experts_fp4(p, packed_v[:, c].reshape(outer * piece, K // 2), sf_v[:, c].reshape(-1), gs, w, K)
        dst = out[c * piece:(c + 1) * piece]
        if scatter:
            part = combine(p, y, w.first, w.last, out_dtype=dt)
            works.append(dist.reduce_scatter_tensor(dst, part, group=group, async_op=True))
            keep.append(part)
        else:
            combine(p, y, w.first, w.last, out=dst)
            works.append(dist.all_reduce(dst, group=group, async_op=True))
    for wk in works:
        wk.wait()
    return out


def moe_forward(x: torch.Tensor, logits: torch.Tensor, w: MoEWeights, k: int, *, renormalize: bool = True,
                out_dtype=torch.float32, group=None, reduce: str = "all_reduce", exchange_dtype=None,
                dispatch: str = "replicated", chunks: int = 1, act_global_scale=None) -> torch.Tensor:
    """One MoE feed-forward layer: x [tokens, K], router logits [tokens, experts] -> [tokens, D].
    dispatch "all_to_all": x / logits are this rank's OWN token rows and the result is theirs
    (`moe_forward_all_to_all`); the remaining arguments below apply to "replicated".
    When `w` covers only part of the experts the per-rank partial results are summed over `group` (default: the
    default process group of torch.distributed): reduce "all_reduce" leaves the whole result on every rank,
    "reduce_scatter" leaves rank r with token rows [r * tokens / world, (r + 1) * tokens / world) - half the
    traffic, and what a sequence-sharded consumer wants; "pull" gives the same rows without a data-moving collective:
    the shares sit in symmetric memory and `dsl_moe_reduce_pull` reads the rank's rows of every share over NVLink
    and adds them in rank order (`sharding.PeerReducer`; one small all-reduce per layer serves as the barrier).  `exchange_dtype` (e.g. torch.bfloat16) rounds the
    partial results before they travel; default fp32.  `chunks` > 1 (NVFP4 / MXFP4 weights, expert-parallel) runs the
    layer in that many pieces so that each piece's collective overlaps the next piece's GEMMs; every piece must be a
    multiple of 128 token rows.  Per token the arithmetic is that of chunks = 1 (the ranks' sums may associate
    differently inside the collective when there are more than two ranks).  `act_global_scale` (NVFP4 weights): a
    calibrated global scale of x (number or one-element tensor) instead of amax / 2688 - one quantiser pass, no
    collective for it in the all-to-all form."""
    if dispatch not in ("replicated", "all_to_all"):
        raise ValueError("dispatch must be 'replicated' or 'all_to_all'")
    if dispatch == "all_to_all":
        return moe_forward_all_to_all(x, logits, w, k, renormalize=renormalize, out_dtype=out_dtype, group=group,
                                      act_global_scale=act_global_scale)
    if reduce not in ("all_reduce", "reduce_scatter", "pull"):
        raise ValueError("reduce must be 'all_reduce', 'reduce_scatter' or 'pull'")
    partial = (w.last - w.first) < w.experts
    if chunks > 1 and reduce == "pull":
        raise ValueError("chunks > 1 goes with reduce='all_reduce' or 'reduce_scatter'")
    if chunks > 1 and partial and w.gate_up.format in ("nvfp4", "mxfp4"):
        import torch.distributed as dist
        if not dist.is_available() or not dist.is_initialized():
            raise RuntimeError("these weights cover only part of the experts: initialise torch.distributed")
        out = _moe_forward_chunked(x, logits, w, k, renormalize, group, reduce, exchange_dtype, chunks, act_global_scale)
        return out if out.dtype == out_dtype else out.to(out_dtype)
    if partial and reduce == "pull":
        # every rank writes its share into symmetric memory and reads its own token rows of all shares over NVLink
        import torch.distributed as dist
        from .sharding import peer_reducer
        if not dist.is_available() or not dist.is_initialized():
            raise RuntimeError("these weights cover only part of the experts: initialise torch.distributed")
        dt = exchange_dtype if exchange_dtype is not None else torch.float32
        red = peer_reducer(x.shape[0], w.down.n, dt, x.device, group)
        moe_partial(x, logits, w, k, renormalize=renormalize, act_global_scale=act_global_scale, out=red.buffer())
        return red.reduce(out_dtype)
    # shares that travel in bf16 are written in bf16 by the combine itself (fp32 sum, one rounding)
    direct = partial and exchange_dtype == torch.bfloat16
    out = moe_partial(x, logits, w, k, renormalize=renormalize, out_dtype=torch.bfloat16 if direct else torch.float32,
                      act_global_scale=act_global_scale)
    if partial:
        import torch.distributed as dist
        if not dist.is_available() or not dist.is_initialized():
            raise RuntimeError("these weights cover only part of the experts: initialise torch.distributed")
        if exchange_dtype is not None and exchange_dtype != out.dtype:
            out = out.to(exchange_dtype)
        if reduce == "all_reduce":
            dist.all_reduce(out, group=group)
        else:
            world = dist.get_world_size(group)
            if out.shape[0] % world:
                raise ValueError(f"reduce_scatter needs the token count ({out.shape[0]}) to be a multiple of the group size ({world})")
            shard = torch.empty((out.shape[0] // world, out.shape[1]), dtype=out.dtype, device=out.device)
            dist.reduce_scatter_tensor(shard, out, group=group)
            out = shard
    return out if out.dtype == out_dtype else out.to(out_dtype)
