"""Mixture-of-experts steps around the grouped GEMM (router top-k, expert-sorted plan, dispatch of
quantised rows, combine) against plain numpy / torch restatements, and the whole layer against the same
layer composed from the library's unfused pieces.  The reference has no counterpart for these steps
(it stops at the grouped GEMM), so there are no reference vectors to pin them to."""
import numpy as np
import pytest
import torch

import dsl_tool_b200 as D
from dsl_tool_b200 import _lib, moe
from dsl_tool_b200.gemm_kernels import gemm_fp4_quantized
from oracle import moe_oracle as MO
from tests.helpers import activations

pytestmark = pytest.mark.gpu


_route_np = lambda logits, k, renorm: MO.route(logits, k, renorm)
_plan_np = MO.plan


@pytest.mark.parametrize("T,E,k", [(1, 8, 2), (9, 33, 4), (50, 40, 6), (257, 64, 8), (70, 65, 8), (100, 200, 5), (64, 1000, 32)])
@pytest.mark.parametrize("renorm", [True, False])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_route(cuda_device, T, E, k, renorm, dtype):
    rng = np.random.default_rng(T + E)
    logits = rng.standard_normal((T, E)).astype(np.float32)
    logits[0, :4] = logits[0, 0]                          # ties inside one token
    lt = torch.from_numpy(logits).to(dtype)
    ids, w = moe.route(lt.to(cuda_device), k, renorm)
    ids_np, w_np = _route_np(lt.float().numpy(), k, renorm)
    assert np.array_equal(ids.cpu().numpy(), ids_np)
    assert np.allclose(w.cpu().numpy(), w_np, rtol=2e-5, atol=1e-8)


@pytest.mark.parametrize("T,E,k", [(1, 4, 1), (300, 64, 8), (1000, 7, 3)])
def test_plan_is_the_stable_sort(cuda_device, T, E, k):
    rng = np.random.default_rng(T)
    ids = rng.integers(0, E, (T, k)).astype(np.int32)
    if E > 3:
        ids[ids == 2] = 3                                 # an expert nobody chose
    p = moe.plan(torch.from_numpy(ids).to(cuda_device), torch.ones(T, k, device=cuda_device), E)
    offsets, tile0, dest = _plan_np(ids, E)
    assert np.array_equal(p.offsets.cpu().numpy(), offsets)
    assert np.array_equal(p.tile0.cpu().numpy(), tile0)
    assert np.array_equal(p.dest.cpu().numpy(), dest)


@pytest.mark.parametrize("fmt", ["nvfp4", "mxfp4"])
@pytest.mark.parametrize("first,last", [(0, 16), (5, 11)])
def test_dispatch_of_quantised_rows_equals_quantising_dispatched_rows(cuda_device, fmt, first, last):
    rng = np.random.default_rng(first)
    T, E, k, K = 200, 16, 4, 256
    x = torch.from_numpy(activations(rng, T, K, outliers=True)).bfloat16().to(cuda_device)
    ids = torch.from_numpy(rng.integers(0, E, (T, k)).astype(np.int32)).to(cuda_device)
    p = moe.plan(ids, torch.ones(T, k, device=cuda_device), E)
    packed, sf, gs = D.quantize_fp4(x, fmt)
    q_rows, sf_rows = moe.dispatch_fp4(p, packed, sf, K, fmt, first, last)
    offsets, _, dest = _plan_np(ids.cpu().numpy(), E)
    n_local = int(offsets[last] - offsets[first])
    token_of_row = np.empty(T * k, np.int64)
    token_of_row[dest] = np.arange(T * k) // k
    rows = x[torch.from_numpy(token_of_row[offsets[first]:offsets[last]]).to(cuda_device)]
    loc = torch.from_numpy((offsets[first:last + 1] - offsets[first]).astype(np.int32)).to(cuda_device)
    pe, sfe, _ = D.quantize_fp4(rows, fmt, global_scale=gs, group_offsets=loc)
    assert torch.equal(q_rows[:n_local], pe)
    assert torch.equal(sf_rows[:sfe.numel()], sfe)
    plain = moe.dispatch_rows(p, x, first, last)
    assert torch.equal(plain[:n_local], rows)


def test_combine(cuda_device):
    rng = np.random.default_rng(9)
    T, E, k, Dm = 150, 8, 3, 200
    ids = rng.integers(0, E, (T, k)).astype(np.int32)
    w = rng.random((T, k)).astype(np.float32)
    p = moe.plan(torch.from_numpy(ids).to(cuda_device), torch.from_numpy(w).to(cuda_device), E)
    offsets, _, dest = _plan_np(ids, E)
    y = rng.standard_normal((T * k, Dm)).astype(np.float32)
    for first, last in ((0, E), (2, 5)):
        yl = np.zeros_like(y)
        n_local = offsets[last] - offsets[first]
        yl[:n_local] = y[offsets[first]:offsets[last]]
        want = np.zeros((T, Dm), np.float64)
        for t in range(T):
            for s in range(k):
                if first <= ids[t, s] < last:
                    want[t] += w[t, s] * y[dest[t * k + s]]
        for ydt in (torch.float32, torch.bfloat16):
            yt = torch.from_numpy(yl).to(ydt)
            ref = want if ydt == torch.float32 else None
            got = moe.combine(p, yt.to(cuda_device), first, last).cpu().numpy()
            if ref is None:
                ref = np.zeros((T, Dm), np.float64)
                yb = yt.float().numpy()
                for t in range(T):
                    for s in range(k):
                        if first <= ids[t, s] < last:
                            ref[t] += w[t, s] * yb[dest[t * k + s] - offsets[first]]
            assert np.allclose(got, ref, rtol=1e-5, atol=1e-5)


def _layer_inputs(rng, T, E, K, H, Dm, device):
    x = torch.from_numpy(activations(rng, T, K)).bfloat16().to(device)
    logits = torch.from_numpy(rng.standard_normal((T, E)).astype(np.float32)).to(device)
    w1 = torch.from_numpy((rng.standard_normal((E, 2 * H, K)) * 0.05).astype(np.float32)).bfloat16().to(device)
    w2 = torch.from_numpy((rng.standard_normal((E, Dm, H)) * 0.05).astype(np.float32)).bfloat16().to(device)
    return x, logits, w1, w2


def test_layer_equals_its_unfused_composition(cuda_device):
    """NVFP4 layer, fused path (quantise once + dispatch, SwiGLU and hidden quantisation in the epilogue) ==
    gather bf16 rows, quantise them, GEMM, activation tensor in fp32, quantise, GEMM, combine in torch."""
    rng = np.random.default_rng(40)
    T, E, k, K, H, Dm = 96, 6, 2, 256, 128, 192
    x, logits, w1, w2 = _layer_inputs(rng, T, E, K, H, Dm, cuda_device)
    hgs = 0.004
    wts = D.MoEWeights.pack(w1, w2, "nvfp4", hidden_global_scale=hgs)
    got = D.moe_forward(x, logits, wts, k)
    _lib.check_status()
    ids, rw = moe.route(logits, k)
    offsets, _, dest = _plan_np(ids.cpu().numpy(), E)
    token_of_row = np.empty(T * k, np.int64)
    token_of_row[dest] = np.arange(T * k) // k
    rows = x[torch.from_numpy(token_of_row).to(cuda_device)]
    offs = torch.from_numpy(offsets).to(cuda_device)
    gsx = x.float().abs().amax() / 2688.0
    pa, sfa, ga = D.quantize_fp4(rows, "nvfp4", global_scale=gsx, group_offsets=offs)
    h = gemm_fp4_quantized(pa, wts.gate_up.q, sfa, wts.gate_up.scale, format="nvfp4", n=2 * H, global_scale_a=ga,
                                                    global_scale_b=wts.gate_up.global_scale, expert_offsets=offs, activation="swiglu")
    hp, hsf, hg = D.quantize_fp4(h, "nvfp4", global_scale=hgs, group_offsets=offs)
    y = gemm_fp4_quantized(hp, wts.down.q, hsf, wts.down.scale, format="nvfp4", n=Dm, global_scale_a=hg,
                           global_scale_b=wts.down.global_scale, expert_offsets=offs, out_dtype=torch.bfloat16).float()
    want = torch.zeros(T, Dm, device=cuda_device)
    d = torch.from_numpy(dest.reshape(T, k).astype(np.int64)).to(cuda_device)
    for s in range(k):
        want = want + rw[:, s:s + 1] * y[d[:, s]]
    assert torch.allclose(got, want, rtol=1e-5, atol=1e-6)
    # and it is the layer: against fp32 math on the unquantised tensors, within the formats' error
    xf, w1f, w2f = x.float(), w1.float(), w2.float()
    dense = torch.zeros(T, Dm, device=cuda_device)
    for s in range(k):
        e = ids[:, s].long()
        gu = torch.einsum("tk,tnk->tn", xf, w1f[e])
        hh = torch.nn.functional.silu(gu[:, :H]) * gu[:, H:]
        dense += rw[:, s:s + 1] * torch.einsum("th,tdh->td", hh, w2f[e])
    rel = ((got - dense).norm() / dense.norm()).item()
    assert rel < 0.25


@pytest.mark.parametrize("fmt", ["nvfp4", "mxfp4", "bf16", "fp8", "fp8_block128"])
def test_expert_parallel_partials_add_up(cuda_device, fmt):
    """Two ranks' shares of the experts, computed on this one GPU, sum to the single-rank result."""
    rng = np.random.default_rng(41)
    T, E, k, K, H, Dm = 64, 5, 2, 256, 128, 128
    x, logits, w1, w2 = _layer_inputs(rng, T, E, K, H, Dm, cuda_device)
    hgs = 0.004 if fmt == "nvfp4" else None
    whole = moe.moe_partial(x, logits, D.MoEWeights.pack(w1, w2, fmt, hidden_global_scale=hgs), k)
    parts = [moe.moe_partial(x, logits, D.MoEWeights.pack(w1, w2, fmt, rank=r, world=2, hidden_global_scale=hgs), k) for r in range(2)]
    _lib.check_status()
    if fmt == "fp8":      # the hidden activation's per-tensor scale is each rank's own: equal up to E4M3 rounding
        rel = ((parts[0] + parts[1] - whole).norm() / whole.norm()).item()
        assert rel < 0.05, rel
    else:
        assert torch.allclose(parts[0] + parts[1], whole, rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("fmt,hgs", [("nvfp4", 0.004), ("nvfp4", None), ("mxfp4", None)])
def test_all_to_all_path_on_one_rank_equals_the_replicated_layer(cuda_device, fmt, hgs):
    """dispatch="all_to_all" with a single rank sends nothing, but runs every kernel of that path (records packed
    for the wire, unpacked into expert-sorted rows and scale tiles, results put back in arrival order): it must
    give the very bits of the ordinary layer.  Shapes with an expert nobody chose and rows that do not fill tiles."""
    rng = np.random.default_rng(60)
    T, E, k, K, H, Dm = 333, 7, 3, 384, 128, 160
    x, logits, w1, w2 = _layer_inputs(rng, T, E, K, H, Dm, cuda_device)
    logits[:, 2] = -1e9
    wts = D.MoEWeights.pack(w1, w2, fmt, hidden_global_scale=hgs)
    base = D.moe_forward(x, logits, wts, k)
    got = D.moe_forward(x, logits, wts, k, dispatch="all_to_all")
    _lib.check_status()
    assert torch.equal(got, base)


def test_calibrated_activation_scale_in_the_layer(cuda_device):
    """act_global_scale replaces amax / 2688 of the tokens: given the very scale the dynamic path derives, the layer's
    bits do not change (both dispatch forms); given another one, the result moves by FP4 rounding noise and both forms still agree."""
    rng = np.random.default_rng(62)
    T, E, k, K, H, Dm = 200, 5, 2, 256, 128, 192
    x, logits, w1, w2 = _layer_inputs(rng, T, E, K, H, Dm, cuda_device)
    wts = D.MoEWeights.pack(w1, w2, "nvfp4", hidden_global_scale=0.004)
    base = D.moe_forward(x, logits, wts, k)
    _, _, gs = D.quantize_fp4(x, "nvfp4")
    for given in (gs, float(gs.item())):
        assert torch.equal(D.moe_forward(x, logits, wts, k, act_global_scale=given), base)
        assert torch.equal(D.moe_forward(x, logits, wts, k, act_global_scale=given, dispatch="all_to_all"), base)
    other = D.moe_forward(x, logits, wts, k, act_global_scale=float(gs.item()) * 1.3)
    assert torch.equal(D.moe_forward(x, logits, wts, k, act_global_scale=float(gs.item()) * 1.3, dispatch="all_to_all"), other)
    rel = float((other - base).norm() / base.norm())
    assert 0 < rel < 0.5, rel          # another block-scale grid: FP4 rounding noise of the same order as the layer's own
    _lib.check_status()


def test_wire_records_round_trip(cuda_device):
    """pack -> unpack of the wire records reproduces dispatch_fp4's expert-sorted rows and scale tiles bit for bit."""
    rng = np.random.default_rng(61)
    T, E, k, K = 300, 9, 4, 416                     # 26 scale blocks per row: the last scale tile is partly padding
    x = torch.from_numpy(activations(rng, T, K, outliers=True)).bfloat16().to(cuda_device)
    ids = torch.from_numpy(rng.integers(0, E, (T, k)).astype(np.int32)).to(cuda_device)
    p = moe.plan(ids, torch.ones(T, k, device=cuda_device), E)
    for fmt in ("nvfp4", "mxfp4"):
        packed, sf, _ = D.quantize_fp4(x, fmt)
        want_q, want_sf = moe.dispatch_fp4(p, packed, sf, K, fmt, 0, E)
        wire = moe.pack_wire(p, packed, sf, K, fmt)
        assert wire.shape == (T * k, int(_lib.lib().dsl_moe_wire_bytes(K, _lib.FP4_NV if fmt == "nvfp4" else _lib.FP4_MX)))
        # on arrival the records are planned again, one slot each: the expert of record r is that of sorted row r
        expert_of_row = torch.repeat_interleave(torch.arange(E, device=cuda_device, dtype=torch.int32),
                                                (p.offsets[1:] - p.offsets[:-1]).long())
        p2 = moe.plan(expert_of_row.reshape(-1, 1).contiguous(), torch.ones(T * k, 1, device=cuda_device), E)
        q, sf2 = moe.unpack_wire(p2, wire, K, fmt)
        assert torch.equal(q, want_q) and torch.equal(sf2, want_sf)


def test_token_permutation_invariance_at_scale(cuda_device):
    """Size-independent property of the whole layer: permuting the tokens permutes the result rows and changes
    nothing else (a row's value depends only on the token, its experts and the fixed summation orders)."""
    rng = np.random.default_rng(50)
    T, E, k, K, H, Dm = 4096, 64, 8, 1024, 512, 1024
    x, logits, w1, w2 = _layer_inputs(rng, T, E, K, H, Dm, cuda_device)
    wts = D.MoEWeights.pack(w1, w2, "nvfp4", hidden_global_scale=0.004)
    perm = torch.from_numpy(rng.permutation(T)).to(cuda_device)
    base = D.moe_forward(x, logits, wts, k)
    again = D.moe_forward(x[perm].contiguous(), logits[perm].contiguous(), wts, k)
    _lib.check_status()
    assert torch.equal(again, base[perm])
    assert torch.isfinite(base).all() and float(base.abs().max()) > 0
