"""Benchmark of the quantised-GEMM hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl ours|reference]

One "step" = one pass of the hot path over one batch of synthetic input: quantise / scale-pack
the activations (one kernel) and run the GEMM against weights that were quantised once.  The
default workload is the FP8 groupwise GEMM at the Llama-3-8B MLP shape (M=4096, K=4096,
N=14336; 1x128 activation scales, 128x128 weight-block scales, bf16 output).  Inputs are
seeded synthetic tensors of the stated shapes and distributions.

Prints ONE JSON line (rank 0).  `value` is aggregate TFLOP/s over all ranks with inputs
resident in HBM; `e2e` is the same metric through the public callable with activations in
pinned host memory (host->device copy of the activations and device->host copy of the result
inside the timed region).  With N > 1 each rank holds its own column shard of the weight
(dense) or its own experts (MoE) of the same per-rank size, no data-path collective.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (kind, M, K, N, act std/outliers, weight std, description)
    "fp8_groupwise_llama8b_mlp": dict(kind="fp8_block128", M=4096, K=4096, N=14336, wstd=0.02, outliers=False),
    "fp8_groupwise_m1024": dict(kind="fp8_block128", M=1024, K=4096, N=14336, wstd=0.02, outliers=False),
    "fp8_per_tensor_1024": dict(kind="fp8", M=1024, K=1024, N=1024, wstd=1.0, outliers=False),
    "fp8_groupwise_8192": dict(kind="fp8_block128", M=8192, K=8192, N=8192, wstd=0.02, outliers=False),
    "nvfp4_8192": dict(kind="nvfp4", M=8192, K=8192, N=8192, wstd=0.02, outliers=True),
    "nvfp4_m1024": dict(kind="nvfp4", M=1024, K=8192, N=8192, wstd=0.02, outliers=True),
    "nvfp4_m128": dict(kind="nvfp4", M=128, K=8192, N=8192, wstd=0.02, outliers=True),
    "nvfp4_m16": dict(kind="nvfp4", M=16, K=8192, N=8192, wstd=0.02, outliers=True),
    "nvfp4_m1": dict(kind="nvfp4", M=1, K=8192, N=8192, wstd=0.02, outliers=True),
    "mxfp4_llama70b_up": dict(kind="mxfp4", M=8192, K=8192, N=28672, wstd=0.015, outliers=False),
    "mxfp4_llama70b_down": dict(kind="mxfp4", M=8192, K=28672, N=8192, wstd=0.015, outliers=False),
    "moe_nvfp4": dict(kind="nvfp4", moe=True, tokens=16384, topk=8, experts=64, K=4096, N=3072, wstd=0.02),
    "moe_fp8_groupwise": dict(kind="fp8_block128", moe=True, tokens=16384, topk=8, experts=64, K=4096, N=3072, wstd=0.02),
    "moe_nvfp4_swiglu": dict(kind="nvfp4", moe=True, tokens=16384, topk=8, experts=64, K=4096, N=3072, wstd=0.02, act="swiglu"),
    "moe_nvfp4_swiglu_nvfp4out": dict(kind="nvfp4", moe=True, tokens=16384, topk=8, experts=64, K=4096, N=3072, wstd=0.02,
                                      act="swiglu", out="nvfp4"),
    "moe_fp8_groupwise_swiglu": dict(kind="fp8_block128", moe=True, tokens=16384, topk=8, experts=64, K=4096, N=3072, wstd=0.02,
                                     act="swiglu"),
    # config C5 fed the way a layer feeds it: 16384 token rows + their routing; the tokens are quantised ONCE and the
    # packed rows dispatched to expert-sorted order (step = plan + quantise + dispatch + grouped GEMM)
    "moe_nvfp4_tokens": dict(kind="nvfp4", tokens_in=True, tokens=16384, topk=8, experts=64, K=4096, N=3072, wstd=0.02),
    # the whole MoE feed-forward layer around the two grouped GEMMs (router, plan, quantise once, dispatch,
    # gate/up GEMM with SwiGLU and NVFP4 result, down GEMM, combine); 0.01 = calibrated hidden global scale
    "moe_layer_nvfp4": dict(kind="nvfp4", layer=True, tokens=16384, topk=8, experts=64, K=4096, H=1536, D=4096, wstd=0.02,
                            hidden_gs=0.01),
    "bf16_8192": dict(kind="bf16", M=8192, K=8192, N=8192, wstd=0.02, outliers=False),
}
DTYPE_NAME = {"fp8": "fp8_e4m3", "fp8_block128": "fp8_e4m3", "nvfp4": "fp4_e2m1", "mxfp4": "fp4_e2m1", "bf16": "bf16"}
# dram__bytes_read.sum + dram__bytes_write.sum of the GEMM kernel per launch, from an ncu capture of the
# full-size workload (profiles/): bytes.  None where no capture exists.
NCU_TRAFFIC = {"fp8_groupwise_llama8b_mlp": 77.1e6 + 74.9e6,
               "nvfp4_8192": 164.5e6 + 105.9e6,
               "nvfp4_m16": 37.93e6 + 0.28e6}      # decode: GEMM + quantiser launch (whole step)
PEAK_MULT = {"fp8": 2.0, "fp8_block128": 2.0, "nvfp4": 4.0, "mxfp4": 4.0, "bf16": 1.0}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return p["bf16_tflops"], p["hbm_gbs"], "measured"
    return 1590.0, 6650.0, "fallback"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "20"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm = [float(r[0]) for r in self.rows if len(r) >= 6 and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) >= 6 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) >= 6 and r[2 + i] == "Active" for r in self.rows)]
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


def make_moe_offsets(rng, tokens, experts, topk):
    logits = rng.standard_normal((tokens, experts)).astype(np.float32)
    top = np.argpartition(-logits, topk - 1, axis=1)[:, :topk]
    counts = np.bincount(top.reshape(-1), minlength=experts)
    return np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)


def build_workload(name, rank, world, device, sets, strong=False):
    """Returns dict(step=callable(i)->out, gemm=callable, flops, rows, desc...) with `sets`
    rotating copies of inputs so consecutive steps never reuse L2-resident operands."""
    from dsl_tool_b200 import pack_weight
    from dsl_tool_b200.gemm_kernels import linear
    cfg = WORKLOADS[name]
    kind = cfg["kind"]
    g = torch.Generator(device=device).manual_seed(1234 + rank)
    if cfg.get("layer"):
        return build_layer_workload(cfg, rank, world, device, sets, strong, g)
    if cfg.get("tokens_in"):
        return build_token_moe_workload(cfg, rank, device, sets)
    offs = None
    if cfg.get("moe"):
        experts = cfg["experts"]          # weak scaling keeps 64 local experts (and their routed rows) per GPU
        if strong:                        # strong scaling: one global routing, this rank owns experts/world of them
            from dsl_tool_b200.sharding import expert_ranges, local_rows
            glob = make_moe_offsets(np.random.default_rng(99), cfg["tokens"], experts, cfg["topk"])
            first, last = expert_ranges(experts, world)[rank]
            _, _, loc = local_rows(glob, first, last)
            offs_np = np.asarray(loc, dtype=np.int32)
            experts = last - first
        else:
            offs_np = make_moe_offsets(np.random.default_rng(99 + rank), cfg["tokens"], experts, cfg["topk"])
        offs = torch.from_numpy(offs_np).to(device)
        M, K, N = int(offs_np[-1]), cfg["K"], cfg["N"]
        wshape = (experts, N, K)
    else:
        M, K, N = cfg["M"], cfg["K"], cfg["N"]
        if strong:                        # this rank's 128-aligned column range of the one weight
            from dsl_tool_b200.sharding import column_ranges
            c0, c1 = column_ranges(N, world)[rank]
            N = c1 - c0
        wshape = (1, N, K)
    acts, wts = [], []
    for s in range(sets):
        a = torch.randn((M, K), generator=g, device=device, dtype=torch.float32)
        if cfg.get("outliers"):
            mask = torch.rand((M, K), generator=g, device=device) < 1e-3
            sign = torch.where(torch.rand((M, K), generator=g, device=device) < 0.5, -20.0, 20.0)
            a = torch.where(mask, sign, a)
        acts.append(a.to(torch.bfloat16))
        del a
        w = (torch.randn(wshape, generator=g, device=device, dtype=torch.float32) * cfg["wstd"]).to(torch.bfloat16)
        wts.append(pack_weight(w, kind, layout="nk", gate_up_interleave=cfg.get("act") == "swiglu"))
        del w
    torch.cuda.synchronize()

    def step(i, a=None):
        if cfg.get("out") == "nvfp4":    # result quantised in the epilogue with a fixed (calibrated) global scale
            return linear(acts[i % sets] if a is None else a, wts[i % sets], out_dtype="nvfp4", out_global_scale=1.0 / 2688.0,
                          expert_offsets=offs, activation=cfg.get("act"))[0]
        return linear(acts[i % sets] if a is None else a, wts[i % sets], out_dtype=torch.bfloat16, expert_offsets=offs,
                      activation=cfg.get("act"))

    return dict(step=step, acts=acts, wts=wts, offs=offs, M=M, K=K, N=N, kind=kind, flops=2.0 * M * N * K,
                moe=bool(cfg.get("moe")), act=cfg.get("act"), out=cfg.get("out"))


def build_layer_workload(cfg, rank, world, device, sets, strong, g):
    """Whole MoE layer.  Weak scaling: every rank owns a full set of experts and its own tokens; strong
    scaling: the experts of one layer are split over the ranks, tokens replicated, partial results all-reduced."""
    from dsl_tool_b200 import MoEWeights, moe_forward
    T, E, k, K, H, D = cfg["tokens"], cfg["experts"], cfg["topk"], cfg["K"], cfg["H"], cfg["D"]
    acts, logits, wts = [], [], []
    for s in range(sets):
        gen = torch.Generator(device=device).manual_seed(77 + s + (0 if strong else 1000 * rank))
        acts.append(torch.randn((T, K), generator=gen, device=device, dtype=torch.float32).to(torch.bfloat16))
        logits.append(torch.randn((T, E), generator=gen, device=device, dtype=torch.float32))
        w1 = (torch.randn((E, 2 * H, K), generator=gen, device=device, dtype=torch.float32) * cfg["wstd"]).to(torch.bfloat16)
        w2 = (torch.randn((E, D, H), generator=gen, device=device, dtype=torch.float32) * cfg["wstd"]).to(torch.bfloat16)
        wts.append(MoEWeights.pack(w1, w2, cfg["kind"], rank=rank if strong else 0, world=world if strong else 1,
                                   hidden_global_scale=cfg.get("hidden_gs")))
        del w1, w2
    torch.cuda.synchronize()

    def step(i, a=None):
        # expert-parallel ranks exchange bf16 partial results and keep their own token rows (reduce-scatter)
        return moe_forward(acts[i % sets] if a is None else a, logits[i % sets], wts[i % sets], k, out_dtype=torch.bfloat16,
                           reduce="reduce_scatter", exchange_dtype=torch.bfloat16)

    flops = 2.0 * T * k * (2 * H * K + D * H) / (world if strong else 1)
    return dict(step=step, acts=acts, wts=wts, offs=None, M=T * k, K=K, N=2 * H, kind=cfg["kind"], flops=flops, moe=True,
                act="swiglu", out=None, layer=True, out_cols=D, out_rows=T // (world if strong else 1))


def build_token_moe_workload(cfg, rank, device, sets):
    """Grouped GEMM of an MoE layer from token-level input: x [tokens, K], ids [tokens, k] (seeded top-k routing)."""
    from dsl_tool_b200 import moe, pack_weight, quantize_fp4
    from dsl_tool_b200.gemm_kernels import gemm_fp4_quantized
    T, E, k, K, N = cfg["tokens"], cfg["experts"], cfg["topk"], cfg["K"], cfg["N"]
    acts, ids, wts = [], [], []
    for s in range(sets):
        gen = torch.Generator(device=device).manual_seed(55 + s + 1000 * rank)
        acts.append(torch.randn((T, K), generator=gen, device=device, dtype=torch.float32).to(torch.bfloat16))
        logits = torch.randn((T, E), generator=gen, device=device, dtype=torch.float32)
        ids.append(torch.topk(logits, k, dim=1).indices.to(torch.int32).contiguous())
        w = (torch.randn((E, N, K), generator=gen, device=device, dtype=torch.float32) * cfg["wstd"]).to(torch.bfloat16)
        wts.append(pack_weight(w, "nvfp4", layout="nk"))
        del w
    ones = torch.ones((T, k), dtype=torch.float32, device=device)
    torch.cuda.synchronize()

    def quant(i, a=None):
        p = moe.plan(ids[i % sets], ones, E)
        packed, sf, gs = quantize_fp4(acts[i % sets] if a is None else a, "nvfp4")
        q, s = moe.dispatch_fp4(p, packed, sf, K, "nvfp4", 0, E)
        return q, s, gs, p.offsets

    def gemm(i, qs):
        w = wts[i % sets]
        return gemm_fp4_quantized(qs[0], w.q, qs[1], w.scale, format="nvfp4", n=N, global_scale_a=qs[2],
                                  global_scale_b=w.global_scale, expert_offsets=qs[3], out_dtype=torch.bfloat16, b_static=True)

    def step(i, a=None):
        return gemm(i, quant(i, a))

    return dict(step=step, acts=acts, wts=wts, offs=None, M=T * k, K=K, N=N, kind="nvfp4", flops=2.0 * T * k * N * K, moe=True,
                act=None, out=None, split=(quant, gemm))


def split_step(wl):
    """(quantise, gemm) closures so the GEMM launch can be bracketed by its own events."""
    if wl.get("layer"):
        return (lambda i: None), (lambda i, q: wl["step"](i))
    if wl.get("split"):
        return wl["split"]
    from dsl_tool_b200 import quantize_fp4, quantize_fp8
    from dsl_tool_b200 import gemm_kernels as GK
    kind, offs, sets = wl["kind"], wl["offs"], len(wl["acts"])

    def quant(i):
        a = wl["acts"][i % sets]
        if kind == "fp8":
            return quantize_fp8(a, "per_tensor")
        if kind == "fp8_block128":
            return quantize_fp8(a, "groupwise")
        if kind in ("nvfp4", "mxfp4"):
            return quantize_fp4(a, kind, group_offsets=offs)
        return (a,)

    def gemm(i, q):
        w = wl["wts"][i % sets]
        common = dict(n=w.n, out_dtype=torch.bfloat16, expert_offsets=offs, activation=wl.get("act"))
        if wl.get("out") == "nvfp4":
            common.update(out_dtype="nvfp4", out_global_scale=1.0 / 2688.0)
        if kind == "fp8":
            return GK.gemm_fp8_quantized(q[0], w.q, q[1], w.scale, b_static=True, **common)
        if kind == "fp8_block128":
            return GK.gemm_fp8_groupwise_quantized(q[0], w.q, q[1], w.scale, sb_block=True, **common)
        if kind in ("nvfp4", "mxfp4"):
            return GK.gemm_fp4_quantized(q[0], w.q, q[1], w.scale, format=kind, global_scale_a=q[2],
                                         global_scale_b=w.global_scale, b_static=True, **common)
        return GK.gemm_bf16_raw(q[0], w.q, **common)

    return quant, gemm


def cpu_baseline(name, sample_rows, steps=1, warmup=0):
    """The oracle's fp32-accumulated dequantised GEMM (numpy, all host threads) on the first
    `sample_rows` activation rows of the workload, full N and K.  Returns (TFLOP/s, cores, text)."""
    from oracle import quant_oracle as O
    cfg = WORKLOADS[name]
    kind = cfg["kind"]
    rng = np.random.default_rng(5)
    K, N = cfg["K"], cfg["N"]
    R = sample_rows
    a = rng.standard_normal((R, K)).astype(np.float32)
    w = (rng.standard_normal((N, K)) * cfg["wstd"]).astype(np.float32)
    if kind == "fp8_block128":
        qa, sa = O.quant_fp8_groupwise(a)
        qb, sbb = O.quant_fp8_block(w)
        sb = O.expand_block_scale(sbb, N)
        fn = lambda: O.gemm_fp8_groupwise(qa, qb, sa, sb)
    elif kind == "fp8":
        qa, sa = O.quant_fp8_per_tensor(a)
        qb, sb = O.quant_fp8_per_tensor(w)
        fn = lambda: O.gemm_fp8_per_tensor(qa, qb, sa, sb)
    elif kind == "nvfp4":
        pa, sfa, gsa = O.quant_nvfp4(a)
        pb, sfb, gsb = O.quant_nvfp4(w)
        fn = lambda: O.gemm_nvfp4(pa, sfa, gsa, pb, sfb, gsb)
    elif kind == "mxfp4":
        pa, sfa = O.quant_mxfp4(a)
        pb, sfb = O.quant_mxfp4(w)
        fn = lambda: O.gemm_mxfp4(pa, sfa, pb, sfb)
    else:
        fn = lambda: a @ w.T
    for _ in range(warmup):
        fn()
    t0 = time.perf_counter()
    for _ in range(steps):
        fn()
    dt = (time.perf_counter() - t0) / steps
    cores = os.cpu_count() or 1
    return 2.0 * R * N * K / dt / 1e12, cores, dt, f"first {R} activation rows x full N={N}, K={K} (dequantise + fp32 GEMM per step)"


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cfg = WORKLOADS[args.workload]
    rows = 512 if not cfg.get("moe") else 512
    val, cores, dt, sample = cpu_baseline(args.workload, rows, steps=args.steps, warmup=min(args.warmup, 2))
    line = {
        "impl": "reference", "metric": "gemm_tflops", "value": val, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": DTYPE_NAME[cfg["kind"]], "data": "synthetic",
        "config": {"workload": args.workload, **{k: cfg[k] for k in ("M", "K", "N") if k in cfg},
                   "note": "CPU port of the reference emulation (oracle), bounded sample"},
        "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="fp8_groupwise_llama8b_mlp", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--sets", type=int, default=4, help="rotating input sets (keeps operands out of L2)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--scaling", default="weak", choices=["weak", "strong"],
                    help="weak: every rank holds a full-size shard (default); strong: the one problem is split "
                         "across ranks (columns / experts)")
    ap.add_argument("--graph", action="store_true",
                    help="replay each step (quantise + GEMM) from a CUDA graph: removes host launch gaps, "
                         "which dominate the decode-sized workloads")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)
    if args.warmup < 3:
        args.warmup = 3

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU path)")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)

    from dsl_tool_b200 import _lib
    wl = build_workload(args.workload, rank, world, device, args.sets, strong=args.scaling == "strong")
    quant, gemm = split_step(wl)
    K_steps, W = args.steps, args.warmup

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident timing ------------------------------------------------------------
    for i in range(W):
        gemm(i, quant(i))
    _lib.check_status(device)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(4)] for _ in range(K_steps)]
    barrier()
    t_start = torch.cuda.Event(enable_timing=True)
    t_end = torch.cuda.Event(enable_timing=True)
    t_start.record()
    for i in range(K_steps):
        ev[i][0].record()
        q = quant(i)
        ev[i][1].record()
        out = gemm(i, q)
        ev[i][2].record()
    t_end.record()
    barrier()
    total_ms = t_start.elapsed_time(t_end)
    gemm_ms = statistics.mean(e[1].elapsed_time(e[2]) for e in ev)
    quant_ms = statistics.mean(e[0].elapsed_time(e[1]) for e in ev)
    graph_ms = None
    if args.graph:
        # same steps, captured once per input set and replayed: device time without host gaps
        side = torch.cuda.Stream()
        graphs = []
        with torch.cuda.stream(side):
            for i in range(args.sets):
                gemm(i, quant(i))                     # this stream's scratch exists before capture
            torch.cuda.synchronize()
            for i in range(args.sets):
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=side):
                    keep = gemm(i, quant(i))
                graphs.append((g, keep))
            for i in range(W):
                graphs[i % args.sets][0].replay()
            barrier()
            g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            g0.record()
            for i in range(K_steps):
                graphs[i % args.sets][0].replay()
            g1.record()
            barrier()
            graph_ms = g0.elapsed_time(g1) / K_steps
        total_ms = graph_ms * K_steps
    clocks = sampler.stop() if rank == 0 else None
    _lib.check_status(device)

    # ---- end to end: activations from pinned host memory, result back to the host -----------
    host_a = [torch.empty_like(wl["acts"][0], device="cpu").pin_memory() for _ in range(2)]
    for j, h in enumerate(host_a):
        h.copy_(wl["acts"][j % len(wl["acts"])])
    dev_a = torch.empty_like(wl["acts"][0])
    out_cols = wl["N"] // 2 if wl.get("act") else wl["N"]
    if wl.get("layer"):
        out_cols = wl["out_cols"]
        host_out = torch.empty((wl["out_rows"], out_cols), dtype=torch.bfloat16).pin_memory()
    elif wl.get("out") == "nvfp4":
        host_out = torch.empty((wl["M"], out_cols // 2), dtype=torch.uint8).pin_memory()
    else:
        host_out = torch.empty((wl["M"], out_cols), dtype=torch.bfloat16).pin_memory()
    e2e_steps = max(4, min(K_steps, 12))
    for i in range(2):
        dev_a.copy_(host_a[i % 2], non_blocking=True)
        host_out.copy_(wl["step"](i, dev_a), non_blocking=True)
    barrier()
    # one step at a time: copy in, compute, copy out on one stream (the latency of a single call)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(3):
        dev_a.copy_(host_a[i % 2], non_blocking=True)
        host_out.copy_(wl["step"](i, dev_a), non_blocking=True)
    e1.record()
    barrier()
    e2e_serial_ms = e0.elapsed_time(e1) / 3
    # throughput: the same steps through the library's host pipeline (copy-in of step i+1 and copy-out of
    # step i-1 overlap the compute of step i); every step's copies are inside the timed region
    from dsl_tool_b200.host_io import HostPipeline
    cell = [0]
    pipe = HostPipeline(lambda a: wl["step"](cell[0], a), device)
    host_outs = [host_out, torch.empty_like(host_out).pin_memory()]
    for i in range(3):
        cell[0] = i
        pipe.submit(host_a[i % 2], host_outs[i % 2])
    pipe.join()
    barrier()
    e0.record()
    for i in range(e2e_steps):
        cell[0] = i
        pipe.submit(host_a[i % 2], host_outs[i % 2])
    pipe.join()
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1) / e2e_steps

    # ---- aggregate over ranks (max time, summed work) ------------------------------------------
    stats = torch.tensor([total_ms, e2e_ms, wl["flops"], gemm_ms, quant_ms], dtype=torch.float64, device=device)
    if dist is not None:
        mx = stats.clone()
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        sm = stats.clone()
        dist.all_reduce(sm, op=dist.ReduceOp.SUM)
        total_ms, e2e_ms, gemm_ms, quant_ms = mx[0].item(), mx[1].item(), mx[3].item(), mx[4].item()
        flops_all = sm[2].item()
    else:
        flops_all = wl["flops"]
    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return

    ms_per_step = total_ms / K_steps
    value = flops_all / (ms_per_step * 1e-3) / 1e12
    bf16_peak, hbm_peak, basis = measured_peaks()
    kind = wl["kind"]
    achieved = wl["flops"] / (gemm_ms * 1e-3) / 1e12
    peak = bf16_peak * PEAK_MULT[kind]
    decode = wl["M"] <= 128 and not wl["moe"]
    if decode and kind in ("nvfp4", "mxfp4"):
        # weight streaming: the step is bound by HBM; algorithmic bytes = operands + scales + output, each once
        sfdiv = 16 if kind == "nvfp4" else 32
        step_bytes = (wl["M"] + wl["N"]) * wl["K"] * (0.5 + 1.0 / sfdiv) + 2.0 * wl["M"] * wl["N"] + 2.0 * wl["M"] * wl["K"]
        hbm = {"bound": "hbm", "achieved": step_bytes / (ms_per_step * 1e-3) / 1e9, "peak": hbm_peak, "unit": "GB/s",
               "frac": step_bytes / (ms_per_step * 1e-3) / 1e9 / hbm_peak, "traffic": NCU_TRAFFIC.get(args.workload),
               "kernel": "activation quantise + weight-streaming gemm (whole step)", "bytes_per_step": step_bytes,
               "peak_basis": f"{basis} HBM copy {hbm_peak} GB/s"}
    else:
        hbm = None
    line = {
        "metric": "gemm_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": K_steps, "warmup": W,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None,
        "dtype": DTYPE_NAME[kind], "data": "synthetic",
        "config": {"workload": args.workload, "M": wl["M"], "K": wl["K"], "N": wl["N"],
                   "out": ("bf16" if not wl.get("act") else "bf16 [M, N/2] = silu(gate) * up, folded in the GEMM epilogue")
                   if not wl.get("out") else "NVFP4 [M, N/2] = quantise(silu(gate) * up), both folded in the GEMM epilogue",
                   "moe": wl["moe"], "per_rank": ("own weight shard / experts of this size, no collective" if args.scaling == "weak" else
                                "this rank's column range / experts of the one problem, no collective"),
                   "step": "activation quantise + GEMM, weights quantised once",
                   "l2": f"inputs rotate over {args.sets} sets (larger than the 126 MB L2)"},
        "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                     "frac": achieved / peak, "traffic": NCU_TRAFFIC.get(args.workload),
                     "kernel": "gemm", "kernel_ms": gemm_ms, "quant_kernel_ms": quant_ms,
                     "peak_basis": f"{PEAK_MULT[kind]:g} x {basis} bf16 burst {bf16_peak} TFLOP/s"},
        "e2e": {"value": flops_all / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
                "h2d_bytes_per_step": wl["acts"][0].numel() * 2, "d2h_bytes_per_step": host_out.numel() * host_out.element_size(),
                "ms_per_step": e2e_ms, "single_step_ms": e2e_serial_ms,
                "how": "HostPipeline: pinned host buffers, copy-in / compute / copy-out on three streams, two staging buffers"},
        # kernels of this library per step: quantiser passes + one GEMM kernel (NVFP4 tensors of up to
        # 2^18 elements are quantised by a single launch, larger ones by an amax pass + a quantise pass)
        "gpu_launches": K_steps * 9 if wl.get("layer") else K_steps * 7 if wl.get("split") else K_steps * ({"fp8": 3, "fp8_block128": 2, "mxfp4": 2, "bf16": 1,
                                    "nvfp4": 2 if (not wl["moe"] and wl["M"] * wl["K"] <= (256 << 10)) else 3}[kind]),
        "cuda_graph": bool(args.graph),
        "clocks": clocks,
    }
    if hbm is not None:
        line["roofline_tensor"] = line["roofline"]
        line["roofline"] = hbm
    if not args.no_cpu_baseline and world == 1:
        rows = 512
        val, cores, dt, sample = cpu_baseline(args.workload, rows)
        line["cpu_baseline"] = {"value": val, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample,
                                "seconds": dt}
    print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
