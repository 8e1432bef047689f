"""Benchmark of the quantised-GEMM hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl ours|reference]
                    [--scaling strong|weak] [--no-sweep] [--min-seconds S] [--graph]

One "step" = one pass of the hot path over one batch of synthetic input: quantise / scale-pack
the activations and run the GEMM against weights that were quantised once, through the library's
public callable (`linear`).  The default workload is the FP8 groupwise GEMM at the Llama-3-8B MLP
shape (M=4096, K=4096, N=14336; 1x128 activation scales, 128x128 weight-block scales, bf16
output).  Inputs are seeded synthetic tensors of the stated shapes and distributions.

Prints ONE JSON line (rank 0).
  * `value`: aggregate TFLOP/s over all ranks with inputs resident in HBM.  K steps are timed between
    two barriers with CUDA events, and that K-step block is repeated until the timed region lasts at
    least `--min-seconds` (default 1 s), so that the figure is taken at the clocks the part sustains;
    `ms_per_step` is the median block, `burst` the first one.
  * `roofline`: the GEMM kernel alone, from its own pair of events in a K-step pass that follows the
    timed blocks without a pause.
  * `e2e`: the same metric through the public callable with the activations in pinned host memory
    (host->device copy of the activations and device->host copy of the result inside the timed region).
  * `sweep`: one short record per further configuration (decode shapes replayed as CUDA graphs).
  * `cpu_baseline`: the reference's own CPU emulation (a copy made by `make -C oracle ref_py`) on a
    bounded slab of the workload, the numpy restatement beside it.
With N > 1 the ONE problem is split across the ranks (`--scaling strong`, the default): 128-aligned
column ranges of the weight for the dense GEMMs, contiguous expert ranges for the MoE GEMMs, no
data-path collective.  `--scaling weak` gives every rank a full-size shard instead.
"""
from __future__ import annotations

import argparse
import importlib.util
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
    "fp8_groupwise_llama8b_mlp": dict(kind="fp8_block128", M=4096, K=4096, N=14336, wstd=0.02, outliers=False),
    "fp8_groupwise_m1024": dict(kind="fp8_block128", M=1024, K=4096, N=14336, wstd=0.02, outliers=False),
    "fp8_per_tensor_1024": dict(kind="fp8", M=1024, K=1024, N=1024, wstd=1.0, outliers=False),
    "fp8_groupwise_8192": dict(kind="fp8_block128", M=8192, K=8192, N=8192, wstd=0.02, outliers=False),
    "nvfp4_8192": dict(kind="nvfp4", M=8192, K=8192, N=8192, wstd=0.02, outliers=True),
    # the same with a calibrated (static) global scale of the activations: the quantiser is one pass over them
    "nvfp4_8192_static_scale": dict(kind="nvfp4", M=8192, K=8192, N=8192, wstd=0.02, outliers=True, act_gs=20.0 / 2688.0),
    # ... and with one dynamic global scale per token (row): also one pass, no calibration needed
    "nvfp4_8192_token_scale": dict(kind="nvfp4", M=8192, K=8192, N=8192, wstd=0.02, outliers=True, act_gs="per_token"),
    "nvfp4_m1024": dict(kind="nvfp4", M=1024, K=8192, N=8192, wstd=0.02, outliers=True),
    "nvfp4_m128": dict(kind="nvfp4", M=128, K=8192, N=8192, wstd=0.02, outliers=True),
    "nvfp4_m16": dict(kind="nvfp4", M=16, K=8192, N=8192, wstd=0.02, outliers=True),
    "nvfp4_m1": dict(kind="nvfp4", M=1, K=8192, N=8192, wstd=0.02, outliers=True),
    "mxfp4_llama70b_up": dict(kind="mxfp4", M=8192, K=8192, N=28672, wstd=0.015, outliers=False),
    "mxfp4_llama70b_down": dict(kind="mxfp4", M=8192, K=28672, N=8192, wstd=0.015, outliers=False),
    # the up projection with the full result wanted on every rank: one NCCL all-gather of the column shards per step
    "mxfp4_llama70b_up_gather": dict(kind="mxfp4", M=8192, K=8192, N=28672, wstd=0.015, outliers=False, gather=True),
    "moe_nvfp4": dict(kind="nvfp4", moe=True, tokens=16384, topk=8, experts=64, K=4096, N=3072, wstd=0.02),
    # expert-sorted rows quantised with per-token global scales (one pass over the 1.07 GB of routed rows)
    "moe_nvfp4_token_scale": dict(kind="nvfp4", moe=True, tokens=16384, topk=8, experts=64, K=4096, N=3072, wstd=0.02,
                                  act_gs="per_token"),
    # the same layer under skewed routing: per-expert logit bias N(0, 0.6), one expert nobody is routed to
    "moe_nvfp4_skewed": dict(kind="nvfp4", moe=True, tokens=16384, topk=8, experts=64, K=4096, N=3072, wstd=0.02, skew=0.6),
    "moe_fp8_groupwise": dict(kind="fp8_block128", moe=True, tokens=16384, topk=8, experts=64, K=4096, N=3072, wstd=0.02),
    "moe_nvfp4_swiglu": dict(kind="nvfp4", moe=True, tokens=16384, topk=8, experts=64, K=4096, N=3072, wstd=0.02, act="swiglu"),
    "moe_nvfp4_swiglu_nvfp4out": dict(kind="nvfp4", moe=True, tokens=16384, topk=8, experts=64, K=4096, N=3072, wstd=0.02,
                                      act="swiglu", out="nvfp4"),
    "moe_fp8_groupwise_swiglu": dict(kind="fp8_block128", moe=True, tokens=16384, topk=8, experts=64, K=4096, N=3072, wstd=0.02,
                                     act="swiglu"),
    # the MoE GEMM fed the way a layer feeds it: 16384 token rows + their routing; the tokens are quantised ONCE and the
    # packed rows dispatched to expert-sorted order (step = plan + quantise + dispatch + grouped GEMM)
    "moe_nvfp4_tokens": dict(kind="nvfp4", tokens_in=True, tokens=16384, topk=8, experts=64, K=4096, N=3072, wstd=0.02),
    "moe_fp8_groupwise_tokens": dict(kind="fp8_block128", tokens_in=True, tokens=16384, topk=8, experts=64, K=4096, N=3072, wstd=0.02),
    # the whole MoE feed-forward layer around the two grouped GEMMs (router, plan, quantise once, dispatch,
    # gate/up GEMM with SwiGLU and NVFP4 result, down GEMM, combine); 0.01 = calibrated hidden global scale
    "moe_layer_nvfp4": dict(kind="nvfp4", layer=True, tokens=16384, topk=8, experts=64, K=4096, H=1536, D=4096, wstd=0.02,
                            hidden_gs=0.01),
    # the same layer with the tokens split over the ranks and a token all-to-all either side of the expert GEMMs
    "moe_layer_nvfp4_a2a": dict(kind="nvfp4", layer=True, tokens=16384, topk=8, experts=64, K=4096, H=1536, D=4096, wstd=0.02,
                                hidden_gs=0.01, a2a=True),
    # the replicated-routing layer in 2 pipelined pieces: each piece's reduce-scatter overlaps the next piece's GEMMs
    # (measured slower than the unchunked layer on 2 and 4 GPUs, so it is not part of the sweep; --workload runs it)
    "moe_layer_nvfp4_overlap": dict(kind="nvfp4", layer=True, tokens=16384, topk=8, experts=64, K=4096, H=1536, D=4096, wstd=0.02,
                                    hidden_gs=0.01, chunks=2),
    # the replicated-routing layer whose shares are summed by the library's own kernel over peer memory (symmetric
    # memory, plain NVLink loads) instead of NCCL's reduce-scatter
    "moe_layer_nvfp4_pull": dict(kind="nvfp4", layer=True, tokens=16384, topk=8, experts=64, K=4096, H=1536, D=4096, wstd=0.02,
                                 hidden_gs=0.01, pull=True),
    "bf16_8192": dict(kind="bf16", M=8192, K=8192, N=8192, wstd=0.02, outliers=False),
}
DEFAULT_WORKLOAD = "fp8_groupwise_llama8b_mlp"
# further configurations reported in `sweep` (one GPU) ...
SWEEP_1GPU = ["fp8_per_tensor_1024", "fp8_groupwise_8192", "nvfp4_8192", "nvfp4_8192_static_scale", "nvfp4_8192_token_scale", "nvfp4_m1", "nvfp4_m16", "nvfp4_m128", "nvfp4_m1024",
              "mxfp4_llama70b_up", "mxfp4_llama70b_down", "moe_nvfp4", "moe_nvfp4_token_scale", "moe_nvfp4_tokens", "moe_nvfp4_skewed",
              "moe_fp8_groupwise", "moe_fp8_groupwise_tokens", "moe_layer_nvfp4"]
# ... and the sharded ones when the problem is split over several GPUs
SWEEP_SHARDED = ["mxfp4_llama70b_up", "mxfp4_llama70b_up_gather", "mxfp4_llama70b_down", "moe_nvfp4", "moe_fp8_groupwise",
                 "moe_layer_nvfp4", "moe_layer_nvfp4_pull", "moe_layer_nvfp4_a2a"]
DTYPE_NAME = {"fp8": "fp8_e4m3", "fp8_block128": "fp8_e4m3", "nvfp4": "fp4_e2m1", "mxfp4": "fp4_e2m1", "bf16": "bf16"}
# dram__bytes_read.sum + dram__bytes_write.sum of the GEMM kernel per launch, from ncu captures of the
# full-size workloads: bytes.  None where no capture exists.
NCU_TRAFFIC = {"fp8_groupwise_llama8b_mlp": 77.1e6 + 74.9e6,
               "nvfp4_8192": 164.5e6 + 105.9e6,
               "nvfp4_m16": 37.93e6 + 0.28e6}      # decode: GEMM + quantiser launch (whole step)
PEAK_MULT = {"fp8": 2.0, "fp8_block128": 2.0, "nvfp4": 4.0, "mxfp4": 4.0, "bf16": 1.0}
STATED_PEAK = {"fp8": 4500.0, "fp8_block128": 4500.0, "nvfp4": 9000.0, "mxfp4": 9000.0, "bf16": 2250.0}   # dense TFLOP/s
STATED_HBM = 8000.0                                                                                      # GB/s


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return p["bf16_tflops"], p.get("bf16_tflops_sustained"), p["hbm_gbs"], "measured"
    return 1590.0, 1400.0, 6650.0, "fallback"


class ClockSampler:
    """Samples nvidia-smi clocks, power and throttle reasons while a timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap,power.draw")

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
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def mark(self) -> int:
        return len(self.rows)

    def summary(self, first: int = 0, last=None):
        rows = self.rows[first:last]
        num = lambda s: s.replace(".", "", 1).isdigit()
        sm = [float(r[0]) for r in rows if len(r) >= 7 and num(r[0])]
        mx = [float(r[1]) for r in rows if len(r) >= 7 and num(r[1])]
        pw = [float(r[6]) for r in rows if len(r) >= 7 and num(r[6])]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) >= 7 and r[2 + i] == "Active" for r in rows)]
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm), "power_w_max": max(pw) if pw else None}

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.1)
        self.proc.terminate()
        return self.summary()


def make_moe_offsets(rng, tokens, experts, topk, skew=0.0):
    logits = rng.standard_normal((tokens, experts)).astype(np.float32)
    if skew > 0:
        bias = (rng.standard_normal(experts) * skew).astype(np.float32)
        bias[5 % experts] = -1e9                      # an expert without rows
        logits += bias[None, :]
    top = np.argpartition(-logits, topk - 1, axis=1)[:, :topk]
    counts = np.bincount(top.reshape(-1), minlength=experts)
    return np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)


def workload_config(name, scaling, sets):
    """The `config` object of the JSON line: identical in both arms (--impl ours / reference)."""
    cfg = WORKLOADS[name]
    out = {"workload": name, "format": cfg["kind"]}
    if cfg.get("moe") or cfg.get("tokens_in") or cfg.get("layer"):
        out.update(M=cfg["tokens"] * cfg["topk"], K=cfg["K"], N=cfg.get("N", 2 * cfg.get("H", 0)), experts=cfg["experts"],
                   tokens=cfg["tokens"], topk=cfg["topk"], moe=True)
    else:
        out.update(M=cfg["M"], K=cfg["K"], N=cfg["N"], moe=False)
    out["out"] = ("NVFP4 [M, N/2] = quantise(silu(gate) * up), both folded in the GEMM epilogue" if cfg.get("out") == "nvfp4"
                  else "bf16 [M, N/2] = silu(gate) * up, folded in the GEMM epilogue" if cfg.get("act") else "bf16")
    out["step"] = "activation quantise + GEMM, weights quantised once"
    out["scaling"] = ("one problem split across the ranks (column ranges / expert ranges), no collective" if scaling == "strong"
                      else "every rank holds a full-size shard, no collective")
    out["l2"] = f"inputs rotate over {sets} sets (larger than the 126 MB L2)"
    return out


def build_workload(name, rank, world, device, sets, strong=False):
    """Returns dict(step=callable(i)->out, ...) with `sets` rotating copies of the inputs so that
    consecutive steps never reuse L2-resident operands."""
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
            glob = make_moe_offsets(np.random.default_rng(99), cfg["tokens"], experts, cfg["topk"], cfg.get("skew", 0.0))
            first, last = expert_ranges(experts, world)[rank]
            _, _, loc = local_rows(glob, first, last)
            offs_np = np.asarray(loc, dtype=np.int32)
            experts = last - first
        else:
            offs_np = make_moe_offsets(np.random.default_rng(99 + rank), cfg["tokens"], experts, cfg["topk"], cfg.get("skew", 0.0))
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
        # strong scaling: the activations of the one problem are the same on every rank
        ga = torch.Generator(device=device).manual_seed(4321 + s) if (strong and not cfg.get("moe")) else g
        a = torch.randn((M, K), generator=ga, device=device, dtype=torch.float32)
        if cfg.get("outliers"):
            mask = torch.rand((M, K), generator=ga, device=device) < 1e-3
            sign = torch.where(torch.rand((M, K), generator=ga, device=device) < 0.5, -20.0, 20.0)
            a = torch.where(mask, sign, a)
        acts.append(a.to(torch.bfloat16))
        del a
        w = (torch.randn(wshape, generator=g, device=device, dtype=torch.float32) * cfg["wstd"]).to(torch.bfloat16)
        wts.append(pack_weight(w, kind, layout="nk", gate_up_interleave=cfg.get("act") == "swiglu"))
        del w
    torch.cuda.synchronize()
    gather_ranges = None
    if cfg.get("gather") and strong and world > 1:
        from dsl_tool_b200.sharding import all_gather_columns, column_ranges
        gather_ranges = column_ranges(cfg["N"], world)

    def step(i, a=None):
        if gather_ranges is not None:
            return all_gather_columns(linear(acts[i % sets] if a is None else a, wts[i % sets], out_dtype=torch.bfloat16), gather_ranges)
        if cfg.get("out") == "nvfp4":    # result quantised in the epilogue with a fixed (calibrated) global scale
            return linear(acts[i % sets] if a is None else a, wts[i % sets], out_dtype="nvfp4", out_global_scale=1.0 / 2688.0,
                          expert_offsets=offs, activation=cfg.get("act"))[0]
        return linear(acts[i % sets] if a is None else a, wts[i % sets], out_dtype=torch.bfloat16, expert_offsets=offs,
                      activation=cfg.get("act"), act_global_scale=cfg.get("act_gs"))

    return dict(step=step, acts=acts, wts=wts, offs=offs, M=M, K=K, N=N, kind=kind, flops=2.0 * M * N * K,
                moe=bool(cfg.get("moe")), act=cfg.get("act"), out=cfg.get("out"), act_gs=cfg.get("act_gs"))


def build_layer_workload(cfg, rank, world, device, sets, strong, g):
    """Whole MoE layer.  Weak scaling: every rank owns a full set of experts and its own tokens; strong
    scaling: the experts of one layer are split over the ranks, tokens replicated, partial results reduce-scattered."""
    from dsl_tool_b200 import MoEWeights, moe_forward
    T, E, k, K, H, D = cfg["tokens"], cfg["experts"], cfg["topk"], cfg["K"], cfg["H"], cfg["D"]
    a2a = bool(cfg.get("a2a")) and strong and world > 1
    chunks = int(cfg.get("chunks", 1)) if strong and world > 1 else 1
    red = "pull" if cfg.get("pull") and strong and world > 1 else "reduce_scatter"
    mine = slice(rank * (T // world), (rank + 1) * (T // world)) if a2a else slice(0, T)
    acts, logits, wts = [], [], []
    for s in range(sets):
        gen = torch.Generator(device=device).manual_seed(77 + s + (0 if strong else 1000 * rank))
        acts.append(torch.randn((T, K), generator=gen, device=device, dtype=torch.float32).to(torch.bfloat16)[mine].contiguous())
        logits.append(torch.randn((T, E), generator=gen, device=device, dtype=torch.float32)[mine].contiguous())
        w1 = (torch.randn((E, 2 * H, K), generator=gen, device=device, dtype=torch.float32) * cfg["wstd"]).to(torch.bfloat16)
        w2 = (torch.randn((E, D, H), generator=gen, device=device, dtype=torch.float32) * cfg["wstd"]).to(torch.bfloat16)
        wts.append(MoEWeights.pack(w1, w2, cfg["kind"], rank=rank if strong else 0, world=world if strong else 1,
                                   hidden_global_scale=cfg.get("hidden_gs")))
        del w1, w2
    torch.cuda.synchronize()

    def step(i, a=None):
        if a2a:     # every rank owns T / world tokens; routed rows travel to the experts' ranks and back
            return moe_forward(acts[i % sets] if a is None else a, logits[i % sets], wts[i % sets], k, out_dtype=torch.bfloat16,
                               dispatch="all_to_all")
        # expert-parallel ranks exchange bf16 partial results and keep their own token rows (reduce-scatter)
        return moe_forward(acts[i % sets] if a is None else a, logits[i % sets], wts[i % sets], k, out_dtype=torch.bfloat16,
                           reduce=red, exchange_dtype=torch.bfloat16, chunks=chunks)

    flops = 2.0 * T * k * (2 * H * K + D * H) / (world if strong else 1)
    return dict(step=step, acts=acts, wts=wts, offs=None, M=T * k, K=K, N=2 * H, kind=cfg["kind"], flops=flops, moe=True,
                act="swiglu", out=None, layer=True, out_cols=D, out_rows=T // (world if strong else 1))


def build_token_moe_workload(cfg, rank, device, sets):
    """Grouped GEMM of an MoE layer from token-level input: x [tokens, K], ids [tokens, k] (seeded top-k routing).
    The tokens are quantised ONCE (16384 rows) and the quantised rows - packed e2m1 bytes + scale tiles, or E4M3 bytes +
    1x128 scale rows - are dispatched to expert-sorted order; the grouped GEMM consumes them as they are."""
    from dsl_tool_b200 import moe, pack_weight, quantize_fp4, quantize_fp8
    from dsl_tool_b200.gemm_kernels import gemm_fp4_quantized, gemm_fp8_groupwise_quantized
    T, E, k, K, N = cfg["tokens"], cfg["experts"], cfg["topk"], cfg["K"], cfg["N"]
    kind = cfg["kind"]
    acts, ids, wts = [], [], []
    for s in range(sets):
        gen = torch.Generator(device=device).manual_seed(55 + s + 1000 * rank)
        acts.append(torch.randn((T, K), generator=gen, device=device, dtype=torch.float32).to(torch.bfloat16))
        logits = torch.randn((T, E), generator=gen, device=device, dtype=torch.float32)
        ids.append(torch.topk(logits, k, dim=1).indices.to(torch.int32).contiguous())
        w = (torch.randn((E, N, K), generator=gen, device=device, dtype=torch.float32) * cfg["wstd"]).to(torch.bfloat16)
        wts.append(pack_weight(w, kind, layout="nk"))
        del w
    ones = torch.ones((T, k), dtype=torch.float32, device=device)
    torch.cuda.synchronize()

    def quant(i, a=None):
        p = moe.plan(ids[i % sets], ones, E)
        x = acts[i % sets] if a is None else a
        if kind == "nvfp4":
            packed, sf, gs = quantize_fp4(x, "nvfp4")
            q, s = moe.dispatch_fp4(p, packed, sf, K, "nvfp4", 0, E)
            return q, s, gs, p.offsets
        qa, sa = quantize_fp8(x, "groupwise")                  # [T, K] bytes, [T, K/128] fp32 (128-byte rows)
        return moe.dispatch_rows(p, qa, 0, E), moe.dispatch_rows(p, sa, 0, E), None, p.offsets

    def gemm(i, qs):
        w = wts[i % sets]
        if kind == "nvfp4":
            return gemm_fp4_quantized(qs[0], w.q, qs[1], w.scale, format="nvfp4", n=N, global_scale_a=qs[2],
                                      global_scale_b=w.global_scale, expert_offsets=qs[3], out_dtype=torch.bfloat16, b_static=True)
        return gemm_fp8_groupwise_quantized(qs[0], w.q, qs[1], w.scale, n=N, sb_block=True, expert_offsets=qs[3],
                                            out_dtype=torch.bfloat16)

    def step(i, a=None):
        return gemm(i, quant(i, a))

    return dict(step=step, acts=acts, wts=wts, offs=None, M=T * k, K=K, N=N, kind=kind, flops=2.0 * T * k * N * K, moe=True,
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
            return quantize_fp4(a, kind, global_scale=wl.get("act_gs"), group_offsets=offs)
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
            if wl.get("act_gs") == "per_token":
                return GK.gemm_fp4_quantized(q[0], w.q, q[1], w.scale, format=kind, token_scale=q[2],
                                             global_scale_b=w.global_scale, b_static=True, **common)
            return GK.gemm_fp4_quantized(q[0], w.q, q[1], w.scale, format=kind, global_scale_a=q[2],
                                         global_scale_b=w.global_scale, b_static=True, **common)
        return GK.gemm_bf16_raw(q[0], w.q, **common)

    return quant, gemm


# ------------------------------------------------------------------------------------------------
# CPU arm: the reference's own emulation where a copy of it was built, the numpy restatement otherwise
# ------------------------------------------------------------------------------------------------

def reference_emulation():
    """The reference's CPU-runnable tiled GEMMs (`fp8_gemm_tiled`, `grouped_gemm_tiled`), loaded from the copy
    that `make -C oracle ref_py REFERENCE_ROOT=...` places under oracle/_ref/ (never from the package)."""
    path = os.path.join(ROOT, "oracle", "_ref", "tilelang_gemm_kernels.py")
    if not os.path.exists(path):
        return None
    import contextlib
    import io
    spec = importlib.util.spec_from_file_location("reference_tilelang_gemm_kernels", path)
    mod = importlib.util.module_from_spec(spec)
    with contextlib.redirect_stdout(io.StringIO()):      # it prints "TileLang not installed" on import
        spec.loader.exec_module(mod)
    return mod


def cpu_operands(name, rows):
    """Seeded operands of the workload, quantised by the oracle: (dequantised A [rows, K], dequantised B [N, K],
    closure computing the oracle's product).  MoE workloads: one expert's rows against that expert's weight."""
    from oracle import quant_oracle as O
    cfg = WORKLOADS[name]
    kind = cfg["kind"]
    rng = np.random.default_rng(5)
    K, N = cfg["K"], cfg.get("N", 2 * cfg.get("H", 0))
    a = rng.standard_normal((rows, K)).astype(np.float32)
    w = (rng.standard_normal((N, K)) * cfg["wstd"]).astype(np.float32)
    if kind == "fp8_block128":
        qa, sa = O.quant_fp8_groupwise(a)
        qb, sbb = O.quant_fp8_block(w)
        sb = O.expand_block_scale(sbb, N)
        A = O.e4m3_decode(qa) * np.repeat(sa, 128, axis=1)[:, :K]
        B = O.e4m3_decode(qb) * np.repeat(sb.T, 128, axis=1)[:, :K]
        port = lambda: O.gemm_fp8_groupwise(qa, qb, sa, sb)
    elif kind == "fp8":
        qa, sa = O.quant_fp8_per_tensor(a)
        qb, sb = O.quant_fp8_per_tensor(w)
        A, B = O.e4m3_decode(qa) * sa, O.e4m3_decode(qb) * sb
        port = lambda: O.gemm_fp8_per_tensor(qa, qb, sa, sb)
    elif kind == "nvfp4":
        pa, sfa, gsa = O.quant_nvfp4(a)
        pb, sfb, gsb = O.quant_nvfp4(w)
        A = O.dequant_fp4_values(pa, O.e4m3_decode(sfa), 16) * gsa
        B = O.dequant_fp4_values(pb, O.e4m3_decode(sfb), 16) * gsb
        port = lambda: O.gemm_nvfp4(pa, sfa, gsa, pb, sfb, gsb)
    elif kind == "mxfp4":
        pa, sfa = O.quant_mxfp4(a)
        pb, sfb = O.quant_mxfp4(w)
        A = O.dequant_fp4_values(pa, O.e8m0_decode(sfa), 32)
        B = O.dequant_fp4_values(pb, O.e8m0_decode(sfb), 32)
        port = lambda: O.gemm_mxfp4(pa, sfa, pb, sfb)
    else:
        A, B = a, w
        port = lambda: a @ w.T
    return A.astype(np.float32), B.astype(np.float32), port


def cpu_arm(name, steps=1, warmup=0, rows_reference=64, rows_port=512, want_port=True):
    """Times the CPU arm on a bounded slab of the workload (the first rows of A against the full weight).
    Returns the `cpu_baseline` object.  kind "reference": the reference's own `fp8_gemm_tiled` (Python tile loops
    of 64 x 64 x 32 over torch CPU matmuls, all host threads) fed the oracle's dequantised operands - it is
    format-agnostic (`tile.float() @ tile.float()`); kind "port": the oracle's numpy dequantise + fp32 GEMM."""
    cfg = WORKLOADS[name]
    K, N = cfg["K"], cfg.get("N", 2 * cfg.get("H", 0))
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    ref = reference_emulation()
    out = {"unit": "TFLOP/s", "cores": cores}
    if ref is not None:
        R = rows_reference
        A, B, _ = cpu_operands(name, R)
        At, Bt = torch.from_numpy(A), torch.from_numpy(np.ascontiguousarray(B.T))        # the reference takes B [K, N]
        for _ in range(warmup):
            ref.fp8_gemm_tiled(At[:8], Bt, 1.0, 1.0)
        t0 = time.perf_counter()
        for _ in range(steps):
            ref.fp8_gemm_tiled(At, Bt, 1.0, 1.0)
        dt = (time.perf_counter() - t0) / steps
        out.update(value=2.0 * R * N * K / dt / 1e12, kind="reference", seconds=dt,
                   sample=f"reference fp8_gemm_tiled (tilelang/gemm/gemm_kernels.py:96-113), first {R} activation rows x full "
                          f"N={N}, K={K}, dequantised operands, {steps} step(s)")
    if ref is None or want_port:
        R = rows_port
        _, _, port = cpu_operands(name, R)
        for _ in range(min(warmup, 1)):
            port()
        n = steps if ref is None else 1
        t0 = time.perf_counter()
        for _ in range(n):
            port()
        dt = (time.perf_counter() - t0) / n
        val = 2.0 * R * N * K / dt / 1e12
        sample = f"numpy restatement (dequantise + fp32 GEMM), first {R} activation rows x full N={N}, K={K}"
        if ref is None:
            out.update(value=val, kind="port", seconds=dt, sample=sample)
        else:
            out["port"] = {"value": val, "unit": "TFLOP/s", "seconds": dt, "sample": sample}
    return out


def reference_cuda(name):
    """The reference's own CUDA kernel for the workload (FP8 dense workloads only), timed on this GPU through the
    driver program `oracle/_ref/ref_time_fp8`, which compiles the reference's cuda/gemm/fp8_gemm.cu unmodified.  Context
    beside the CPU arm; None where the binary was not built or the workload has no reference kernel."""
    cfg = WORKLOADS[name]
    exe = os.path.join(ROOT, "oracle", "_ref", "ref_time_fp8")
    if cfg["kind"] not in ("fp8", "fp8_block128") or cfg.get("moe") or not os.path.exists(exe):
        return None
    M, N, K = cfg["M"], cfg["N"], cfg["K"]
    try:
        out = subprocess.run([exe, str(M), str(N), str(K), "128", "1"], capture_output=True, text=True, timeout=180)
        words = out.stdout.split()
        ms = float(words[1] if cfg["kind"] == "fp8_block128" else words[3])
    except Exception as exc:
        return {"error": f"{type(exc).__name__}: {exc}"[:200]}
    kernel = ("fp8_gemm_groupwise_kernel (cuda/gemm/fp8_gemm.cu:69-99)" if cfg["kind"] == "fp8_block128"
              else "fp8_gemm_per_tensor_kernel (cuda/gemm/fp8_gemm.cu:29-65)")
    return {"value": 2.0 * M * N * K / (ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms": ms, "kernel": kernel,
            "sample": f"the reference's kernel, unmodified, one launch at the full {M} x {K} x {N} on this GPU (operands already quantised)"}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cfg = WORKLOADS[args.workload]
    steps = args.steps if args.steps is not None else 5
    warmup = args.warmup if args.warmup is not None else 1
    cb = cpu_arm(args.workload, steps=steps, warmup=min(warmup, 2), want_port=False)
    sets = args.sets
    line = {
        "impl": "reference", "metric": "gemm_tflops", "value": cb["value"], "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": steps, "warmup": warmup, "ms_per_step": cb["seconds"] * 1e3, "higher_is_better": True,
        "scaling": args.scaling, "vs_baseline": None, "dtype": DTYPE_NAME[cfg["kind"]], "data": "synthetic",
        "config": workload_config(args.workload, args.scaling, sets),
        "cpu_baseline": {k: cb[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": cb["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


# ------------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------------

class Timer:
    """Device timing of one workload: K-step blocks between barriers, repeated; max over ranks."""

    def __init__(self, dist, device, rank, world):
        self.dist, self.device, self.rank, self.world = dist, device, rank, world

    def barrier(self):
        if self.dist is not None:
            self.dist.barrier()
        torch.cuda.synchronize()

    def reduce_max(self, values):
        t = torch.tensor(values, dtype=torch.float64, device=self.device)
        if self.dist is not None:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return t.tolist()

    def gather(self, value):
        t = torch.tensor([value], dtype=torch.float64, device=self.device)
        if self.dist is None:
            return [value]
        out = [torch.zeros_like(t) for _ in range(self.world)]
        self.dist.all_gather(out, t)
        return [o.item() for o in out]

    def block(self, run_steps, K):
        """One K-step block: barrier + synchronize on both sides, CUDA events on the launching stream."""
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        self.barrier()
        e0.record()
        run_steps(K)
        e1.record()
        self.barrier()
        return e0.elapsed_time(e1)

    def blocks(self, run_steps, K, min_seconds, max_repeats=2000):
        """Repeats the K-step block until the timed region (sum of the blocks) reaches `min_seconds`.
        The number of repeats is fixed from the first block (max over ranks) so that all ranks agree.
        Returns the per-block times in ms: (max over ranks, this rank's own)."""
        mine = [self.block(run_steps, K)]
        first = self.reduce_max(mine)[0]
        repeats = int(min(max_repeats, max(0, np.ceil(min_seconds * 1e3 / max(first, 1e-3)) - 1)))
        mine += [self.block(run_steps, K) for _ in range(repeats)]
        return self.reduce_max(mine), mine


def measure(name, args, timer, sampler, K, W, min_seconds, graph, strong, sets, full):
    """Times one workload.  `full`: also the end-to-end path and per-rank detail (the headline workload)."""
    from dsl_tool_b200 import _lib
    rank, world, device = timer.rank, timer.world, timer.device
    wl = build_workload(name, rank, world, device, sets, strong=strong)
    quant, gemm = split_step(wl)
    step = wl["step"]
    decode = wl["M"] <= 128 and not wl["moe"]

    for i in range(W):
        step(i)
    _lib.check_status(device)

    def run_eager(n):
        for i in range(n):
            step(i)

    runner = run_eager
    graphs = None
    steps_per_graph = None
    if graph:
        # the same steps captured eight at a time (over the rotating input sets) and replayed: device time without host
        # launch gaps, and without charging every 17-us step a whole graph launch of its own - a decode step never runs
        # as a graph by itself, it is one of the many small GEMMs of a layer stack
        steps_per_graph = 8 if K >= 8 else K
        K = max(steps_per_graph, K // steps_per_graph * steps_per_graph)
        side = torch.cuda.Stream()
        with torch.cuda.stream(side):
            for i in range(sets):
                step(i)                               # this stream's scratch exists before capture
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            keep = []
            with torch.cuda.graph(g, stream=side):
                for i in range(steps_per_graph):
                    keep.append(step(i))
            graphs = [(g, keep)]
            for i in range(max(1, W // steps_per_graph)):
                g.replay()
            torch.cuda.synchronize()

        def run_graph(n):
            side.wait_stream(torch.cuda.current_stream())      # the block's start event comes first
            with torch.cuda.stream(side):
                for i in range(n // steps_per_graph):
                    graphs[0][0].replay()
            torch.cuda.current_stream().wait_stream(side)
        runner = run_graph

    # the kernels alone: same steps with an event between quantise and GEMM - once before the timed blocks
    # (the part is cool: burst clocks) and once straight after them (the clocks the part sustains)
    kk = min(K, 50)

    def kernel_pass():
        ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(kk)]
        for i in range(kk):
            ev[i][0].record()
            q = quant(i)
            ev[i][1].record()
            gemm(i, q)
            ev[i][2].record()
        torch.cuda.synchronize()
        return (statistics.mean(e[1].elapsed_time(e[2]) for e in ev), statistics.mean(e[0].elapsed_time(e[1]) for e in ev))

    gemm_ms_burst, _ = kernel_pass() if full else (None, None)
    mark0 = sampler.mark() if sampler is not None else 0
    times, mine = timer.blocks(runner, K, min_seconds)
    eager_ms = None
    if graph:       # the same steps launched one by one from the host (what a caller without a graph gets)
        eager_ms = timer.reduce_max([timer.block(run_eager, K)])[0] / K
    gemm_ms, quant_ms = kernel_pass()
    mark1 = sampler.mark() if sampler is not None else 0
    _lib.check_status(device)

    ms_blocks = [t / K for t in times]
    ms_med = statistics.median(ms_blocks)
    gemm_ms_max, quant_ms_max = timer.reduce_max([gemm_ms, quant_ms])
    flops_all = sum(timer.gather(wl["flops"]))
    per_rank_ms = timer.gather(statistics.median(t / K for t in mine))
    per_rank_gemm, per_rank_quant = timer.gather(gemm_ms), timer.gather(quant_ms)

    bf16_peak, bf16_sus, hbm_peak, basis = measured_peaks()
    kind = wl["kind"]
    rec = {
        "workload": name, "format": kind, "M": wl["M"], "K": wl["K"], "N": wl["N"],
        "value": flops_all / (ms_med * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms_med,
        "burst": {"value": flops_all / (ms_blocks[0] * 1e-3) / 1e12, "ms_per_step": ms_blocks[0]},
        "repeats": len(ms_blocks), "steps": K, "timed_region_s": sum(times) / 1e3,
        "ms_per_step_min_median_max": [min(ms_blocks), ms_med, max(ms_blocks)],
        "kernel_ms": gemm_ms_max, "quant_kernel_ms": quant_ms_max, "cuda_graph": bool(graph), "steps_per_graph": steps_per_graph,
        "host_gap_ms": max(0.0, ms_med - gemm_ms_max - quant_ms_max),
    }
    if eager_ms is not None:
        rec["eager_ms_per_step"] = eager_ms
    achieved = wl["flops"] / (gemm_ms * 1e-3) / 1e12
    # The kernel is timed inside a region of a second or more (sustained clocks, usually at the power cap), so the
    # denominator is the cuBLAS bf16 rate measured the same way; the headline workload also carries the pair
    # "timed cool / burst peak".  Sweep entries run a quarter of a second each: they are compared with the burst peak.
    sustained = full and bool(bf16_sus) and sum(times) >= 900.0
    base = bf16_sus if sustained else bf16_peak
    peak = base * PEAK_MULT[kind]
    tensor = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
              "frac_of_stated_peak": achieved / STATED_PEAK[kind], "traffic": NCU_TRAFFIC.get(name), "kernel": "gemm",
              "kernel_ms": gemm_ms, "quant_kernel_ms": quant_ms,
              "peak_basis": f"{PEAK_MULT[kind]:g} x {basis} bf16 {'sustained' if sustained else 'burst'} {base} TFLOP/s"}
    if not sustained and bf16_sus:
        # a sweep entry runs on a part the headline has already heated (see its `clocks`): beside the conservative
        # fraction against the burst rate, the same figure against what cuBLAS bf16 sustains at the power cap
        tensor["vs_sustained"] = {"peak": bf16_sus * PEAK_MULT[kind], "frac": achieved / (bf16_sus * PEAK_MULT[kind]),
                                  "peak_basis": f"{PEAK_MULT[kind]:g} x {basis} bf16 sustained {bf16_sus} TFLOP/s"}
    if gemm_ms_burst:
        ab = wl["flops"] / (gemm_ms_burst * 1e-3) / 1e12
        tensor["burst"] = {"achieved": ab, "peak": bf16_peak * PEAK_MULT[kind], "frac": ab / (bf16_peak * PEAK_MULT[kind]),
                           "kernel_ms": gemm_ms_burst, "peak_basis": f"{PEAK_MULT[kind]:g} x {basis} bf16 burst {bf16_peak} TFLOP/s"}
    if decode and kind in ("nvfp4", "mxfp4"):
        # weight streaming: the step is bound by HBM; algorithmic bytes = operands + scales + output, each once
        sfdiv = 16 if kind == "nvfp4" else 32
        step_bytes = (wl["M"] + wl["N"]) * wl["K"] * (0.5 + 1.0 / sfdiv) + 2.0 * wl["M"] * wl["N"] + 2.0 * wl["M"] * wl["K"]
        gbs = step_bytes / (ms_med * 1e-3) / 1e9
        rec["roofline"] = {"bound": "hbm", "achieved": gbs, "peak": hbm_peak, "unit": "GB/s", "frac": gbs / hbm_peak,
                           "frac_of_stated_peak": gbs / STATED_HBM, "traffic": NCU_TRAFFIC.get(name),
                           "kernel": "activation quantise + weight-streaming gemm (whole step)", "bytes_per_step": step_bytes,
                           "peak_basis": f"{basis} HBM copy {hbm_peak} GB/s"}
        rec["roofline_tensor"] = tensor
    else:
        rec["roofline"] = tensor
    if sampler is not None:
        rec["clocks"] = sampler.summary(mark0, mark1)
    if world > 1:
        rec["per_rank"] = {"ms_per_step": per_rank_ms, "gemm_ms": per_rank_gemm, "quant_ms": per_rank_quant,
                           "host_gap_ms": [max(0.0, a - b - c) for a, b, c in zip(per_rank_ms, per_rank_gemm, per_rank_quant)]}
    if wl.get("layer"):
        launches = 9
    elif wl.get("split"):
        launches = 7
    else:
        launches = {"fp8": 3, "fp8_block128": 2, "mxfp4": 2, "bf16": 1,
                    "nvfp4": 2 if (not wl["moe"] and wl["M"] * wl["K"] <= (256 << 10)) else 3}[kind]
    rec["launches_per_step"] = launches
    rec["gpu_launches"] = launches * (K * len(ms_blocks) + kk * (2 if full else 1))
    if full:
        rec["_wl"] = wl
        rec["_flops_all"] = flops_all
    else:
        del wl, graphs
        torch.cuda.empty_cache()
    return rec


def measure_e2e(wl, timer, K_steps):
    """The step through the public callable with host buffers: H2D of the activations and D2H of the result inside
    the timed region, pipelined by HostPipeline; plus one step at a time (latency of a single call)."""
    from dsl_tool_b200.host_io import HostPipeline
    device = timer.device
    host_a = [torch.empty_like(wl["acts"][0], device="cpu").pin_memory() for _ in range(2)]
    for j, h in enumerate(host_a):
        h.copy_(wl["acts"][j % len(wl["acts"])])
    dev_a = torch.empty_like(wl["acts"][0])
    out_cols = wl["N"] // 2 if wl.get("act") else wl["N"]
    if wl.get("layer"):
        host_out = torch.empty((wl["out_rows"], wl["out_cols"]), dtype=torch.bfloat16).pin_memory()
    elif wl.get("out") == "nvfp4":
        host_out = torch.empty((wl["M"], out_cols // 2), dtype=torch.uint8).pin_memory()
    else:
        host_out = torch.empty((wl["M"], out_cols), dtype=torch.bfloat16).pin_memory()
    e2e_steps = max(4, min(K_steps, 12))
    for i in range(2):
        dev_a.copy_(host_a[i % 2], non_blocking=True)
        host_out.copy_(wl["step"](i, dev_a), non_blocking=True)
    timer.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(3):
        dev_a.copy_(host_a[i % 2], non_blocking=True)
        host_out.copy_(wl["step"](i, dev_a), non_blocking=True)
    e1.record()
    timer.barrier()
    serial_ms = e0.elapsed_time(e1) / 3
    cell = [0]
    pipe = HostPipeline(lambda a: wl["step"](cell[0], a), device)
    host_outs = [host_out, torch.empty_like(host_out).pin_memory()]
    for i in range(3):
        cell[0] = i
        pipe.submit(host_a[i % 2], host_outs[i % 2])
    pipe.join()
    timer.barrier()
    e0.record()
    for i in range(e2e_steps):
        cell[0] = i
        pipe.submit(host_a[i % 2], host_outs[i % 2])
    pipe.join()
    e1.record()
    timer.barrier()
    e2e_ms = timer.reduce_max([e0.elapsed_time(e1) / e2e_steps])[0]
    # the host link alone: this step's result copied device -> pinned host and its input host -> device, all ranks at once
    # (the ceiling the end-to-end figure can reach however fast the kernels are)
    dev_out = torch.empty(host_out.shape, dtype=host_out.dtype, device=device)
    timer.barrier()
    e0.record()
    for _ in range(3):
        host_out.copy_(dev_out, non_blocking=True)
    e1.record()
    timer.barrier()
    d2h_ms = timer.reduce_max([e0.elapsed_time(e1) / 3])[0]
    e0.record()
    for _ in range(3):
        dev_a.copy_(host_a[0], non_blocking=True)
    e1.record()
    timer.barrier()
    h2d_ms = timer.reduce_max([e0.elapsed_time(e1) / 3])[0]
    link = {"d2h_gbs_per_rank": host_out.numel() * host_out.element_size() / (d2h_ms * 1e-3) / 1e9,
            "h2d_gbs_per_rank": wl["acts"][0].numel() * 2 / (h2d_ms * 1e-3) / 1e9, "d2h_ms": d2h_ms, "h2d_ms": h2d_ms}
    return e2e_ms, serial_ms, wl["acts"][0].numel() * 2, host_out.numel() * host_out.element_size(), link


def host_cost_us(wl, n=200):
    """Host time of one call of the public callable with the stream left to drain first (time.perf_counter
    around the call; nothing waits for the GPU inside)."""
    step = wl["step"]
    for i in range(5):
        step(i)
    torch.cuda.synchronize()
    best = []
    for _ in range(3):
        t0 = time.perf_counter()
        for i in range(n):
            step(i)
        best.append((time.perf_counter() - t0) / n * 1e6)
        torch.cuda.synchronize()
    return min(best)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None, help="steps per timed block (default 50; reference arm 5)")
    ap.add_argument("--warmup", type=int, default=None, help="untimed warm-up steps (default 5, at least 3)")
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--sets", type=int, default=4, help="rotating input sets (keeps operands out of L2)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-sweep", action="store_true", help="only the headline workload")
    ap.add_argument("--sweep-limit", type=float, default=420.0,
                    help="seconds after which the line is printed with the sweep entries measured so far")
    ap.add_argument("--min-seconds", type=float, default=1.0, help="the K-step block is repeated until the timed region is this long")
    ap.add_argument("--scaling", default="strong", choices=["weak", "strong"],
                    help="strong (default): the one problem is split across the ranks (columns / experts); "
                         "weak: every rank holds a full-size shard")
    ap.add_argument("--graph", action="store_true",
                    help="replay each step (quantise + GEMM) from a CUDA graph: removes host launch gaps, "
                         "which dominate the decode-sized workloads")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)
    K_steps = args.steps if args.steps is not None else 50
    W = max(3, args.warmup if args.warmup is not None else 5)

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
    timer = Timer(dist, device, rank, world)
    strong = args.scaling == "strong"
    sampler = ClockSampler(local).start() if rank == 0 else None

    cfg0 = WORKLOADS[args.workload]
    decode0 = (not cfg0.get("moe")) and cfg0.get("M", 1 << 30) <= 128
    head = measure(args.workload, args, timer, sampler, K_steps, W, args.min_seconds, args.graph or False, strong, args.sets, True)
    wl = head.pop("_wl")
    flops_all = head.pop("_flops_all")
    clocks = head.pop("clocks", None)
    e2e_ms, serial_ms, h2d, d2h, link = measure_e2e(wl, timer, K_steps)
    host_us = host_cost_us(wl) if not wl.get("layer") else None
    del wl
    torch.cuda.empty_cache()

    # The headline line is complete here; the sweep only adds to it.  A watchdog guarantees that the line is printed
    # (and every rank exits) even if a sweep entry fails on one rank and leaves the others waiting in a collective.
    line = None
    if rank == 0:
        line = {
            "metric": "gemm_tflops", "value": head["value"], "unit": "TFLOP/s", "n_gpus": world, "steps": K_steps, "warmup": W,
            "ms_per_step": head["ms_per_step"], "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None,
            "dtype": DTYPE_NAME[head["format"]], "data": "synthetic",
            "config": workload_config(args.workload, args.scaling, args.sets),
            "repeats": head["repeats"], "timed_region_s": head["timed_region_s"],
            "ms_per_step_min_median_max": head["ms_per_step_min_median_max"], "burst": head["burst"],
            "roofline": head["roofline"],
            "e2e": {"value": flops_all / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms, "single_step_ms": serial_ms, "host_link_alone": link,
                    "how": "HostPipeline: pinned host buffers, copy-in / compute / copy-out on three streams, two staging buffers"},
            "host_us_per_call": host_us,
            "gpu_launches": head["gpu_launches"], "launches_per_step": head["launches_per_step"],
            "cuda_graph": bool(args.graph), "steps_per_graph": head.get("steps_per_graph"),
            "clocks": clocks if clocks is not None else (sampler.summary() if sampler is not None else None),
        }
        if "roofline_tensor" in head:
            line["roofline_tensor"] = head["roofline_tensor"]
        if "per_rank" in head:
            line["per_rank"] = head["per_rank"]
            line["kernel_ms"], line["quant_kernel_ms"], line["host_gap_ms"] = head["kernel_ms"], head["quant_kernel_ms"], head["host_gap_ms"]
        if not args.no_cpu_baseline and world == 1:
            line["cpu_baseline"] = cpu_arm(args.workload, steps=1, warmup=1)
            rc = reference_cuda(args.workload)
            if rc is not None:
                line["reference_cuda"] = rc

    sweep = []
    printed = threading.Lock()

    def give_up():
        if printed.acquire(blocking=False):
            if line is not None:
                line["sweep"] = sweep
                line["sweep_error"] = f"the sweep did not finish within {args.sweep_limit:.0f} s; entries measured so far are kept"
                print(json.dumps(line), flush=True)
            os._exit(0)

    if not args.no_sweep and args.workload == DEFAULT_WORKLOAD:
        watchdog = threading.Timer(args.sweep_limit, give_up)
        watchdog.daemon = True
        watchdog.start()
        names = SWEEP_1GPU if world == 1 else SWEEP_SHARDED
        for name in names:
            c = WORKLOADS[name]
            is_decode = (not c.get("moe")) and not c.get("tokens_in") and not c.get("layer") and c.get("M", 1 << 30) <= 128
            big = c.get("moe") or c.get("tokens_in") or c.get("layer") or c.get("K", 0) * c.get("N", 0) >= (1 << 27)
            try:
                rec = measure(name, args, timer, sampler, min(K_steps, 20 if big else 50), 3, 0.25, is_decode, strong,
                              2 if big else args.sets, False)
            except Exception as exc:     # a sweep entry must not take the headline down with it
                rec = {"workload": name, "error": f"{type(exc).__name__}: {exc}"}
            sweep.append(rec)
        watchdog.cancel()
    if not printed.acquire(blocking=False):
        return                                    # the watchdog is printing / has printed
    if sampler is not None:
        sampler.stop()
    if rank == 0:
        if sweep:
            line["sweep"] = sweep
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
