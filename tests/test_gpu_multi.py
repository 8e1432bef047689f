"""Column-parallel / expert-parallel split on real GPUs with the CUDA kernels and an NCCL gather.
Runs as child processes, one per GPU; skipped with fewer than two GPUs."""
import os
import socket
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

WORKER = r'''
import os, sys
import numpy as np, torch, torch.distributed as dist
sys.path.insert(0, os.environ["REPO_ROOT"])
from dsl_tool_b200 import linear, pack_weight
from dsl_tool_b200.sharding import ColumnParallelLinear, ExpertParallelGroupedLinear, shard_weight_columns, shard_weight_experts
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
g = torch.Generator(device="cuda").manual_seed(0)
x = torch.randn(300, 512, generator=g, device="cuda").bfloat16()
w = (torch.randn(1024, 512, generator=g, device="cuda") * 0.02).bfloat16()
ok = True
for fmt in ("nvfp4", "fp8_block128"):
    full = linear(x, pack_weight(w, fmt), out_dtype="float32")
    gs = w.float().abs().amax() / 2688.0 if fmt == "nvfp4" else None     # the whole weight's global scale
    lin = ColumnParallelLinear(pack_weight(shard_weight_columns(w, rank, world).contiguous(), fmt, global_scale=gs), 1024, linear)
    y = lin.forward(x, gather=True, out_dtype="float32")
    err = float((y - full).norm() / full.norm())
    print(rank, fmt, "column-parallel relF", err, tuple(y.shape), flush=True)
    ok &= err < 1e-6
G = 4
wg = (torch.randn(G, 256, 512, generator=g, device="cuda") * 0.02).bfloat16()
offs = [0, 100, 100, 180, 300]
full = linear(x, pack_weight(wg, "mxfp4"), expert_offsets=torch.tensor(offs, dtype=torch.int32, device="cuda"), out_dtype="float32")
ep = ExpertParallelGroupedLinear(pack_weight(shard_weight_experts(wg, rank, world).contiguous(), "mxfp4"), G, linear)
y = ep.forward_from_global(x, offs, gather=True, out_dtype="float32")
err = float((y - full).norm() / full.norm())
print(rank, "expert-parallel relF", err, tuple(y.shape), flush=True)
ok &= err < 1e-6
# whole MoE layer, experts split over the ranks, partial results summed by all-reduce
from dsl_tool_b200 import MoEWeights, moe_forward
T, E, k, K, H, D = 96, 6, 2, 256, 128, 192
xm = torch.randn(T, K, generator=g, device="cuda").bfloat16()
lg = torch.randn(T, E, generator=g, device="cuda")
w1 = (torch.randn(E, 2 * H, K, generator=g, device="cuda") * 0.05).bfloat16()
w2 = (torch.randn(E, D, H, generator=g, device="cuda") * 0.05).bfloat16()
for fmt in ("nvfp4", "bf16"):
    hgs = 0.004 if fmt == "nvfp4" else None
    whole = moe_forward(xm, lg, MoEWeights.pack(w1, w2, fmt, hidden_global_scale=hgs), k)
    part = moe_forward(xm, lg, MoEWeights.pack(w1, w2, fmt, rank=rank, world=world, hidden_global_scale=hgs), k)
    err = float((part - whole).norm() / whole.norm())
    print(rank, fmt, "moe layer expert-parallel relF", err, flush=True)
    ok &= err < 1e-5
    shard = moe_forward(xm, lg, MoEWeights.pack(w1, w2, fmt, rank=rank, world=world, hidden_global_scale=hgs), k,
                        reduce="reduce_scatter", exchange_dtype=torch.bfloat16)
    rows = T // world
    ref = whole[rank * rows:(rank + 1) * rows]
    err = float((shard - ref).norm() / ref.norm())
    print(rank, fmt, "moe layer reduce-scatter (bf16 exchange) relF", err, tuple(shard.shape), flush=True)
    ok &= err < 1e-2 and tuple(shard.shape) == (rows, D)
# the same layer in pipelined pieces (each piece's collective overlaps the next piece's GEMMs): on two ranks the sums are
# those of the unchunked layer, bit for bit, in both reduce modes; tokens 512 = 2 ranks x 2 pieces x 128 rows
Tc = 512
xc = torch.randn(Tc, K, generator=g, device="cuda").bfloat16()
lc = torch.randn(Tc, E, generator=g, device="cuda")
for fmt, hgs in (("nvfp4", 0.004), ("mxfp4", None)):
    wc = MoEWeights.pack(w1, w2, fmt, rank=rank, world=world, hidden_global_scale=hgs)
    for red, dt in (("reduce_scatter", torch.bfloat16), ("reduce_scatter", None), ("all_reduce", None)):
        base = moe_forward(xc, lc, wc, k, reduce=red, exchange_dtype=dt)
        got = moe_forward(xc, lc, wc, k, reduce=red, exchange_dtype=dt, chunks=2)
        same = bool(torch.equal(got, base))
        print(rank, fmt, red, dt, "chunked layer identical", same, tuple(got.shape), flush=True)
        ok &= same
try:
    moe_forward(xc[:384], lc[:384], wc, k, reduce="reduce_scatter", chunks=2)
    ok = False
except ValueError:
    pass
# the same reduce-scatter with the library's own kernel reading the peers' shares over NVLink (symmetric memory).  Shares
# that travel in fp32: on two ranks a + b is one addition whichever way, so the bits are NCCL's.  Shares in bf16: the kernel
# returns the fp32 sum of the two bf16 shares where NCCL rounds it to bf16, so the two agree to bf16 precision and the
# kernel's rounds agree with each other exactly.  Three rounds, so that both buffers are used again.
for fmt, hgs in (("nvfp4", 0.004), ("bf16", None)):
    wp = MoEWeights.pack(w1, w2, fmt, rank=rank, world=world, hidden_global_scale=hgs)
    for dt in (torch.bfloat16, None):
        base = moe_forward(xc, lc, wp, k, reduce="reduce_scatter", exchange_dtype=dt)
        first = None
        for rnd in range(3):
            got = moe_forward(xc, lc, wp, k, reduce="pull", exchange_dtype=dt)
            first = got if first is None else first
            if dt is None:
                same = bool(torch.equal(got, base))
            else:
                same = bool(torch.equal(got, first)) and bool(torch.equal(got.bfloat16(), base.bfloat16()))
            print(rank, fmt, dt, "pull round", rnd, "agrees with reduce-scatter", same, tuple(got.shape), flush=True)
            ok &= same
    # a different input in between: a stale buffer would show
    other = moe_forward((xc * 0.5).contiguous(), lc, wp, k, reduce="reduce_scatter")
    got = moe_forward((xc * 0.5).contiguous(), lc, wp, k, reduce="pull")
    same = bool(torch.equal(got, other))
    print(rank, fmt, "pull after a different input identical", same, flush=True)
    ok &= same
# token all-to-all: every rank owns half of the tokens and half of the experts; bit-identical to one GPU holding all
for fmt, hgs in (("nvfp4", 0.004), ("nvfp4", None), ("mxfp4", None)):
    whole = moe_forward(xm, lg, MoEWeights.pack(w1, w2, fmt, hidden_global_scale=hgs), k)
    rows = T // world
    mine = slice(rank * rows, (rank + 1) * rows)
    got = moe_forward(xm[mine].contiguous(), lg[mine].contiguous(),
                      MoEWeights.pack(w1, w2, fmt, rank=rank, world=world, hidden_global_scale=hgs), k, dispatch="all_to_all")
    same = bool(torch.equal(got, whole[mine]))
    print(rank, fmt, hgs, "moe layer token all-to-all identical", same, tuple(got.shape), flush=True)
    ok &= same
# a calibrated activation scale: no amax collective, still the bits of one GPU holding every token
whole = moe_forward(xm, lg, MoEWeights.pack(w1, w2, "nvfp4", hidden_global_scale=0.004), k, act_global_scale=0.002)
got = moe_forward(xm[mine].contiguous(), lg[mine].contiguous(),
                  MoEWeights.pack(w1, w2, "nvfp4", rank=rank, world=world, hidden_global_scale=0.004), k, dispatch="all_to_all",
                  act_global_scale=0.002)
same = bool(torch.equal(got, whole[mine]))
print(rank, "all-to-all with a calibrated activation scale identical", same, flush=True)
ok &= same
# a rank that receives nothing: every token prefers the experts of rank 0
lg0 = lg.clone(); lg0[:, E // 2:] = -1e9
whole = moe_forward(xm, lg0, MoEWeights.pack(w1, w2, "nvfp4", hidden_global_scale=None), k)
got = moe_forward(xm[mine].contiguous(), lg0[mine].contiguous(), MoEWeights.pack(w1, w2, "nvfp4", rank=rank, world=world), k,
                  dispatch="all_to_all")
same = bool(torch.equal(got, whole[mine]))
print(rank, "all-to-all with an idle rank identical", same, flush=True)
ok &= same
torch.cuda.synchronize()
dist.destroy_process_group()
sys.exit(0 if ok else 3)
'''


def test_two_gpu_split_matches_single_gpu(cuda_device, tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    procs = []
    for r in range(2):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE="2", MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port),
                   REPO_ROOT=root, NCCL_NVLS_ENABLE="0")
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE,
                                      stderr=subprocess.STDOUT, text=True))
    outs = [p.communicate(timeout=300)[0] for p in procs]
    assert all(p.returncode == 0 for p in procs), "\n".join(o[-1500:] for o in outs)


def test_one_process_driving_two_devices(cuda_device):
    """Kernel attributes, occupancy and SM counts are kept per device: a process that has used the library on one GPU
    gets the same results, bit for bit, on a second one (every kernel family: pair, group-scaled pair, decode, 1-CTA)."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from dsl_tool_b200 import _lib, linear, pack_weight
    g = torch.Generator().manual_seed(3)
    w = (torch.randn(640, 512, generator=g) * 0.02).bfloat16()
    outs = {}
    for dev in ("cuda:0", "cuda:1"):
        torch.cuda.set_device(dev)
        for fmt in ("nvfp4", "mxfp4", "fp8", "fp8_block128", "bf16"):
            pw = pack_weight(w.to(dev), fmt)
            for M in (5, 100, 300):
                a = torch.randn(M, 512, generator=torch.Generator().manual_seed(M)).bfloat16().to(dev)
                outs[(dev, fmt, M)] = linear(a, pw, out_dtype="float32").cpu()
        _lib.check_status(torch.device(dev))
    torch.cuda.set_device(0)
    for (dev, fmt, M), v in outs.items():
        if dev == "cuda:1":
            assert torch.equal(v, outs[("cuda:0", fmt, M)]), (fmt, M)
