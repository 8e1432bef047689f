"""bench.py on a machine without a GPU: the reference arm (the oracle's CPU GEMM) prints the contract's JSON line,
other ranks of that arm stay silent, and the product arm refuses to run instead of falling back to the CPU."""
import json
import os
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(args, env=None, timeout=600):
    e = dict(os.environ)
    e.update(env or {})
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True, cwd=ROOT,
                          env=e, timeout=timeout)


def test_reference_arm_line():
    r = _run(["--impl", "reference", "--steps", "1", "--warmup", "1"])
    assert r.returncode == 0, r.stderr[-2000:]
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["metric"] == "gemm_tflops" and line["unit"] == "TFLOP/s"
    assert line["value"] > 0 and line["ms_per_step"] > 0 and line["higher_is_better"] is True and line["vs_baseline"] is None
    assert line["n_gpus"] == 1 and line["steps"] == 1 and line["warmup"] == 1 and line["data"] == "synthetic"
    cfg = line["config"]
    assert cfg["workload"] == "fp8_groupwise_llama8b_mlp" and (cfg["M"], cfg["K"], cfg["N"]) == (4096, 4096, 14336)
    cb = line["cpu_baseline"]
    assert cb["kind"] in ("port", "reference") and cb["cores"] >= 1 and cb["value"] == line["value"] and cb["sample"]
    e2e = line["e2e"]
    assert e2e["value"] == line["value"] and e2e["h2d_bytes_per_step"] == 0 and e2e["d2h_bytes_per_step"] == 0


def test_reference_arm_other_ranks_are_silent():
    r = _run(["--impl", "reference", "--steps", "1", "--warmup", "1"], env={"RANK": "1", "WORLD_SIZE": "2", "LOCAL_RANK": "1"})
    assert r.returncode == 0 and r.stdout.strip() == ""


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the behaviour of a machine without a GPU")
def test_product_arm_refuses_without_a_gpu():
    r = _run(["--steps", "1", "--warmup", "1"], timeout=300)
    assert r.returncode != 0 and "CUDA" in r.stderr and '"value"' not in r.stdout


def test_both_arms_describe_the_workload_with_the_same_config_object():
    """The product arm and the reference arm build `config` with one function; the reference arm's line (above) carries
    it, and it names the workload's shape and format, so the two lines can be matched by comparing `config`."""
    sys.path.insert(0, ROOT)
    import bench
    for name in ("fp8_groupwise_llama8b_mlp", "nvfp4_8192", "moe_nvfp4", "moe_layer_nvfp4"):
        for scaling in ("strong", "weak"):
            c = bench.workload_config(name, scaling, 4)
            assert c == bench.workload_config(name, scaling, 4)
            assert c["workload"] == name and c["format"] == bench.WORKLOADS[name]["kind"] and {"M", "K", "N"} <= set(c)
    r = _run(["--impl", "reference", "--steps", "1", "--warmup", "1"])
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert line["config"] == bench.workload_config("fp8_groupwise_llama8b_mlp", line["scaling"], 4)
