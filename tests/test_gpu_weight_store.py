"""Packed weights through the file format and the identity cache on the GPU: a weight that was saved and
loaded, or served from the cache, multiplies exactly like the freshly packed one."""
import numpy as np
import pytest
import torch

import dsl_tool_b200 as D
from dsl_tool_b200.dispatcher import KernelDispatcher
from dsl_tool_b200.dispatcher.dispatcher import serialize_tensor
from dsl_tool_b200.weight_store import default_cache
from tests.helpers import activations, weights

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("fmt", ["fp8", "fp8_block128", "nvfp4", "mxfp4", "bf16"])
def test_saved_weight_multiplies_identically(cuda_device, tmp_path, fmt):
    rng = np.random.default_rng(3)
    M, N, K = 40, 384, 512
    a = torch.from_numpy(activations(rng, M, K)).bfloat16().to(cuda_device)
    w = torch.from_numpy(weights(rng, N, K)).bfloat16().to(cuda_device)
    pw = D.pack_weight(w, fmt)
    D.save_packed(tmp_path / "w.dslw", pw)
    back = D.load_packed(tmp_path / "w.dslw", cuda_device)
    assert torch.equal(D.linear(a, back), D.linear(a, pw))


def test_grouped_weight_round_trip(cuda_device, tmp_path):
    rng = np.random.default_rng(4)
    G, N, K = 3, 200, 256                      # N not a multiple of 128: every expert's scales start a fresh tile
    w = torch.from_numpy((rng.standard_normal((G, N, K)) * 0.02).astype(np.float32)).bfloat16().to(cuda_device)
    a = torch.from_numpy(activations(rng, 90, K)).bfloat16().to(cuda_device)
    offs = torch.tensor([0, 17, 17, 90], dtype=torch.int32, device=cuda_device)
    pw = D.pack_weight(w, "nvfp4")
    D.save_packed(tmp_path / "e.dslw", pw)
    back = D.load_packed(tmp_path / "e.dslw", cuda_device)
    assert back.groups == G and torch.equal(D.linear(a, back, expert_offsets=offs), D.linear(a, pw, expert_offsets=offs))


def test_cache_weights_flag(cuda_device):
    rng = np.random.default_rng(5)
    a = torch.from_numpy(activations(rng, 33, 256)).to(cuda_device)
    b = torch.from_numpy(weights(rng, 320, 256).T.copy()).to(cuda_device)          # reference layout [K, N] = [256, 320]
    cache = default_cache()
    cache.clear()
    h0, m0 = cache.hits, cache.misses
    want = D.fp4_gemm(a, b)
    assert torch.equal(D.fp4_gemm(a, b, cache_weights=True), want) and cache.misses == m0 + 1
    assert torch.equal(D.fp4_gemm(a, b, cache_weights=True), want) and cache.hits == h0 + 1
    b.mul_(2)                                  # an in-place update must not be served from the cache
    assert torch.equal(D.fp4_gemm(a, b, cache_weights=True), D.fp4_gemm(a, b)) and cache.misses == m0 + 2
    for mode in ("per_tensor", "block128"):
        assert torch.equal(D.fp8_gemm(a, b, mode=mode, cache_weights=True), D.fp8_gemm(a, b, mode=mode))
    g = torch.stack([b, -b])
    a3 = torch.stack([a, a])
    assert torch.equal(D.grouped_gemm(a3, g, format="mxfp4", cache_weights=True), D.grouped_gemm(a3, g, format="mxfp4"))
    cache.clear()


def test_run_from_spec_with_packed_file(cuda_device, tmp_path):
    rng = np.random.default_rng(6)
    a = torch.from_numpy(activations(rng, 20, 256)).to(cuda_device)
    w = torch.from_numpy(weights(rng, 384, 256)).to(cuda_device)
    D.save_packed(tmp_path / "w.dslw", D.pack_weight(w, "nvfp4"))
    disp = KernelDispatcher()
    res = disp.run_from_spec("gemm.fp4_gemm", "cuda", tensor_specs=[serialize_tensor(a), {"packed_file": str(tmp_path / "w.dslw")}],
                             scalar_params={"format": "nvfp4"})
    assert torch.equal(res.output, D.fp4_gemm(a, w, b_layout="nk"))
