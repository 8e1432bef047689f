"""Packed-weight cache and file format (CPU part): container round trip, malformed files, identity
cache semantics, and the dispatcher's wire-format additions that carry packed weights."""
import base64
import json
import os
import struct

import numpy as np
import pytest
import torch

from dsl_tool_b200.dispatcher.dispatcher import deserialize_tensor, serialize_tensor
from dsl_tool_b200.quantize import PackedWeight
from dsl_tool_b200.weight_store import WeightCache, load_packed, load_packed_cached, packed_nbytes, save_packed


def _fake(fmt, g=2, n=256, k=512, seed=0):
    gen = torch.Generator().manual_seed(seed)
    rb = lambda *shape: torch.randint(0, 256, shape, dtype=torch.uint8, generator=gen)
    if fmt == "bf16":
        return PackedWeight(fmt, torch.randn(g * n, k, generator=gen).bfloat16(), None, None, g, n, k)
    if fmt == "fp8":
        return PackedWeight(fmt, rb(g * n, k), torch.rand(1, generator=gen), None, g, n, k)
    if fmt == "fp8_block128":
        return PackedWeight(fmt, rb(g * n, k), torch.rand(g, n // 128, k // 128, generator=gen), None, g, n, k)
    sf = rb(g * (n // 128) * ((k // (16 if fmt == "nvfp4" else 32) + 3) // 4) * 512)
    gs = torch.rand(1, generator=gen) if fmt == "nvfp4" else None
    return PackedWeight(fmt, rb(g * n, k // 2), sf, gs, g, n, k)


def _same(a: PackedWeight, b: PackedWeight):
    assert (a.format, a.groups, a.n, a.k) == (b.format, b.groups, b.n, b.k)
    for x, y in ((a.q, b.q), (a.scale, b.scale), (a.global_scale, b.global_scale)):
        assert (x is None) == (y is None)
        if x is not None:
            assert x.dtype == y.dtype and x.shape == y.shape and torch.equal(x.view(torch.uint8), y.view(torch.uint8))


@pytest.mark.parametrize("fmt", ["fp8", "fp8_block128", "nvfp4", "mxfp4", "bf16"])
def test_file_round_trip(tmp_path, fmt):
    w = _fake(fmt)
    path = tmp_path / f"w_{fmt}.dslw"
    save_packed(path, w)
    _same(load_packed(path, "cpu"), w)
    # the container is the plain "length + JSON + data" layout: a generic reader can list the tensors
    raw = path.read_bytes()
    (n,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + n])
    assert header["__metadata__"]["format"] == fmt and all(isinstance(v, str) for v in header["__metadata__"].values())
    q = header["q"]
    assert q["data_offsets"][1] - q["data_offsets"][0] == w.q.numel() * w.q.element_size() and (8 + n) % 8 == 0
    assert len(raw) == 8 + n + packed_nbytes(w)


def test_malformed_files(tmp_path):
    good = tmp_path / "good.dslw"
    save_packed(good, _fake("nvfp4"))
    raw = good.read_bytes()
    (n,) = struct.unpack("<Q", raw[:8])
    cases = {
        "short": raw[:5],
        "hugeheader": struct.pack("<Q", 1 << 40) + raw[8:],
        "notjson": raw[:8] + b"\xff" * n + raw[8 + n:],
        "truncated": raw[:-100],
        "foreign": None,
    }
    hdr = json.loads(raw[8:8 + n])
    hdr["__metadata__"]["producer"] = "someone else"
    f = json.dumps(hdr).encode()
    cases["foreign"] = struct.pack("<Q", len(f)) + f + raw[8 + n:]
    hdr = json.loads(raw[8:8 + n])
    hdr["q"]["shape"][0] += 1
    f = json.dumps(hdr).encode()
    cases["shape"] = struct.pack("<Q", len(f)) + f + raw[8 + n:]
    for name, blob in cases.items():
        p = tmp_path / f"{name}.dslw"
        p.write_bytes(blob)
        with pytest.raises(ValueError):
            load_packed(p, "cpu")
    with pytest.raises(ValueError):
        save_packed(tmp_path / "x", PackedWeight("int3", torch.zeros(1, dtype=torch.uint8), None, None, 1, 1, 1))


def test_cached_file_load_follows_the_file(tmp_path):
    p = tmp_path / "w.dslw"
    save_packed(p, _fake("mxfp4", seed=1))
    a = load_packed_cached(p, "cpu")
    assert load_packed_cached(p, "cpu") is a
    save_packed(p, _fake("mxfp4", seed=2, n=384))
    os.utime(p, (1, 1))                                   # whatever the clock granularity, the stamp differs
    b = load_packed_cached(p, "cpu")
    assert b is not a and b.n == 384


def test_identity_cache():
    calls = []

    def packer(w, fmt, layout):
        calls.append((fmt, layout))
        return PackedWeight(fmt, torch.zeros(1000, dtype=torch.uint8), None, None, 1, 1, 1)

    cache = WeightCache(max_bytes=2500)
    w = torch.randn(8, 8)
    a = cache.get(w, "fp8", "nk", packer)
    assert cache.get(w, "fp8", "nk", packer) is a and len(calls) == 1 and cache.hits == 1
    cache.get(w, "fp8", "kn", packer)                     # another layout is another entry
    cache.get(w.t(), "fp8", "nk", packer)                 # so is another view of the same storage
    assert len(calls) == 3
    w.add_(1)                                              # in-place update: the old entry must not be served
    cache.get(w, "fp8", "nk", packer)
    assert len(calls) == 4
    assert cache.nbytes <= 2500 and len(cache) == 2       # 1000-byte entries, 2500-byte budget: oldest evicted
    big = WeightCache(max_bytes=10)
    big.get(w, "fp8", "nk", packer)                       # larger than the budget: packed, returned, not kept
    assert len(big) == 0
    cache.clear()
    assert len(cache) == 0 and cache.nbytes == 0


@pytest.mark.parametrize("name,dtype", [("uint8", torch.uint8), ("e8m0", torch.float8_e8m0fnu), ("float8_e8m0fnu", torch.float8_e8m0fnu),
                                        ("fp4x2", torch.float4_e2m1fn_x2), ("float4_e2m1fn_x2", torch.float4_e2m1fn_x2),
                                        ("fp8", torch.float8_e4m3fn)])
def test_wire_format_byte_dtypes(name, dtype):
    raw = np.arange(24, dtype=np.uint8).reshape(2, 12)
    spec = {"shape": [2, 12], "dtype": name, "data": base64.b64encode(raw.tobytes()).decode()}
    t = deserialize_tensor(spec, device="cpu")
    assert t.dtype == dtype and tuple(t.shape) == (2, 12) and np.array_equal(t.view(torch.uint8).numpy(), raw)
    back = serialize_tensor(t)
    assert base64.b64decode(back["data"]) == raw.tobytes() and back["shape"] == [2, 12]
    assert deserialize_tensor({"shape": [3], "dtype": name, "fill": "zeros"}, device="cpu").view(torch.uint8).sum() == 0
    assert deserialize_tensor({"shape": [64], "dtype": name, "fill": "random"}, device="cpu").dtype == dtype
    if dtype in (torch.float8_e8m0fnu, torch.float4_e2m1fn_x2):
        with pytest.raises(ValueError):
            deserialize_tensor({"shape": [3], "dtype": name, "fill": 1.5}, device="cpu")


def test_packed_file_spec(tmp_path):
    p = tmp_path / "w.dslw"
    w = _fake("nvfp4")
    save_packed(p, w)
    got = deserialize_tensor({"packed_file": str(p)}, device="cpu")
    assert isinstance(got, PackedWeight)
    _same(got, w)


def test_host_pipeline_chunk_bounds_and_no_cpu_path():
    from dsl_tool_b200.host_io import HostPipeline, chunk_bounds
    assert chunk_bounds(10, 4) == [(0, 4), (4, 8), (8, 10)] and chunk_bounds(0, 4) == [] and chunk_bounds(4, 4) == [(0, 4)]
    with pytest.raises(ValueError):
        chunk_bounds(4, 0)
    if not torch.cuda.is_available():
        with pytest.raises(RuntimeError):
            HostPipeline(lambda a: a, "cuda:0")
