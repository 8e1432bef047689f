"""The dispatch layer keeps the reference's surface (dispatcher/dispatcher.py, registry.py). CPU."""
import base64

import numpy as np
import pytest
import torch

from dsl_tool_b200.dispatcher import (KernelDispatcher, KernelRegistry, deserialize_tensor, get_registry,
                                      serialize_tensor, summarize_tensor)


def test_registry_entries_and_order():
    reg = get_registry()
    rows = reg.list_kernels()
    assert [r["kernel_name"] for r in rows] == sorted(r["kernel_name"] for r in rows)
    names = {(r["kernel_name"], r["backend"]) for r in rows}
    assert {("gemm.fp8_gemm", "cuda"), ("gemm.fp4_gemm", "cuda"), ("gemm.grouped_gemm", "cuda")} <= names
    assert {r["backend"] for r in rows} == {"cuda"}            # one backend, no multi-backend dispatch
    assert set(rows[0]) == {"kernel_name", "backend", "description"}
    assert reg.list_backends_for("GEMM.FP8_GEMM") == ["cuda"]  # keys are lower-cased
    assert reg.get("Gemm.Fp4_Gemm", "CUDA") is not None
    assert get_registry() is reg                               # singleton


def test_register_signature_and_overwrite():
    reg = KernelRegistry()
    reg.register("Cat.Fn", "CUDA", lambda: 1, "d", {"x": "int"})
    e = reg.get("cat.fn", "cuda")
    assert (e.kernel_name, e.backend, e.description, e.input_schema, e.output_schema) == ("cat.fn", "cuda", "d", {"x": "int"}, {})
    reg.register("cat.fn", "cuda", lambda: 2)
    assert reg.get("cat.fn", "cuda").fn() == 2 and len(reg.list_kernels()) == 1


def test_kernel_info_schema_keys():
    d = KernelDispatcher()
    info = d.kernel_info("gemm.fp8_gemm", "cuda")
    assert set(info) == {"kernel_name", "backend", "description", "input_schema", "output_schema"}
    assert {"A", "B", "scale_a", "scale_b"} <= set(info["input_schema"])
    assert info["input_schema"]["A"] == "Tensor[M, K] bf16" and info["input_schema"]["B"] == "Tensor[K, N] bf16"
    assert "num_groups" in d.kernel_info("gemm.grouped_gemm", "cuda")["input_schema"]
    assert d.list_backends("gemm.fp4_gemm") == ["cuda"]


def test_unknown_kernel_and_backend_messages():
    d = KernelDispatcher()
    with pytest.raises(KeyError, match="Unknown kernel 'gemm.nope'"):
        d.run("gemm.nope", "cuda")
    with pytest.raises(KeyError, match=r"Backend 'triton' not available for kernel 'gemm.fp8_gemm'. Available backends: \['cuda'\]"):
        d.run("gemm.fp8_gemm", "triton")


def test_exceptions_are_wrapped():
    reg = get_registry()

    def boom(*a, **k):
        raise ValueError("bad shape")
    reg.register("test.boom", "cuda", boom)
    with pytest.raises(RuntimeError, match=r"Kernel 'test.boom' \[cuda\] raised: bad shape"):
        KernelDispatcher().run("test.boom", "cuda")


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the no-GPU behaviour")
def test_no_cpu_fallback():
    d = KernelDispatcher()
    assert d.device == "cpu"
    specs = [{"shape": [16, 32], "dtype": "float32", "fill": "ones"}, {"shape": [32, 16], "dtype": "float32", "fill": "ones"}]
    for name in ("gemm.fp8_gemm", "gemm.fp4_gemm"):
        with pytest.raises(RuntimeError, match="no CPU fallback"):
            d.run_from_spec(name, "cuda", specs, {})


def test_wire_format_roundtrip():
    x = torch.arange(12, dtype=torch.float32).reshape(3, 4) / 7
    s = serialize_tensor(x)
    assert s["shape"] == [3, 4] and s["dtype"] == "float32"
    assert torch.equal(deserialize_tensor(s, device="cpu"), x)
    xb = x.bfloat16()
    sb = serialize_tensor(xb)                       # bf16 travels as fp32 bytes labelled bfloat16
    assert sb["dtype"] == "bfloat16" and len(base64.b64decode(sb["data"])) == 12 * 4
    assert torch.equal(deserialize_tensor(sb, device="cpu"), xb)
    u = torch.arange(16, dtype=torch.uint8).reshape(2, 8)
    assert torch.equal(deserialize_tensor(serialize_tensor(u), device="cpu"), u)
    f8 = torch.tensor([[1.0, -2.5, 448.0]]).to(torch.float8_e4m3fn)
    assert torch.equal(deserialize_tensor(serialize_tensor(f8), device="cpu").view(torch.uint8), f8.view(torch.uint8))
    for fill, val in (("zeros", 0.0), ("ones", 1.0), (2.5, 2.5)):
        t = deserialize_tensor({"shape": [2, 2], "dtype": "fp16", "fill": fill}, device="cpu")
        assert t.dtype == torch.float16 and (t == val).all()
    assert deserialize_tensor({"shape": [4], "dtype": "int32", "fill": "random"}, device="cpu").dtype == torch.int32
    with pytest.raises(ValueError, match="Unknown dtype"):
        deserialize_tensor({"shape": [1], "dtype": "float128"}, device="cpu")
    summ = summarize_tensor(x)
    assert set(summ) == {"shape", "dtype", "numel", "min", "max", "mean", "std"} and summ["numel"] == 12


def test_dispatch_result_to_dict():
    reg = get_registry()
    reg.register("test.pair", "cuda", lambda a: [a, 3])
    r = KernelDispatcher().run("test.pair", "cuda", args=[torch.ones(2)])
    d = r.to_dict()
    assert set(d) == {"kernel_name", "backend", "elapsed_ms", "device_info", "output"}
    assert d["output"][1] == 3 and d["output"][0]["shape"] == [2]
    assert np.frombuffer(base64.b64decode(d["output"][0]["data"]), np.float32).tolist() == [1.0, 1.0]
