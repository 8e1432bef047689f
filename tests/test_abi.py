"""The C-ABI library loads and exports every symbol include/dslgemm.h declares; argument
validation that needs no GPU.  CPU."""
import ctypes
import os
import re

import pytest

from dsl_tool_b200 import _lib
from dsl_tool_b200.build import build_library

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def cdll():
    build_library()
    return _lib.lib()


def declared_functions():
    text = open(os.path.join(ROOT, "include", "dslgemm.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(dsl_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported(cdll):
    names = declared_functions()
    assert len(names) >= 11
    for n in names:
        assert hasattr(cdll, n), n
    assert set(names) == set(_lib._SIGNATURES)        # the Python binding covers the whole header


def test_version_and_sizes(cdll):
    assert b"sm_100a" in cdll.dsl_version()
    assert cdll.dsl_sf_bytes(1, 1) == 512
    assert cdll.dsl_sf_bytes(128, 4) == 512
    assert cdll.dsl_sf_bytes(129, 5) == 4 * 512
    assert cdll.dsl_sf_bytes(8192, 512) == 64 * 128 * 512
    assert cdll.dsl_sf_bytes_grouped(300, 8, 4) == (3 + 4) * 2 * 512
    assert cdll.dsl_sf_bytes(0, 4) == 0


def test_argument_validation_without_gpu(cdll):
    buf = ctypes.create_string_buffer(4096)
    p = ctypes.addressof(buf) & ~15
    ep = _lib.Epilogue()
    assert cdll.dsl_quant_fp8(None, 0, 4, 16, 0, p, 0, p, p, None) == -1          # NULL input
    assert cdll.dsl_quant_fp8(p, 7, 4, 16, 0, p, 0, p, p, None) == -4             # bad dtype
    assert cdll.dsl_quant_fp8(p, 0, 4, 24, 1, p, 0, p, p, None) == -2             # cols % 16 for grouped modes
    assert cdll.dsl_quant_fp8(p + 4, 0, 4, 16, 0, p, 0, p, p, None) == -3         # misaligned
    assert cdll.dsl_quant_fp4(p, 0, 4, 48, 0, p, 0, p, p, None, 0, p, None) == -2 # K % 32
    assert cdll.dsl_quant_fp4(p, 0, 4, 64, 5, p, 0, p, p, None, 0, p, None) == -4
    assert cdll.dsl_quant_fp4(p, 0, 4, 64, 0, p, 0, p, p, p, 5000, p, None) == -6 # too many groups
    assert cdll.dsl_gemm_fp8(p, p, p, 16, 4, 16, 24, None, 1, ctypes.byref(ep), None, None) == -2   # K % 16
    assert cdll.dsl_gemm_fp8(p, p, p, 8, 4, 16, 32, None, 1, ctypes.byref(ep), None, None) == -2    # ldc < N
    assert cdll.dsl_gemm_fp8(p, p, p, 16, 4, 16, 32, None, 1, None, None, None) == -1
    assert cdll.dsl_gemm_fp4(p, p, p, p, 0, p, 16, 4, 16, 48, None, 1, ctypes.byref(ep), None, None) == -2
    assert cdll.dsl_gemm_fp4(p, p, None, p, 0, p, 16, 4, 16, 64, None, 1, ctypes.byref(ep), None, None) == -1
    assert cdll.dsl_gemm_fp8_groupwise(p, p, p, p, 1, p, 16, 4, 16, 192, None, 1, ctypes.byref(ep), None, None) == -2
    ep.out_dtype = 9
    assert cdll.dsl_gemm_bf16(p, p, p, 16, 4, 16, 32, None, 1, ctypes.byref(ep), None, None) == -4
    # empty problems are a no-op, not an error
    ep.out_dtype = 0
    assert cdll.dsl_gemm_fp8(p, p, p, 16, 0, 16, 32, None, 1, ctypes.byref(ep), None, None) == 0
    assert cdll.dsl_quant_fp8(p, 0, 0, 16, 0, p, 0, p, p, None) == 0


def test_missing_library_fails_loudly(monkeypatch):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", "/nonexistent/libdslgemm.so")
    with pytest.raises(RuntimeError, match="no fallback"):
        _lib.lib()


def test_epilogue_struct_layout_matches_the_header(tmp_path):
    """The ctypes mirror of dsl_epilogue has the size and field offsets the C compiler gives the header's struct."""
    import subprocess
    fields = [name for name, _ in _lib.Epilogue._fields_]
    src = tmp_path / "layout.c"
    lines = ['#include <stdio.h>', '#include <stddef.h>', '#include "dslgemm.h"', 'int main(void) {',
             '  printf("%zu\\n", sizeof(dsl_epilogue));']
    lines += [f'  printf("{f} %zu\\n", offsetof(dsl_epilogue, {f}));' for f in fields]
    lines += ['  return 0;', '}']
    src.write_text("\n".join(lines))
    exe = tmp_path / "layout"
    subprocess.run(["gcc", "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe)], check=True)
    out = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.split("\n")
    assert int(out[0]) == ctypes.sizeof(_lib.Epilogue)
    for line in out[1:]:
        if line:
            name, off = line.split()
            assert getattr(_lib.Epilogue, name).offset == int(off), name
    # and the header's enum values are the ones the binding uses
    text = open(os.path.join(ROOT, "include", "dslgemm.h")).read()
    for cname, value in (("DSL_ACT_SWIGLU", _lib.ACT_SWIGLU), ("DSL_ACT_GEGLU", _lib.ACT_GEGLU), ("DSL_OUT_NVFP4", _lib.OUT_NVFP4)):
        assert re.search(rf"\b{cname}\s*=\s*{value}\b", text), cname


def test_new_argument_validation_without_gpu(cdll):
    buf = ctypes.create_string_buffer(4096)
    p = ctypes.addressof(buf) & ~15
    ep = _lib.Epilogue()
    ep.activation = 7
    assert cdll.dsl_gemm_fp8(p, p, p, 16, 4, 16, 32, None, 1, ctypes.byref(ep), None, None) == -4      # unknown activation
    ep.activation = _lib.ACT_SWIGLU
    assert cdll.dsl_gemm_fp8(p, p, p, 16, 4, 15, 32, None, 1, ctypes.byref(ep), None, None) == -2      # odd column count
    assert cdll.dsl_gemm_fp8(p, p, p, 4, 4, 16, 32, None, 1, ctypes.byref(ep), None, None) == -2       # ldc < N/2
    ep.activation = 0
    ep.out_dtype = _lib.OUT_NVFP4
    assert cdll.dsl_gemm_fp8(p, p, p, 32, 4, 32, 32, None, 1, ctypes.byref(ep), None, None) == -1      # no out_sf
    ep.out_sf = p
    assert cdll.dsl_gemm_fp8(p, p, p, 32, 4, 32, 32, None, 1, ctypes.byref(ep), None, None) == -2      # no global scale
    ep.out_gs_host = 0.01
    assert cdll.dsl_gemm_fp8(p, p, p, 24, 4, 24, 32, None, 1, ctypes.byref(ep), None, None) == -2      # columns % 16
    assert cdll.dsl_gemm_fp8_groupwise(p, p, p, p, 1, p, 32, 4, 32, 128, None, 1, ctypes.byref(ep), None, None) == -4
    assert cdll.dsl_moe_route(p, 0, 4, 8, 9, 1, p, p, None) == -2                                      # k > experts
    assert cdll.dsl_moe_route(p, 2, 4, 8, 2, 1, p, p, None) == -4                                      # fp16 logits
    assert cdll.dsl_moe_plan(p, 8, 5000, p, p, p, p, None) == -2
    assert cdll.dsl_moe_plan_scratch_bytes(4096, 64) == (2 + 1) * 64 * 4
    assert cdll.dsl_moe_dispatch_fp4(p, p, p, p, p, p, 4, 2, 48, 0, 0, 4, p, p, None) == -2            # K % 32
    assert cdll.dsl_moe_dispatch_rows(p, p, p, p, 4, 2, 24, 0, 4, p, None) == -2                       # row bytes % 16
    assert cdll.dsl_moe_combine(p, 0, p, p, p, p, 4, 40, 16, 0, 4, p, 0, None) == -2                   # k > 32
    ptrs = (ctypes.c_void_p * 2)(p, p)
    assert cdll.dsl_moe_reduce_pull(ptrs, 17, 0, 4, 64, 1, p, 1, None) != 0                             # more ranks than DSL_MAX_PEERS
    assert cdll.dsl_moe_reduce_pull(ptrs, 2, 0, 4, 60, 1, p, 1, None) == -2                            # row not whole 16-byte vectors
    assert cdll.dsl_moe_reduce_pull(ptrs, 2, 0, 4, 64, 2, p, 1, None) == -4                            # fp16 shares
    assert cdll.dsl_moe_reduce_pull((ctypes.c_void_p * 2)(p, None), 2, 0, 4, 64, 1, p, 1, None) == -1  # a missing peer buffer
    assert cdll.dsl_moe_reduce_pull(ptrs, 2, 0, 0, 64, 1, p, 1, None) == 0                             # nothing to do
    assert cdll.dsl_quant_fp4_ref32(None, 0, 64, p, p, None) == -1
    assert cdll.dsl_gemm_fp4_ref32(p, p, p, p, p, 4, 8, 48, None) == -2                                # K % 32
