"""The allocation-free FP4 GEMM entry point (`dsl_gemm_fp4_static_scratch`) against the ordinary
one (`dsl_gemm_fp4`), both called through the C ABI.

Who needs it: hosts that cannot give the GEMM a scratch buffer - code inside a stream capture
or a memory-planned region of another framework, plugin interfaces that pass only inputs and
outputs, processes that must not allocate after start-up.  The entry point keeps the scratch
for its partial sums along K in a fixed array inside the library.

The shapes here are ones whose kernel really goes through that array (16 tokens against 150
column tiles: more tiles than SMs, so the K runs cross tile borders and their partial tiles and
arrival words live in scratch).  Before the calls the whole array is filled with foreign bytes
(NaN patterns) and another shape is run through it, so the test also shows that
  * a call writes the partial sums it later reads (the result is right although the array held
    NaNs, and the NaNs in the part it uses are gone afterwards),
  * stale bytes where the arrival words live are taken as "empty" (they carry no valid epoch),
  * two calls in a row give bit-identical answers, equal to the ordinary entry point's,
  * problems whose scratch would not fit the array are refused.
"""
import ctypes

import numpy as np
import pytest
import torch

from oracle import quant_oracle as O
from tests.helpers import REL_FROB_TOL, activations, rel_frobenius, weights

pytestmark = pytest.mark.gpu

NAN_WORD = 0x7FC00000


def _t(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _epilogue(lib_mod, gsa, gsb, workspace=None):
    ep = lib_mod.Epilogue()
    ep.scale_a_host, ep.scale_b_host = float(gsa), float(gsb)
    ep.out_dtype = lib_mod.F32
    if workspace is not None:
        ep.workspace, ep.workspace_bytes = workspace.data_ptr(), workspace.numel()
    return ep


def _quantised(fmt, a, w):
    from dsl_tool_b200 import _lib
    if fmt == "nvfp4":
        pa, sfa, gsa = O.quant_nvfp4(a)
        pb, sfb, gsb = O.quant_nvfp4(w)
        return pa, sfa, gsa, pb, sfb, gsb, O.gemm_nvfp4(pa, sfa, gsa, pb, sfb, gsb), _lib.FP4_NV
    pa, sfa = O.quant_mxfp4(a)
    pb, sfb = O.quant_mxfp4(w)
    return pa, sfa, 1.0, pb, sfb, 1.0, O.gemm_mxfp4(pa, sfa, pb, sfb), _lib.FP4_MX


def _poison_array(lib, stream):
    from dsl_tool_b200 import _lib
    junk = torch.full((_lib.STATIC_SCRATCH_BYTES // 4,), NAN_WORD, dtype=torch.int32, device="cuda")
    assert lib.dsl_selftest_static_scratch_copy(junk.data_ptr(), 0, _lib.STATIC_SCRATCH_BYTES, 1, stream) == 0
    return junk


def _read_array(lib, stream):
    from dsl_tool_b200 import _lib
    out = torch.empty(_lib.STATIC_SCRATCH_BYTES // 4, dtype=torch.int32, device="cuda")
    assert lib.dsl_selftest_static_scratch_copy(out.data_ptr(), 0, _lib.STATIC_SCRATCH_BYTES, 0, stream) == 0
    torch.cuda.synchronize()
    return out.cpu().numpy()


@pytest.mark.parametrize("fmt", ["nvfp4", "mxfp4"])
def test_static_scratch_matches_regular_entry_point(cuda_device, fmt):
    from dsl_tool_b200 import _lib
    lib = _lib.lib()
    rng = np.random.default_rng(77)
    M, N, K = 16, 19200, 2048                       # 150 column tiles on at most 148 SMs: the scratch combine
    op = _lib.OP_GEMM_FP4_NV if fmt == "nvfp4" else _lib.OP_GEMM_FP4_MX
    need = lib.dsl_workspace_bytes(op, M, N, K, 1)
    assert _lib.WS_HEADER_BYTES < need <= _lib.STATIC_SCRATCH_BYTES, "the shape must be one that uses the array"
    a, w = activations(rng, M, K, outliers=True), weights(rng, N, K)
    pa, sfa, gsa, pb, sfb, gsb, want, code = _quantised(fmt, a, w)
    A, B, SFA, SFB = _t(pa), _t(pb), _t(O.swizzle_sf(sfa)), _t(O.swizzle_sf(sfb))
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    stream = _lib.stream_ptr()

    ws = torch.empty(_lib.STATIC_SCRATCH_BYTES, dtype=torch.uint8, device="cuda")
    ref = torch.full((M, N), float("nan"), device="cuda")
    ep = _epilogue(_lib, gsa, gsb, ws)
    rc = lib.dsl_gemm_fp4(A.data_ptr(), B.data_ptr(), SFA.data_ptr(), SFB.data_ptr(), code, ref.data_ptr(), N, M, N, K,
                          None, 1, ctypes.byref(ep), status.data_ptr(), stream)
    assert rc == 0

    ep2 = _epilogue(_lib, gsa, gsb)                  # no workspace is passed
    keep = _poison_array(lib, stream)                # foreign bytes everywhere, the arrival words' place included
    # a different problem first (32 tokens: partial tiles twice the size and fewer CTAs, so every offset differs)
    M0, N0, K0 = 32, 19200, 768
    assert _lib.WS_HEADER_BYTES < lib.dsl_workspace_bytes(op, M0, N0, K0, 1) <= _lib.STATIC_SCRATCH_BYTES
    pa0, sfa0, gsa0, pb0, sfb0, gsb0, want0, _ = _quantised(fmt, activations(rng, M0, K0), weights(rng, N0, K0))
    out0 = torch.full((M0, N0), float("nan"), device="cuda")
    t0 = [_t(pa0), _t(pb0), _t(O.swizzle_sf(sfa0)), _t(O.swizzle_sf(sfb0))]
    ep0 = _epilogue(_lib, gsa0, gsb0)
    rc = lib.dsl_gemm_fp4_static_scratch(t0[0].data_ptr(), t0[1].data_ptr(), t0[2].data_ptr(), t0[3].data_ptr(), code,
                                         out0.data_ptr(), N0, M0, N0, K0, ctypes.byref(ep0), status.data_ptr(), stream)
    assert rc == 0
    outs = []
    for _ in range(2):                              # the second call finds the first call's partial sums in the array
        out = torch.full((M, N), float("nan"), device="cuda")
        rc = lib.dsl_gemm_fp4_static_scratch(A.data_ptr(), B.data_ptr(), SFA.data_ptr(), SFB.data_ptr(), code,
                                             out.data_ptr(), N, M, N, K, ctypes.byref(ep2), status.data_ptr(), stream)
        assert rc == 0
        outs.append(out)
    torch.cuda.synchronize()
    assert status.item() == 0
    assert rel_frobenius(out0.cpu().numpy(), want0) <= REL_FROB_TOL
    for out in outs:
        assert rel_frobenius(out.cpu().numpy(), ref.cpu().numpy()) <= REL_FROB_TOL
        assert rel_frobenius(out.cpu().numpy(), want) <= REL_FROB_TOL
    assert torch.equal(outs[0], outs[1])
    assert torch.equal(outs[0], ref)                 # same kernel, same plan: bit-identical to the ordinary entry point

    # what the calls left in the array: partial sums where the NaN patterns were, arrival words back at zero
    after = _read_array(lib, stream)
    header_words = _lib.WS_HEADER_BYTES // 4
    tiles = (N + 127) // 128
    words = after[: 2 * tiles].view(np.int64)
    stale = np.int64(NAN_WORD) << 32 | np.int64(NAN_WORD)
    # a tile whose K runs were shared leaves a zeroed word; a tile one CTA did alone never touched its word
    assert np.all((words == 0) | (words == stale)), "an arrival word was left tagged"
    assert (words == 0).sum() > tiles // 2
    used = after[header_words: need // 4]
    assert (used != np.int32(NAN_WORD)).mean() > 0.25, "the calls did not write their partial sums into the array"
    del keep


def test_static_scratch_rejects_what_does_not_fit(cuda_device):
    from dsl_tool_b200 import _lib
    lib = _lib.lib()
    ep = _epilogue(_lib, 1.0, 1.0)
    dummy = torch.zeros(4096, dtype=torch.uint8, device="cuda")
    p = dummy.data_ptr()
    # 32 tokens against 512 column tiles: one CTA per SM, two 16 KiB partial tiles each -> more than the 4 MiB array
    M, N, K = 32, 65536, 2048
    assert lib.dsl_workspace_bytes(_lib.OP_GEMM_FP4_NV, M, N, K, 1) > _lib.STATIC_SCRATCH_BYTES
    rc = lib.dsl_gemm_fp4_static_scratch(p, p, p, p, _lib.FP4_NV, p, N, M, N, K, ctypes.byref(ep), None, _lib.stream_ptr())
    assert rc == -6
    with pytest.raises(ValueError, match="fixed capacity"):
        _lib.check(rc, "dsl_gemm_fp4_static_scratch")
    assert lib.dsl_gemm_fp4_static_scratch(p, p, p, p, _lib.FP4_NV, p, 64, 16, 64, 64, None, None, None) == -1
    # the test hook stays inside the array
    assert lib.dsl_selftest_static_scratch_copy(p, _lib.STATIC_SCRATCH_BYTES, 16, 0, _lib.stream_ptr()) == -6
