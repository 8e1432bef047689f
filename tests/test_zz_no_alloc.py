"""The allocation-free FP4 GEMM entry point (`dsl_gemm_fp4_static_scratch`) against the ordinary
one (`dsl_gemm_fp4`), both called through the C ABI.

Who needs it: hosts that cannot give the GEMM a scratch buffer - code inside a stream capture
or a memory-planned region of another framework, plugin interfaces that pass only inputs and
outputs, processes that must not allocate after start-up.  The entry point keeps its split-K
scratch in a fixed array inside the library, so the test also checks that calling it twice in
a row (the array still holds the first call's partial sums) gives the same answer, and that
problems whose partial sums would not fit are refused.
"""
import ctypes

import numpy as np
import pytest
import torch

from oracle import quant_oracle as O
from tests.helpers import REL_FROB_TOL, activations, rel_frobenius, weights

pytestmark = pytest.mark.gpu


def _t(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _epilogue(lib_mod, gsa, gsb, workspace=None):
    ep = lib_mod.Epilogue()
    ep.scale_a_host, ep.scale_b_host = float(gsa), float(gsb)
    ep.out_dtype = lib_mod.F32
    if workspace is not None:
        ep.workspace, ep.workspace_bytes = workspace.data_ptr(), workspace.numel()
    return ep


@pytest.mark.parametrize("fmt", ["nvfp4", "mxfp4"])
def test_static_scratch_matches_regular_entry_point(cuda_device, fmt):
    from dsl_tool_b200 import _lib
    lib = _lib.lib()
    rng = np.random.default_rng(77)
    M, N, K = 16, 1024, 4096                        # a decode shape: the GEMM is cut along K
    a, w = activations(rng, M, K, outliers=True), weights(rng, N, K)
    if fmt == "nvfp4":
        pa, sfa, gsa = O.quant_nvfp4(a)
        pb, sfb, gsb = O.quant_nvfp4(w)
        want = O.gemm_nvfp4(pa, sfa, gsa, pb, sfb, gsb)
        code = _lib.FP4_NV
    else:
        pa, sfa = O.quant_mxfp4(a)
        pb, sfb = O.quant_mxfp4(w)
        gsa = gsb = 1.0
        want = O.gemm_mxfp4(pa, sfa, pb, sfb)
        code = _lib.FP4_MX
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
    outs = []
    for _ in range(2):                              # second call finds the first call's partial sums in the array
        out = torch.full((M, N), float("nan"), device="cuda")
        rc = lib.dsl_gemm_fp4_static_scratch(A.data_ptr(), B.data_ptr(), SFA.data_ptr(), SFB.data_ptr(), code,
                                             out.data_ptr(), N, M, N, K, ctypes.byref(ep2), status.data_ptr(), stream)
        assert rc == 0
        outs.append(out)
    torch.cuda.synchronize()
    assert status.item() == 0
    for out in outs:
        assert rel_frobenius(out.cpu().numpy(), ref.cpu().numpy()) <= REL_FROB_TOL
        assert rel_frobenius(out.cpu().numpy(), want) <= REL_FROB_TOL
    assert torch.equal(outs[0], outs[1])


def test_static_scratch_rejects_what_does_not_fit(cuda_device):
    from dsl_tool_b200 import _lib
    lib = _lib.lib()
    ep = _epilogue(_lib, 1.0, 1.0)
    dummy = torch.zeros(4096, dtype=torch.uint8, device="cuda")
    p = dummy.data_ptr()
    # 2 * M * N * 4 bytes must fit in the 4 MiB array: 1024 x 1024 does not
    rc = lib.dsl_gemm_fp4_static_scratch(p, p, p, p, _lib.FP4_NV, p, 1024, 1024, 1024, 64, ctypes.byref(ep), None,
                                         _lib.stream_ptr())
    assert rc == -6
    with pytest.raises(ValueError, match="fixed capacity"):
        _lib.check(rc, "dsl_gemm_fp4_static_scratch")
    assert lib.dsl_gemm_fp4_static_scratch(p, p, p, p, _lib.FP4_NV, p, 64, 16, 64, 64, None, None, None) == -1
