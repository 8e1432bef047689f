"""Host-resident batches through HostPipeline: the overlapped copies change no bit of the result."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _setup(kind, M=1024, K=512, N=768, seed=0):
    from dsl_tool_b200 import pack_weight
    dev = torch.device("cuda:0")
    g = torch.Generator(device=dev).manual_seed(seed)
    w = (torch.randn((1, N, K), generator=g, device=dev) * 0.05).to(torch.bfloat16)
    acts = [torch.randn((M, K), generator=g, device=dev).to(torch.bfloat16) for _ in range(5)]
    return dev, pack_weight(w, kind, layout="nk"), acts


@pytest.mark.parametrize("kind", ["fp8_block128", "mxfp4", "nvfp4"])
def test_pipeline_matches_direct_calls(kind):
    from dsl_tool_b200 import HostPipeline
    from dsl_tool_b200.gemm_kernels import linear
    dev, w, acts = _setup(kind)
    step = lambda a: linear(a, w, out_dtype=torch.bfloat16)
    want = [step(a).cpu() for a in acts]
    host_in = [a.cpu().pin_memory() for a in acts]
    host_out = [torch.empty_like(x).pin_memory() for x in want]
    pipe = HostPipeline(step, dev)
    for rounds in range(2):                                   # the second round reuses every staging buffer
        for o in host_out:
            o.zero_()
        for i, o in zip(host_in, host_out):
            pipe.submit(i, o)
        pipe.synchronize()
        for got, ref in zip(host_out, want):
            assert torch.equal(got.view(torch.int16), ref.view(torch.int16))


@pytest.mark.parametrize("kind,chunk", [("fp8_block128", 256), ("mxfp4", 384), ("fp8_block128", 1000)])
def test_row_chunks_are_bit_identical_for_row_local_scales(kind, chunk):
    """1x128 FP8 scales and MXFP4 block scales depend on one row only, so cutting the batch by rows changes nothing
    (the last chunk is short for 384 and 1000)."""
    from dsl_tool_b200 import HostPipeline
    from dsl_tool_b200.gemm_kernels import linear
    dev, w, acts = _setup(kind, seed=3)
    step = lambda a: linear(a, w, out_dtype=torch.bfloat16)
    want = step(acts[0]).cpu()
    host_in = acts[0].cpu().pin_memory()
    host_out = torch.zeros_like(want).pin_memory()
    pipe = HostPipeline(step, dev, depth=3)
    pipe.submit(host_in, host_out, rows_per_chunk=chunk)
    pipe.join()
    torch.cuda.current_stream().synchronize()                 # join() ordered the current stream behind the pipeline
    assert torch.equal(host_out.view(torch.int16), want.view(torch.int16))


def test_argument_errors():
    from dsl_tool_b200 import HostPipeline
    dev = torch.device("cuda:0")
    pipe = HostPipeline(lambda a: a, dev)
    pinned = torch.zeros(4, 4).pin_memory()
    with pytest.raises(ValueError):
        pipe.submit(torch.zeros(4, 4), pinned)                # pageable
    with pytest.raises(ValueError):
        pipe.submit(pinned.to(dev), pinned)                   # a device tensor
    with pytest.raises(ValueError):
        pipe.submit(pinned, torch.zeros(8, 4).pin_memory())   # the step returns another shape
    pipe.synchronize()
    with pytest.raises(ValueError):
        HostPipeline(lambda a: a, dev, depth=0)
