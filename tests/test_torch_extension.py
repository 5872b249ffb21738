"""The `fastmax_cuda` torch extension: the reference's forwardpass/backwardpass boundary
(reference fastmax_cuda.cpp:17-37) over the C ABI."""
import pytest
import torch

from gpu_util import assert_close, oracle

fastmax_cuda = pytest.importorskip("fastmax_cuda", reason="build with python -m fastmax_b200.build --torch-ext")


def test_module_surface_and_cpu_rejection():
    assert callable(fastmax_cuda.forwardpass) and callable(fastmax_cuda.backwardpass)
    q = torch.randn(2, 8, 32)
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        fastmax_cuda.forwardpass(q, q, q, None, True, 0.0, False, 1.0, 1.0, 1.0, 0.5, 1.0, 2)
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        fastmax_cuda.forwardpass(q, q, q, None, None, True, 0.0, False, 1.0, 1.0, 1.0, 0.5, 1.0, 2)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["fp32", "bf16"])
def test_reference_wrapper_flow_through_the_extension(dtype):
    """What the reference's autograd wrapper does (model.py:29-75): forwardpass, slice off the
    denominator channel, later backwardpass with the saved o -- both forwardpass arities."""
    g = torch.Generator().manual_seed(21)
    q, k, v, go = [torch.randn(1, 4, 300, 64, generator=g) for _ in range(4)]
    q, k = q / 8, k / 8
    kw = dict(mask=1, normalize=0, p=2, a0=1.0, a1=1.0, a2=0.5, lim=1.0)
    ref = oracle(q, k, v, go, dtype, dense=True, **kw)
    qc, kc, vc, gc = [t[0].to(dtype).cuda().contiguous() for t in (q, k, v, go)]
    noise = torch.zeros_like(qc)
    o13 = fastmax_cuda.forwardpass(qc, kc, vc, noise, True, 0.0, False, 1.0, 1.0, 1.0, 0.5, 1.0, 2)
    o14 = fastmax_cuda.forwardpass(qc, kc, vc, noise, torch.zeros(599, 64, device="cuda"), True, 0.0, False, 1.0,
                                   1.0, 1.0, 0.5, 1.0, 2)
    assert o13.shape == (4, 300, 65) and o13.dtype == torch.float32 and torch.equal(o13, o14)
    gq, gk, gv = fastmax_cuda.backwardpass(qc, kc, vc, o13, gc, True, 1.0, 1.0, 0.5, 2)
    got = [t.float().cpu()[None] for t in (o13[:, :, :64], gq, gk, gv)]
    assert_close(got, ref, dtype, "extension")
    assert gq.dtype == dtype and gk.shape == kc.shape


@pytest.mark.gpu
def test_extension_rejects_bad_p_and_noncontiguous():
    q = torch.randn(2, 16, 32, device="cuda")
    with pytest.raises(RuntimeError, match="p must be 1 or 2"):
        fastmax_cuda.forwardpass(q, q, q, None, True, 0.0, False, 1.0, 1.0, 1.0, 0.5, 1.0, 3)
    with pytest.raises(RuntimeError, match="contiguous"):
        fastmax_cuda.forwardpass(q.transpose(0, 1), q, q, None, True, 0.0, False, 1.0, 1.0, 1.0, 0.5, 1.0, 2)
