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


class _ReferenceWrapper(torch.autograd.Function):
    """The reference's autograd wrapper, as its model file writes it (model.py:20-75): reshape to
    (b*h, n, d), 13-argument forwardpass, save (q, k, v, o), slice off the denominator channel;
    later backwardpass with the saved tensors and gradk / temperature."""

    @staticmethod
    def forward(ctx, q, k, v, drop_noise, mask, dropout, normalize, temperature, a0, a1, a2, lim, p):
        b = 0
        if q.dim() == 4:
            b, h, nq, d = q.shape
            nk = k.shape[2]
            q = q.reshape(b * h, nq, d)
            k = k.reshape(b * h, nk, d)
            v = v.reshape(b * h, nk, d)
            drop_noise = drop_noise.reshape(b * h, nq, d)
        o = fastmax_cuda.forwardpass(q, k, v, drop_noise, mask, dropout, normalize, temperature, a0, a1, a2, lim, p)
        ctx.save_for_backward(q, k, v, o)
        ctx.mask, ctx.p, ctx.b, ctx.t, ctx.a0, ctx.a1, ctx.a2 = mask, p, b, temperature, a0, a1, a2
        o = o[:, :, :q.shape[2]]
        if b != 0:
            o = o.reshape(b, o.shape[0] // b, o.shape[1], o.shape[2])
        return o

    @staticmethod
    def backward(ctx, grad_output):
        q, k, v, o = ctx.saved_tensors
        if ctx.b != 0:
            grad_output = grad_output.reshape(grad_output.shape[0] * grad_output.shape[1], grad_output.shape[2],
                                              grad_output.shape[3]).contiguous()
        gradq, gradk, gradv = fastmax_cuda.backwardpass(q, k, v, o, grad_output, ctx.mask, ctx.a0, ctx.a1, ctx.a2,
                                                        ctx.p)
        if ctx.b != 0:
            gradq = gradq.reshape(ctx.b, gradq.shape[0] // ctx.b, gradq.shape[1], gradq.shape[2])
            gradk = gradk.reshape(ctx.b, gradk.shape[0] // ctx.b, gradk.shape[1], gradk.shape[2])
            gradv = gradv.reshape(ctx.b, gradv.shape[0] // ctx.b, gradv.shape[1], gradv.shape[2])
        return gradq, gradk / ctx.t, gradv, None, None, None, None, None, None, None, None, None, None


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["fp32", "bf16"])
@pytest.mark.parametrize("mask,p,lim", [(True, 1, 1.0), (True, 2, 1.0), (False, 2, 1.5)])
def test_reference_wrapper_with_normalize(dtype, mask, p, lim):
    """normalize=True, which the reference's model always passes (model.py:560-569): the wrapper hands
    backwardpass only (q, k, v, o, grad), and must still get the gradients of the normalised attention
    with respect to its own q and k -- what autograd through the reference's PyTorch path gives.  Two
    results are kept alive at once so that each backwardpass has to find its own record."""
    g = torch.Generator().manual_seed(23)
    cases = []
    for n in (300, 257):
        q, k, v, go = [torch.randn(2, 2, n, 64, generator=g) for _ in range(4)]
        kw = dict(mask=int(mask), normalize=1, p=p, a0=1.0, a1=1.0, a2=0.5, lim=lim)
        ref = oracle(q, k, v, go, dtype, dense=True, **kw)
        qc, kc, vc = [t.to(dtype).cuda().requires_grad_(True) for t in (q, k, v)]
        q0, k0 = qc.detach().clone(), kc.detach().clone()
        out = _ReferenceWrapper.apply(qc, kc, vc, torch.zeros_like(qc), mask, 0.0, True, 1.0, 1.0, 1.0, 0.5, lim, p)
        cases.append((out, go, ref, qc, kc, vc, q0, k0))
    for out, go, ref, qc, kc, vc, q0, k0 in cases:
        out.backward(go.to(dtype).cuda())
        assert torch.equal(qc.detach(), q0) and torch.equal(kc.detach(), k0), "inputs were modified"
        got = [t.detach().float().cpu() for t in (out, qc.grad, kc.grad, vc.grad)]
        assert_close(got, ref, dtype, f"normalised wrapper n={out.shape[2]}")


@pytest.mark.gpu
def test_backwardpass_on_a_foreign_o_differentiates_what_it_is_given():
    """An o that forwardpass did not make (here a copy) carries no record: backwardpass then treats q and k
    as they are, like the reference's."""
    g = torch.Generator().manual_seed(24)
    q, k, v, go = [torch.randn(1, 2, 130, 32, generator=g) for _ in range(4)]
    q, k = q / 6, k / 6
    kw = dict(mask=1, normalize=0, p=2, a0=1.0, a1=1.0, a2=0.5, lim=1.0)
    ref = oracle(q, k, v, go, torch.float32, dense=True, **kw)
    qc, kc, vc, gc = [t[0].cuda().contiguous() for t in (q, k, v, go)]
    o = fastmax_cuda.forwardpass(qc, kc, vc, None, True, 0.0, False, 1.0, 1.0, 1.0, 0.5, 1.0, 2)
    gq, gk, gv = fastmax_cuda.backwardpass(qc, kc, vc, o.clone(), gc, True, 1.0, 1.0, 0.5, 2)
    assert_close([t.cpu()[None] for t in (o[:, :, :32], gq, gk, gv)], ref, torch.float32, "foreign o")


@pytest.mark.gpu
@pytest.mark.parametrize("noise_dtype", [torch.float32, torch.bfloat16], ids=["noise_fp32", "noise_bf16"])
def test_forwardpass_output_dropout(noise_dtype):
    """o[..., :d] *= 1 + dropout * drop_noise, the denominator channel untouched
    (reference fastmax_cuda_forward.cu:271-280, 396-399)."""
    g = torch.Generator().manual_seed(25)
    q, k, v = [torch.randn(3, 77, 32, generator=g).cuda() for _ in range(3)]
    noise = torch.randn(3, 77, 32, generator=g).to(noise_dtype).cuda()
    args = (True, 1.0, 1.0, 1.0, 0.5, 1.0, 2)
    plain = fastmax_cuda.forwardpass(q, k, v, noise, True, 0.0, *args)
    noised = fastmax_cuda.forwardpass(q, k, v, noise, True, 0.25, *args)
    want = plain.clone()
    want[:, :, :32] *= 1 + 0.25 * noise.float()
    assert torch.allclose(noised, want, rtol=1e-6, atol=1e-7)
    assert torch.equal(noised[:, :, 32], plain[:, :, 32])
    with pytest.raises(RuntimeError, match="drop_noise"):
        fastmax_cuda.forwardpass(q, k, v, None, True, 0.25, *args)


@pytest.mark.gpu
def test_extension_rejects_bad_p_and_noncontiguous():
    q = torch.randn(2, 16, 32, device="cuda")
    with pytest.raises(RuntimeError, match="p must be 1 or 2"):
        fastmax_cuda.forwardpass(q, q, q, None, True, 0.0, False, 1.0, 1.0, 1.0, 0.5, 1.0, 3)
    with pytest.raises(RuntimeError, match="contiguous"):
        fastmax_cuda.forwardpass(q.transpose(0, 1), q, q, None, True, 0.0, False, 1.0, 1.0, 1.0, 0.5, 1.0, 2)
