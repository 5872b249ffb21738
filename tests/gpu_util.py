"""Helpers shared by the GPU parity tests."""
import torch

from oracle.fastmax_oracle import fastmax_fwd_bwd, rel_err

from fastmax_b200 import _cabi

TOL = {torch.float32: 1e-4, torch.bfloat16: 2e-2}   # relative, outputs and gradients


def run_cabi(q, k, v, go, dtype, impl="auto", **kw):
    """Forward+backward through the C ABI on cuda:0; inputs are (b,h,n,d) CPU tensors."""
    dev = torch.device("cuda", 0)
    def prep(t):
        return t.to(dtype).reshape(-1, t.shape[-2], t.shape[-1]).contiguous().to(dev)
    q3, k3, v3, g3 = prep(q), prep(k), prep(v), prep(go)
    out, den, stats = _cabi.forward(q3, k3, v3, impl=impl, **kw)
    gq, gk, gv = _cabi.backward(q3, k3, v3, out, den, stats, g3, impl=impl, **kw)
    torch.cuda.synchronize()
    return [t.float().cpu().reshape(s.shape) for t, s in ((out, q), (gq, q), (gk, k), (gv, v))], den.cpu()


def oracle(q, k, v, go, dtype, dense=False, **kw):
    """Oracle on the inputs as the kernel sees them (rounded to `dtype`), in fp64."""
    r = lambda t: t.to(dtype).double()
    return fastmax_fwd_bwd(r(q), r(k), r(v), r(go), dense=dense, **kw)


def assert_close(got, ref, dtype, what="", floor=1e-2):
    """Relative max error per tensor; the denominator is floored at 1e-2 (inputs
    are O(1) Gaussians) so that gradients that are zero by construction, such as
    grad_q and grad_k at n == 1, compare by absolute error (callers raise the
    floor to the magnitude of the cancelling terms where bf16 rounding of an
    intermediate makes that cancellation inexact)."""
    for g, r, name in zip(got, ref, ("out", "dq", "dk", "dv")):
        e = float((g.double() - r.double()).abs().max() / r.double().abs().max().clamp_min(floor))
        assert e < TOL[dtype], f"{what} {name}: rel err {e:.3e} >= {TOL[dtype]}"
