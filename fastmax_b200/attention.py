"""Host-side mirror of the reference's Python interface for Fastmax attention.

Same names, argument order and meaning as the reference's ``example.py``:

* ``FASTMultiHeadAttention_Function`` -- autograd function over the CUDA kernels
  (reference ``example.py:6-80``),
* ``FASTMultiHeadAttention``          -- the ``nn.Module`` front end
  (reference ``example.py:214-221``),
* ``fastmax_function``                -- the pure-PyTorch evaluation selected by
  ``use_custom_gradient=False`` (reference ``example.py:83-212``),
* ``rpe_matrix_creator``              -- helper of the reference's timing script
  (reference ``test_fastmax.py:251-280``); the matrix is accepted and unused, as
  in every kernel version of the reference.

Differences from the reference, all deliberate: inputs are never modified
(the reference rescales q and k in place), no layout permutes are made, bf16 is
supported besides fp32, the custom path serves unmasked as well as causal
attention, its gradients include the derivative of the max-norm scaling, and a
CPU tensor on the custom path is an error instead of a silent pass-through.
"""
from __future__ import annotations

import math

import torch

from . import _cabi

__all__ = ["FASTMultiHeadAttention_Function", "FASTMultiHeadAttention", "fastmax_function",
           "rpe_matrix_creator"]


def _to3d(t: torch.Tensor) -> torch.Tensor:
    if t.dim() == 4:
        return t.reshape(t.shape[0] * t.shape[1], t.shape[2], t.shape[3]).contiguous()
    if t.dim() == 3:
        return t.contiguous()
    raise ValueError("q, k, and v should be either 3 or 4 dimensional tensors. "
                     "If 3D: (b*h,n,d), if 4D: (b,h,n,d).")


class FASTMultiHeadAttention_Function(torch.autograd.Function):
    """Fastmax attention with hand-written forward and backward kernels.

    ``apply(q, k, v, drop_noise, mask, dropout, normalize, temperature, a0, a1,
    a2, lim, p)`` -- the reference's argument list.  q, k, v are (b,h,n,d) or
    (b*h,n,d) CUDA tensors in float32 or bfloat16; the result has q's shape and
    dtype.  With ``dropout > 0`` the result is multiplied elementwise by
    ``1 + dropout * drop_noise`` (``drop_noise`` shaped like q), the reference's
    output dropout (``fastmax_cuda_forward.cu:271-280, 396-399``); the gradient
    is the exact derivative of that product (the reference's backward instead
    feeds the noised output into its gradient formulas).  ``temperature`` has no effect on the value (as in the reference's
    PyTorch path); grad_k is divided by it as the reference wrapper does
    (reference ``example.py:80``).  ``impl`` selects a kernel family and is
    meant for tests.
    """

    @staticmethod
    def forward(ctx, q, k, v, drop_noise=None, mask=False, dropout=0.0, normalize=False,
                temperature=1.0, a0=1.0, a1=1.0, a2=0.5, lim=1.0, p=2, impl="auto"):
        if not q.is_cuda:
            raise RuntimeError("FASTMultiHeadAttention_Function needs CUDA tensors; "
                               "use fastmax_function for the pure-PyTorch path")
        if dropout < 0.0:
            raise ValueError(f"dropout must be non-negative, got: {dropout}")
        if dropout > 0.0 and (drop_noise is None or drop_noise.shape != q.shape):
            raise ValueError("dropout > 0 needs drop_noise with the shape of q")
        shape_q, shape_k = q.shape, k.shape
        q3, k3, v3 = _to3d(q), _to3d(k), _to3d(v)
        kw = dict(mask=bool(mask), normalize=bool(normalize), temperature=temperature,
                  a0=a0, a1=a1, a2=a2, lim=lim, p=p, impl=impl)
        out, den, stats = _cabi.forward(q3, k3, v3, **kw)
        noise = None
        if dropout > 0.0:
            noise = _to3d(drop_noise.to(q3.dtype))
        ctx.save_for_backward(q3, k3, v3, out, den, stats, noise)
        ctx.kw = kw
        ctx.dropout = float(dropout)
        ctx.shape_q, ctx.shape_k = shape_q, shape_k
        if noise is not None:
            out = _cabi.scale_by_noise(out, noise, ctx.dropout)
        return out.reshape(shape_q)

    @staticmethod
    def backward(ctx, grad_output):
        q3, k3, v3, out, den, stats, noise = ctx.saved_tensors
        go = grad_output.reshape(q3.shape).contiguous()
        if go.dtype != q3.dtype:
            go = go.to(q3.dtype)
        if noise is not None:
            go = _cabi.scale_by_noise(go, noise, ctx.dropout)
        gq, gk, gv = _cabi.backward(q3, k3, v3, out, den, stats, go, **ctx.kw)
        t = ctx.kw["temperature"]
        if t != 1.0:
            gk = gk / t
        return (gq.reshape(ctx.shape_q), gk.reshape(ctx.shape_k), gv.reshape(ctx.shape_k),
                None, None, None, None, None, None, None, None, None, None, None)


def fastmax_function(q, k, v, mask=0, dropout_rate=0.0, normalize=0, temperature=1, a0=1, a1=1,
                     a2=0.5, lim=1, p=2, create_attn_matrix=0, block=1024):
    """Pure-PyTorch Fastmax on (b,h,n,d) tensors, differentiable by autograd.

    Same signature and results as the reference's ``fastmax_function``
    (``example.py:83-212``); runs on whatever device the tensors live on.  The
    causal branch carries the running moments over blocks of ``block`` tokens
    instead of materialising an (n, d^2, d) cumulative sum, so memory is linear
    in n.  ``create_attn_matrix != 0`` returns ``(ans, attn)`` from the dense
    n x n form; there ``mask`` is a tensor (or None) marking allowed pairs and,
    as in the reference, q and k are not normalised.
    """
    if create_attn_matrix:
        s = q @ k.transpose(-2, -1)
        attn = a0 + a1 * s / temperature + a2 * s * s / (temperature * temperature)
        if mask is not None:
            attn = torch.where(mask == 0, 0, attn)
        attn = attn / attn.sum(-1, keepdim=True)
        return attn @ v, attn
    if p not in (1, 2):
        raise ValueError(f"p must be 1 or 2, got: {p}")
    if normalize:
        qn = torch.linalg.norm(q, dim=3).amax(dim=2)[..., None, None]
        kn = torch.linalg.norm(k, dim=3).amax(dim=2)[..., None, None]
        q, k = lim * q / qn, lim * k / kn
    if dropout_rate:
        drop = torch.nn.Dropout(p=dropout_rate)
    d = q.shape[-1]
    if p == 2:
        def feat(x):
            x2 = (x.unsqueeze(-1) * x.unsqueeze(-2)).flatten(-2)
            return torch.cat([x, drop(x2) if dropout_rate else x2], -1)
        wts = torch.cat([q.new_full((d,), float(a1)), q.new_full((d * d,), float(a2))])
    else:
        def feat(x):
            return drop(x) if dropout_rate else x
        wts = q.new_full((d,), float(a1))
    ones = v.new_ones(v.shape[:-1] + (1,))
    vt = torch.cat([v, ones], -1)                       # value columns + the normaliser column
    if not mask:
        fk = feat(k)
        state = fk.transpose(-2, -1) @ vt               # (b,h,F,d+1)
        num = (feat(q) * wts) @ state + a0 * vt.sum(-2, keepdim=True)
        return num[..., :d] / num[..., d:]
    n = q.shape[2]
    outs = []
    state = None
    s0 = vt.new_zeros(vt.shape[:2] + (1, d + 1))
    for lo in range(0, n, block):
        hi = min(lo + block, n)
        fq = feat(q[:, :, lo:hi]) * wts
        fk = feat(k[:, :, lo:hi])
        vb = vt[:, :, lo:hi]
        sc = fq @ fk.transpose(-2, -1) + a0            # scores inside the block
        num = torch.tril(sc) @ vb + a0 * s0
        if state is not None:
            num = num + fq @ state
        outs.append(num[..., :d] / num[..., d:])
        upd = fk.transpose(-2, -1) @ vb
        state = upd if state is None else state + upd
        s0 = s0 + vb.sum(-2, keepdim=True)
    return torch.cat(outs, 2)


class FASTMultiHeadAttention(torch.nn.Module):
    """``FASTMultiHeadAttention(use_custom_gradient=True)(q, k, v, drop_noise=None,
    mask=False, dropout=0.0, normalize=False, temperature=1.0, a0=1.0, a1=1.0,
    a2=0.5, lim=1.0, p=2)`` -> tensor shaped like q.

    With ``use_custom_gradient`` the CUDA kernels run, for causal and unmasked
    attention alike (the dispatch of the reference's ``model.py:207-216`` and
    ``test_fastmax.py:242-249``); otherwise ``fastmax_function`` does.
    ``rpe_matrix`` may be passed by keyword, as the reference's timing script
    does, and is ignored.
    """

    def __init__(self, use_custom_gradient=True):
        super().__init__()
        self.use_custom_gradient = use_custom_gradient

    def forward(self, q, k, v, drop_noise=None, mask=False, dropout=0.0, normalize=False,
                temperature=1.0, a0=1.0, a1=1.0, a2=0.5, lim=1.0, p=2, rpe_matrix=None):
        if self.use_custom_gradient:
            return FASTMultiHeadAttention_Function.apply(q, k, v, drop_noise, mask, dropout, normalize,
                                                         temperature, a0, a1, a2, lim, p)
        if q.dim() == 3:
            return fastmax_function(q[None], k[None], v[None], mask, dropout, normalize, temperature,
                                    a0, a1, a2, lim, p)[0]
        return fastmax_function(q, k, v, mask, dropout, normalize, temperature, a0, a1, a2, lim, p)


def rpe_matrix_creator(n, d, device, dtype, structured=False, is_zero=True):
    """(2n-1, d) relative-position matrix: zeros, Gaussian, or sin/cos when ``structured``."""
    if not structured:
        if is_zero:
            return torch.zeros(2 * n - 1, d, device=device, dtype=dtype)
        return torch.randn(2 * n - 1, d, device=device, dtype=dtype)
    pos = torch.arange(n, device=device, dtype=dtype).unsqueeze(1)
    freq = torch.exp(torch.arange(0, d, 2, device=device, dtype=dtype) * -(math.log(10000.0) / d))
    plus = torch.zeros(n, d, device=device, dtype=dtype)
    minus = torch.zeros(n, d, device=device, dtype=dtype)
    plus[:, 0::2], plus[:, 1::2] = torch.sin(pos * freq), torch.cos(pos * freq)
    minus[:, 0::2], minus[:, 1::2] = torch.sin(-pos * freq), torch.cos(-pos * freq)
    return torch.cat([plus.flip(0), minus[1:]], 0)
