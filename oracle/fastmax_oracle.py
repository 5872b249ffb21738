"""CPU oracle for Fastmax attention -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.

This module restates, on the CPU, the algorithm of the reference's pure-PyTorch
path ``fastmax_function`` (reference ``example.py:83-197``), which is the only
self-consistent, fully general implementation the reference ships and the one
its ``use_custom_gradient=False`` switch selects.  It exists so that the CUDA
kernels can be checked against it.  Only the test-suite, the smoke check and the
CPU-baseline leg of the benchmark may import it; the product package never does.

Parity pin: ``tests/golden/make_golden.py`` runs the reference's own
``fastmax_function`` (lifted from the reference source with ``ast`` at
generation time) on seeded inputs and stores inputs, outputs and autograd
gradients in ``tests/golden/*.npz``; ``tests/test_oracle.py`` checks every
function in this file against those vectors.  The reference holds no golden
vectors or assertions of its own, so those generated fixtures are the pin.

Three evaluators are provided:

``fastmax_moments``   factorised (moment) evaluation following the reference's
                      operation order: normalise, build Sum v, Sum k(x)v,
                      Sum k(x)k(x)v and their v=1 counterparts (cumulative sums
                      when masked), contract with q and q(x)q, divide.  The
                      masked branch carries the running moments block by block,
                      so memory stays bounded at long n; with ``block=None`` it
                      is one cumulative sum over n as in the reference.
``fastmax_dense``     independent O(n^2) evaluation of
                      a0 + a1 (q.k) + a2 (q.k)^2, row-normalised
                      (semantics of reference ``example.py:199-212`` applied to
                      the normalised q, k); used to cross-check the factorised
                      form and for spot rows at lengths the factorised oracle
                      cannot hold in memory.
``fastmax_fwd_bwd``   forward plus autograd backward of either evaluator for a
                      fixed upstream gradient.
``fastmax_dense_fwd_bwd_blocked``
                      the same result as ``fastmax_fwd_bwd(dense=True)`` with the
                      query rows taken block by block, so that a head of 10^4 to
                      3x10^4 tokens fits in host memory.
"""
from __future__ import annotations

import torch

__all__ = [
    "normalize_qk",
    "fastmax_moments",
    "fastmax_dense",
    "fastmax_fwd_bwd",
    "fastmax_dense_fwd_bwd_blocked",
    "rel_err",
]


def normalize_qk(q: torch.Tensor, k: torch.Tensor, lim: float):
    """Per-head max-norm scaling (reference ``example.py:101-108``).

    ``x <- lim * x / max_n ||x_n||_2`` separately for q and k, the maximum taken
    over the sequence axis of each (batch, head).
    """
    qmax = torch.linalg.norm(q, dim=3).amax(dim=2)[..., None, None]
    kmax = torch.linalg.norm(k, dim=3).amax(dim=2)[..., None, None]
    return lim * q / qmax, lim * k / kmax


def _features(x: torch.Tensor, p: int):
    """Second-order features x (x) x flattened to d*d (reference ``example.py:117-120``)."""
    if p == 1:
        return None
    return (x.unsqueeze(-1) * x.unsqueeze(-2)).flatten(-2)


def fastmax_moments(q, k, v, mask=0, dropout_rate=0.0, normalize=0, temperature=1.0,
                    a0=1.0, a1=1.0, a2=0.5, lim=1.0, p=2, block=None):
    """Factorised Fastmax, (b, h, n, d) -> (b, h, nq, d).

    Follows reference ``example.py:100-197``.  ``temperature`` is accepted and,
    as in the reference (``example.py:102`` and ``:110-111`` both overwrite it
    with 1), has no effect.  ``dropout_rate`` must be 0: the reference's feature
    dropout is random and has no parity meaning.
    """
    if p not in (1, 2):
        raise ValueError(f"p must be 1 or 2, got: {p}")  # reference example.py:195-196
    if dropout_rate != 0.0:
        raise NotImplementedError("oracle covers dropout_rate == 0 only")
    if normalize:
        q, k = normalize_qk(q, k, lim)
    b, h, nq, d = q.shape
    nk = k.shape[2]
    q2, k2 = _features(q, p), _features(k, p)

    if not mask:
        # reference example.py:125-145 (p=2) and :167-181 (p=1): total moments.
        num = a0 * v.sum(-2, keepdim=True) + a1 * (q @ (k.transpose(-2, -1) @ v))
        den = a0 * nk + a1 * (q @ k.sum(-2).unsqueeze(-1))
        if p == 2:
            num = num + a2 * (q2 @ (k2.transpose(-2, -1) @ v))
            den = den + a2 * (q2 @ k2.sum(-2).unsqueeze(-1))
        return num / den

    # reference example.py:147-160 (p=2) and :183-193 (p=1): cumulative moments.
    if nq != nk:
        raise ValueError("the reference's masked branch needs nq == nk")
    n = nq
    step = n if block is None else int(block)
    out = []
    s_v = q.new_zeros(b, h, 1, d)
    s_k = q.new_zeros(b, h, 1, d)
    s_kv = q.new_zeros(b, h, 1, d, d)
    s_k2 = q.new_zeros(b, h, 1, d * d) if p == 2 else None
    s_k2v = q.new_zeros(b, h, 1, d * d, d) if p == 2 else None
    cnt = 0
    for lo in range(0, n, step):
        hi = min(lo + step, n)
        qb, kb, vb = q[:, :, lo:hi], k[:, :, lo:hi], v[:, :, lo:hi]
        c_v = s_v + torch.cumsum(vb, 2)
        c_k = s_k + torch.cumsum(kb, 2)
        c_kv = s_kv + torch.cumsum(kb.unsqueeze(-1) * vb.unsqueeze(-2), 2)
        ones = torch.arange(cnt + 1, cnt + hi - lo + 1, dtype=q.dtype, device=q.device)
        num = a0 * c_v + a1 * torch.einsum("bhij,bhijk->bhik", qb, c_kv)
        den = a0 * ones[None, None, :] + a1 * torch.einsum("bhij,bhij->bhi", qb, c_k)
        s_v, s_k, s_kv = c_v[:, :, -1:], c_k[:, :, -1:], c_kv[:, :, -1:]
        if p == 2:
            q2b, k2b = q2[:, :, lo:hi], k2[:, :, lo:hi]
            c_k2 = s_k2 + torch.cumsum(k2b, 2)
            c_k2v = s_k2v + torch.cumsum(k2b.unsqueeze(-1) * vb.unsqueeze(-2), 2)
            num = num + a2 * torch.einsum("bhij,bhijk->bhik", q2b, c_k2v)
            den = den + a2 * torch.einsum("bhij,bhij->bhi", q2b, c_k2)
            s_k2, s_k2v = c_k2[:, :, -1:], c_k2v[:, :, -1:]
        out.append(num / den.unsqueeze(-1))
        cnt += hi - lo
    return torch.cat(out, 2)


def fastmax_dense(q, k, v, mask=0, normalize=0, a0=1.0, a1=1.0, a2=0.5, lim=1.0, p=2,
                  rows=None):
    """Independent O(n^2) evaluation; ``rows`` restricts the query rows computed.

    Row-normalised polynomial attention (reference ``example.py:199-212``
    semantics) on the normalised q, k.  Causal alignment for nq != nk puts the
    queries on the last nq keys (reference ``fastmax_cuda_forward.cu:109``).
    """
    if p not in (1, 2):
        raise ValueError(f"p must be 1 or 2, got: {p}")
    if normalize:
        q, k = normalize_qk(q, k, lim)
    nq, nk = q.shape[2], k.shape[2]
    idx = torch.arange(nq) if rows is None else torch.as_tensor(rows)
    s = q[:, :, idx] @ k.transpose(-2, -1)
    attn = a0 + a1 * s
    if p == 2:
        attn = attn + a2 * s * s
    if mask:
        allowed = torch.arange(nk)[None, :] <= (idx[:, None] + (nk - nq))
        attn = attn * allowed.to(attn.dtype)
    return (attn @ v) / attn.sum(-1, keepdim=True)


def fastmax_fwd_bwd(q, k, v, go, *, dense=False, **kw):
    """Forward and autograd backward; returns (out, dq, dk, dv) detached."""
    q = q.detach().clone().requires_grad_(True)
    k = k.detach().clone().requires_grad_(True)
    v = v.detach().clone().requires_grad_(True)
    if dense:
        kw = {a: b for a, b in kw.items() if a not in ("temperature", "dropout_rate", "block")}
        out = fastmax_dense(q, k, v, **kw)
    else:
        out = fastmax_moments(q, k, v, **kw)
    out.backward(go)
    return out.detach(), q.grad, k.grad, v.grad


def fastmax_dense_fwd_bwd_blocked(q, k, v, go, *, mask=0, normalize=0, a0=1.0, a1=1.0, a2=0.5, lim=1.0,
                                  p=2, block=1024):
    """``fastmax_fwd_bwd(dense=True)`` evaluated over blocks of ``block`` query rows.

    The max-norm scaling (reference ``example.py:101-108``) is taken once, outside the blocks,
    and autograd is run in two stages: every row block back-propagates into the scaled q and k
    (a causal block only touches the keys it may see), and the accumulated gradients are then
    pushed through the scaling.  Memory is ``block x nk`` instead of ``nq x nk``.
    Returns (out, dq, dk, dv) detached.
    """
    q = q.detach().clone().requires_grad_(True)
    k = k.detach().clone().requires_grad_(True)
    qs, ks = normalize_qk(q, k, lim) if normalize else (q, k)
    qd = qs.detach().requires_grad_(True)
    kd = ks.detach().requires_grad_(True)
    vd = v.detach().clone().requires_grad_(True)
    nq, nk = q.shape[2], k.shape[2]
    outs = []
    for lo in range(0, nq, block):
        hi = min(lo + block, nq)
        kcut = min(nk, hi + (nk - nq)) if mask else nk      # keys the block's last row may see
        sc = qd[:, :, lo:hi] @ kd[:, :, :kcut].transpose(-2, -1)
        attn = a0 + a1 * sc
        if p == 2:
            attn = attn + a2 * sc * sc
        if mask:
            rows = torch.arange(lo, hi)
            attn = attn * (torch.arange(kcut)[None, :] <= rows[:, None] + (nk - nq)).to(attn.dtype)
        ob = (attn @ vd[:, :, :kcut]) / attn.sum(-1, keepdim=True)
        ob.backward(go[:, :, lo:hi])
        outs.append(ob.detach())
    if normalize:
        torch.autograd.backward([qs, ks], [qd.grad, kd.grad])
        dq, dk = q.grad, k.grad
    else:
        dq, dk = qd.grad, kd.grad
    return torch.cat(outs, 2), dq, dk, vd.grad


def rel_err(x: torch.Tensor, ref: torch.Tensor) -> float:
    """max|x - ref| / max|ref| over the whole tensor (the parity metric).

    The denominator is floored at 1e-6 so that an identically zero reference
    (the n=1 gradients of q and k) compares by absolute error."""
    ref = ref.double()
    return float((x.double() - ref).abs().max() / ref.abs().max().clamp_min(1e-6))
