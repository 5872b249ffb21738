"""CPU oracle for the attention call site -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.

Restates, with plain torch ops on the CPU, what the reference's model does
between its fused projection and its output projection when the Fastmax branch
is taken:

``rope``                    ``apply_rope`` (reference ``model.py:812-825``);
``call_site``               view / permute / split / expand / rotate / attention /
                            transpose (reference ``model.py:472-499, 557-603``),
                            the attention itself being ``fastmax_dense`` of the
                            attention oracle;
``output_dropout``          ``o * (1 + dropout * drop_noise)`` (reference
                            ``fastmax_cuda_forward.cu:271-280``, applied at
                            ``:396-399``);
``MomentState``             the recurrence a decoder can keep instead of the
                            reference's key/value cache (``model.py:501-504,
                            828-852``): running sums of (v,1), k (x) (v,1) and
                            k (x) k (x) (v,1) over raw keys plus the running
                            max |k|; ``tests/test_oracle.py`` checks that a step
                            equals the dense attention row over the tokens so far.

Parity pin: ``tests/golden/make_golden_rope.py`` lifts ``apply_rope`` out of the
reference source with ``ast`` and stores its outputs on seeded inputs in
``tests/golden/rope.npz``; ``tests/test_oracle.py`` checks ``rope`` against them.
The rest of the call site is tensor reshaping whose reference (``model.py``)
cannot be imported here (it needs the absent ``litgpt`` package), so those lines
are restated by reading and the parity of the reshaping is unpinned.  The output
dropout is pinned by reading as well: the reference extension that holds it does
not link at its current head.

Only the test-suite may import this module.
"""
from __future__ import annotations

import torch

from .fastmax_oracle import fastmax_dense

__all__ = ["rope", "split_heads", "call_site", "output_dropout", "MomentState"]


def rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x (..., T, r), cos / sin (T, r): x * cos + (-x2, x1) * sin, rounded to x's dtype."""
    r = x.size(-1)
    x1, x2 = x[..., : r // 2], x[..., r // 2:]
    rotated = torch.cat((-x2, x1), dim=-1)
    return (x * cos + rotated * sin).to(x.dtype)


def split_heads(qkv, cos, sin, n_head, n_query_groups, head_size, rope_n, expand=True):
    """qkv (B, T, (n_head + 2 G) hs) -> q (B, H, T, hs), k, v (B, H or G, T, hs), q and k rotated."""
    b, t, _ = qkv.shape
    qper = n_head // n_query_groups
    x = qkv.view(b, t, n_query_groups, qper + 2, head_size).permute(0, 2, 3, 1, 4)
    q, k, v = x.split((qper, 1, 1), dim=2)
    if expand:
        k = k.expand(b, n_query_groups, qper, t, head_size)
        v = v.expand(b, n_query_groups, qper, t, head_size)
    q, k, v = [y.reshape(b, -1, t, head_size) for y in (q, k, v)]
    if rope_n:
        q = torch.cat((rope(q[..., :rope_n], cos, sin), q[..., rope_n:]), dim=-1)
        k = torch.cat((rope(k[..., :rope_n], cos, sin), k[..., rope_n:]), dim=-1)
    return q, k, v


def call_site(qkv, cos, sin, n_head, n_query_groups, head_size, rope_n, round_dtype=None, **kw):
    """(B, T, n_head * hs): the reference's Fastmax branch, differentiable by autograd.

    With ``round_dtype`` the rotated q, k (and v) are rounded to that dtype before the attention, as
    they are in a reduced-precision model (``apply_rope`` ends in ``.to(dtype=x.dtype)``); the
    rounding passes gradients straight through, which is what a backward pass in that precision
    computes."""
    q, k, v = split_heads(qkv, cos, sin, n_head, n_query_groups, head_size, rope_n)
    if round_dtype is not None:
        q, k, v = [y + (y.detach().to(round_dtype).to(y.dtype) - y.detach()) for y in (q, k, v)]
    o = fastmax_dense(q, k, v, **kw)
    b, _, t, _ = o.shape
    return o.transpose(1, 2).reshape(b, t, n_head * head_size)


def output_dropout(o: torch.Tensor, drop_noise: torch.Tensor, dropout: float) -> torch.Tensor:
    return o * (1 + dropout * drop_noise)


class MomentState:
    """Per-head running moments of raw keys and values; float64, CPU, heads on the leading axis."""

    def __init__(self, heads, d, p=2, normalize=True, a0=1.0, a1=1.0, a2=0.5, lim=1.0):
        self.p, self.normalize, self.a0, self.a1, self.a2, self.lim = p, normalize, a0, a1, a2, lim
        self.s0 = torch.zeros(heads, d + 1, dtype=torch.float64)
        self.s1 = torch.zeros(heads, d, d + 1, dtype=torch.float64)
        self.s2 = torch.zeros(heads, d, d, d + 1, dtype=torch.float64)
        self.kmax = torch.zeros(heads, dtype=torch.float64)

    def append(self, k, v):
        """k, v: (heads, n, d)."""
        vt = torch.cat([v.double(), torch.ones_like(v[..., :1], dtype=torch.float64)], dim=-1)
        k = k.double()
        self.s0 += vt.sum(1)
        self.s1 += torch.einsum("hna,hnc->hac", k, vt)
        if self.p == 2:
            self.s2 += torch.einsum("hna,hnb,hnc->habc", k, k, vt)
        self.kmax = torch.maximum(self.kmax, k.norm(dim=-1).amax(dim=-1))

    def step(self, q, k, v):
        """Add one token (heads, 1, d) and return the attention row of q (heads, 1, d)."""
        self.append(k, v)
        q = q.double()[:, 0]
        s = (self.lim / q.norm(dim=-1)) * (self.lim / self.kmax) if self.normalize else torch.ones_like(self.kmax)
        num = self.a0 * self.s0 + self.a1 * s[:, None] * torch.einsum("ha,hac->hc", q, self.s1)
        if self.p == 2:
            num = num + self.a2 * (s * s)[:, None] * torch.einsum("ha,hb,habc->hc", q, q, self.s2)
        return (num[:, :-1] / num[:, -1:])[:, None]
