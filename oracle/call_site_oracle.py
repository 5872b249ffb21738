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
                            ``:396-399``).

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

__all__ = ["rope", "split_heads", "call_site", "output_dropout"]


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
