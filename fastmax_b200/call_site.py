"""Fastmax attention at the transformer call site of the reference's model.

The reference's ``CausalSelfAttention.forward`` (``model.py:472-499``) views the
packed projection as (B, T, G, Q+2, hs), permutes and splits it into q, k, v,
expands k and v to the query head count, applies rotary embeddings
(``apply_rope``, ``model.py:812-825``), copies the three views with
``.contiguous()`` and calls the attention (``model.py:557-575``); the result is
transposed back (``model.py:603``) and flattened to (B, T, H*hs) by the caller.

``fastmax_attention_from_qkv`` does the same with two kernel passes around the
attention kernels instead of a dozen elementwise ones: one that reads the
projection once and writes rotated per-head q, k, v (k and v stay at G heads;
the attention kernels take grouped heads natively) and its mirror image in the
backward pass.  The transposition to (B, T, H, hs) costs no pass where the
tensor-core kernels run (bf16, head size 64 or 128): the forward kernel writes
its result in that layout and the backward's preparation pass reads the
incoming gradient from it.  Other problems (fp32, small heads) swap the axes
with one more pass each way.  Every pass goes through the C ABI; nothing here
computes on the CPU.
"""
from __future__ import annotations

import torch

from . import _cabi

__all__ = ["fastmax_attention_from_qkv"]


class _FromQKV(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv5, cos, sin, rope_n, kw):
        b, n, g, total, d = qkv5.shape
        heads = g * (total - 2)
        q, k, v = _cabi.qkv_split_rope(qkv5, cos, sin, rope_n)
        ctx.kw, ctx.rope_n, ctx.dims = kw, rope_n, (b, n, heads, d)
        ctx.bt = _cabi.bt_layout_supported(q, k, heads, **kw)
        if ctx.bt:      # the attention kernel writes (B, T, H, hs) itself
            out, den, stats = _cabi.forward_bt(q, k, v, heads, **kw)
            ctx.save_for_backward(q, k, v, out, den, stats, cos, sin)
            return out.view(b, n, heads * d)
        out, den, stats = _cabi.forward(q, k, v, **kw)
        ctx.save_for_backward(q, k, v, out, den, stats, cos, sin)
        return _cabi.swap_middle_axes(out.view(b, heads, n, d)).view(b, n, heads * d)

    @staticmethod
    def backward(ctx, grad_y):
        q, k, v, out, den, stats, cos, sin = ctx.saved_tensors
        b, n, heads, d = ctx.dims
        gy = grad_y.to(q.dtype).contiguous().view(b, n, heads, d)
        if ctx.bt:
            gq, gk, gv = _cabi.backward_bt(q, k, v, out, den, stats, gy, heads, **ctx.kw)
        else:
            go = _cabi.swap_middle_axes(gy).view(b * heads, n, d)
            gq, gk, gv = _cabi.backward(q, k, v, out, den, stats, go, **ctx.kw)
        t = ctx.kw["temperature"]
        if t != 1.0:
            gk = gk / t               # as the reference wrapper does (example.py:80)
        return _cabi.qkv_merge_rope_grad(gq, gk, gv, cos, sin, ctx.rope_n, b), None, None, None, None


def fastmax_attention_from_qkv(qkv, cos, sin, n_head, n_query_groups, head_size, rope_n_elem, mask=True,
                               normalize=True, temperature=1.0, a0=1.0, a1=1.0, a2=0.5, lim=1.0, p=1,
                               impl="auto"):
    """Rotary embedding + Fastmax attention on the packed projection.

    ``qkv`` is the output of the model's fused projection, (B, T, (n_head + 2 *
    n_query_groups) * head_size), float32 or bfloat16 on a CUDA device; ``cos``
    and ``sin`` are the rotary tables for these T positions, (T, rope_n_elem).
    Returns (B, T, n_head * head_size), ready for the output projection.  The
    defaults are the constants of the reference's call site
    (``model.py:561-570``: causal, normalised, a = (1, 1, 0.5), lim = 1, p = 1).
    """
    if qkv.dim() != 3:
        raise ValueError("qkv must be (B, T, (n_head + 2 * n_query_groups) * head_size)")
    if n_head % n_query_groups:
        raise ValueError("n_head must be a multiple of n_query_groups")
    qper = n_head // n_query_groups
    b, n, width = qkv.shape
    if width != (qper + 2) * n_query_groups * head_size:
        raise ValueError(f"qkv width {width} does not match the head configuration")
    if not qkv.is_cuda:
        raise RuntimeError("fastmax_attention_from_qkv needs CUDA tensors (there is no CPU path)")
    kw = dict(mask=bool(mask), normalize=bool(normalize), temperature=temperature, a0=a0, a1=a1, a2=a2,
              lim=lim, p=p, impl=impl)
    qkv5 = qkv.contiguous().view(b, n, n_query_groups, qper + 2, head_size)
    if rope_n_elem:
        cos = cos.to(device=qkv.device, dtype=torch.float32).contiguous()
        sin = sin.to(device=qkv.device, dtype=torch.float32).contiguous()
    else:
        cos = sin = torch.empty(0, device=qkv.device)
    return _FromQKV.apply(qkv5, cos, sin, int(rope_n_elem), kw)
