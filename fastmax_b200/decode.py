"""Decoding with a persistent moment state instead of a key/value cache.

The reference's model keeps every earlier key and value and calls the attention with one
query row per new token (``model.py:501-504, 828-852``).  For causal Fastmax attention the
same row follows from a fixed-size state per key/value head -- the sums of ``(v, 1)``,
``k (x) (v, 1)`` and, for p = 2, ``k (x) k (x) (v, 1)`` over the tokens so far -- so a step
costs the same at every length.  ``FastmaxDecodeState`` owns that state on the GPU;
``append`` consumes a prompt, ``step`` one new token.  All arithmetic runs in the CUDA
library (``fastmax_b200_decode_*``); there is no CPU path.
"""
from __future__ import annotations

import torch

from . import _cabi

__all__ = ["FastmaxDecodeState"]


class FastmaxDecodeState:
    """State of ``bhkv`` key/value heads serving ``bh`` query heads (``bh`` a multiple of ``bhkv``).

    ``step(q, k, v)`` with q (bh, 1, d) and k, v (bhkv, 1, d) returns what the attention gives
    for that query row over all tokens added so far: keys scaled by ``lim / max |k|`` over all of
    them and the query by ``lim / |q|`` when ``normalize`` is set.
    """

    def __init__(self, bh, bhkv, d, dtype=torch.bfloat16, device="cuda", normalize=True, a0=1.0, a1=1.0,
                 a2=0.5, lim=1.0, p=2):
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise RuntimeError("FastmaxDecodeState lives on a CUDA device (there is no CPU path)")
        if self.device.index is None:
            self.device = torch.device("cuda", torch.cuda.current_device())
        if p not in (1, 2):
            raise ValueError(f"p must be 1 or 2, got: {p}")
        self.bh, self.bhkv, self.d, self.dtype = int(bh), int(bhkv), int(d), dtype
        probe = torch.empty(0, dtype=dtype)
        self.prob = _cabi.Problem(dtype=_cabi._dtype_code(probe), bh=self.bh, bhkv=self.bhkv, nq=1, nk=1, d=self.d,
                                  mask=1, normalize=int(bool(normalize)), p=int(p), impl=0, a0=float(a0),
                                  a1=float(a1), a2=float(a2), lim=float(lim), temperature=1.0, chunk=0)
        L = _cabi.lib()
        with torch.cuda.device(self.device):
            self.state = torch.zeros(max(L.fastmax_b200_decode_state_bytes(self.prob), 4) // 4,
                                     dtype=torch.float32, device=self.device)
            self.scratch = torch.empty(max(L.fastmax_b200_decode_scratch_bytes(self.prob), 4) // 4,
                                       dtype=torch.float32, device=self.device)
        self.tokens = 0

    def reset(self):
        self.state.zero_()
        self.tokens = 0

    def _check(self, t, heads, name):
        if t.device != self.device or t.dtype != self.dtype or not t.is_contiguous() or t.dim() != 3 \
                or t.shape[0] != heads or t.shape[2] != self.d:
            raise ValueError(f"{name} must be a contiguous ({heads}, n, {self.d}) {self.dtype} tensor on {self.device}")

    def append(self, k, v):
        """Add the tokens of k, v (bhkv, n, d) to the state."""
        self._check(k, self.bhkv, "k")
        self._check(v, self.bhkv, "v")
        if k.shape != v.shape:
            raise ValueError("k and v differ in shape")
        with torch.cuda.device(self.device):
            rc = _cabi.lib().fastmax_b200_decode_append(self.prob, k.data_ptr(), v.data_ptr(), k.shape[1],
                                                        self.state.data_ptr(), _cabi._stream(k))
        _cabi._check(rc, "fastmax_b200_decode_append")
        self.tokens += k.shape[1]

    def step(self, q, k, v):
        """Add one token and return the attention row of q (bh, 1, d) over all tokens so far."""
        self._check(q, self.bh, "q")
        self._check(k, self.bhkv, "k")
        self._check(v, self.bhkv, "v")
        if q.shape[1] != 1 or k.shape[1] != 1 or v.shape[1] != 1:
            raise ValueError("step takes exactly one token")
        out = torch.empty_like(q)
        with torch.cuda.device(self.device):
            rc = _cabi.lib().fastmax_b200_decode_step(self.prob, q.data_ptr(), k.data_ptr(), v.data_ptr(),
                                                      self.state.data_ptr(), self.scratch.data_ptr(),
                                                      out.data_ptr(), _cabi._stream(q))
        _cabi._check(rc, "fastmax_b200_decode_step")
        self.tokens += 1
        return out
