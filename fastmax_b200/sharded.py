"""Fastmax attention (causal, or unmasked) over a sequence that is split across GPUs.

One process per GPU (``torch.distributed``); rank r holds the r-th contiguous
slice of the sequence for every head: ``q, k, v : (b*h, n_local, d)``.  The
reference has nothing like this (single device, hard-wired to ``cuda:0``,
reference ``fastmax_cuda_forward.cu:347``); what makes it possible is that the
reference's moment tensors (Sum v, Sum k(x)v, Sum k(x)k(x)v and their v=1
counterparts) are sums over tokens, so a shard only needs the *sum of the
totals* of the shards before it (forward, grad_q) or after it (grad_k, grad_v).

Per pass the ranks exchange

* with ``normalize``: one MAX all-reduce of the per-head statistics words
  (max row norm and its global row, packed in an int64) and, in backward, one
  SUM all-reduce of ``2*b*h`` floats for the gradient of the max-norm scaling;
* one all-gather of each rank's total state, ``b*h * (d*d+d+1) * (d+1)`` floats
  rounded up, followed by a local sum over the earlier (or later) ranks; unmasked
  attention needs the sum over all ranks instead, one SUM all-reduce of the totals.

Everything else is local and runs through the C ABI's ``fastmax_b200_shard_*``
stage calls.  The stage calls are reached through a small backend object so that
the exchange logic can be exercised on CPU ranks (gloo) with a stand-in backend.
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from . import _cabi

__all__ = ["CudaShardBackend", "SequenceShardedFastmax", "fastmax_sequence_parallel", "exclusive_rank_sum"]


class _Exchange:
    """Exchange of per-shard totals on CUDA without staging copies.

    One persistent ``(world, floats)`` buffer per (device, kind): the state kernels write this
    rank's total straight into its row, an in-place ``all_gather_into_tensor`` issued on a side
    stream fills the other rows while the caller's stream keeps computing, and one library
    kernel (``fastmax_b200_shard_sum_totals``) adds up the rows of the earlier (or later) ranks.
    """

    _buffers = {}
    _streams = {}

    @classmethod
    def buffer(cls, kind, device, world, floats):
        key = (kind, device, world, floats)
        buf = cls._buffers.get(key)
        if buf is None:
            buf = torch.empty(world, floats, dtype=torch.float32, device=device)
            cls._buffers[key] = buf
            cls._buffers[key + ("sum",)] = torch.empty(floats, dtype=torch.float32, device=device)
        return buf

    @classmethod
    def start(cls, gathered, rank, group):
        """Begin the all-gather of row ``rank`` of ``gathered`` into all rows; returns a handle."""
        dev = gathered.device
        side = cls._streams.get(dev)
        if side is None:
            side = cls._streams[dev] = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream(dev))        # the row has been written
        with torch.cuda.stream(side):
            return dist.all_gather_into_tensor(gathered, gathered[rank], group=group, async_op=True)

    @classmethod
    def finish(cls, kind, work, gathered, rank, reverse):
        """Wait (on the current stream) for the gather and return the sum over the ranks before
        ``rank`` (after it when ``reverse``), or None when there are none."""
        work.wait()
        world, floats = gathered.shape
        if (rank == world - 1) if reverse else (rank == 0):
            return None
        out = cls._buffers[(kind, gathered.device, world, floats, "sum")]
        with torch.cuda.device(gathered.device):
            _cabi._check(_cabi.lib().fastmax_b200_shard_sum_totals(
                gathered.data_ptr(), world, rank, int(reverse), floats, out.data_ptr(), _cabi._stream(gathered)),
                "shard_sum_totals")
        return out


def exclusive_rank_sum(total: torch.Tensor, group=None, reverse: bool = False):
    """Sum of ``total`` over the ranks before this one (after it when ``reverse``); None if there are none."""
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    parts = [torch.empty_like(total) for _ in range(world)]
    dist.all_gather(parts, total.contiguous(), group=group)
    pick = parts[rank + 1:] if reverse else parts[:rank]
    if not pick:
        return None
    acc = pick[0].clone()
    for t in pick[1:]:
        acc += t
    return acc


class CudaShardBackend:
    """The stage calls of ``include/fastmax_b200.h`` on the current CUDA device."""

    def __init__(self, mask=True, **kw):
        self.mask = bool(mask)
        self.kw = kw  # normalize, a0.., p, chunk as for _cabi.make_problem

    def _prob(self, q, k):
        kw = self.kw
        return _cabi.make_problem(q, k, self.mask, kw["normalize"], 1.0, kw["a0"], kw["a1"], kw["a2"], kw["lim"],
                                  kw["p"], "auto", kw.get("chunk", 0))

    @staticmethod
    def _ptr(t):
        return None if t is None else t.data_ptr()

    def rowmax(self, q, k, row_offset):
        L, prob = _cabi.lib(), self._prob(q, k)
        stats = torch.empty(q.shape[0] + k.shape[0], dtype=torch.int64, device=q.device)
        _cabi._check(L.fastmax_b200_shard_rowmax(prob, q.data_ptr(), k.data_ptr(), int(row_offset),
                                                 stats.data_ptr(), _cabi._stream(q)), "shard_rowmax")
        return stats

    def total_floats(self, k):
        return _cabi.lib().fastmax_b200_moment_total_bytes(self._prob(k, k)) // 4

    def kv_state(self, k, v, total_out=None):
        L, prob = _cabi.lib(), self._prob(k, k)
        states = torch.empty(L.fastmax_b200_moment_state_bytes(prob) // 4, dtype=torch.float32, device=k.device)
        total = total_out if total_out is not None else \
            torch.empty(L.fastmax_b200_moment_total_bytes(prob) // 4, dtype=torch.float32, device=k.device)
        _cabi._check(L.fastmax_b200_shard_kv_state(prob, k.data_ptr(), v.data_ptr(), states.data_ptr(),
                                                   total.data_ptr(), _cabi._stream(k)), "shard_kv_state")
        return states, total

    def forward(self, q, k, v, stats, kv_states, s_base):
        L, prob = _cabi.lib(), self._prob(q, k)
        out = torch.empty_like(q)
        den = torch.empty(q.shape[:2], dtype=torch.float32, device=q.device)
        wsb = L.fastmax_b200_shard_forward_workspace_bytes(prob)
        ws = torch.empty(max(wsb, 1), dtype=torch.uint8, device=q.device)
        _cabi._check(L.fastmax_b200_shard_forward(prob, q.data_ptr(), k.data_ptr(), v.data_ptr(), self._ptr(stats),
                                                  self._ptr(kv_states), self._ptr(s_base), out.data_ptr(),
                                                  den.data_ptr(), ws.data_ptr(), wsb, _cabi._stream(q)),
                     "shard_forward")
        return out, den

    def qg_state(self, q, out, den, go, total_out=None):
        L, prob = _cabi.lib(), self._prob(q, q)
        delta = torch.empty(q.shape[:2], dtype=torch.float32, device=q.device)
        states = torch.empty(L.fastmax_b200_moment_state_bytes(prob) // 4, dtype=torch.float32, device=q.device)
        total = total_out if total_out is not None else \
            torch.empty(L.fastmax_b200_moment_total_bytes(prob) // 4, dtype=torch.float32, device=q.device)
        wsb = L.fastmax_b200_shard_backward_workspace_bytes(prob)
        self._bwd_ws = torch.empty(max(wsb, 1), dtype=torch.uint8, device=q.device)   # reused by backward()
        _cabi._check(L.fastmax_b200_shard_qg_state(prob, q.data_ptr(), out.data_ptr(), den.data_ptr(), go.data_ptr(),
                                                   delta.data_ptr(), states.data_ptr(), total.data_ptr(),
                                                   self._bwd_ws.data_ptr(), wsb, _cabi._stream(q)), "shard_qg_state")
        return delta, states, total

    def dq_far(self, q, den, stats, go, delta, kv_states):
        """The part of grad_q that needs nothing from later shards (see ``fastmax_b200_shard_dq_far``); its
        result stays in the workspace that ``qg_state`` made and ``backward`` reuses."""
        L, prob = _cabi.lib(), self._prob(q, q)
        ws = self._bwd_ws
        _cabi._check(L.fastmax_b200_shard_dq_far(prob, q.data_ptr(), den.data_ptr(), self._ptr(stats), go.data_ptr(),
                                                 delta.data_ptr(), kv_states.data_ptr(), ws.data_ptr(), ws.numel(),
                                                 _cabi._stream(q)), "shard_dq_far")

    def backward(self, q, k, v, out, den, stats, go, delta, kv_states, qg_states, r_base, dq_far_done=False):
        L, prob = _cabi.lib(), self._prob(q, k)
        gq, gk, gv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        dots = torch.empty(q.shape[0] + k.shape[0], dtype=torch.float32, device=q.device)
        wsb = L.fastmax_b200_shard_backward_workspace_bytes(prob)
        ws = getattr(self, "_bwd_ws", None)
        if ws is None or ws.numel() < wsb or ws.device != q.device:
            ws = torch.empty(max(wsb, 1), dtype=torch.uint8, device=q.device)
        _cabi._check(L.fastmax_b200_shard_backward(
            prob, q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), den.data_ptr(), self._ptr(stats),
            go.data_ptr(), delta.data_ptr(), kv_states.data_ptr(), self._ptr(qg_states), self._ptr(r_base),
            dots.data_ptr(), gq.data_ptr(), gk.data_ptr(), gv.data_ptr(), int(bool(dq_far_done)), ws.data_ptr(), wsb,
            _cabi._stream(q)),
            "shard_backward")
        return gq, gk, gv, dots

    def norm_fixup(self, q, k, stats, dots, row_offset, gq, gk):
        L, prob = _cabi.lib(), self._prob(q, k)
        _cabi._check(L.fastmax_b200_shard_norm_fixup(prob, q.data_ptr(), k.data_ptr(), stats.data_ptr(),
                                                     dots.data_ptr(), int(row_offset), gq.data_ptr(), gk.data_ptr(),
                                                     _cabi._stream(q)), "shard_norm_fixup")


class SequenceShardedFastmax(torch.autograd.Function):
    """``apply(q, k, v, backend, normalize, group)`` on this rank's slice; returns its slice of the output."""

    @staticmethod
    def forward(ctx, q, k, v, backend, normalize, group):
        rank = dist.get_rank(group)
        n_local = q.shape[1]
        lens = [torch.zeros(1, dtype=torch.int64, device=q.device) for _ in range(dist.get_world_size(group))]
        dist.all_gather(lens, torch.tensor([n_local], dtype=torch.int64, device=q.device), group=group)
        if any(int(x) != n_local for x in lens):
            raise ValueError("every rank must hold the same number of tokens")
        row_offset = rank * n_local
        stats = None
        if normalize:
            stats = backend.rowmax(q, k, row_offset)
            dist.all_reduce(stats, op=dist.ReduceOp.MAX, group=group)
        fused = q.is_cuda and isinstance(backend, CudaShardBackend) and getattr(backend, "mask", True)
        if fused:
            # this rank's total is written straight into its row of the gather buffer
            world = dist.get_world_size(group)
            gathered = _Exchange.buffer("kv", q.device, world, backend.total_floats(k))
            kv_states, kv_total = backend.kv_state(k, v, total_out=gathered[rank])
            work = _Exchange.start(gathered, rank, group)
            s_base = _Exchange.finish("kv", work, gathered, rank, reverse=False)
            out, den = backend.forward(q, k, v, stats, kv_states, s_base)
            ctx.fused = True
            ctx.backend, ctx.group, ctx.normalize, ctx.row_offset = backend, group, normalize, row_offset
            ctx.save_for_backward(q, k, v, out, den, kv_states, *([stats] if normalize else []))
            return out
        ctx.fused = False
        kv_states, kv_total = backend.kv_state(k, v)
        if getattr(backend, "mask", True):
            s_base = exclusive_rank_sum(kv_total, group)
            out, den = backend.forward(q, k, v, stats, kv_states, s_base)
        else:
            # unmasked: every token reads the total of all shards
            kv_states = kv_total.clone()
            dist.all_reduce(kv_states, op=dist.ReduceOp.SUM, group=group)
            out, den = backend.forward(q, k, v, stats, None, kv_states)
        ctx.backend, ctx.group, ctx.normalize, ctx.row_offset = backend, group, normalize, row_offset
        ctx.save_for_backward(q, k, v, out, den, kv_states, *([stats] if normalize else []))
        return out

    @staticmethod
    def backward(ctx, grad_out):
        q, k, v, out, den, kv_states, *rest = ctx.saved_tensors
        stats = rest[0] if rest else None
        backend, group = ctx.backend, ctx.group
        go = grad_out.contiguous().to(q.dtype)
        if ctx.fused:
            rank, world = dist.get_rank(group), dist.get_world_size(group)
            gathered = _Exchange.buffer("qg", q.device, world, backend.total_floats(q))
            delta, qg_states, _ = backend.qg_state(q, out, den, go, total_out=gathered[rank])
            work = _Exchange.start(gathered, rank, group)
            backend.dq_far(q, den, stats, go, delta, kv_states)       # runs while the totals travel
            r_base = _Exchange.finish("qg", work, gathered, rank, reverse=True)
            gq, gk, gv, dots = backend.backward(q, k, v, out, den, stats, go, delta, kv_states, qg_states, r_base,
                                                dq_far_done=True)
            if ctx.normalize:
                dist.all_reduce(dots, op=dist.ReduceOp.SUM, group=group)
                backend.norm_fixup(q, k, stats, dots, ctx.row_offset, gq, gk)
            return gq, gk, gv, None, None, None
        delta, qg_states, qg_total = backend.qg_state(q, out, den, go)
        if getattr(backend, "mask", True):
            r_base = exclusive_rank_sum(qg_total, group, reverse=True)
        else:
            # unmasked: kv_states already holds the key/value total of all shards
            r_base, qg_states = qg_total.clone(), None
            dist.all_reduce(r_base, op=dist.ReduceOp.SUM, group=group)
        gq, gk, gv, dots = backend.backward(q, k, v, out, den, stats, go, delta, kv_states, qg_states, r_base)
        if ctx.normalize:
            dist.all_reduce(dots, op=dist.ReduceOp.SUM, group=group)
            backend.norm_fixup(q, k, stats, dots, ctx.row_offset, gq, gk)
        return gq, gk, gv, None, None, None


def fastmax_sequence_parallel(q, k, v, *, mask=True, normalize=False, a0=1.0, a1=1.0, a2=0.5, lim=1.0, p=2,
                              chunk=0, group=None, backend=None):
    """Fastmax (causal, or unmasked with ``mask=False``) on this rank's ``(b*h, n_local, d)`` slices of q, k, v
    (CUDA, float32 or bfloat16).

    Rank r of ``group`` must hold tokens ``[r*n_local, (r+1)*n_local)``, the same ``n_local`` on every rank
    (chunks of ``chunk`` tokens, default 2048, are laid out from the start of each shard).  Differentiable;
    gradients come back sharded the same way.
    """
    if backend is None:
        if not q.is_cuda:
            raise RuntimeError("fastmax_sequence_parallel needs CUDA tensors")
        backend = CudaShardBackend(mask=mask, normalize=bool(normalize), a0=a0, a1=a1, a2=a2, lim=lim, p=p, chunk=chunk)
    return SequenceShardedFastmax.apply(q.contiguous(), k.contiguous(), v.contiguous(), backend, bool(normalize),
                                        group)
