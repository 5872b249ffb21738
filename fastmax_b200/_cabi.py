"""ctypes binding of the fastmax_b200 C ABI (``include/fastmax_b200.h``).

torch supplies device memory and the current stream; every compute call goes
through the shared library.  There is no fallback: if the library is missing
or a call fails, a ``RuntimeError`` is raised.
"""
from __future__ import annotations

import ctypes
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libfastmax_b200.so")

F32, BF16 = 0, 1
IMPL = {"auto": 0, "dense_ffma": 1, "dense_tc": 2, "moments": 3, "moments_ffma": 4}

EXPORTS = (
    "fastmax_b200_version", "fastmax_b200_last_error", "fastmax_b200_stats_bytes", "fastmax_b200_selected_impl",
    "fastmax_b200_forward_workspace_bytes", "fastmax_b200_backward_workspace_bytes",
    "fastmax_b200_forward", "fastmax_b200_forward_packed", "fastmax_b200_backward",
    "fastmax_b200_forward_bt", "fastmax_b200_backward_bt", "fastmax_b200_bt_layout_supported",
    "fastmax_b200_launch_count", "fastmax_b200_profile_enable", "fastmax_b200_profile_count",
    "fastmax_b200_profile_get", "fastmax_b200_device_status", "fastmax_b200_device_status_reset",
    "fastmax_b200_wait_selftest",
    "fastmax_b200_moment_state_bytes", "fastmax_b200_moment_total_bytes",
    "fastmax_b200_shard_forward_workspace_bytes", "fastmax_b200_shard_backward_workspace_bytes",
    "fastmax_b200_shard_rowmax", "fastmax_b200_shard_kv_state", "fastmax_b200_shard_forward",
    "fastmax_b200_shard_qg_state", "fastmax_b200_shard_backward", "fastmax_b200_shard_norm_fixup",
    "fastmax_b200_shard_dq_far", "fastmax_b200_shard_sum_totals",
    "fastmax_b200_static_scratch_bytes", "fastmax_b200_backward_static",
    "fastmax_b200_qkv_split_rope", "fastmax_b200_qkv_merge_rope_grad", "fastmax_b200_swap_middle_axes",
    "fastmax_b200_scale_by_noise", "fastmax_b200_scale_packed_by_noise",
    "fastmax_b200_decode_state_bytes", "fastmax_b200_decode_scratch_bytes", "fastmax_b200_decode_append",
    "fastmax_b200_decode_step",
)


class Problem(ctypes.Structure):
    """``struct fastmax_problem``."""
    _fields_ = [(n, ctypes.c_int32) for n in
                ("dtype", "bh", "bhkv", "nq", "nk", "d", "mask", "normalize", "p", "impl")] + \
               [(n, ctypes.c_float) for n in ("a0", "a1", "a2", "lim", "temperature")] + \
               [("chunk", ctypes.c_int32)]


_lib = None


def lib() -> ctypes.CDLL:
    """Load the shared library once; raise if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m fastmax_b200.build` "
                "(fastmax_b200 has no fallback path)")
        L = ctypes.CDLL(LIB_PATH)
        vp, sz, pp = ctypes.c_void_p, ctypes.c_size_t, ctypes.POINTER(Problem)
        L.fastmax_b200_version.restype = ctypes.c_int
        L.fastmax_b200_last_error.restype = ctypes.c_char_p
        for f in ("stats_bytes", "forward_workspace_bytes", "backward_workspace_bytes"):
            fn = getattr(L, "fastmax_b200_" + f)
            fn.restype, fn.argtypes = sz, [pp]
        L.fastmax_b200_selected_impl.restype = ctypes.c_int
        L.fastmax_b200_selected_impl.argtypes = [pp, ctypes.POINTER(ctypes.c_int32)]
        L.fastmax_b200_forward.restype = ctypes.c_int
        L.fastmax_b200_forward.argtypes = [pp, vp, vp, vp, vp, vp, vp, vp, sz, vp]
        L.fastmax_b200_forward_packed.restype = ctypes.c_int
        L.fastmax_b200_forward_packed.argtypes = [pp, vp, vp, vp, vp, vp, vp, sz, vp]
        L.fastmax_b200_backward.restype = ctypes.c_int
        L.fastmax_b200_backward.argtypes = [pp] + [vp] * 11 + [sz, vp]
        L.fastmax_b200_forward_bt.argtypes = [pp, vp, vp, vp, vp, vp, vp, ctypes.c_int32, vp, sz, vp]
        L.fastmax_b200_backward_bt.argtypes = [pp] + [vp] * 7 + [ctypes.c_int32] + [vp] * 4 + [sz, vp]
        L.fastmax_b200_bt_layout_supported.argtypes = [pp, ctypes.c_int32]
        for f in ("moment_state_bytes", "moment_total_bytes", "shard_forward_workspace_bytes",
                  "shard_backward_workspace_bytes"):
            fn = getattr(L, "fastmax_b200_" + f)
            fn.restype, fn.argtypes = sz, [pp]
        i32 = ctypes.c_int32
        L.fastmax_b200_shard_rowmax.argtypes = [pp, vp, vp, i32, vp, vp]
        L.fastmax_b200_shard_kv_state.argtypes = [pp, vp, vp, vp, vp, vp]
        L.fastmax_b200_shard_forward.argtypes = [pp] + [vp] * 9 + [sz, vp]
        L.fastmax_b200_shard_qg_state.argtypes = [pp] + [vp] * 8 + [sz, vp]
        L.fastmax_b200_shard_backward.argtypes = [pp] + [vp] * 15 + [i32, vp, sz, vp]
        L.fastmax_b200_shard_dq_far.argtypes = [pp] + [vp] * 7 + [sz, vp]
        L.fastmax_b200_shard_sum_totals.argtypes = [vp, i32, i32, i32, sz, vp, vp]
        L.fastmax_b200_shard_norm_fixup.argtypes = [pp, vp, vp, vp, vp, i32, vp, vp, vp]
        L.fastmax_b200_device_status.argtypes = [ctypes.POINTER(ctypes.c_int), vp]
        L.fastmax_b200_device_status_reset.argtypes = [vp]
        L.fastmax_b200_wait_selftest.argtypes = [ctypes.c_longlong, vp]
        L.fastmax_b200_launch_count.restype = ctypes.c_ulonglong
        L.fastmax_b200_profile_enable.argtypes = [ctypes.c_int]
        L.fastmax_b200_profile_get.argtypes = [ctypes.c_int, ctypes.c_char_p, ctypes.c_int,
                                               ctypes.POINTER(ctypes.c_float)]
        i64, ci = ctypes.c_longlong, ctypes.c_int
        L.fastmax_b200_qkv_split_rope.argtypes = [vp] * 6 + [i64, i64, ci, ci, ci, ci, ci, vp]
        L.fastmax_b200_qkv_merge_rope_grad.argtypes = [vp] * 6 + [i64, i64, ci, ci, ci, ci, ci, vp]
        L.fastmax_b200_swap_middle_axes.argtypes = [vp, vp, i64, i64, i64, ci, ci, vp]
        L.fastmax_b200_scale_by_noise.argtypes = [vp, vp, vp, ctypes.c_float, sz, ci, vp]
        for f in ("decode_state_bytes", "decode_scratch_bytes"):
            fn = getattr(L, "fastmax_b200_" + f)
            fn.restype, fn.argtypes = sz, [pp]
        L.fastmax_b200_decode_append.argtypes = [pp, vp, vp, i64, vp, vp]
        L.fastmax_b200_decode_step.argtypes = [pp, vp, vp, vp, vp, vp, vp, vp]
        _lib = L
    return _lib


def device_status(device=None) -> int:
    """Synchronise the current stream and return the tensor-core kernels' status word (0 = fine)."""
    st = ctypes.c_int(0)
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else device
    with torch.cuda.device(dev):
        _check(lib().fastmax_b200_device_status(ctypes.byref(st), torch.cuda.current_stream(dev).cuda_stream),
               "fastmax_b200_device_status")
    return int(st.value)


def device_status_reset(device=None):
    """Clear the status word (synchronises the current stream)."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else device
    with torch.cuda.device(dev):
        _check(lib().fastmax_b200_device_status_reset(torch.cuda.current_stream(dev).cuda_stream),
               "fastmax_b200_device_status_reset")


def wait_selftest(limit_clocks: int, device=None):
    """Launch the one-warp kernel whose bounded wait is designed to run out (status 99 afterwards)."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else device
    with torch.cuda.device(dev):
        _check(lib().fastmax_b200_wait_selftest(int(limit_clocks), torch.cuda.current_stream(dev).cuda_stream),
               "fastmax_b200_wait_selftest")


def launch_count() -> int:
    """Kernels launched through the library by this process so far."""
    return int(lib().fastmax_b200_launch_count())


def profile(on: bool):
    """Start (discarding earlier records) or stop per-launch event timing."""
    lib().fastmax_b200_profile_enable(int(bool(on)))


def profile_records():
    """[(kernel name, milliseconds)] for every launch since ``profile(True)``; waits for them."""
    L = lib()
    out = []
    buf = ctypes.create_string_buffer(64)
    ms = ctypes.c_float()
    for i in range(L.fastmax_b200_profile_count()):
        _check(L.fastmax_b200_profile_get(i, buf, 64, ctypes.byref(ms)), "fastmax_b200_profile_get")
        out.append((buf.value.decode(), float(ms.value)))
    return out


def _check(rc: int, what: str):
    if rc != 0:
        msg = lib().fastmax_b200_last_error().decode()
        if rc == -1:
            raise ValueError(f"{what}: {msg}")
        raise RuntimeError(f"{what} failed (code {rc}): {msg}")


def _dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.bfloat16:
        return BF16
    raise TypeError(f"fastmax_b200 supports float32 and bfloat16 tensors, got {t.dtype}")


def make_problem(q, k, mask, normalize, temperature, a0, a1, a2, lim, p, impl="auto", chunk=0) -> Problem:
    if p not in (1, 2):
        raise ValueError(f"p must be 1 or 2, got: {p}")
    return Problem(dtype=_dtype_code(q), bh=q.shape[0], bhkv=k.shape[0], nq=q.shape[1], nk=k.shape[1],
                   d=q.shape[2], mask=int(bool(mask)), normalize=int(bool(normalize)), p=int(p),
                   impl=IMPL[impl] if isinstance(impl, str) else int(impl),
                   a0=float(a0), a1=float(a1), a2=float(a2), lim=float(lim),
                   temperature=float(temperature), chunk=int(chunk))


def _require(q, k, v, *more):
    if not q.is_cuda:
        raise RuntimeError("fastmax_b200 runs on CUDA tensors only (there is no CPU path)")
    if q.dim() != 3 or k.dim() != 3 or v.dim() != 3:
        raise ValueError("q, k and v must be (b*h, n, d) here")
    if k.shape != v.shape or q.shape[2] != k.shape[2]:
        raise ValueError(f"shape mismatch: q {tuple(q.shape)}, k {tuple(k.shape)}, v {tuple(v.shape)}")
    for t in (q, k, v) + more:
        if t.device != q.device or t.dtype != q.dtype:
            raise ValueError("all tensors must share one device and dtype")
        if not t.is_contiguous():
            raise ValueError("tensors must be contiguous")


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def _workspace(nbytes: int, device) -> torch.Tensor:
    return torch.empty(max(int(nbytes), 1), dtype=torch.uint8, device=device)


def forward(q, k, v, *, mask, normalize, temperature=1.0, a0=1.0, a1=1.0, a2=0.5, lim=1.0, p=2,
            impl="auto", chunk=0, buffers=None):
    """q (bh,nq,d), k/v (bhkv,nk,d) -> out (bh,nq,d), den (bh,nq) fp32, stats (opaque).

    ``buffers`` may hold preallocated ``out``, ``den``, ``stats`` and ``workspace`` tensors
    (see ``forward_buffers``); otherwise they are allocated here."""
    _require(q, k, v)
    L = lib()
    prob = make_problem(q, k, mask, normalize, temperature, a0, a1, a2, lim, p, impl, chunk)
    with torch.cuda.device(q.device):
        wsb = L.fastmax_b200_forward_workspace_bytes(prob)
        if buffers is None:
            out = torch.empty_like(q)
            den = torch.empty(q.shape[:2], dtype=torch.float32, device=q.device)
            stats = torch.empty(max(L.fastmax_b200_stats_bytes(prob), 8), dtype=torch.uint8, device=q.device)
            ws = _workspace(wsb, q.device)
        else:
            out, den, stats, ws = buffers["out"], buffers["den"], buffers["stats"], buffers["workspace"]
            if ws.numel() < wsb:
                raise ValueError("preallocated forward workspace is too small")
        rc = L.fastmax_b200_forward(prob, q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(),
                                    den.data_ptr(), stats.data_ptr(), ws.data_ptr(), wsb, _stream(q))
    _check(rc, "fastmax_b200_forward")
    return out, den, stats


def bt_layout_supported(q, k, heads_per_batch, **kw) -> bool:
    """Whether ``forward_bt`` / ``backward_bt`` can serve a problem of these shapes."""
    prob = make_problem(q, k, kw["mask"], kw["normalize"], kw.get("temperature", 1.0), kw.get("a0", 1.0),
                        kw.get("a1", 1.0), kw.get("a2", 0.5), kw.get("lim", 1.0), kw.get("p", 2),
                        kw.get("impl", "auto"), kw.get("chunk", 0))
    return bool(lib().fastmax_b200_bt_layout_supported(prob, int(heads_per_batch)))


def forward_bt(q, k, v, heads_per_batch, *, mask, normalize, temperature=1.0, a0=1.0, a1=1.0, a2=0.5, lim=1.0,
               p=2, impl="auto", chunk=0):
    """As ``forward`` but the result is (batch, nq, heads_per_batch, d) -- what the model's output projection
    takes after a ``view`` -- written in that layout by the attention kernel itself."""
    _require(q, k, v)
    L = lib()
    prob = make_problem(q, k, mask, normalize, temperature, a0, a1, a2, lim, p, impl, chunk)
    bh, nq, d = q.shape
    with torch.cuda.device(q.device):
        wsb = L.fastmax_b200_forward_workspace_bytes(prob)
        out = torch.empty(bh // heads_per_batch, nq, heads_per_batch, d, dtype=q.dtype, device=q.device)
        den = torch.empty(bh, nq, dtype=torch.float32, device=q.device)
        stats = torch.empty(max(L.fastmax_b200_stats_bytes(prob), 8), dtype=torch.uint8, device=q.device)
        ws = _workspace(wsb, q.device)
        rc = L.fastmax_b200_forward_bt(prob, q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(),
                                       den.data_ptr(), stats.data_ptr(), int(heads_per_batch), ws.data_ptr(), wsb,
                                       _stream(q))
    _check(rc, "fastmax_b200_forward_bt")
    return out, den, stats


def backward_bt(q, k, v, out_bt, den, stats, grad_out_bt, heads_per_batch, *, mask, normalize, temperature=1.0,
                a0=1.0, a1=1.0, a2=0.5, lim=1.0, p=2, impl="auto", chunk=0):
    """Gradients from ``forward_bt``'s result and an upstream gradient in the same (batch, nq, heads, d) layout."""
    _require(q, k, v)
    for t in (out_bt, grad_out_bt):
        if t.device != q.device or t.dtype != q.dtype or not t.is_contiguous() or t.numel() != q.numel():
            raise ValueError("out and grad_out must be contiguous (batch, nq, heads, d) tensors of q's dtype")
    L = lib()
    prob = make_problem(q, k, mask, normalize, temperature, a0, a1, a2, lim, p, impl, chunk)
    with torch.cuda.device(q.device):
        wsb = L.fastmax_b200_backward_workspace_bytes(prob)
        gq, gk, gv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        ws = _workspace(wsb, q.device)
        rc = L.fastmax_b200_backward_bt(prob, q.data_ptr(), k.data_ptr(), v.data_ptr(), out_bt.data_ptr(),
                                        den.data_ptr(), stats.data_ptr(), grad_out_bt.data_ptr(),
                                        int(heads_per_batch), gq.data_ptr(), gk.data_ptr(), gv.data_ptr(),
                                        ws.data_ptr(), wsb, _stream(q))
    _check(rc, "fastmax_b200_backward_bt")
    return gq, gk, gv


def forward_packed(q, k, v, *, mask, normalize, temperature=1.0, a0=1.0, a1=1.0, a2=0.5, lim=1.0,
                   p=2, impl="auto"):
    """Reference layout: (bh, nq, d+1) fp32, denominator in the last channel."""
    _require(q, k, v)
    L = lib()
    prob = make_problem(q, k, mask, normalize, temperature, a0, a1, a2, lim, p, impl)
    with torch.cuda.device(q.device):
        o = torch.empty(q.shape[0], q.shape[1], q.shape[2] + 1, dtype=torch.float32, device=q.device)
        stats = torch.empty(max(L.fastmax_b200_stats_bytes(prob), 8), dtype=torch.uint8, device=q.device)
        wsb = L.fastmax_b200_forward_workspace_bytes(prob)
        ws = _workspace(wsb, q.device)
        rc = L.fastmax_b200_forward_packed(prob, q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(),
                                           stats.data_ptr(), ws.data_ptr(), wsb, _stream(q))
    _check(rc, "fastmax_b200_forward_packed")
    return o, stats


def selected_impl(prob: Problem) -> str:
    """Name of the kernel family a call with this problem runs (host arithmetic only, no device needed)."""
    got = ctypes.c_int32(0)
    rc = lib().fastmax_b200_selected_impl(prob, ctypes.byref(got))
    if rc:
        raise RuntimeError(lib().fastmax_b200_last_error().decode())
    return {v: k for k, v in IMPL.items()}[got.value]


def workspace_bytes(q, k, **kw):
    """(forward, backward, stats) scratch sizes in bytes for a problem of these shapes."""
    L = lib()
    prob = make_problem(q, k, kw["mask"], kw["normalize"], kw.get("temperature", 1.0), kw.get("a0", 1.0),
                        kw.get("a1", 1.0), kw.get("a2", 0.5), kw.get("lim", 1.0), kw.get("p", 2),
                        kw.get("impl", "auto"), kw.get("chunk", 0))
    return (L.fastmax_b200_forward_workspace_bytes(prob), L.fastmax_b200_backward_workspace_bytes(prob),
            max(L.fastmax_b200_stats_bytes(prob), 8))


def backward(q, k, v, out, den, stats, grad_out, *, mask, normalize, temperature=1.0, a0=1.0, a1=1.0,
             a2=0.5, lim=1.0, p=2, impl="auto", chunk=0, buffers=None):
    """Gradients (grad_q, grad_k, grad_v) in the dtype of the inputs; ``buffers`` as in ``forward``
    with ``grad_q``, ``grad_k``, ``grad_v`` and ``workspace``."""
    _require(q, k, v, out, grad_out)
    L = lib()
    prob = make_problem(q, k, mask, normalize, temperature, a0, a1, a2, lim, p, impl, chunk)
    with torch.cuda.device(q.device):
        wsb = L.fastmax_b200_backward_workspace_bytes(prob)
        if buffers is None:
            gq, gk, gv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
            ws = _workspace(wsb, q.device)
        else:
            gq, gk, gv, ws = buffers["grad_q"], buffers["grad_k"], buffers["grad_v"], buffers["workspace"]
            if ws.numel() < wsb:
                raise ValueError("preallocated backward workspace is too small")
        rc = L.fastmax_b200_backward(prob, q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(),
                                     den.data_ptr(), stats.data_ptr(), grad_out.data_ptr(),
                                     gq.data_ptr(), gk.data_ptr(), gv.data_ptr(), ws.data_ptr(), wsb,
                                     _stream(q))
    _check(rc, "fastmax_b200_backward")
    return gq, gk, gv


# ---- the transformer call site around the attention ---------------------------------------------

def _rope_tables(cos, sin, n, rope_n, device):
    if rope_n == 0:
        return None, None
    out = []
    for t in (cos, sin):
        if t.shape != (n, rope_n):
            raise ValueError(f"cos / sin must be ({n}, {rope_n}), got {tuple(t.shape)}")
        out.append(t.to(device=device, dtype=torch.float32).contiguous())
    return out


def _ptr(t):
    return None if t is None else t.data_ptr()


def qkv_split_rope(qkv, cos, sin, rope_n):
    """``qkv`` (B, T, G, Q+2, hs) -> q (B*G*Q, T, hs), k and v (B*G, T, hs), the first ``rope_n`` features
    of q and k rotated by the (T, rope_n) tables.  One pass over HBM."""
    if not qkv.is_cuda or qkv.dim() != 5 or not qkv.is_contiguous():
        raise ValueError("qkv must be a contiguous CUDA tensor (B, T, G, Q+2, hs)")
    b, n, g, total, d = qkv.shape
    qper = total - 2
    cs, sn = _rope_tables(cos, sin, n, rope_n, qkv.device)
    q = torch.empty(b * g * qper, n, d, dtype=qkv.dtype, device=qkv.device)
    k = torch.empty(b * g, n, d, dtype=qkv.dtype, device=qkv.device)
    v = torch.empty_like(k)
    with torch.cuda.device(qkv.device):
        rc = lib().fastmax_b200_qkv_split_rope(qkv.data_ptr(), _ptr(cs), _ptr(sn), q.data_ptr(), k.data_ptr(),
                                               v.data_ptr(), b, n, g, qper, d, rope_n, _dtype_code(qkv),
                                               _stream(qkv))
    _check(rc, "fastmax_b200_qkv_split_rope")
    return q, k, v


def qkv_merge_rope_grad(gq, gk, gv, cos, sin, rope_n, batch):
    """Gradient of the packed projection (B, T, G, Q+2, hs) from the per-head gradients."""
    for t in (gq, gk, gv):
        if not t.is_cuda or t.dim() != 3 or not t.is_contiguous() or t.dtype != gq.dtype:
            raise ValueError("gradients must be contiguous CUDA tensors (heads, T, hs) of one dtype")
    n, d = gq.shape[1], gq.shape[2]
    g = gk.shape[0] // batch
    qper = gq.shape[0] // gk.shape[0]
    if gk.shape != gv.shape or g * batch != gk.shape[0] or qper * gk.shape[0] != gq.shape[0]:
        raise ValueError("head counts do not match the batch size")
    cs, sn = _rope_tables(cos, sin, n, rope_n, gq.device)
    out = torch.empty(batch, n, g, qper + 2, d, dtype=gq.dtype, device=gq.device)
    with torch.cuda.device(gq.device):
        rc = lib().fastmax_b200_qkv_merge_rope_grad(gq.data_ptr(), gk.data_ptr(), gv.data_ptr(), _ptr(cs), _ptr(sn),
                                                    out.data_ptr(), batch, n, g, qper, d, rope_n,
                                                    _dtype_code(gq), _stream(gq))
    _check(rc, "fastmax_b200_qkv_merge_rope_grad")
    return out


def swap_middle_axes(x):
    """(B, X, Y, hs) -> contiguous (B, Y, X, hs)."""
    if not x.is_cuda or x.dim() != 4 or not x.is_contiguous():
        raise ValueError("expected a contiguous CUDA tensor (B, X, Y, hs)")
    b, nx, ny, d = x.shape
    out = torch.empty(b, ny, nx, d, dtype=x.dtype, device=x.device)
    with torch.cuda.device(x.device):
        rc = lib().fastmax_b200_swap_middle_axes(x.data_ptr(), out.data_ptr(), b, nx, ny, d, _dtype_code(x),
                                                 _stream(x))
    _check(rc, "fastmax_b200_swap_middle_axes")
    return out


def scale_by_noise(x, noise, dropout, out=None):
    """``x * (1 + dropout * noise)``; ``out`` may be ``x``."""
    if not x.is_cuda or not x.is_contiguous() or not noise.is_contiguous() or noise.shape != x.shape \
            or noise.dtype != x.dtype or noise.device != x.device:
        raise ValueError("x and noise must be contiguous CUDA tensors of one shape and dtype")
    out = torch.empty_like(x) if out is None else out
    with torch.cuda.device(x.device):
        rc = lib().fastmax_b200_scale_by_noise(x.data_ptr(), noise.data_ptr(), out.data_ptr(), float(dropout),
                                               x.numel(), _dtype_code(x), _stream(x))
    _check(rc, "fastmax_b200_scale_by_noise")
    return out
