"""The allocation-free backward entry point (scratch in a fixed array inside the
library) must give what the ordinary backward gives.

It exists for embedders that cannot give the library memory or let it take any:
a host program whose own arena already owns the whole GPU, or a loop that cannot
afford the device-wide synchronisation of cudaMalloc/cudaFree.  The test calls it
through the C ABI with raw pointers, twice in a row on different problems (the
array is shared and keeps the previous call's contents), and compares with
fastmax_b200_backward and with the CPU oracle within the tolerances of the other GPU
tests, and checks that the device's free memory does not move across a call.  The file
name sorts last so a failure here cannot hide another test's result.
"""
import ctypes

import pytest
import torch

from fastmax_b200 import _cabi
from gpu_util import assert_close, oracle

pytestmark = pytest.mark.gpu


def _static_backward(q, k, v, out, den, stats, go, **kw):
    L = _cabi.lib()
    fn = L.fastmax_b200_backward_static
    fn.restype = ctypes.c_int
    vp = ctypes.c_void_p
    fn.argtypes = [ctypes.POINTER(_cabi.Problem)] + [vp] * 10 + [vp]
    prob = _cabi.make_problem(q, k, kw["mask"], kw["normalize"], 1.0, 1.0, 1.0, 0.5, 1.0, kw["p"], "dense_ffma")
    gq, gk, gv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    rc = fn(prob, q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), den.data_ptr(), stats.data_ptr(),
            go.data_ptr(), gq.data_ptr(), gk.data_ptr(), gv.data_ptr(),
            torch.cuda.current_stream().cuda_stream)
    return rc, (gq, gk, gv)


def _case(bh, bhkv, nq, nk, d, dtype, seed, **kw):
    g = torch.Generator(device="cuda").manual_seed(seed)
    mk = lambda h, n: torch.randn(h, n, d, generator=g, device="cuda").to(dtype)
    q, go, k, v = mk(bh, nq), mk(bh, nq), mk(bhkv, nk), mk(bhkv, nk)
    out, den, stats = _cabi.forward(q, k, v, impl="dense_ffma", **kw)
    want = _cabi.backward(q, k, v, out, den, stats, go, impl="dense_ffma", **kw)
    rc, got = _static_backward(q, k, v, out, den, stats, go, **kw)
    assert rc == 0, _cabi.lib().fastmax_b200_last_error()
    torch.cuda.synchronize()
    tol = 1e-4 if dtype == torch.float32 else 2e-2
    for a, b, name in zip(got, want, ("grad_q", "grad_k", "grad_v")):
        err = float((a.float() - b.float()).abs().max() / b.float().abs().max().clamp_min(1e-2))
        assert err < tol, (name, err)
    if bh == bhkv:   # the CPU oracle beside the library's own backward
        ref = oracle(q.float().cpu()[None], k.float().cpu()[None], v.float().cpu()[None], go.float().cpu()[None],
                     dtype, dense=True, a0=1.0, a1=1.0, a2=0.5, lim=1.0, **{x: int(y) for x, y in kw.items()})
        assert_close([t.float().cpu()[None] for t in (out,) + tuple(got)], ref, dtype, "static scratch vs oracle")


def test_static_scratch_backward_matches_workspace_backward_twice_in_a_row():
    L = _cabi.lib()
    L.fastmax_b200_static_scratch_bytes.restype = ctypes.c_size_t
    assert L.fastmax_b200_static_scratch_bytes() == 8 << 20
    # two different problems back to back: the second sees the first one's leftovers
    _case(6, 6, 300, 300, 32, torch.float32, 1, mask=True, normalize=True, p=2)
    _case(4, 2, 70, 100, 64, torch.bfloat16, 2, mask=True, normalize=True, p=2)
    _case(6, 6, 300, 300, 32, torch.float32, 1, mask=True, normalize=True, p=2)


def test_static_scratch_backward_leaves_free_memory_alone():
    """An empty problem does the one-time set-up (device check, address lookup); after that a real call
    must not change how much device memory is free."""
    L = _cabi.lib()
    fn = L.fastmax_b200_backward_static
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.POINTER(_cabi.Problem)] + [ctypes.c_void_p] * 11
    empty = _cabi.Problem(dtype=0, bh=0, bhkv=0, nq=0, nk=0, d=32, mask=1, normalize=0, p=2, impl=0,
                          a0=1, a1=1, a2=0.5, lim=1, temperature=1)
    assert fn(empty, *([None] * 11)) == 0
    g = torch.Generator(device="cuda").manual_seed(3)
    q, k, v, go = [torch.randn(4, 200, 32, generator=g, device="cuda") for _ in range(4)]
    kw = dict(mask=True, normalize=True, p=2)
    out, den, stats = _cabi.forward(q, k, v, impl="dense_ffma", **kw)
    rc, _ = _static_backward(q, k, v, out, den, stats, go, **kw)     # warm: kernels loaded
    assert rc == 0
    gq, gk, gv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    prob = _cabi.make_problem(q, k, True, True, 1.0, 1.0, 1.0, 0.5, 1.0, 2, "dense_ffma")
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info()
    rc = fn(prob, q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), den.data_ptr(), stats.data_ptr(),
            go.data_ptr(), gq.data_ptr(), gk.data_ptr(), gv.data_ptr(), torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    free1, _ = torch.cuda.mem_get_info()
    assert rc == 0 and free1 == free0, (rc, free0, free1)


def test_static_scratch_backward_rejects_oversized_problems():
    q = torch.zeros(1, 8, 32, device="cuda")
    prob = _cabi.Problem(dtype=0, bh=64, bhkv=64, nq=40000, nk=40000, d=32, mask=1, normalize=1, p=2, impl=0,
                         a0=1, a1=1, a2=0.5, lim=1, temperature=1)
    L = _cabi.lib()
    fn = L.fastmax_b200_backward_static
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.POINTER(_cabi.Problem)] + [ctypes.c_void_p] * 11
    p = q.data_ptr()
    rc = fn(prob, p, p, p, p, p, p, p, p, p, p, None)
    assert rc == -2 and b"built-in array" in L.fastmax_b200_last_error()
