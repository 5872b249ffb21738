"""CPU-side checks: the C ABI library loads and exports what the header declares,
the host wrappers validate their arguments, and the pure-PyTorch path of the
package agrees with the reference-generated vectors."""
import ctypes
import os
import re

import pytest
import torch

from conftest import ROOT, case_kwargs, load_small_cases
from oracle.fastmax_oracle import rel_err

import fastmax_b200
from fastmax_b200 import _cabi

CASES = load_small_cases()


def _declared_functions():
    names = set()
    for fn in os.listdir(os.path.join(ROOT, "include")):
        if fn.endswith(".h"):
            txt = open(os.path.join(ROOT, "include", fn)).read()
            txt = re.sub(r"/\*.*?\*/", "", txt, flags=re.S)
            names |= set(re.findall(r"\b(fastmax_b200_\w+)\s*\(", txt))
    return sorted(names)


def test_library_exports_every_declared_symbol():
    lib = ctypes.CDLL(_cabi.LIB_PATH)
    declared = _declared_functions()
    assert len(declared) >= 8
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in include/ but not exported"
    assert set(_cabi.EXPORTS) <= set(declared)


def test_version_and_size_queries_need_no_gpu():
    L = _cabi.lib()
    assert L.fastmax_b200_version() >= 100
    prob = _cabi.Problem(dtype=0, bh=6, bhkv=3, nq=10, nk=12, d=32, mask=1, normalize=1, p=2, impl=0,
                         a0=1, a1=1, a2=0.5, lim=1, temperature=1)
    assert L.fastmax_b200_stats_bytes(prob) == 8 * 9
    assert L.fastmax_b200_backward_workspace_bytes(prob) >= 4 * (9 + 60)
    assert ctypes.sizeof(_cabi.Problem) == 64


def test_family_selection_follows_the_measured_break_even_points():
    """The library's choice of kernel family (host arithmetic, no device): tensor-core score kernels for short
    rows, the moment family where it was measured faster -- causal bf16 p=2 d=64 from about 9 500 keys on (the
    headline shape has 10 000), unmasked from about 5 500, p=1 at almost any length -- and never for a few
    query rows against many keys; fp32 stays on the CUDA-core score kernels."""
    def pick(**kw):
        base = dict(dtype=_cabi.BF16, bh=1024, bhkv=1024, nq=10000, nk=10000, d=64, mask=1, normalize=1, p=2,
                    impl=0, a0=1, a1=1, a2=0.5, lim=1, temperature=1)
        base.update(kw)
        return _cabi.selected_impl(_cabi.Problem(**base))

    assert pick() == "moments"                                           # the headline shape
    assert pick(nq=8192, nk=8192) == "dense_tc"
    assert pick(nq=9216, nk=9216) == "dense_tc"
    assert pick(nq=12288, nk=12288) == "moments"
    assert pick(bh=32, bhkv=32, nq=262144, nk=262144) == "moments"       # the long-context configuration
    assert pick(mask=0, nq=4096, nk=4096) == "dense_tc"
    assert pick(mask=0, nq=6144, nk=6144) == "moments"
    assert pick(mask=0, nq=256, nk=6000) == "dense_tc"                   # few query rows, many keys
    assert pick(mask=0, nq=1, nk=100000) == "dense_tc"
    assert pick(mask=0, p=1, d=128, nq=16384, nk=16384, normalize=0) == "moments"
    assert pick(mask=0, d=128, nq=16384, nk=16384, normalize=0) == "dense_tc"
    assert pick(dtype=_cabi.F32, d=32, nq=1000, nk=1000) == "dense_ffma"
    assert pick(impl=_cabi.IMPL["dense_tc"]) == "dense_tc"               # a forced family is reported as such
    assert pick(impl=_cabi.IMPL["moments_ffma"]) == "moments"
    with pytest.raises(RuntimeError):
        pick(impl=_cabi.IMPL["dense_tc"], dtype=_cabi.F32, d=32)


def test_bad_arguments_are_rejected_before_any_launch():
    L = _cabi.lib()
    prob = _cabi.Problem(dtype=0, bh=2, bhkv=2, nq=4, nk=4, d=32, mask=1, normalize=0, p=3, impl=0,
                         a0=1, a1=1, a2=0.5, lim=1, temperature=1)
    rc = L.fastmax_b200_forward(prob, 1, 1, 1, 1, 1, 1, None, 0, None)
    assert rc == -1 and b"p must be 1 or 2" in L.fastmax_b200_last_error()
    assert L.fastmax_b200_backward(prob, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, None, 0, None) == -1
    assert L.fastmax_b200_forward_packed(prob, 1, 1, 1, 1, 1, None, 0, None) == -1
    prob.p, prob.d = 2, 24
    assert L.fastmax_b200_forward(prob, 1, 1, 1, 1, 1, 1, None, 0, None) == -1
    prob.d, prob.nk = 32, 3
    assert L.fastmax_b200_forward(prob, 1, 1, 1, 1, 1, 1, None, 0, None) == -1
    prob.nk, prob.bhkv = 4, 3
    assert L.fastmax_b200_forward(prob, 1, 1, 1, 1, 1, 1, None, 0, None) == -1


def test_custom_path_refuses_cpu_tensors():
    q = torch.randn(1, 2, 8, 8)
    with pytest.raises(RuntimeError):
        fastmax_b200.FASTMultiHeadAttention()(q, q, q, None, True)
    with pytest.raises(ValueError):
        fastmax_b200.fastmax_function(q, q, q, p=3)


@pytest.mark.parametrize("c", CASES, ids=[c["tag"] for c in CASES])
def test_pytorch_path_matches_reference_vectors(c):
    q, k, v, go = [c[x].double().requires_grad_(x != "go") for x in ("q", "k", "v", "go")]
    mod = fastmax_b200.FASTMultiHeadAttention(use_custom_gradient=False)
    out = mod(q, k, v, None, c["mask"], 0.0, c["normalize"], 1.0, c["a0"], c["a1"], c["a2"], c["lim"], c["p"])
    out.backward(go)
    tol = 1e-9 if c["a0"] == 1.0 else 1e-6   # see tests/test_oracle.py::tol64
    for got, name in ((out.detach(), "out"), (q.grad, "dq"), (k.grad, "dk"), (v.grad, "dv")):
        assert rel_err(got, c[name + "64"]) < tol, name


def test_pytorch_path_blocked_scan_and_attn_matrix():
    c = [x for x in CASES if x["tag"] == "m1p2n0_a"][0]
    q, k, v = [c[x].double() for x in ("q", "k", "v")]
    kw = dict(mask=1, normalize=0, a0=c["a0"], a1=c["a1"], a2=c["a2"], lim=c["lim"], p=2)
    a = fastmax_b200.fastmax_function(q, k, v, block=5, **kw)
    assert rel_err(a, c["out64"]) < 1e-10
    n = q.shape[2]
    tri = torch.tril(torch.ones(n, n))
    ans, attn = fastmax_b200.fastmax_function(q, k, v, mask=tri, a0=c["a0"], a1=c["a1"], a2=c["a2"],
                                              create_attn_matrix=1)
    assert rel_err(ans, c["out64"]) < 1e-10
    assert torch.allclose(attn.sum(-1), torch.ones_like(attn.sum(-1)))


def test_rpe_matrix_creator_shapes():
    r = fastmax_b200.rpe_matrix_creator(5, 8, "cpu", torch.float32)
    assert r.shape == (9, 8) and float(r.abs().sum()) == 0.0
    r = fastmax_b200.rpe_matrix_creator(5, 8, "cpu", torch.float32, structured=True)
    assert r.shape == (9, 8) and torch.allclose(r[4], torch.tensor([0., 1.] * 4))


def test_numa_preference_is_a_no_op_without_a_gpu():
    """The helper must never raise: without CUDA (or without a readable topology) it reports -1."""
    from fastmax_b200.host import prefer_gpu_numa_node
    if not torch.cuda.is_available():
        assert prefer_gpu_numa_node("cuda:0") == -1
    else:
        assert prefer_gpu_numa_node("cuda:0") >= -1
