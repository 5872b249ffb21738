"""GPU parity of the tcgen05 tensor-core family (bf16, head dimension 64) against the
CPU oracle, through the C ABI.  Tolerance: 2e-2 relative on outputs and gradients."""
import pytest
import torch

from gpu_util import assert_close, oracle, run_cabi

from fastmax_b200 import _cabi

pytestmark = pytest.mark.gpu


def randn(*shape, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g)


# bh, nq, nk, mask, p, normalize
EDGE = [(1, 1, 1, 1, 2, 1), (2, 2, 2, 1, 2, 1), (1, 17, 17, 0, 2, 1), (3, 127, 127, 1, 2, 1),
        (3, 128, 128, 1, 1, 1), (2, 129, 129, 0, 1, 0), (3, 255, 255, 1, 2, 1), (2, 256, 256, 1, 2, 0),
        (2, 257, 257, 1, 2, 1), (2, 300, 300, 0, 2, 1), (5, 1000, 1000, 1, 2, 1), (2, 1500, 1500, 0, 2, 0),
        (2, 70, 100, 1, 2, 1), (2, 70, 100, 0, 2, 1), (2, 200, 457, 1, 1, 1), (1, 2500, 2500, 1, 2, 1)]


@pytest.mark.parametrize("cfg", EDGE, ids=[f"bh{c[0]}nq{c[1]}nk{c[2]}m{c[3]}p{c[4]}z{c[5]}" for c in EDGE])
def test_tensor_core_family_against_dense_oracle(cfg):
    bh, nq, nk, mask, p, norm = cfg
    q, go = randn(1, bh, nq, 64, seed=nq), randn(1, bh, nq, 64, seed=nq + 1)
    k, v = randn(1, bh, nk, 64, seed=nk + 2), randn(1, bh, nk, 64, seed=nk + 3)
    if not norm:
        q, k = q / 8, k / 8
    kw = dict(mask=mask, normalize=norm, p=p, a0=1.0, a1=1.0, a2=0.5, lim=1.0)
    got, _ = run_cabi(q, k, v, go, torch.bfloat16, impl="dense_tc", **kw)
    assert _cabi.device_status() == 0
    ref = oracle(q, k, v, go, torch.bfloat16, dense=True, **kw)
    # at n == 1 grad_q and grad_k are exact zeros made of O(1) terms that cancel
    assert_close(got, ref, torch.bfloat16, str(cfg), floor=1.0 if nq == 1 else 1e-2)


# bh, nq, nk, mask, p, normalize  -- head dimension 128
EDGE128 = [(1, 1, 1, 1, 2, 0), (2, 127, 127, 1, 2, 1), (2, 128, 128, 0, 2, 0), (3, 129, 129, 1, 1, 1),
           (2, 300, 300, 1, 2, 1), (2, 257, 257, 0, 1, 0), (1, 1000, 1000, 1, 2, 0), (2, 70, 100, 1, 2, 1),
           (2, 200, 457, 0, 2, 0), (1, 1500, 1500, 0, 2, 0)]


@pytest.mark.parametrize("cfg", EDGE128, ids=[f"bh{c[0]}nq{c[1]}nk{c[2]}m{c[3]}p{c[4]}z{c[5]}" for c in EDGE128])
def test_tensor_core_family_head_dimension_128(cfg):
    bh, nq, nk, mask, p, norm = cfg
    q, go = randn(1, bh, nq, 128, seed=nq), randn(1, bh, nq, 128, seed=nq + 1)
    k, v = randn(1, bh, nk, 128, seed=nk + 2), randn(1, bh, nk, 128, seed=nk + 3)
    if not norm:
        q, k = q * 128 ** -0.5, k * 128 ** -0.5
    kw = dict(mask=mask, normalize=norm, p=p, a0=1.0, a1=1.0, a2=0.5, lim=1.0)
    got, _ = run_cabi(q, k, v, go, torch.bfloat16, impl="dense_tc", **kw)
    assert _cabi.device_status() == 0
    ref = oracle(q, k, v, go, torch.bfloat16, dense=True, **kw)
    assert_close(got, ref, torch.bfloat16, str(cfg), floor=1.0 if nq == 1 else 1e-2)


def test_other_coefficients_and_lim():
    q, k, v, go = [randn(1, 3, 333, 64, seed=s) for s in (1, 2, 3, 4)]
    kw = dict(mask=1, normalize=1, p=2, a0=0.7, a1=1.3, a2=0.4, lim=1.5)
    got, _ = run_cabi(q, k, v, go, torch.bfloat16, impl="dense_tc", **kw)
    ref = oracle(q, k, v, go, torch.bfloat16, dense=True, **kw)
    assert_close(got, ref, torch.bfloat16, "coefficients")


def test_negative_second_order_coefficient_takes_the_general_polynomial_path():
    """With a2 > 0 the fused grad_k + grad_v kernel evaluates the polynomial in completed-square form; a
    negative a2 (still a positive kernel for |s| <= lim^2) must go through the general form."""
    q, k, v, go = [randn(1, 2, 400, 64, seed=s) for s in (11, 12, 13, 14)]
    kw = dict(mask=1, normalize=1, p=2, a0=1.0, a1=0.8, a2=-0.1, lim=1.0)
    got, _ = run_cabi(q, k, v, go, torch.bfloat16, impl="dense_tc", **kw)
    ref = oracle(q, k, v, go, torch.bfloat16, dense=True, **kw)
    assert_close(got, ref, torch.bfloat16, "negative a2")


def test_auto_dispatch_picks_tensor_cores_and_matches_cuda_core_family():
    """Both families on the same device inputs at a size the CPU oracle would take long on."""
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(5)
    q, k, v, go = [torch.randn(4, 4096, 64, generator=g, device=dev).bfloat16() for _ in range(4)]
    kw = dict(mask=True, normalize=True, p=2)
    res = {}
    for impl in ("auto", "dense_ffma"):
        _cabi.profile(True)
        out, den, stats = _cabi.forward(q, k, v, impl=impl, **kw)
        grads = _cabi.backward(q, k, v, out, den, stats, go, impl=impl, **kw)
        names = {n for n, _ in _cabi.profile_records()}
        _cabi.profile(False)
        res[impl] = (out, den) + tuple(grads)
        if impl == "auto":
            assert "fm_dense_tc_fwd" in names and "fm_dense_tc_dq" in names
    assert _cabi.device_status() == 0
    for a, b, name in zip(res["auto"], res["dense_ffma"], ("out", "den", "dq", "dk", "dv")):
        e = float((a.float() - b.float()).abs().max() / b.float().abs().max())
        assert e < 2e-2, (name, e)


def test_unsupported_requests_fail_loudly():
    q = torch.randn(2, 64, 32, device="cuda").bfloat16()
    with pytest.raises(RuntimeError):
        _cabi.forward(q, q, q, mask=True, normalize=False, p=2, impl="dense_tc")   # d = 32
    q = torch.randn(2, 64, 64, device="cuda")
    with pytest.raises(RuntimeError):
        _cabi.forward(q, q, q, mask=True, normalize=False, p=2, impl="dense_tc")   # fp32
    with pytest.raises(ValueError):
        _cabi.forward(q.bfloat16(), q.bfloat16(), q.bfloat16(), mask=True, normalize=False, p=2, impl=7)


_NARROW_CHILD = r"""
import sys, torch
sys.path.insert(0, sys.argv[1]); sys.path.insert(0, sys.argv[1] + "/tests")
from gpu_util import assert_close, oracle, run_cabi
from fastmax_b200 import _cabi
for bh, nq, nk, mask, p, norm, d in [(2, 257, 257, 1, 2, 1, 64), (2, 70, 100, 1, 2, 1, 64), (2, 300, 300, 0, 1, 0, 64),
                                     (2, 300, 300, 1, 2, 1, 128)]:
    g = torch.Generator().manual_seed(nq)
    q, go = torch.randn(1, bh, nq, d, generator=g), torch.randn(1, bh, nq, d, generator=g)
    k, v = torch.randn(1, bh, nk, d, generator=g), torch.randn(1, bh, nk, d, generator=g)
    if not norm:
        q, k = q / 8, k / 8
    kw = dict(mask=mask, normalize=norm, p=p, a0=1.0, a1=1.0, a2=0.5, lim=1.0)
    _cabi.profile(True)
    got, _ = run_cabi(q, k, v, go, torch.bfloat16, impl="dense_tc", **kw)
    names = {n for n, _ in _cabi.profile_records()}
    _cabi.profile(False)
    assert "fm_dense_tc_dv" in names and "fm_dense_tc_dkdv" not in names, names
    assert _cabi.device_status() == 0
    assert_close(got, oracle(q, k, v, go, torch.bfloat16, dense=True, **kw), torch.bfloat16, "narrow")
print("NARROW-OK")
"""


def test_three_kernel_backward_stays_correct_when_the_fused_one_is_switched_off():
    """FASTMAX_B200_NO_WIDE=1 is read once per process, so the check runs in a child."""
    import os, subprocess, sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, FASTMAX_B200_NO_WIDE="1")
    r = subprocess.run([sys.executable, "-c", _NARROW_CHILD, root], env=env, capture_output=True, text=True,
                       timeout=600)
    assert r.returncode == 0 and "NARROW-OK" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]


@pytest.mark.parametrize("d", [64, 128])
def test_fused_backward_is_the_default(d):
    q, k, v, go = [randn(1, 2, 384, d, seed=s) for s in (11, 12, 13, 14)]
    _cabi.profile(True)
    run_cabi(q, k, v, go, torch.bfloat16, impl="dense_tc", mask=1, normalize=1, p=2)
    names = {n for n, _ in _cabi.profile_records()}
    _cabi.profile(False)
    assert {"fm_dense_tc_dq", "fm_dense_tc_dkdv"} <= names and "fm_dense_tc_dv" not in names, names


@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("mask", [0, 1])
def test_grouped_kv_heads_on_the_tensor_core_family(mask, d):
    """bh = 3 * bhkv, nk > nq: each key/value head serves three query heads inside the kernels."""
    from oracle.fastmax_oracle import fastmax_dense
    q, go = randn(1, 6, 200, d, seed=1), randn(1, 6, 200, d, seed=2)
    k, v = randn(1, 2, 300, d, seed=3), randn(1, 2, 300, d, seed=4)
    kw = dict(mask=mask, normalize=1, p=2, a0=1.0, a1=1.0, a2=0.5, lim=1.0)
    _cabi.profile(True)
    got, _ = run_cabi(q, k, v, go, torch.bfloat16, impl="dense_tc", **kw)
    names = {n for n, _ in _cabi.profile_records()}
    _cabi.profile(False)
    assert "fm_dense_tc_dkdv" in names and _cabi.device_status() == 0
    r = lambda t: t.bfloat16().double()
    kx, vx = [r(t).repeat_interleave(3, dim=1).requires_grad_(True) for t in (k, v)]
    qx = r(q).requires_grad_(True)
    out = fastmax_dense(qx, kx, vx, **kw)
    out.backward(r(go))
    ref = [out.detach(), qx.grad, kx.grad.reshape(1, 2, 3, 300, d).sum(2), vx.grad.reshape(1, 2, 3, 300, d).sum(2)]
    assert_close(got, ref, torch.bfloat16, f"gqa mask={mask}")


def test_few_query_rows_against_many_keys_of_many_heads():
    """nq != nk with one row tile per head: every resident CTA streams the column tiles of a different
    head from DRAM, so loads arrive late and out of order.  (With an odd number of ring stages the two
    S / W issuer warps could pass a stage barrier one phase early in this regime and the launch failed;
    the ring is even now.)  Repeated launches must give identical results, match the CUDA-core family
    and leave the status word at zero."""
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(9)
    k, v = [torch.randn(512, 6000, 64, generator=g, device=dev).bfloat16() for _ in range(2)]
    for nq, mask in ((1, True), (128, True), (256, False)):
        q = torch.randn(512, nq, 64, generator=g, device=dev).bfloat16()
        kw = dict(mask=mask, normalize=True, p=2)
        want, wden, _ = _cabi.forward(q, k, v, impl="dense_ffma", **kw)
        _cabi.profile(True)
        first, fden, _ = _cabi.forward(q, k, v, **kw)               # AUTO takes the tensor cores here
        names = {n for n, _ in _cabi.profile_records()}
        _cabi.profile(False)
        assert "fm_dense_tc_fwd" in names
        for _ in range(25):
            out, den, _ = _cabi.forward(q, k, v, impl="dense_tc", **kw)
        assert _cabi.device_status() == 0
        assert torch.equal(out, first) and torch.equal(den, fden)
        assert float((out.float() - want.float()).abs().max() / want.float().abs().max()) < 2e-2
        assert float((den - wden).abs().max() / wden.abs().max()) < 1e-3
