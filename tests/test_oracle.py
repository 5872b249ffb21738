"""Pins the CPU oracle to vectors produced by the reference's own fastmax_function."""
import os

import numpy as np
import pytest
import torch

from conftest import GOLDEN, case_kwargs, load_small_cases
from oracle.fastmax_oracle import fastmax_dense, fastmax_fwd_bwd, fastmax_moments, rel_err

CASES = load_small_cases()


def tol64(c):
    """fp64 agreement bound.  The reference builds the a0*count term of the
    denominator from a float32 ``torch.ones`` (reference example.py:132,155), so
    for an a0 that float32 cannot hold exactly (the ``_b`` cases use 0.7) its
    fp64 run carries a ~1e-8 relative rounding that the oracle does not copy."""
    return 1e-11 if c["a0"] == 1.0 else 1e-6


@pytest.mark.parametrize("c", CASES, ids=[c["tag"] for c in CASES])
def test_moments_oracle_matches_reference_fp64(c):
    q, k, v, go = [c[x].double() for x in ("q", "k", "v", "go")]
    out, dq, dk, dv = fastmax_fwd_bwd(q, k, v, go, **case_kwargs(c))
    for got, name in ((out, "out"), (dq, "dq"), (dk, "dk"), (dv, "dv")):
        assert rel_err(got, c[name + "64"]) < tol64(c), name


@pytest.mark.parametrize("c", CASES, ids=[c["tag"] for c in CASES])
def test_blocked_scan_equals_full_cumsum(c):
    if not c["mask"]:
        pytest.skip("unmasked has no scan")
    q, k, v, go = [c[x].double() for x in ("q", "k", "v", "go")]
    res = fastmax_fwd_bwd(q, k, v, go, block=7, **case_kwargs(c))
    for got, name in zip(res, ("out", "dq", "dk", "dv")):
        assert rel_err(got, c[name + "64"]) < tol64(c), name


@pytest.mark.parametrize("c", CASES, ids=[c["tag"] for c in CASES])
def test_dense_oracle_matches_reference_fp64(c):
    q, k, v, go = [c[x].double() for x in ("q", "k", "v", "go")]
    res = fastmax_fwd_bwd(q, k, v, go, dense=True, **case_kwargs(c))
    for got, name in zip(res, ("out", "dq", "dk", "dv")):
        assert rel_err(got, c[name + "64"]) < max(1e-9, tol64(c)), name


@pytest.mark.parametrize("c", CASES, ids=[c["tag"] for c in CASES])
def test_oracle_fp32_close_to_reference_fp32(c):
    res = fastmax_fwd_bwd(c["q"], c["k"], c["v"], c["go"], **case_kwargs(c))
    for got, name in zip(res, ("out", "dq", "dk", "dv")):
        # both sides are fp32 evaluations of the same formula; they agree to rounding
        for ref in (c[name + "32"], c[name + "64"]):
            diff = float((got.double() - ref.double()).abs().max())
            # absolute floor: the n=1 gradients of q and k are exactly zero
            assert diff <= 2e-4 * float(ref.abs().max()) + 1e-6, name


def test_c1_configuration_sampled_rows():
    z = np.load(os.path.join(GOLDEN, "c1_sampled.npz"))
    b, h, n, d = [int(x) for x in z["cfg"][:4]]
    g = torch.Generator().manual_seed(int(z["seed"]))
    q, k, v, go = [torch.randn(b, h, n, d, generator=g) for _ in range(4)]
    chk = np.array([float(t.double().sum()) for t in (q, k, v, go)])
    if not np.allclose(chk, z["input_checksum"], rtol=0, atol=1e-6):
        pytest.skip("torch RNG stream differs from the one the fixture was made with")
    res = fastmax_fwd_bwd(q.double(), k.double(), v.double(), go.double(),
                          mask=0, normalize=1, p=2)
    st = int(z["row_stride"])
    for got, name in zip(res, ("out", "dq", "dk", "dv")):
        pick = torch.stack([got[bb, hh, ::st] for bb, hh in z["heads"]])
        ref = torch.from_numpy(z[name + "64"])
        assert float((pick - ref).abs().max()) < 1e-11 * float(z[name + "64_absmax"]), name


def test_temperature_is_ignored_and_bad_p_raises():
    c = CASES[0]
    a = fastmax_moments(c["q"], c["k"], c["v"], temperature=1.0, p=2)
    b = fastmax_moments(c["q"], c["k"], c["v"], temperature=7.5, p=2)
    assert torch.equal(a, b)
    with pytest.raises(ValueError):
        fastmax_moments(c["q"], c["k"], c["v"], p=3)
    with pytest.raises(ValueError):
        fastmax_dense(c["q"], c["k"], c["v"], p=0)


def test_dense_rows_subset():
    c = [x for x in CASES if x["tag"] == "m1p2n1_d32"][0]
    q, k, v = [c[x].double() for x in ("q", "k", "v")]
    rows = [0, 3, 69]
    part = fastmax_dense(q, k, v, rows=rows, **case_kwargs(c))
    assert rel_err(part, c["out64"][:, :, rows]) < 1e-10


@pytest.mark.parametrize("tag", ["a", "b"])
@pytest.mark.parametrize("tables", ["rot", "gen"])
def test_rope_oracle_matches_reference_vectors(tag, tables):
    """The call-site oracle's rotary embedding against outputs of the reference's apply_rope."""
    from oracle.call_site_oracle import rope
    z = np.load(os.path.join(GOLDEN, "rope.npz"))
    x = torch.from_numpy(z[f"{tag}_x"]).requires_grad_(True)
    cos, sin = [torch.from_numpy(z[f"{tag}_{tables}_{n}"]) for n in ("cos", "sin")]
    y = rope(x, cos, sin)
    (gx,) = torch.autograd.grad(y, x, torch.from_numpy(z[f"{tag}_go"]))
    assert torch.equal(y.detach(), torch.from_numpy(z[f"{tag}_{tables}_y"]))
    assert torch.equal(gx, torch.from_numpy(z[f"{tag}_{tables}_gx"]))


def test_call_site_oracle_shapes_and_grouping():
    """Expanded and grouped key/value heads describe the same attention."""
    from oracle.call_site_oracle import call_site, split_heads
    g = torch.Generator().manual_seed(3)
    b, t, heads, groups, hs, r = 2, 11, 4, 2, 8, 8
    qkv = torch.randn(b, t, (heads + 2 * groups) * hs, generator=g, dtype=torch.float64)
    cos, sin = torch.randn(t, r, generator=g, dtype=torch.float64), torch.randn(t, r, generator=g, dtype=torch.float64)
    q, k, v = split_heads(qkv, cos, sin, heads, groups, hs, r)
    qg, kg, vg = split_heads(qkv, cos, sin, heads, groups, hs, r, expand=False)
    assert q.shape == (b, heads, t, hs) and kg.shape == (b, groups, t, hs)
    assert torch.equal(k, kg.repeat_interleave(heads // groups, dim=1)) and torch.equal(q, qg)
    y = call_site(qkv, cos, sin, heads, groups, hs, r, mask=1, normalize=1, p=1)
    assert y.shape == (b, t, heads * hs)


@pytest.mark.parametrize("p", [1, 2])
@pytest.mark.parametrize("normalize", [0, 1])
def test_moment_state_recurrence_equals_dense_rows(p, normalize):
    """The fixed-size decode state gives, token by token, the causal attention row over the tokens so far."""
    from oracle.call_site_oracle import MomentState
    g = torch.Generator().manual_seed(17)
    heads, n, d, n0 = 3, 14, 8, 5
    scale = 1.0 if normalize else d ** -0.5
    q, k = [torch.randn(heads, n, d, generator=g, dtype=torch.float64) * scale for _ in range(2)]
    v = torch.randn(heads, n, d, generator=g, dtype=torch.float64)
    st = MomentState(heads, d, p=p, normalize=bool(normalize), a0=0.7, a1=1.3, a2=0.4, lim=1.5)
    st.append(k[:, :n0], v[:, :n0])
    for t in range(n0, n):
        got = st.step(q[:, t:t + 1], k[:, t:t + 1], v[:, t:t + 1])
        want = fastmax_dense(q[None, :, t:t + 1], k[None, :, :t + 1], v[None, :, :t + 1], mask=1,
                             normalize=normalize, p=p, a0=0.7, a1=1.3, a2=0.4, lim=1.5)[0]
        assert rel_err(got, want) < 1e-12


def test_restatement_matches_the_compiled_reference_function():
    """Where oracle/_ref has been built from a reference tree (oracle/make_ref.py), the oracle is held
    against the reference's own function directly, on fresh seeded inputs."""
    from oracle.make_ref import load
    ref = load()
    if ref is None:
        pytest.skip("oracle/_ref has not been built")
    g = torch.Generator().manual_seed(41)
    for mask in (0, 1):
        for p in (1, 2):
            for norm in (0, 1):
                q, k, v, go = [torch.randn(2, 2, 37, 8, generator=g, dtype=torch.float64) * 0.5 for _ in range(4)]
                kw = dict(mask=mask, normalize=norm, a0=1.0, a1=1.2, a2=0.4, lim=1.1, p=p)
                qr, kr, vr = [t.clone().requires_grad_(True) for t in (q, k, v)]
                out = ref(qr, kr, vr, **kw)
                out.backward(go)
                got = fastmax_fwd_bwd(q, k, v, go, **kw)
                for a, b, name in zip(got, (out.detach(), qr.grad, kr.grad, vr.grad), ("out", "dq", "dk", "dv")):
                    assert rel_err(a, b) < 1e-11, (mask, p, norm, name)
