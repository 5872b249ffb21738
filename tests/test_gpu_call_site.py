"""GPU parity of the call-site kernels (packed projection -> rotary embedding -> heads and back,
axis swap, output dropout) through the C ABI, against the reference's rotary vectors and the CPU
oracle.  Layout moves are exact; rotated values agree to fp32 rounding (1e-6 relative) in float32
and to one bf16 rounding in bfloat16; the whole call site meets the attention tolerances
(1e-4 / 2e-2 relative)."""
import os

import numpy as np
import pytest
import torch

from conftest import GOLDEN
from gpu_util import TOL
from oracle.call_site_oracle import call_site, output_dropout, split_heads
from oracle.fastmax_oracle import fastmax_dense

import fastmax_b200
from fastmax_b200 import _cabi
from fastmax_b200.call_site import fastmax_attention_from_qkv

pytestmark = pytest.mark.gpu


def rel(a, b, floor=1e-2):
    return float((a.double().cpu() - b.double()).abs().max() / b.double().abs().max().clamp_min(floor))


def tables(t, r, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(t, r, generator=g), torch.randn(t, r, generator=g)


@pytest.mark.parametrize("tag", ["a", "b"])
@pytest.mark.parametrize("kind", ["rot", "gen"])
def test_rotation_and_its_gradient_match_reference_vectors(tag, kind):
    """Heads of the golden x become query heads of a packed projection whose head size is the
    rotated width; the kernel's q must equal the reference's apply_rope output, and the merged
    gradient its autograd gradient."""
    z = np.load(os.path.join(GOLDEN, "rope.npz"))
    x, go = torch.from_numpy(z[f"{tag}_x"]), torch.from_numpy(z[f"{tag}_go"])
    cos, sin = [torch.from_numpy(z[f"{tag}_{kind}_{n}"]) for n in ("cos", "sin")]
    b, h, t, r = x.shape
    kv = torch.zeros(b, t, h, 2, r, dtype=torch.float64)
    qkv = torch.cat([x.permute(0, 2, 1, 3)[:, :, :, None, :], kv], dim=3).float().contiguous().cuda()
    q, k, v = _cabi.qkv_split_rope(qkv, cos, sin, r)
    assert q.shape == (b * h, t, r) and k.shape == (b * h, t, r)
    assert rel(q.view(b, h, t, r), torch.from_numpy(z[f"{tag}_{kind}_y"]), 1.0) < 2e-6
    assert not k.any() and not v.any()
    g3 = go.float().reshape(b * h, t, r).contiguous().cuda()
    gqkv = _cabi.qkv_merge_rope_grad(g3, torch.zeros_like(g3), torch.zeros_like(g3), cos, sin, r, b)
    got = gqkv[:, :, :, 0, :].permute(0, 2, 1, 3)
    assert rel(got, torch.from_numpy(z[f"{tag}_{kind}_gx"]), 1.0) < 2e-6
    assert not gqkv[:, :, :, 1:, :].any()


SITES = [
    # batch, tokens, heads, groups, head size, rotated features
    (2, 37, 4, 4, 32, 32), (2, 37, 4, 2, 32, 8), (1, 130, 6, 1, 64, 16), (3, 5, 2, 2, 8, 0), (1, 1, 8, 2, 16, 16),
]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["fp32", "bf16"])
@pytest.mark.parametrize("cfg", SITES, ids=[f"b{c[0]}t{c[1]}h{c[2]}g{c[3]}d{c[4]}r{c[5]}" for c in SITES])
def test_split_and_merge_against_oracle(cfg, dtype):
    b, t, heads, groups, hs, r = cfg
    g = torch.Generator().manual_seed(11 + t)
    qkv = torch.randn(b, t, (heads + 2 * groups) * hs, generator=g).to(dtype)
    cos, sin = tables(t, max(r, 1), 5)
    cos, sin = cos[:, :r], sin[:, :r]
    qper = heads // groups
    q, k, v = _cabi.qkv_split_rope(qkv.cuda().view(b, t, groups, qper + 2, hs), cos, sin, r)
    rq, rk, rv = split_heads(qkv.double(), cos.double(), sin.double(), heads, groups, hs, r, expand=False)
    eps = 2e-6 if dtype == torch.float32 else 2 ** -8
    assert rel(q.view(b, heads, t, hs), rq, 1.0) < eps and rel(k.view(b, groups, t, hs), rk, 1.0) < eps
    assert torch.equal(v.view(b, groups, t, hs).cpu().double(), rv)          # values are only moved
    if r < hs:                                                               # so are unrotated features
        assert torch.equal(q.view(b, heads, t, hs)[..., r:].cpu().double(), rq[..., r:])
    # the merge is the transpose of the split: <split(x), g> == <x, merge(g)>
    gq, gk, gv = [torch.randn(s.shape, generator=g).to(dtype) for s in (q, k, v)]
    x = qkv.double().requires_grad_(True)
    sq, sk, sv = split_heads(x, cos.double(), sin.double(), heads, groups, hs, r, expand=False)
    dot = (sq.reshape(q.shape) * gq.double()).sum() + (sk.reshape(k.shape) * gk.double()).sum() \
        + (sv.reshape(v.shape) * gv.double()).sum()
    dot.backward()
    got = _cabi.qkv_merge_rope_grad(gq.cuda(), gk.cuda(), gv.cuda(), cos, sin, r, b)
    assert got.shape == (b, t, groups, qper + 2, hs)
    assert rel(got.view(b, t, -1), x.grad, 1.0) < eps


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["fp32", "bf16"])
def test_axis_swap_is_an_exact_transpose(dtype):
    x = torch.randn(3, 7, 33, 24).to(dtype).cuda()
    y = _cabi.swap_middle_axes(x)
    assert y.shape == (3, 33, 7, 24) and y.is_contiguous()
    assert torch.equal(y, x.transpose(1, 2).contiguous())
    assert torch.equal(_cabi.swap_middle_axes(y), x)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["fp32", "bf16"])
@pytest.mark.parametrize("count", [0, 1, 3, 4, 1023, 70000])
def test_noise_scaling_matches_oracle_and_runs_in_place(count, dtype):
    g = torch.Generator().manual_seed(count)
    x, noise = [torch.randn(count, generator=g).to(dtype) for _ in range(2)]
    want = output_dropout(x.double(), noise.double(), 0.2)
    xc = x.cuda()
    got = _cabi.scale_by_noise(xc, noise.cuda(), 0.2)
    eps = 1e-6 if dtype == torch.float32 else 2 ** -8
    if count:
        assert float((got.double().cpu() - want).abs().max() / want.abs().max()) < eps
    same = _cabi.scale_by_noise(xc, noise.cuda(), 0.2, out=xc)
    assert same.data_ptr() == xc.data_ptr() and torch.equal(same, got)


FULL = [
    # batch, tokens, heads, groups, head size, rotated features, mask, p
    (2, 70, 4, 2, 32, 8, 1, 1), (1, 150, 4, 4, 64, 64, 1, 2), (2, 33, 6, 2, 16, 16, 0, 2), (1, 300, 4, 1, 64, 32, 1, 1),
    (2, 200, 2, 1, 128, 128, 1, 2), (1, 4400, 2, 2, 64, 64, 1, 1), (2, 140, 4, 2, 64, 64, 0, 2),
]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["fp32", "bf16"])
@pytest.mark.parametrize("cfg", FULL, ids=[f"b{c[0]}t{c[1]}h{c[2]}g{c[3]}d{c[4]}r{c[5]}m{c[6]}p{c[7]}" for c in FULL])
def test_call_site_forward_and_backward_against_oracle(cfg, dtype):
    b, t, heads, groups, hs, r, mask, p = cfg
    g = torch.Generator().manual_seed(21 + t)
    qkv = torch.randn(b, t, (heads + 2 * groups) * hs, generator=g).to(dtype)
    gy = torch.randn(b, t, heads * hs, generator=g).to(dtype)
    ang = torch.outer(torch.arange(t, dtype=torch.float32), 1.0 / (10000 ** (torch.arange(0, r, 2) / r)))
    cos, sin = torch.cos(ang).repeat(1, 2), torch.sin(ang).repeat(1, 2)
    xq = qkv.cuda().requires_grad_(True)
    _cabi.profile(True)
    y = fastmax_attention_from_qkv(xq, cos, sin, heads, groups, hs, r, mask=bool(mask), normalize=True, p=p)
    assert y.shape == (b, t, heads * hs) and y.dtype == dtype
    y.backward(gy.cuda())
    names = [n for n, _ in _cabi.profile_records()]
    _cabi.profile(False)
    if dtype == torch.bfloat16 and hs in (64, 128):
        # the tensor-core kernels write and read the (B, T, H, hs) layout themselves: no transposition pass
        assert "fm_swap_axes" not in names, names
    else:
        assert names.count("fm_swap_axes") == 2, names
    x = qkv.double().requires_grad_(True)
    want = call_site(x, cos.double(), sin.double(), heads, groups, hs, r, round_dtype=dtype, mask=mask,
                     normalize=1, p=p, a0=1.0, a1=1.0, a2=0.5, lim=1.0)
    want.backward(gy.double())
    assert rel(y.detach(), want.detach()) < TOL[dtype]
    assert rel(xq.grad, x.grad) < TOL[dtype]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["fp32", "bf16"])
def test_output_dropout_of_the_autograd_function(dtype):
    g = torch.Generator().manual_seed(8)
    q, k, v, go, noise = [torch.randn(2, 2, 90, 32, generator=g).to(dtype) for _ in range(5)]
    kw = dict(mask=1, normalize=1, p=2, a0=1.0, a1=1.0, a2=0.5, lim=1.0)
    qc, kc, vc = [t.cuda().requires_grad_(True) for t in (q, k, v)]
    mod = fastmax_b200.FASTMultiHeadAttention()
    out = mod(qc, kc, vc, noise.cuda(), True, 0.2, True, 1.0, 1.0, 1.0, 0.5, 1.0, 2)
    out.backward(go.cuda())
    qd, kd, vd = [t.double().requires_grad_(True) for t in (q, k, v)]
    want = output_dropout(fastmax_dense(qd, kd, vd, **kw), noise.double(), 0.2)
    want.backward(go.double())
    for got, ref in ((out.detach(), want.detach()), (qc.grad, qd.grad), (kc.grad, kd.grad), (vc.grad, vd.grad)):
        assert rel(got, ref) < TOL[dtype]
    with pytest.raises(ValueError):
        mod(qc, kc, vc, None, True, 0.2, True, 1.0, 1.0, 1.0, 0.5, 1.0, 2)


def test_bad_shapes_surface_as_value_errors():
    qkv = torch.randn(1, 4, 2, 3, 16, device="cuda")
    cos, sin = tables(4, 4, 1)
    with pytest.raises(ValueError):
        _cabi.qkv_split_rope(qkv, cos, sin, 4)                   # rotated width not a multiple of 8
    with pytest.raises(ValueError):
        _cabi.qkv_split_rope(torch.randn(1, 4, 2, 3, 12, device="cuda"), None, None, 0)   # head size
    with pytest.raises(ValueError):
        fastmax_attention_from_qkv(torch.randn(1, 4, 100, device="cuda"), cos, sin, 4, 2, 16, 8)
