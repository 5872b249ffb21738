"""GPU parity of decoding against a persistent moment state: every step must reproduce the
attention row the oracle computes for that query over all tokens so far (the reference's
key/value-cache call: one query row, all keys, causal), 1e-4 relative in float32 and 2e-2 in
bfloat16, and agree with the library's own forward on the same shapes."""
import pytest
import torch

from gpu_util import TOL
from oracle.fastmax_oracle import fastmax_dense

from fastmax_b200 import FastmaxDecodeState, _cabi

pytestmark = pytest.mark.gpu

CASES = [
    # key/value heads, query heads per key/value head, d, p, normalize, prompt tokens, decoded tokens
    (3, 1, 32, 2, 1, 20, 6), (2, 2, 64, 2, 1, 37, 5), (2, 1, 64, 1, 1, 0, 8), (1, 4, 32, 1, 0, 17, 4),
    (1, 1, 128, 2, 1, 9, 3), (2, 1, 64, 2, 0, 1, 3),
]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["fp32", "bf16"])
@pytest.mark.parametrize("cfg", CASES, ids=[f"kv{c[0]}x{c[1]}d{c[2]}p{c[3]}z{c[4]}n{c[5]}+{c[6]}" for c in CASES])
def test_steps_match_oracle_rows_and_library_forward(cfg, dtype):
    bhkv, ratio, d, p, norm, n0, steps = cfg
    bh, n = bhkv * ratio, n0 + steps
    g = torch.Generator().manual_seed(31 + d + n)
    scale = 1.0 if norm else d ** -0.5
    q = (torch.randn(bh, n, d, generator=g) * scale).to(dtype)
    k = (torch.randn(bhkv, n, d, generator=g) * scale).to(dtype)
    v = torch.randn(bhkv, n, d, generator=g).to(dtype)
    kw = dict(mask=1, normalize=norm, p=p, a0=1.0, a1=1.0, a2=0.5, lim=1.0)
    st = FastmaxDecodeState(bh, bhkv, d, dtype=dtype, device="cuda:0", normalize=bool(norm), p=p)
    qc, kc, vc = q.cuda(), k.cuda(), v.cuda()
    if n0:
        st.append(kc[:, :n0].contiguous(), vc[:, :n0].contiguous())
    for t in range(n0, n):
        out = st.step(qc[:, t:t + 1].contiguous(), kc[:, t:t + 1].contiguous(), vc[:, t:t + 1].contiguous())
        kx = k[:, :t + 1].double().repeat_interleave(ratio, dim=0)[None]
        vx = v[:, :t + 1].double().repeat_interleave(ratio, dim=0)[None]
        want = fastmax_dense(q[:, t:t + 1].double()[None], kx, vx, **kw)[0]
        err = float((out.double().cpu() - want).abs().max() / want.abs().max().clamp_min(1e-2))
        assert err < TOL[dtype], (t, err)
        lib_out, _, _ = _cabi.forward(qc[:, t:t + 1].contiguous(), kc[:, :t + 1].contiguous(),
                                      vc[:, :t + 1].contiguous(), mask=True, normalize=bool(norm), p=p)
        err = float((out.double() - lib_out.double()).abs().max() / want.abs().max().clamp_min(1e-2))
        assert err < TOL[dtype], ("library forward", t, err)
    assert st.tokens == n


def test_prompt_in_pieces_equals_prompt_at_once_and_reset_clears():
    g = torch.Generator().manual_seed(5)
    k, v = [torch.randn(2, 50, 64, generator=g).cuda() for _ in range(2)]
    a = FastmaxDecodeState(2, 2, 64, dtype=torch.float32, device="cuda:0")
    b = FastmaxDecodeState(2, 2, 64, dtype=torch.float32, device="cuda:0")
    a.append(k, v)
    for lo, hi in ((0, 1), (1, 18), (18, 50)):
        b.append(k[:, lo:hi].contiguous(), v[:, lo:hi].contiguous())
    assert torch.allclose(a.state, b.state, rtol=1e-5, atol=1e-5)
    assert float(a.state.view(2, -1)[0, 0]) == pytest.approx(float((k[0] ** 2).sum(-1).max()), rel=1e-6)
    a.reset()
    assert not a.state.any() and a.tokens == 0


def test_bad_arguments_raise():
    with pytest.raises(ValueError):
        FastmaxDecodeState(2, 2, 48, dtype=torch.float32, device="cuda:0").append(
            torch.zeros(2, 1, 48, device="cuda"), torch.zeros(2, 1, 48, device="cuda"))
    st = FastmaxDecodeState(2, 2, 32, dtype=torch.float32, device="cuda:0")
    with pytest.raises(ValueError):
        st.step(torch.zeros(2, 2, 32, device="cuda"), torch.zeros(2, 1, 32, device="cuda"),
                torch.zeros(2, 1, 32, device="cuda"))
    with pytest.raises(ValueError):
        st.append(torch.zeros(2, 3, 32, device="cuda").bfloat16(), torch.zeros(2, 3, 32, device="cuda").bfloat16())


@pytest.mark.parametrize("p", [1, 2])
def test_steps_match_the_oracle_recurrence_with_other_coefficients(p):
    """Against the CPU restatement of the recurrence itself, with a0, a1, a2, lim away from their defaults."""
    from oracle.call_site_oracle import MomentState
    g = torch.Generator().manual_seed(3)
    heads, n, d, n0 = 4, 30, 32, 21
    q, k, v = [torch.randn(heads, n, d, generator=g) for _ in range(3)]
    coef = dict(a0=0.7, a1=1.3, a2=0.4, lim=1.5)
    ref = MomentState(heads, d, p=p, normalize=True, **coef)
    st = FastmaxDecodeState(heads, heads, d, dtype=torch.float32, device="cuda:0", normalize=True, p=p, **coef)
    ref.append(k[:, :n0], v[:, :n0])
    st.append(k[:, :n0].contiguous().cuda(), v[:, :n0].contiguous().cuda())
    for t in range(n0, n):
        sl = slice(t, t + 1)
        want = ref.step(q[:, sl], k[:, sl], v[:, sl])
        got = st.step(q[:, sl].contiguous().cuda(), k[:, sl].contiguous().cuda(), v[:, sl].contiguous().cuda())
        err = float((got.double().cpu() - want).abs().max() / want.abs().max())
        assert err < TOL[torch.float32], (t, err)
