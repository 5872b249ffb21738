"""GPU parity of the moment-state family (chunk states, prefix, read-outs, coupled to the
score-form kernels for each chunk's own block) and of the sequence-shard stage calls,
through the C ABI.  Tolerances: 1e-4 (float32), 2e-2 (bfloat16), relative max error."""
import pytest
import torch

from conftest import case_kwargs, load_small_cases
from gpu_util import assert_close, oracle, run_cabi

from fastmax_b200 import _cabi
from fastmax_b200.sharded import CudaShardBackend

pytestmark = pytest.mark.gpu
CASES = load_small_cases()


def randn(*shape, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g)


@pytest.mark.parametrize("c", CASES, ids=[c["tag"] for c in CASES])
def test_reference_vectors_through_the_moment_family(c):
    """Sequences shorter than one chunk: states are built and summed, the score-form part covers everything."""
    got, _ = run_cabi(c["q"], c["k"], c["v"], c["go"], torch.float32, impl="moments", chunk=256,
                      **case_kwargs(c))
    assert_close(got, [c[n + "64"] for n in ("out", "dq", "dk", "dv")], torch.float32, c["tag"])


# bh, n, d, mask, p, normalize, chunk
MOM = [(2, 700, 32, 1, 2, 1, 256), (2, 700, 32, 0, 2, 1, 256), (3, 1024, 32, 1, 1, 1, 256),
       (2, 600, 16, 1, 2, 0, 256), (1, 900, 64, 1, 2, 1, 256), (2, 520, 64, 0, 2, 0, 256),
       (1, 600, 128, 1, 2, 0, 256), (2, 515, 128, 0, 1, 0, 256), (2, 1030, 64, 1, 2, 1, 512),
       (2, 900, 64, 1, 1, 1, 256), (2, 700, 128, 1, 1, 1, 256), (3, 640, 64, 0, 1, 0, 256)]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["fp32", "bf16"])
@pytest.mark.parametrize("cfg", MOM, ids=[f"bh{c[0]}n{c[1]}d{c[2]}m{c[3]}p{c[4]}z{c[5]}L{c[6]}" for c in MOM])
def test_moment_family_over_several_chunks(cfg, dtype):
    bh, n, d, mask, p, norm, chunk = cfg
    q, k, v, go = [randn(1, bh, n, d, seed=300 + i + n) for i in range(4)]
    if not norm:
        q, k = q * d ** -0.5, k * d ** -0.5
    kw = dict(mask=mask, normalize=norm, p=p, a0=1.0, a1=1.0, a2=0.5, lim=1.0)
    got, _ = run_cabi(q, k, v, go, dtype, impl="moments", chunk=chunk, **kw)
    assert _cabi.device_status() == 0
    ref = oracle(q, k, v, go, dtype, dense=True, **kw)
    assert_close(got, ref, dtype, str(cfg))


def test_unmasked_moments_with_more_keys_than_queries():
    q, go = randn(1, 2, 300, 32, seed=1), randn(1, 2, 300, 32, seed=2)
    k, v = randn(1, 2, 777, 32, seed=3), randn(1, 2, 777, 32, seed=4)
    kw = dict(mask=0, normalize=1, p=2, a0=1.0, a1=1.0, a2=0.5, lim=1.0)
    got, _ = run_cabi(q, k, v, go, torch.float32, impl="moments", chunk=256, **kw)
    ref = oracle(q, k, v, go, torch.float32, dense=True, **kw)
    assert_close(got, ref, torch.float32, "unmasked nq != nk")


@pytest.mark.parametrize("dtype,d,normalize", [(torch.float32, 32, True), (torch.bfloat16, 64, True),
                                               (torch.float32, 16, False)])
def test_shard_stage_calls_reproduce_the_unsharded_result(dtype, d, normalize):
    """Three shards of one sequence evaluated one after another on this GPU, with the exchange
    of totals done by hand, against the single-call result on the whole sequence."""
    dev = torch.device("cuda", 0)
    G, nl, bh = 3, 384, 3
    g = torch.Generator(device=dev).manual_seed(9)
    q, k, v, go = [torch.randn(bh, G * nl, d, generator=g, device=dev).to(dtype) for _ in range(4)]
    kw = dict(mask=True, normalize=normalize, p=2)
    out, den, stats = _cabi.forward(q, k, v, impl="dense_ffma", **kw)
    want = (out,) + tuple(_cabi.backward(q, k, v, out, den, stats, go, impl="dense_ffma", **kw))

    be = CudaShardBackend(normalize=normalize, a0=1.0, a1=1.0, a2=0.5, lim=1.0, p=2, chunk=256)
    sh = lambda t, r: t[:, r * nl:(r + 1) * nl].contiguous()
    qs, ks, vs, gs = [[sh(t, r) for r in range(G)] for t in (q, k, v, go)]
    st = None
    if normalize:
        st = torch.stack([be.rowmax(qs[r], ks[r], r * nl) for r in range(G)]).max(0).values
    kv = [be.kv_state(ks[r], vs[r]) for r in range(G)]
    outs, dens = [], []
    for r in range(G):
        base = sum(kv[j][1] for j in range(r)) if r else None
        o, dn = be.forward(qs[r], ks[r], vs[r], st, kv[r][0], base)
        outs.append(o); dens.append(dn)
    qg = [be.qg_state(qs[r], outs[r], dens[r], gs[r]) for r in range(G)]
    grads = []
    for r in range(G):
        base = sum(qg[j][2] for j in range(r + 1, G)) if r < G - 1 else None
        grads.append(be.backward(qs[r], ks[r], vs[r], outs[r], dens[r], st, gs[r], qg[r][0], kv[r][0], qg[r][1], base))
    # the split backward (grad_q's far part issued early, as the multi-GPU driver does while the totals
    # travel) and the library's sum over gathered totals give the same numbers
    gathered = torch.stack([x[2] for x in qg])
    for r in range(G):
        delta_r, states_r, _ = be.qg_state(qs[r], outs[r], dens[r], gs[r])
        be.dq_far(qs[r], dens[r], st, gs[r], delta_r, kv[r][0])
        base = None
        if r < G - 1:
            base = torch.empty_like(gathered[0])
            _cabi._check(_cabi.lib().fastmax_b200_shard_sum_totals(gathered.data_ptr(), G, r, 1, gathered.shape[1],
                                                                   base.data_ptr(), _cabi._stream(base)), "sum_totals")
            want_base = sum(qg[j][2] for j in range(r + 1, G))
            assert torch.allclose(base, want_base, rtol=1e-6, atol=1e-6)
        split = be.backward(qs[r], ks[r], vs[r], outs[r], dens[r], st, gs[r], delta_r, kv[r][0], states_r, base,
                            dq_far_done=True)
        for a, b, name in zip(split, grads[r], ("dq", "dk", "dv", "dots")):
            assert torch.allclose(a.float(), b.float(), rtol=1e-5, atol=1e-6), (r, name)
    if normalize:
        dots = sum(gr[3] for gr in grads)
        for r in range(G):
            be.norm_fixup(qs[r], ks[r], st, dots, r * nl, grads[r][0], grads[r][1])
    torch.cuda.synchronize()
    assert _cabi.device_status() == 0
    got = (torch.cat(outs, 1),) + tuple(torch.cat([gr[i] for gr in grads], 1) for i in range(3))
    tol = 1e-4 if dtype == torch.float32 else 2e-2
    for a, b, name in zip(got, want, ("out", "dq", "dk", "dv")):
        e = float((a.float() - b.float()).abs().max() / b.float().abs().max())
        assert e < tol, (name, e)
    # and against the CPU oracle, not only against another CUDA path
    ref = oracle(*[t.float().cpu()[None] for t in (q, k, v, go)], dtype, dense=True, a0=1.0, a1=1.0, a2=0.5, lim=1.0,
                 **{n_: int(x_) for n_, x_ in kw.items()})
    assert_close([t.float().cpu()[None] for t in got], ref, dtype, "shard stages vs oracle")


@pytest.mark.parametrize("dtype,d,normalize,p", [(torch.float32, 32, True, 2), (torch.bfloat16, 64, True, 2),
                                                 (torch.bfloat16, 128, False, 1), (torch.float32, 16, False, 2)])
def test_unmasked_shard_stage_calls_reproduce_the_unsharded_result(dtype, d, normalize, p):
    """Unmasked attention over three shards: the totals are summed over ALL shards (what an
    all-reduce does) and every shard reads them."""
    dev = torch.device("cuda", 0)
    G, nl, bh = 3, 384, 3
    g = torch.Generator(device=dev).manual_seed(19)
    q, k, v, go = [torch.randn(bh, G * nl, d, generator=g, device=dev).to(dtype) for _ in range(4)]
    if not normalize:
        q, k = q * d ** -0.5, k * d ** -0.5
    kw = dict(mask=False, normalize=normalize, p=p)
    out, den, stats = _cabi.forward(q, k, v, impl="dense_ffma", **kw)
    want = (out,) + tuple(_cabi.backward(q, k, v, out, den, stats, go, impl="dense_ffma", **kw))

    be = CudaShardBackend(mask=False, normalize=normalize, a0=1.0, a1=1.0, a2=0.5, lim=1.0, p=p, chunk=256)
    sh = lambda t, r: t[:, r * nl:(r + 1) * nl].contiguous()
    qs, ks, vs, gs = [[sh(t, r) for r in range(G)] for t in (q, k, v, go)]
    st = None
    if normalize:
        st = torch.stack([be.rowmax(qs[r], ks[r], r * nl) for r in range(G)]).max(0).values
    kv_total = sum(be.kv_state(ks[r], vs[r])[1] for r in range(G))
    outs, dens = zip(*[be.forward(qs[r], ks[r], vs[r], st, None, kv_total) for r in range(G)])
    qg = [be.qg_state(qs[r], outs[r], dens[r], gs[r]) for r in range(G)]
    qg_total = sum(x[2] for x in qg)
    grads = [be.backward(qs[r], ks[r], vs[r], outs[r], dens[r], st, gs[r], qg[r][0], kv_total, None, qg_total)
             for r in range(G)]
    if normalize:
        dots = sum(gr[3] for gr in grads)
        for r in range(G):
            be.norm_fixup(qs[r], ks[r], st, dots, r * nl, grads[r][0], grads[r][1])
    torch.cuda.synchronize()
    assert _cabi.device_status() == 0
    got = (torch.cat(outs, 1),) + tuple(torch.cat([gr[i] for gr in grads], 1) for i in range(3))
    tol = 1e-4 if dtype == torch.float32 else 2e-2
    for a, b, name in zip(got, want, ("out", "dq", "dk", "dv")):
        e = float((a.float() - b.float()).abs().max() / b.float().abs().max())
        assert e < tol, (name, e)
    # and against the CPU oracle, not only against another CUDA path
    ref = oracle(*[t.float().cpu()[None] for t in (q, k, v, go)], dtype, dense=True, a0=1.0, a1=1.0, a2=0.5, lim=1.0,
                 **{n_: int(x_) for n_, x_ in kw.items()})
    assert_close([t.float().cpu()[None] for t in got], ref, dtype, "shard stages vs oracle")


def test_second_order_state_rows_are_mirrored_and_match_the_definition():
    """The tensor-core state build forms each unordered feature pair {a, b} once and writes the row to
    both (a, b) and (b, a): the two rows must be bit-identical, every row must be written (ragged last
    chunk included), and the total must equal sum_j k_j[a] k_j[b] v_j[c] -- with the products of two
    bf16 values rounded to bf16, as the kernel forms them."""
    dev = torch.device("cuda", 0)
    bh, n, d = 3, 1000, 64
    g = torch.Generator(device=dev).manual_seed(21)
    k, v = [torch.randn(bh, n, d, generator=g, device=dev).bfloat16() for _ in range(2)]
    be = CudaShardBackend(normalize=False, a0=1.0, a1=1.0, a2=0.5, lim=1.0, p=2, chunk=256)
    _, total = be.kv_state(k, v)
    dvp, rows = 68, d * d + d + 1
    assert total.numel() >= bh * rows * dvp                          # the size query rounds up to 256 bytes
    t = total[:bh * rows * dvp].view(bh, rows, dvp)
    s2 = t[:, :d * d, :d].reshape(bh, d, d, d)                     # [a][b][c]
    assert torch.equal(s2, s2.transpose(1, 2))
    e2 = t[:, :d * d, d].reshape(bh, d, d)                          # normaliser column
    kf, vf = k.float(), v.float()
    feat = (kf[:, :, :, None] * kf[:, :, None, :]).bfloat16().float()      # (bh, n, a, b), rounded like the kernel's
    want = torch.einsum("hjab,hjc->habc", feat, vf)
    scale = want.abs().max()
    assert float((s2 - want).abs().max() / scale) < 2e-3
    want_e = torch.einsum("hja,hjb->hab", kf, kf)
    assert float((e2 - want_e).abs().max() / want_e.abs().max()) < 1e-2
    s1 = t[:, d * d:d * d + d, :d]                                  # first-order rows
    want1 = torch.einsum("hja,hjc->hac", kf, vf)
    assert float((s1 - want1).abs().max() / want1.abs().max()) < 2e-3
