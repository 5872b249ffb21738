"""The give-up path of the bounded waits, and requests the fast family cannot serve.

Every wait inside the tensor-core kernels is bounded; one that runs out stores a code in a device
word and the kernel returns.  Here that path is taken on purpose without breaking any real kernel's
protocol: a one-warp kernel waits, with a limit of about a millisecond, on a barrier that nothing
ever completes.  Nothing faults or hangs, the context stays usable, and the library computes
correctly afterwards.
"""
import pytest
import torch

from gpu_util import assert_close, oracle, run_cabi

from fastmax_b200 import _cabi

pytestmark = pytest.mark.gpu


def test_a_wait_that_runs_out_reports_a_status_and_leaves_the_library_usable():
    _cabi.device_status_reset()
    assert _cabi.device_status() == 0
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    _cabi.wait_selftest(2_000_000)            # about a millisecond of SM clocks
    ev1.record()
    torch.cuda.synchronize()
    assert ev0.elapsed_time(ev1) < 500.0      # the kernel returned by itself, long before the one-second limit
    assert _cabi.device_status() == 99
    # the word is sticky until it is cleared
    assert _cabi.device_status() == 99
    _cabi.device_status_reset()
    assert _cabi.device_status() == 0
    # and the next real launch is correct
    g = torch.Generator().manual_seed(79)
    q, k, v, go = [torch.randn(1, 3, 255, 64, generator=g) for _ in range(4)]
    kw = dict(mask=1, normalize=1, p=2, a0=1.0, a1=1.0, a2=0.5, lim=1.0)
    got, _ = run_cabi(q, k, v, go, torch.bfloat16, impl="dense_tc", **kw)
    assert _cabi.device_status() == 0
    assert_close(got, oracle(q, k, v, go, torch.bfloat16, dense=True, **kw), torch.bfloat16, "after the selftest")


def test_wait_selftest_rejects_limits_beyond_the_kernels_own():
    with pytest.raises(ValueError):
        _cabi.wait_selftest(10 ** 12)


def test_auto_serves_unaligned_bf16_tensors_on_the_cuda_core_family():
    """Views that start 2 bytes off a 16-byte boundary cannot be read through TMA; the library's own choice
    (impl = auto) must then fall back instead of failing, while a forced tensor-core request still errors."""
    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(78)
    q, k, v, go = [torch.randn(1, 2, 260, 64, generator=g) for _ in range(4)]
    kw = dict(mask=1, normalize=1, p=2, a0=1.0, a1=1.0, a2=0.5, lim=1.0)

    def off_by_one(t):
        flat = torch.empty(t.numel() + 1, dtype=torch.bfloat16, device=dev)
        view = flat[1:].view(t.shape[1:])
        view.copy_(t[0].bfloat16())
        assert view.data_ptr() % 16 == 2 and view.is_contiguous()
        return view

    qc, kc, vc, gc = [off_by_one(t) for t in (q, k, v, go)]
    _cabi.profile(True)
    out, den, stats = _cabi.forward(qc, kc, vc, impl="auto", **kw)
    gq, gk, gv = _cabi.backward(qc, kc, vc, out, den, stats, gc, impl="auto", **kw)
    names = {n for n, _ in _cabi.profile_records()}
    _cabi.profile(False)
    assert "fm_dense_ffma_fwd" in names and not any(n.startswith("fm_dense_tc") for n in names), names
    ref = oracle(q, k, v, go, torch.bfloat16, dense=True, **kw)
    assert_close([t.float().cpu()[None] for t in (out, gq, gk, gv)], ref, torch.bfloat16, "unaligned")
    with pytest.raises((RuntimeError, ValueError)):
        _cabi.forward(qc, kc, vc, impl="dense_tc", **kw)
