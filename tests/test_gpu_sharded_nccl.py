"""Sequence sharding over NCCL on two GPUs (skipped on a one-GPU box): every rank runs
fastmax_sequence_parallel on its half and compares with the single-GPU result of the whole
sequence.  Each rank leaves only after the final barrier, with nothing in flight."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, mask, ret):
    import torch.distributed as dist

    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from fastmax_b200 import _cabi
        from fastmax_b200.sharded import fastmax_sequence_parallel

        g = torch.Generator(device=dev).manual_seed(3)          # same full problem on every rank
        bh, n, d = 4, 4096, 64
        q, k, v, go = [torch.randn(bh, n, d, generator=g, device=dev).bfloat16() for _ in range(4)]
        kw = dict(mask=mask, normalize=True, p=2)
        out, den, stats = _cabi.forward(q, k, v, impl="dense_tc", **kw)
        want = (out,) + tuple(_cabi.backward(q, k, v, out, den, stats, go, impl="dense_tc", **kw))
        nl = n // world
        sl = slice(rank * nl, (rank + 1) * nl)
        ql, kl, vl = [t[:, sl].contiguous().requires_grad_(True) for t in (q, k, v)]
        o = fastmax_sequence_parallel(ql, kl, vl, mask=mask, normalize=True, p=2, chunk=512)
        o.backward(go[:, sl].contiguous())
        torch.cuda.synchronize()
        errs = []
        for a, b in zip((o.detach(), ql.grad, kl.grad, vl.grad), want):
            b = b[:, sl].float()
            errs.append(float((a.float() - b).abs().max() / b.abs().max()))
        ret[rank] = (errs, _cabi.device_status())
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("mask", [True, False], ids=["causal", "unmasked"])
def test_two_gpu_sequence_sharding_matches_single_gpu(mask):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(2, _free_port(), mask, ret), nprocs=2, join=True)
    assert len(ret) == 2
    for rank, (errs, status) in ret.items():
        assert status == 0
        for e, name in zip(errs, ("out", "dq", "dk", "dv")):
            assert e < 2e-2, (rank, name, e)
