"""Sequence sharding on CPU ranks (gloo): the exchange logic of fastmax_b200.sharded --
which shard totals each rank receives, the reverse scan of the backward pass, the reduced
max-norm statistics and the ownership of the max-norm row -- driven with the CPU stand-in
for the stage calls and checked against the unsharded oracle."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle.fastmax_oracle import fastmax_fwd_bwd, rel_err


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, normalize, p, mask, ret):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import sys
        sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
        from shard_cpu_backend import TorchShardBackend

        from fastmax_b200.sharded import fastmax_sequence_parallel

        torch.manual_seed(11)                      # every rank builds the same full problem
        h, n, d = 3, 24 * world, 8
        q, k, v, go = [torch.randn(1, h, n, d, dtype=torch.float64) for _ in range(4)]
        kw = dict(mask=int(mask), normalize=int(normalize), p=p, a0=0.9, a1=1.1, a2=0.45, lim=1.3)
        ref = fastmax_fwd_bwd(q, k, v, go, **kw)
        nl = n // world
        sl = slice(rank * nl, (rank + 1) * nl)
        ql, kl, vl = [t[0, :, sl].clone().requires_grad_(True) for t in (q, k, v)]
        be = TorchShardBackend(normalize, 0.9, 1.1, 0.45, 1.3, p, mask=mask)
        out = fastmax_sequence_parallel(ql, kl, vl, mask=mask, normalize=normalize, backend=be)
        out.backward(go[0, :, sl])
        errs = [rel_err(a, b[0, :, sl]) for a, b in zip((out.detach(), ql.grad, kl.grad, vl.grad), ref)]
        ret[rank] = errs
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
@pytest.mark.parametrize("mask", [True, False], ids=["causal", "unmasked"])
@pytest.mark.parametrize("normalize,p", [(False, 2), (True, 2), (True, 1)])
def test_sequence_sharding_matches_unsharded_oracle(world, normalize, p, mask):
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), normalize, p, mask, ret), nprocs=world, join=True)
    assert len(ret) == world
    for rank, errs in ret.items():
        for e, name in zip(errs, ("out", "dq", "dk", "dv")):
            assert e < 1e-6, (rank, name, e)
