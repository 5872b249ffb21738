"""Forward+backward for tensors that live in host memory.

Batch*head units are independent, so a problem whose q, k, v and upstream gradient sit in
(pinned) host memory is streamed through the GPU in groups of heads: while one group is
being computed, the next group's inputs are on their way in and the previous group's
results on their way out (three CUDA streams, three sets of device buffers).  A set's input
buffers may be refilled as soon as its kernels are done, its output buffers are rewritten only
after they have left the device, so the step costs about max(host->device time, device time,
device->host time) instead of their sum.
The reference has no host-memory path; its wrapper expects device tensors (example.py:8-50).
"""
from __future__ import annotations

import torch

from . import _cabi

__all__ = ["HostPipeline", "prefer_gpu_numa_node"]


def prefer_gpu_numa_node(device) -> int:
    """Make this process prefer host memory on the NUMA node the GPU hangs off (Linux
    ``set_mempolicy(MPOL_PREFERRED)``), so that pinned buffers allocated afterwards are local to
    the GPU's PCIe root and host<->device copies of several ranks do not all cross one socket's
    memory controllers.  Returns the node, or -1 when the topology cannot be read or the call is
    refused (nothing is changed then)."""
    import ctypes
    import os
    try:
        props = torch.cuda.get_device_properties(torch.device(device))
        bdf = "%04x:%02x:%02x.0" % (props.pci_domain_id, props.pci_bus_id, props.pci_device_id)
        with open("/sys/bus/pci/devices/%s/numa_node" % bdf) as f:
            node = int(f.read().strip())
        if node < 0 or node >= 1024 or os.uname().machine != "x86_64":
            return -1
        mask = (ctypes.c_ulong * 16)()
        mask[node // 64] = 1 << (node % 64)
        libc = ctypes.CDLL(None, use_errno=True)
        MPOL_PREFERRED, SYS_set_mempolicy = 1, 238
        rc = libc.syscall(ctypes.c_long(SYS_set_mempolicy), ctypes.c_int(MPOL_PREFERRED), mask,
                          ctypes.c_ulong(16 * 64 + 1))
        return node if rc == 0 else -1
    except Exception:
        return -1


class HostPipeline:
    """``HostPipeline(bh, n, d, dtype, device, heads_per_group=64, **attention kwargs)``;
    ``run(q, k, v, grad_out, out, grad_q, grad_k, grad_v)`` with (bh, n, d) pinned host tensors
    (the last four are written).  Causal or unmasked self-attention (same n for q and k)."""

    SETS = 3

    def __init__(self, bh, n, d, dtype, device, heads_per_group=64, **kw):
        self.dev = torch.device(device)
        self.kw = dict(kw)
        self.group = max(1, min(heads_per_group, bh))
        self.bh, self.n, self.d, self.dtype = bh, n, d, dtype
        g = self.group
        with torch.cuda.device(self.dev):
            probe = torch.empty(g, n, d, dtype=dtype, device=self.dev)
            fwd_b, bwd_b, st_b = _cabi.workspace_bytes(probe, probe, **self.kw)
            self.sets = []
            for _ in range(self.SETS):
                t = lambda: torch.empty(g, n, d, dtype=dtype, device=self.dev)
                self.sets.append(dict(
                    q=t(), k=t(), v=t(), go=t(), out=t(), grad_q=t(), grad_k=t(), grad_v=t(),
                    den=torch.empty(g, n, dtype=torch.float32, device=self.dev),
                    stats=torch.empty(st_b, dtype=torch.uint8, device=self.dev),
                    workspace=torch.empty(max(fwd_b, bwd_b, 1), dtype=torch.uint8, device=self.dev)))
            self.s_in, self.s_cmp, self.s_out = (torch.cuda.Stream(self.dev) for _ in range(3))
            self.ev_in = [torch.cuda.Event() for _ in range(self.SETS)]
            self.ev_cmp = [torch.cuda.Event() for _ in range(self.SETS)]
            self.ev_out = [torch.cuda.Event() for _ in range(self.SETS)]
        torch.cuda.synchronize(self.dev)

    def run(self, q, k, v, go, out, gq, gk, gv):
        cur = torch.cuda.current_stream(self.dev)
        for s in (self.s_in, self.s_cmp, self.s_out):
            s.wait_stream(cur)
        for i, lo in enumerate(range(0, self.bh, self.group)):
            hi = min(lo + self.group, self.bh)
            m = hi - lo
            b = i % self.SETS
            S = self.sets[b]
            with torch.cuda.stream(self.s_in):
                # the input buffers of this set are free once its previous kernels are done
                self.s_in.wait_event(self.ev_cmp[b])
                for name, src in (("q", q), ("k", k), ("v", v), ("go", go)):
                    S[name][:m].copy_(src[lo:hi], non_blocking=True)
                self.ev_in[b].record(self.s_in)
            with torch.cuda.stream(self.s_cmp):
                self.s_cmp.wait_event(self.ev_in[b])
                # ... and its output buffers once their previous contents have left the device
                self.s_cmp.wait_event(self.ev_out[b])
                view = {n_: S[n_][:m] for n_ in ("q", "k", "v", "go", "out", "grad_q", "grad_k", "grad_v", "den")}
                bufs = dict(out=view["out"], den=view["den"], stats=S["stats"], workspace=S["workspace"],
                            grad_q=view["grad_q"], grad_k=view["grad_k"], grad_v=view["grad_v"])
                o, den, stats = _cabi.forward(view["q"], view["k"], view["v"], buffers=bufs, **self.kw)
                _cabi.backward(view["q"], view["k"], view["v"], o, den, stats, view["go"], buffers=bufs, **self.kw)
                self.ev_cmp[b].record(self.s_cmp)
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(self.ev_cmp[b])
                for name, dst in (("out", out), ("grad_q", gq), ("grad_k", gk), ("grad_v", gv)):
                    dst[lo:hi].copy_(S[name][:m], non_blocking=True)
                self.ev_out[b].record(self.s_out)
        for s in (self.s_in, self.s_cmp, self.s_out):
            cur.wait_stream(s)
