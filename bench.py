"""Fastmax forward+backward throughput on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

A step is one forward + backward pass of Fastmax attention over one batch of
synthetic N(0,1) inputs.  The workload is the configuration the headline target
is quoted on: causal, bf16, p=2, B=64, H=16, N=10000, D=64, normalize=True,
lim=1, a=(1,1,0.5).  With N GPUs every rank runs that workload on its own shard
of an N-times larger batch (batch*head units are independent; no collective on
the data path), so `value` is total tokens of all ranks over the slowest rank's
device time ("weak" scaling); `--scaling strong` splits the single batch's
batch*head units over the ranks instead.

Rank 0 prints one JSON line.  `value` is measured with the inputs resident in
HBM; `e2e` is the same metric with pinned host buffers through
fastmax_b200.host.HostPipeline, host<->device copies inside the timed region.  `--impl reference` times
the CPU restatement of the reference's PyTorch path (oracle/) on the host
cores, on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (B, H, N, D, dtype, mask, p, normalize)
    "c3": (64, 16, 10000, 64, "bf16", 1, 2, 1),
    "c1": (2, 8, 1024, 32, "fp32", 0, 2, 1),
    "c2": (64, 8, 1000, 32, "fp32", 1, 2, 1),
    "c4p2": (32, 32, 16384, 128, "bf16", 0, 2, 0),
    "c4p1": (32, 32, 16384, 128, "bf16", 0, 1, 0),
    "c5": (1, 32, 262144, 64, "bf16", 1, 2, 1),   # long context; sharded along the sequence when N > 1
    "c5s": (1, 8, 65536, 64, "bf16", 1, 2, 1),    # reduced long-context case
    "c5u": (1, 32, 262144, 128, "bf16", 0, 1, 0), # long unmasked p = 1 sequence, sharded along the sequence when N > 1
    "tiny": (2, 4, 1024, 64, "bf16", 1, 2, 1),
    "c4s": (4, 8, 16384, 128, "bf16", 0, 2, 0),   # reduced unmasked d=128 case
    "prof": (8, 16, 4096, 64, "bf16", 1, 2, 1),   # small case for ncu captures (inputs 4 x 67 MB)
    "prof1": (2, 8, 16384, 128, "bf16", 0, 1, 0),  # small p = 1 case for ncu captures (inputs 4 x 67 MB)
    # decoding against the persistent moment state: one new token per sequence and step (N is not used)
    "decode": (64, 16, 1, 64, "bf16", 1, 2, 1),
    "decodes": (16, 16, 1, 64, "bf16", 1, 2, 1),   # small case for ncu captures (277 MB of state)
    # the model's call site: packed projection -> rotary embedding -> attention -> (B, T, H*hs), and back
    "site": (8, 32, 4096, 64, "bf16", 1, 1, 1),
}
A = dict(a0=1.0, a1=1.0, a2=0.5, lim=1.0)


def describe(name):
    B, H, N, D, dt, mask, p, norm = WORKLOADS[name]
    return (f"{name}: {'causal' if mask else 'unmasked'} {dt} p={p} B={B} H={H} N={N} D={D} "
            f"normalize={bool(norm)} lim=1 a=(1,1,0.5)")


def alg_flops_per_token_head(D, p):
    """Algorithmic FLOPs of the factorised evaluation, per token and head:
    (forward, grad_q pass, grad_k+grad_v pass) = (4, 4, 6) * F * (D+1), F = D + [p=2] D^2."""
    F = D + (D * D if p == 2 else 0)
    u = F * (D + 1)
    return 4 * u, 4 * u, 6 * u


KERNEL_FLOP_SHARE = {"fwd": "fwd", "dq": "dq", "dkdv": "dkdv", "dk": "dk", "dv": "dv"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.lines, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                 "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def run_decode(args, world, rank, dev, cfg):
    """One step = one new token for each of the B sequences on every rank (B*H heads, grouped 1:1), added to
    the per-head moment state and read by its query.  The state (fp32, larger than L2) is read and written once
    per step: HBM-bound, 2 x state bytes of algorithmic traffic.  Sequences are independent: no collective."""
    import torch
    import torch.distributed as dist

    from fastmax_b200 import FastmaxDecodeState, _cabi

    B, H, _, D, dt, _, p, norm = cfg
    dtype = torch.bfloat16 if dt == "bf16" else torch.float32
    st = FastmaxDecodeState(B * H, B * H, D, dtype=dtype, device=dev, normalize=bool(norm), p=p, **A)
    g = torch.Generator(device=dev).manual_seed(1234 + rank)
    q, k, v = [torch.randn(B * H, 1, D, generator=g, device=dev, dtype=torch.float32).to(dtype) for _ in range(3)]
    st.append(torch.randn(B * H, 64, D, generator=g, device=dev, dtype=torch.float32).to(dtype),
              torch.randn(B * H, 64, D, generator=g, device=dev, dtype=torch.float32).to(dtype))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        st.step(q, k, v)
    barrier()
    sampler = ClockSampler(dev.index)
    if rank == 0:
        sampler.start()
    _cabi.profile(True)
    n0 = _cabi.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(args.steps):
        out = st.step(q, k, v)
    e1.record()
    barrier()
    tms = torch.tensor([e0.elapsed_time(e1)], device=dev)
    launches = _cabi.launch_count() - n0
    recs = _cabi.profile_records()
    _cabi.profile(False)
    clocks = sampler.stop() if rank == 0 else None
    if world > 1:
        dist.all_reduce(tms, op=dist.ReduceOp.MAX)
    ms = float(tms.item())
    # end to end: the new token's q, k, v from pinned host memory, the attention row back to the host
    host = [t.cpu().pin_memory() for t in (q, k, v)]
    host_out = torch.empty_like(out, device="cpu").pin_memory()
    dq, dk, dv = [torch.empty_like(t) for t in (q, k, v)]
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        for d_, h_ in zip((dq, dk, dv), host):
            d_.copy_(h_, non_blocking=True)
        host_out.copy_(st.step(dq, dk, dv), non_blocking=True)
    barrier()
    e2e_ms = torch.tensor([(time.perf_counter() - t0) * 1e3], device=dev)
    if world > 1:
        dist.all_reduce(e2e_ms, op=dist.ReduceOp.MAX)
    if rank == 0:
        peaks = load_peaks()
        step_ms = sum(t for n, t in recs if n == "fm_decode_step") / max(1, sum(1 for n, _ in recs if n == "fm_decode_step"))
        state_bytes = st.state.numel() * 4
        ach = 2 * state_bytes / (step_ms * 1e-3) / 1e9
        nbytes = q.numel() * q.element_size()
        line = {
            "metric": "fastmax_decode_tokens_per_s", "value": B * world * args.steps / (ms * 1e-3), "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": dt, "data": "synthetic",
            "config": {"workload": describe(args.workload) + " (one token per sequence and step; fp32 moment state of "
                                   f"{state_bytes / 1e6:.0f} MB per GPU instead of a key/value cache)",
                       "global_batch": B * world, "parallelism": f"sequences sharded x{world}, no collective",
                       "l2": "the state read and written each step is larger than the 126 MB L2"
                             if state_bytes > 126e6 else "state smaller than L2"},
            "clocks": clocks, "gpu_launches": int(launches),
            "e2e": {"value": B * world * args.steps / (float(e2e_ms.item()) * 1e-3), "unit": "tokens/s",
                    "h2d_bytes_per_step": 3 * nbytes, "d2h_bytes_per_step": nbytes},
            "roofline": {"bound": "hbm", "achieved": ach, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": ach / peaks["hbm_gbs"], "traffic": None, "kernel": "fm_decode_step",
                         "peak_source": peaks["source"]},
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_site(args, world, rank, dev, cfg):
    """One step = forward + backward of `fastmax_attention_from_qkv` on a packed projection (B, T, 3*H*hs) that
    is resident on the GPU: split + rotary embedding, attention, axis swap, and the mirror-image gradient passes.
    Batches are independent: every rank runs its own (weak scaling, no collective)."""
    import torch
    import torch.distributed as dist

    from fastmax_b200 import _cabi, fastmax_attention_from_qkv

    B, H, N, D, dt, mask, p, norm = cfg
    dtype = torch.bfloat16 if dt == "bf16" else torch.float32
    g = torch.Generator(device=dev).manual_seed(1234 + rank)
    qkv = torch.randn(B, N, 3 * H * D, generator=g, device=dev, dtype=torch.float32).to(dtype)
    gy = torch.randn(B, N, H * D, generator=g, device=dev, dtype=torch.float32).to(dtype)
    ang = torch.outer(torch.arange(N, dtype=torch.float32, device=dev),
                      1.0 / (10000 ** (torch.arange(0, D, 2, device=dev) / D)))
    cos, sin = torch.cos(ang).repeat(1, 2), torch.sin(ang).repeat(1, 2)

    def step():
        x = qkv.detach().requires_grad_(True)
        y = fastmax_attention_from_qkv(x, cos, sin, H, H, D, D, mask=bool(mask), normalize=bool(norm), p=p, **A)
        y.backward(gy)
        return x.grad

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        step()
    barrier()
    sampler = ClockSampler(dev.index)
    if rank == 0:
        sampler.start()
    _cabi.profile(True)
    n0 = _cabi.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    tms = torch.tensor([e0.elapsed_time(e1)], device=dev)
    launches = _cabi.launch_count() - n0
    recs = _cabi.profile_records()
    _cabi.profile(False)
    clocks = sampler.stop() if rank == 0 else None
    if world > 1:
        dist.all_reduce(tms, op=dist.ReduceOp.MAX)
    ms = float(tms.item())
    if rank == 0:
        peaks = load_peaks()
        per = {}
        for name, t in recs:
            c, sm = per.get(name, (0, 0.0))
            per[name] = (c + 1, sm + t)
        tot = sum(x[1] for x in per.values())
        c_split, t_split = per.get("fm_qkv_split_rope", (1, 0.0))
        nbytes = qkv.numel() * qkv.element_size()
        ach = 2 * nbytes / (t_split / max(c_split, 1) * 1e-3) / 1e9 if t_split else None
        line = {
            "metric": "fastmax_fwd_bwd_tokens_per_s", "value": B * N * world * args.steps / (ms * 1e-3),
            "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": dt, "data": "synthetic",
            "config": {"workload": describe(args.workload) + " through fastmax_attention_from_qkv (packed projection, "
                                   "rotary embedding on all features)", "global_batch": B * world,
                       "parallelism": f"batches sharded x{world}, no collective",
                       "l2": f"projection of {nbytes / 1e6:.0f} MB larger than the 126 MB L2"},
            "clocks": clocks, "gpu_launches": int(launches),
            "roofline": {"bound": "hbm", "achieved": ach, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": ach / peaks["hbm_gbs"] if ach else None,
                         # ncu, this workload: 412.0 MB read + 360.7 MB written per launch
                         "traffic": 772.7e6 if (B, H, N, D) == (8, 32, 4096, 64) else None,
                         "kernel": "fm_qkv_split_rope", "peak_source": peaks["source"]},
            "kernels": {n: {"launches": c, "ms_total": round(sm, 3), "share": round(sm / tot, 4)}
                        for n, (c, sm) in sorted(per.items(), key=lambda kv: -kv[1][1])},
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        z = json.load(open(path))
        return {"hbm_gbs": z["hbm_gbs"], "bf16_tflops": z["bf16_tflops"],
                "bf16_tflops_sustained": z.get("bf16_tflops_sustained", z["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


# --------------------------------------------------------------------------- CPU arm
def cpu_sample(name, steps, warmup):
    """Time the oracle (CPU restatement of the reference's PyTorch path) on one
    head of the workload at a sequence length it can hold in memory; the
    factorised evaluation is linear in n, so tokens/s per head carries over."""
    import torch

    from oracle.fastmax_oracle import fastmax_moments

    B, H, N, D, dt, mask, p, norm = WORKLOADS[name]
    n = min(N, 1024 if D >= 64 else 2048)
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    g = torch.Generator().manual_seed(1234)
    q, k, v, go = [torch.randn(1, 1, n, D, generator=g) for _ in range(4)]
    if dt == "bf16":
        q, k, v, go = [t.bfloat16().float() for t in (q, k, v, go)]
    times = []
    for it in range(warmup + steps):
        qq, kk, vv = [t.clone().requires_grad_(True) for t in (q, k, v)]
        t0 = time.perf_counter()
        out = fastmax_moments(qq, kk, vv, mask=mask, normalize=norm, p=p, **A)
        out.backward(go)
        dtm = time.perf_counter() - t0
        if it >= warmup:
            times.append(dtm)
    t = statistics.median(times)
    # whole-job tokens/s: a token counts once for all H heads
    value = (n / t) / H
    return {"value": value, "unit": "tokens/s", "cores": cores, "kind": "port",
            "sample": f"1 of {B * H} batch*head units, first {n} of {N} tokens, fp32 math, "
                      f"median of {steps} fwd+bwd ({t:.2f} s each), scaled by 1/H"}, t


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cb, t = cpu_sample(args.workload, max(1, min(args.steps, 5)), max(1, min(args.warmup, 1)))
    line = {"impl": "reference", "metric": "fastmax_fwd_bwd_tokens_per_s", "value": cb["value"], "unit": "tokens/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": t * 1e3,
            "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None,
            "dtype": "f32", "data": "synthetic", "config": {"workload": describe(args.workload)},
            "cpu_baseline": cb,
            "e2e": {"value": cb["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------- GPU arm
def run_ours(args):
    import torch
    import torch.distributed as dist

    import fastmax_b200
    from fastmax_b200 import _cabi

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    B, H, N, D, dt, mask, p, norm = WORKLOADS[args.workload]
    dtype = torch.bfloat16 if dt == "bf16" else torch.float32
    bh_total = B * H
    seq_mode = args.workload.startswith("c5")   # one long sequence, split along n over the ranks
    if seq_mode:
        return run_seq(args, world, rank, dev, (B, H, N, D, dt, mask, p, norm))
    if args.workload.startswith("decode"):
        return run_decode(args, world, rank, dev, (B, H, N, D, dt, mask, p, norm))
    if args.workload == "site":
        return run_site(args, world, rank, dev, (B, H, N, D, dt, mask, p, norm))
    if args.scaling == "strong":
        bh = bh_total // world + (1 if rank < bh_total % world else 0)
        tokens_job = B * N
    else:
        bh = bh_total
        tokens_job = B * N * world
    kw = dict(mask=bool(mask), normalize=bool(norm), p=p, impl=args.family, chunk=args.chunk, **A)

    g = torch.Generator(device=dev).manual_seed(1234 + rank)
    q, k, v, go = [torch.randn(bh, N, D, generator=g, device=dev, dtype=torch.float32).to(dtype) for _ in range(4)]

    def step():
        out, den, stats = _cabi.forward(q, k, v, **kw)
        return out, _cabi.backward(q, k, v, out, den, stats, go, **kw)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        step()
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    _cabi.profile(True)
    n0 = _cabi.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(args.steps):
        res = step()
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    launches = _cabi.launch_count() - n0
    recs = _cabi.profile_records()
    _cabi.profile(False)
    clocks = sampler.stop() if rank == 0 else None
    tms = torch.tensor([ms], device=dev)
    if world > 1:
        dist.all_reduce(tms, op=dist.ReduceOp.MAX)
    ms = float(tms.item())
    value = tokens_job * args.steps / (ms * 1e-3)

    # ---- end to end with host buffers: fastmax_b200.host.HostPipeline streams groups of heads
    # through the GPU (copy-in, forward+backward, copy-out overlapped) ----------------------
    from fastmax_b200.host import HostPipeline, prefer_gpu_numa_node

    numa_node = prefer_gpu_numa_node(dev)     # pinned buffers below land next to this rank's GPU

    del res
    host_in = [t.cpu().pin_memory() for t in (q, k, v, go)]
    host_out = [torch.empty_like(h).pin_memory() for h in host_in]
    del q, k, v, go
    torch.cuda.empty_cache()
    pipe = HostPipeline(bh, N, D, dtype, dev, heads_per_group=args.e2e_group, **kw)

    def e2e_step():
        pipe.run(*host_in, *host_out)

    e2e_steps = max(1, min(args.steps, 3))
    e2e_step()
    barrier()
    e0.record()
    for _ in range(e2e_steps):
        e2e_step()
    e1.record()
    barrier()
    tms = torch.tensor([e0.elapsed_time(e1)], device=dev)
    if world > 1:
        dist.all_reduce(tms, op=dist.ReduceOp.MAX)
    e2e_ms = float(tms.item()) / e2e_steps
    nbytes = sum(h.numel() * h.element_size() for h in host_in)

    if rank == 0:
        per = {}
        for name, t in recs:
            c, s = per.get(name, (0, 0.0))
            per[name] = (c + 1, s + t)
        dom = max(per, key=lambda n: per[n][1]) if per else None
        peaks = load_peaks()
        ff, fq, fkv = alg_flops_per_token_head(D, p)
        flops_of = {"fwd": ff, "dq": fq, "dkdv": fkv, "dk": fkv * 2 // 3, "dv": fkv // 3}
        roof = None
        if dom is not None:
            cnt, tot = per[dom]
            kind = dom.rsplit("_", 1)[-1]
            # DRAM bytes per token-head of the score kernels (bf16, d = 64), from the ncu capture of the
            # small case summarised under profiles/: heads are processed one after another, so every
            # re-read of a head's tiles hits L2 and the traffic grows in proportion to heads x tokens
            ncu_bytes = {"fm_dense_tc_fwd": 483.2, "fm_dense_tc_dq": 621.3, "fm_dense_tc_dkdv": 723.8}
            traffic = ncu_bytes[dom] * bh * N if (dom in ncu_bytes and D == 64 and dt == "bf16") else None
            if kind in flops_of:
                achieved = flops_of[kind] * bh * N / (tot / cnt * 1e-3) / 1e12
                roof = {"bound": "tensor", "kernel": dom, "achieved": achieved, "peak": peaks["bf16_tflops_sustained"],
                        "unit": "TFLOP/s", "frac": achieved / peaks["bf16_tflops_sustained"], "traffic": traffic,
                        "traffic_source": "ncu dram bytes of a small case scaled by heads x tokens" if traffic else None,
                        "peak_source": peaks["source"] + " (sustained cuBLAS bf16)", "ms_per_launch": tot / cnt,
                        "alg_flops_per_launch": flops_of[kind] * bh * N}
            else:
                nb = 2 * bh * N * D * (2 if dt == "bf16" else 4)
                achieved = nb / (tot / cnt * 1e-3) / 1e9
                roof = {"bound": "hbm", "kernel": dom, "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                        "frac": achieved / peaks["hbm_gbs"], "traffic": None, "peak_source": peaks["source"]}
        total_alg = (ff + fq + fkv) * bh * N * args.steps * (world if args.scaling != "strong" else 1)
        line = {
            "metric": "fastmax_fwd_bwd_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": args.scaling, "vs_baseline": None, "dtype": dt, "data": "synthetic",
            "config": {"workload": describe(args.workload), "global_batch": B * (world if args.scaling != "strong" else 1),
                       "batch_heads_per_gpu": bh, "parallelism": f"batch*head sharded x{world}, no collective",
                       "l2": "inputs (4 x %.2f GB per GPU) larger than the 126 MB L2" % (bh * N * D * (2 if dt == "bf16" else 4) / 1e9)},
            "clocks": clocks, "gpu_launches": int(launches),
            "alg_tflops_whole_step": total_alg / world / (ms * 1e-3) / 1e12,
            "kernels": {n: {"launches": c, "ms_total": round(s, 3), "share": round(s / sum(x[1] for x in per.values()), 4)}
                        for n, (c, s) in sorted(per.items(), key=lambda kv: -kv[1][1])},
            "roofline": roof,
            "e2e": {"value": tokens_job / (e2e_ms * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": nbytes,
                    "d2h_bytes_per_step": nbytes, "ms_per_step": e2e_ms, "host_numa_node_rank0": numa_node},
        }
        if world == 1 and not args.no_cpu:
            line["cpu_baseline"] = cpu_sample(args.workload, 2, 1)[0]
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_seq(args, world, rank, dev, cfg):
    """Long-context workload: the sequence is split into `world` contiguous shards (one per GPU, all heads
    on every GPU); per pass the ranks exchange the per-shard moment totals (all-gather) and the
    normalisation statistics (all-reduce).  Total work is fixed, so this is strong scaling."""
    import torch
    import torch.distributed as dist

    import fastmax_b200
    from fastmax_b200 import _cabi
    from fastmax_b200.sharded import fastmax_sequence_parallel

    B, H, N, D, dt, mask, p, norm = cfg
    dtype = torch.bfloat16 if dt == "bf16" else torch.float32
    nl = N // world
    g = torch.Generator(device=dev).manual_seed(1234 + rank)
    q, k, v, go = [torch.randn(B * H, nl, D, generator=g, device=dev, dtype=torch.float32).to(dtype) for _ in range(4)]
    if not norm:   # unnormalised configurations scale q and k by 1/sqrt(D)
        q, k = q * D ** -0.5, k * D ** -0.5
    mod = fastmax_b200.FASTMultiHeadAttention()

    def step():
        qd, kd, vd = [t.detach().requires_grad_(True) for t in (q, k, v)]
        if world > 1:
            out = fastmax_sequence_parallel(qd, kd, vd, mask=bool(mask), normalize=bool(norm), p=p, chunk=args.chunk, **A)
        else:
            out = mod(qd, kd, vd, None, bool(mask), 0.0, bool(norm), 1.0, A["a0"], A["a1"], A["a2"], A["lim"], p)
        out.backward(go)
        return out

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        step()
    barrier()
    sampler = ClockSampler(dev.index)
    if rank == 0:
        sampler.start()
    _cabi.profile(True)
    n0 = _cabi.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    tms = torch.tensor([e0.elapsed_time(e1)], device=dev)
    launches = _cabi.launch_count() - n0
    recs = _cabi.profile_records()
    _cabi.profile(False)
    clocks = sampler.stop() if rank == 0 else None
    if world > 1:
        dist.all_reduce(tms, op=dist.ReduceOp.MAX)
    ms = float(tms.item())
    if rank == 0:
        per = {}
        for name, t in recs:
            c, s = per.get(name, (0, 0.0))
            per[name] = (c + 1, s + t)
        ff, fq, fkv = alg_flops_per_token_head(D, p)
        tot = sum(x[1] for x in per.values())
        line = {
            "metric": "fastmax_fwd_bwd_tokens_per_s", "value": B * N * args.steps / (ms * 1e-3), "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": dt, "data": "synthetic",
            "config": {"workload": describe(args.workload), "tokens_per_gpu": nl,
                       "parallelism": f"sequence sharded x{world}; "
                                      + ("all-gather" if mask else "all-reduce") + " of per-shard moment totals, "
                                      "all-reduce of normalisation statistics",
                       "l2": "inputs larger than the 126 MB L2"},
            "clocks": clocks, "gpu_launches": int(launches),
            "alg_tflops_per_gpu": (ff + fq + fkv) * B * H * nl * args.steps / (ms * 1e-3) / 1e12,
            "kernels": {n: {"launches": c, "ms_total": round(s, 3), "share": round(s / tot, 4)}
                        for n, (c, s) in sorted(per.items(), key=lambda kv: -kv[1][1])},
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c3", choices=sorted(WORKLOADS))
    ap.add_argument("--scaling", default="weak", choices=["weak", "strong"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg")
    ap.add_argument("--family", default="auto", choices=["auto", "dense_ffma", "dense_tc", "moments", "moments_ffma"],
                    help="kernel family to force (default: the library's own choice)")
    ap.add_argument("--chunk", type=int, default=0, help="moment family: tokens per chunk (0 = default)")
    ap.add_argument("--e2e-group", type=int, default=32,
                    help="batch*head units per group of the host-buffer pipeline of the e2e leg")
    args = ap.parse_args()
    if args.warmup < 3 and args.impl == "ours":
        args.warmup = 3
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
