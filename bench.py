"""Fastmax forward+backward throughput on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

A step is one forward + backward pass of Fastmax attention over one batch of synthetic
N(0,1) inputs.  The default workload is the configuration the headline target is quoted on:
causal, bf16, p=2, B=64, H=16, N=10000, D=64, normalize=True, lim=1, a=(1,1,0.5).  With N
GPUs that ONE batch is split: its B*H batch*head units are independent, so each rank takes
B*H/N of them and nothing is exchanged on the data path (`scaling: strong`; `--scaling weak`
gives every rank the whole batch instead, and the default run reports that figure too, under
`weak`).  `value` is tokens of the batch over the slowest rank's device time.

Rank 0 prints one JSON line.  `value` is measured with the inputs resident in HBM; `e2e` is
the same metric with pinned host buffers through fastmax_b200.host.HostPipeline, host<->device
copies inside the timed region.  The line of the default workload also carries `c5`: the
long-context configuration (B=1, H=32, N=262144, D=64) with its sequence split over the same
N ranks, a few steps, so that the sequence-sharded path is measured by the same command.

`--impl reference` times the reference's own pure-PyTorch path on the host cores: the function
compiled into oracle/_ref by oracle/make_ref.py when that has been built, else the oracle's
restatement of it.  It runs the CPU-runnable configuration (B=2, H=8, N=1024, D=32) exactly
(`c1`) and a bounded sample of the selected workload, extrapolated to the whole job (`value`).
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
    "c5u": (1, 32, 262144, 128, "bf16", 0, 1, 0), # long unmasked p = 1 sequence, sharded along the sequence when N > 1
    # decoding against the persistent moment state: one new token per sequence and step (N is not used)
    "decode": (64, 16, 1, 64, "bf16", 1, 2, 1),
    # the model's call site: packed projection -> rotary embedding -> attention -> (B, T, H*hs), and back
    "site": (8, 32, 4096, 64, "bf16", 1, 1, 1),
}
# Reduced shapes for profiler captures (--profile-case NAME): inputs larger than L2, a few hundred MB in all.
PROFILE_CASES = {
    "tiny": (2, 4, 1024, 64, "bf16", 1, 2, 1),
    "prof": (8, 16, 4096, 64, "bf16", 1, 2, 1),      # inputs 4 x 67 MB
    "prof1": (2, 8, 16384, 128, "bf16", 0, 1, 0),    # p = 1, inputs 4 x 67 MB
    "c4s": (4, 8, 16384, 128, "bf16", 0, 2, 0),      # unmasked d = 128
    "c5s": (1, 8, 65536, 64, "bf16", 1, 2, 1),       # long context
    "c2s": (16, 8, 1000, 32, "fp32", 1, 2, 1),       # fp32 CUDA-core family
    "decodes": (16, 16, 1, 64, "bf16", 1, 2, 1),     # 277 MB of decode state
}
A = dict(a0=1.0, a1=1.0, a2=0.5, lim=1.0)
L2_BYTES = 126e6
# FP32 FFMA peak for the fp32 workloads (no measured figure exists): 148 SMs x 128 lanes x 2 FLOP x 1.965 GHz
FFMA_TFLOPS_NOMINAL = 148 * 128 * 2 * 1.965e9 / 1e12
# Version of the library the DRAM-traffic figures below were captured on; another version reports none.
TRAFFIC_LIB_VERSION = 200
# ncu DRAM bytes (read + write) per token-head, bf16, D = 64: the capture of the small case summarised in
# profiles/dense_tc_small_case_ncu_full.md, scaled by heads x tokens
NCU_BYTES_PER_TOKEN_HEAD = {"fm_dense_tc_fwd": 487.0, "fm_dense_tc_dq": 622.7, "fm_dense_tc_dkdv": 722.1,
                            # per token whose chunk builds a state (profiles/moments_tc_small_case_ncu_full.md)
                            "fm_moments_tc_state": 717.5,
                            # per token that is read out (same file, section on the read-outs' traffic)
                            "fm_moments_tc_readout_a": 608.2, "fm_moments_tc_readout_b": 742.4,
                            "fm_moments_tc_readout_ab": 976.1}
# Labels that are launches of one kernel function: the roofline record is of the function with the largest share.
KERNEL_OF_LABEL = {"fm_moments_tc_readout_a": "readout_tc_kernel", "fm_moments_tc_readout_b": "readout_tc_kernel",
                   "fm_moments_tc_readout_ab": "readout_tc_kernel"}


def cfg_of(name):
    return WORKLOADS[name] if name in WORKLOADS else PROFILE_CASES[name]


def describe(name):
    B, H, N, D, dt, mask, p, norm = cfg_of(name)
    return (f"{name}: {'causal' if mask else 'unmasked'} {dt} p={p} B={B} H={H} N={N} D={D} "
            f"normalize={bool(norm)} lim=1 a=(1,1,0.5)")


def alg_flops_per_token_head(D, p):
    """Algorithmic FLOPs of the factorised evaluation, per token and head:
    (forward, grad_q pass, grad_k+grad_v pass) = (4, 4, 6) * F * (D+1), F = D + [p=2] D^2."""
    F = D + (D * D if p == 2 else 0)
    u = F * (D + 1)
    return 4 * u, 4 * u, 6 * u


def l2_note(nbytes_inputs, flushed):
    if flushed:
        return ("inputs (%.1f MB per GPU) fit the 126 MB L2: a 256 MB buffer is rewritten between timed steps"
                % (nbytes_inputs / 1e6))
    return "inputs (%.2f GB per GPU) larger than the 126 MB L2" % (nbytes_inputs / 1e9)


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
def _cpu_function():
    """(function, kind): the reference's own fastmax_function from oracle/_ref, else the oracle's port."""
    from oracle.make_ref import load

    fn = load()
    if fn is not None:
        return fn, "reference"
    from oracle.fastmax_oracle import fastmax_moments

    return fastmax_moments, "port"


def _cpu_time(fn, q, k, v, go, steps, warmup, budget_s, **kw):
    """Median seconds of forward + backward(go); stops early when `budget_s` is used up."""
    times, t_start = [], time.perf_counter()
    for it in range(warmup + steps):
        qq, kk, vv = [t.clone().requires_grad_(True) for t in (q, k, v)]
        t0 = time.perf_counter()
        out = fn(qq, kk, vv, **kw)
        out.backward(go.to(out.dtype))
        dtm = time.perf_counter() - t0
        if it >= warmup:
            times.append(dtm)
        if times and time.perf_counter() - t_start > budget_s:
            break
    return statistics.median(times), len(times)


def cpu_arm(name, steps, warmup, budget_s=120.0):
    """The CPU implementation on all host cores: (i) BASELINE configuration 1 exactly, (ii) one
    batch*head unit of workload `name` at a length the cumulative-moment evaluation can hold in
    memory (it is linear in n, so tokens/s per head carries over), scaled to whole-job tokens/s."""
    import torch

    fn, kind = _cpu_function()
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    g = torch.Generator().manual_seed(1234)
    # (i) configuration 1, exactly as stated: fp32, unmasked, p = 2, normalize, B=2 H=8 N=1024 D=32
    B1, H1, N1, D1 = WORKLOADS["c1"][:4]
    q, k, v, go = [torch.randn(B1, H1, N1, D1, generator=g) for _ in range(4)]
    t1, n1 = _cpu_time(fn, q, k, v, go, min(steps, 5), 1, budget_s / 4, mask=0, normalize=1, p=2, **A)
    c1 = {"seconds_per_step": t1, "tokens_per_s": B1 * N1 / t1, "steps": n1,
          "config": describe("c1") + ", the whole configuration"}
    if name == "c1":
        return {"value": c1["tokens_per_s"], "unit": "tokens/s", "cores": cores, "kind": kind,
                "sample": f"the whole configuration, fp32, median of {n1} fwd+bwd ({t1:.2f} s each)", "c1": c1}, t1, n1
    # (ii) a bounded sample of the selected workload
    B, H, N, D, dt, mask, p, norm = cfg_of(name)
    n = min(N, 1024 if D >= 64 else 2048)
    q, k, v, go = [torch.randn(1, 1, n, D, generator=g) for _ in range(4)]
    if dt == "bf16":
        q, k, v, go = [t.bfloat16().float() for t in (q, k, v, go)]
    if not norm:
        q, k = q * D ** -0.5, k * D ** -0.5
    t, ns = _cpu_time(fn, q, k, v, go, steps, warmup, budget_s, mask=mask, normalize=norm, p=p, **A)
    value = (n / t) / H          # whole-job tokens/s: a token counts once for all H heads
    return {"value": value, "unit": "tokens/s", "cores": cores, "kind": kind, "extrapolated": True,
            "sample": f"1 of {B * H} batch*head units, first {n} of {N} tokens, fp32 math, median of {ns} "
                      f"fwd+bwd ({t:.2f} s each), scaled by 1/H to the whole job", "c1": c1}, t, ns


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cb, t, ns = cpu_arm(args.workload, max(1, args.steps), max(1, min(args.warmup, 1)), budget_s=150.0)
    line = {"impl": "reference", "metric": "fastmax_fwd_bwd_tokens_per_s", "value": cb["value"], "unit": "tokens/s",
            "n_gpus": args.gpus, "steps": ns, "steps_requested": args.steps, "warmup": max(1, min(args.warmup, 1)),
            "ms_per_step": t * 1e3, "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None,
            "dtype": "f32", "data": "synthetic", "config": {"workload": describe(args.workload)},
            "cpu_baseline": cb,
            "e2e": {"value": cb["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------- GPU arm
def _per_kernel(recs):
    per = {}
    for name, t in recs:
        c, s = per.get(name, (0, 0.0))
        per[name] = (c + 1, s + t)
    return per


def _kernel_table(per):
    tot = sum(x[1] for x in per.values()) or 1.0
    return {n: {"launches": c, "ms_total": round(s, 3), "share": round(s / tot, 4)}
            for n, (c, s) in sorted(per.items(), key=lambda kv: -kv[1][1])}


class Harness:
    """Process-group plumbing shared by the timed legs."""

    def __init__(self):
        import torch
        import torch.distributed as dist

        self.torch, self.dist = torch, dist
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(self.local)
        self.dev = torch.device("cuda", self.local)
        if self.world > 1:
            dist.init_process_group("nccl", device_id=self.dev)

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def max_over_ranks(self, x):
        t = self.torch.tensor([x], device=self.dev, dtype=self.torch.float64)
        if self.world > 1:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def close(self):
        if self.world > 1:
            self.dist.barrier()
            self.dist.destroy_process_group()


def timed_region(hz, step, steps, warmup, flush_l2=False, sample_clocks=False):
    """`warmup` untimed steps, then exactly `steps` timed ones between barriers; device time by CUDA events
    on the launching stream, max over ranks.  With flush_l2 every step is timed on its own and a 256 MB
    buffer is rewritten in between (outside the events)."""
    torch = hz.torch
    from fastmax_b200 import _cabi

    for _ in range(warmup):
        step()
    hz.barrier()
    sampler = ClockSampler(hz.local)
    if sample_clocks and hz.rank == 0:
        sampler.start()
    _cabi.profile(True)
    n0 = _cabi.launch_count()
    hz.barrier()
    if flush_l2:
        junk = torch.empty(256 << 20, dtype=torch.uint8, device=hz.dev)
        evs = []
        for _ in range(steps):
            junk.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            step()
            e1.record()
            evs.append((e0, e1))
        hz.barrier()
        ms = sum(a.elapsed_time(b) for a, b in evs)
    else:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            step()
        e1.record()
        hz.barrier()
        ms = e0.elapsed_time(e1)
    launches = _cabi.launch_count() - n0
    recs = _cabi.profile_records()
    _cabi.profile(False)
    clocks = sampler.stop() if (sample_clocks and hz.rank == 0) else None
    return {"ms": hz.max_over_ranks(ms), "launches": int(launches), "per": _per_kernel(recs), "clocks": clocks}


def bh_leg(hz, args, cfg, bh, steps, warmup, sample_clocks):
    """Forward + backward on `bh` batch*head units resident in HBM, through the C ABI."""
    torch = hz.torch
    from fastmax_b200 import _cabi

    B, H, N, D, dt, mask, p, norm = cfg
    dtype = torch.bfloat16 if dt == "bf16" else torch.float32
    kw = dict(mask=bool(mask), normalize=bool(norm), p=p, impl=args.family, chunk=args.chunk, **A)
    g = torch.Generator(device=hz.dev).manual_seed(1234 + hz.rank)
    q, k, v, go = [torch.randn(bh, N, D, generator=g, device=hz.dev, dtype=torch.float32).to(dtype) for _ in range(4)]
    if not norm:   # unnormalised configurations scale q and k by 1/sqrt(D)
        q, k = q * D ** -0.5, k * D ** -0.5
    in_bytes = 4 * q.numel() * q.element_size()
    flush = in_bytes < 2 * L2_BYTES

    def step():
        out, den, stats = _cabi.forward(q, k, v, **kw)
        return out, _cabi.backward(q, k, v, out, den, stats, go, **kw)

    r = timed_region(hz, step, steps, warmup, flush_l2=flush, sample_clocks=sample_clocks)
    r.update(in_bytes=in_bytes, flushed=flush, tensors=(q, k, v, go), kw=kw, dtype=dtype)
    return r


def seq_leg(hz, args, cfg, steps, warmup, sample_clocks=False):
    """One long sequence split into `world` contiguous shards (all heads on every GPU); per pass the ranks
    exchange the per-shard moment totals and the normalisation statistics.  Total work is fixed."""
    torch = hz.torch
    import fastmax_b200
    from fastmax_b200.sharded import fastmax_sequence_parallel

    B, H, N, D, dt, mask, p, norm = cfg
    dtype = torch.bfloat16 if dt == "bf16" else torch.float32
    nl = N // hz.world
    g = torch.Generator(device=hz.dev).manual_seed(1234 + hz.rank)
    q, k, v, go = [torch.randn(B * H, nl, D, generator=g, device=hz.dev, dtype=torch.float32).to(dtype) for _ in range(4)]
    if not norm:
        q, k = q * D ** -0.5, k * D ** -0.5
    mod = fastmax_b200.FASTMultiHeadAttention()

    def step():
        qd, kd, vd = [t.detach().requires_grad_(True) for t in (q, k, v)]
        if hz.world > 1:
            out = fastmax_sequence_parallel(qd, kd, vd, mask=bool(mask), normalize=bool(norm), p=p, chunk=args.chunk, **A)
        else:
            out = mod(qd, kd, vd, None, bool(mask), 0.0, bool(norm), 1.0, A["a0"], A["a1"], A["a2"], A["lim"], p)
        out.backward(go)
        return out

    r = timed_region(hz, step, steps, warmup, sample_clocks=sample_clocks)
    ff, fq, fkv = alg_flops_per_token_head(D, p)
    ms_step = r["ms"] / steps
    in_kernels = sum(s for _, s in r["per"].values()) / steps
    r.update(ms_per_step=ms_step, tokens_per_s=B * N / (ms_step * 1e-3), tokens_per_gpu=nl,
             alg_tflops_per_gpu=(ff + fq + fkv) * B * H * nl / (ms_step * 1e-3) / 1e12,
             ms_in_library_kernels=in_kernels, ms_outside_library_kernels=max(ms_step - in_kernels, 0.0))
    del q, k, v, go
    torch.cuda.empty_cache()
    return r


def moment_kernel_flops(name, D, N, mask, chunk):
    """Products one launch of a tensor-core moment kernel needs, per batch*head unit (None: another kernel).
    The state build forms each unordered pair of features once: D (D + 1) / 2 feature rows by D value columns
    per token (the normaliser column comes from another kernel).  A read-out contracts a token's D x D features
    with D + 1 columns.  Causal: one chunk builds no state and one reads none."""
    L = chunk or 2048
    nchunk = -(-N // L)
    if name == "fm_moments_tc_state":
        tokens = min(N, (nchunk - 1) * L) if mask else N
        return 2 * (D * (D + 1) // 2) * D * tokens
    reads = {"fm_moments_tc_readout_a": 1, "fm_moments_tc_readout_b": 1, "fm_moments_tc_readout_ab": 2}
    if name in reads:
        tokens = max(N - L, 0) if mask else N
        return reads[name] * 2 * D * D * (D + 1) * tokens
    return None


def roofline_of(per, cfg, bh, peaks, lib_version, chunk=0):
    """Roofline record of the kernel with the largest share of the timed region."""
    B, H, N, D, dt, mask, p, norm = cfg
    if not per:
        return None
    share = {}
    for label, (c_, t_) in per.items():
        fn = KERNEL_OF_LABEL.get(label, label)
        share[fn] = share.get(fn, 0.0) + t_
    dom = max(share, key=share.get)
    labels = [n for n in per if KERNEL_OF_LABEL.get(n, n) == dom]
    cnt, tot = sum(per[n][0] for n in labels), sum(per[n][1] for n in labels)
    ms = tot / cnt
    mfs = {n: moment_kernel_flops(n, D, N, mask, chunk) for n in labels} if (dt == "bf16" and p == 2) else {}
    if mfs and all(v is not None for v in mfs.values()):
        # per launch: the average over this function's launches of the step, of FLOPs and of time alike
        flops = sum(per[n][0] * mfs[n] for n in labels) * bh / cnt
        achieved = flops / (ms * 1e-3) / 1e12
        traffic = None
        if all(n in NCU_BYTES_PER_TOKEN_HEAD for n in labels) and D == 64 and lib_version == TRAFFIC_LIB_VERSION:
            traffic = sum(per[n][0] * NCU_BYTES_PER_TOKEN_HEAD[n] * mfs[n] / moment_kernel_flops(n, D, 1, 0, 1)
                          for n in labels) * bh / cnt
        if len(labels) > 1:
            dom = dom + " (" + ", ".join(sorted(labels)) + ")"
        return {"bound": "tensor", "kernel": dom, "achieved": achieved, "peak": peaks["bf16_tflops_sustained"],
                "unit": "TFLOP/s", "frac": achieved / peaks["bf16_tflops_sustained"], "traffic": traffic,
                "traffic_source": "ncu dram bytes of a small case scaled by heads x tokens" if traffic else None,
                "peak_source": peaks["source"] + " (sustained cuBLAS bf16)", "ms_per_launch": ms,
                "alg_flops_per_launch": flops,
                "note": "products this kernel's own formulation needs (read-out: ordered feature pairs; state build: "
                        "unordered ones), averaged over its launches of the step; the step's rate is alg_tflops_per_gpu"}
    ff, fq, fkv = alg_flops_per_token_head(D, p)
    flops_of = {"fwd": ff, "dq": fq, "dkdv": fkv, "dk": fkv * 2 // 3, "dv": fkv // 3}
    kind = dom.rsplit("_", 1)[-1]
    es = 2 if dt == "bf16" else 4
    if kind in flops_of and (p == 2 or dt != "bf16"):
        flops = flops_of[kind] * bh * N
        achieved = flops / (ms * 1e-3) / 1e12
        if dt == "bf16":
            peak, src, bound = peaks["bf16_tflops_sustained"], peaks["source"] + " (sustained cuBLAS bf16)", "tensor"
        else:
            peak, src, bound = FFMA_TFLOPS_NOMINAL, "nominal FP32 FFMA at the maximum SM clock (no measured figure)", "fp32-ffma"
        traffic = None
        if dom in NCU_BYTES_PER_TOKEN_HEAD and D == 64 and dt == "bf16" and lib_version == TRAFFIC_LIB_VERSION:
            traffic = NCU_BYTES_PER_TOKEN_HEAD[dom] * bh * N
        return {"bound": bound, "kernel": dom, "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                "frac": achieved / peak, "traffic": traffic,
                "traffic_source": "ncu dram bytes of a small case scaled by heads x tokens" if traffic else None,
                "peak_source": src, "ms_per_launch": ms, "alg_flops_per_launch": flops}
    nb = 2 * bh * N * D * es     # a streaming kernel of the p = 1 path reads two token tensors once
    achieved = nb / (ms * 1e-3) / 1e9
    return {"bound": "hbm", "kernel": dom, "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
            "frac": achieved / peaks["hbm_gbs"], "traffic": None, "peak_source": peaks["source"],
            "ms_per_launch": ms, "alg_bytes_per_launch": nb}


def run_ours(args):
    hz = Harness()
    torch = hz.torch
    from fastmax_b200 import _cabi

    world, rank, dev = hz.world, hz.rank, hz.dev
    cfg = cfg_of(args.workload)
    B, H, N, D, dt, mask, p, norm = cfg
    if args.workload.startswith("c5"):
        return run_seq(hz, args, cfg)
    if args.workload.startswith("decode"):
        return run_decode(args, world, rank, dev, cfg)
    if args.workload == "site":
        return run_site(args, world, rank, dev, cfg)
    bh_total = B * H
    strong = args.scaling == "strong"
    bh = (bh_total // world + (1 if rank < bh_total % world else 0)) if strong else bh_total
    tokens_job = B * N * (1 if strong else world)

    main = bh_leg(hz, args, cfg, bh, args.steps, args.warmup, sample_clocks=True)
    ms = main["ms"]
    value = tokens_job * args.steps / (ms * 1e-3)
    q, k, v, go = main.pop("tensors")
    kw, dtype = main["kw"], main["dtype"]

    # ---- end to end with host buffers: fastmax_b200.host.HostPipeline streams groups of heads
    # through the GPU (copy-in, forward+backward, copy-out overlapped) ----------------------
    from fastmax_b200.host import HostPipeline, prefer_gpu_numa_node

    numa_node, e2e_ms, nbytes = -1, None, 0
    if args.profile_case is None:              # profiler captures stop after the device-resident leg
        numa_node = prefer_gpu_numa_node(dev)     # pinned buffers below land next to this rank's GPU
        host_in = [t.cpu().pin_memory() for t in (q, k, v, go)]
        host_out = [torch.empty_like(h).pin_memory() for h in host_in]
        del q, k, v, go
        torch.cuda.empty_cache()
        pipe = HostPipeline(bh, N, D, dtype, dev, heads_per_group=args.e2e_group, **kw)
        pipe.run(*host_in, *host_out)
        hz.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            pipe.run(*host_in, *host_out)
        e1.record()
        hz.barrier()
        e2e_ms = hz.max_over_ranks(e0.elapsed_time(e1)) / args.steps
        nbytes = sum(h.numel() * h.element_size() for h in host_in)
        del pipe, host_in, host_out
    torch.cuda.empty_cache()

    # ---- extra legs of the default workload --------------------------------------------------
    weak = c5 = None
    if args.workload == "c3" and not args.no_extras:
        if world > 1 and strong:
            w = bh_leg(hz, args, cfg, bh_total, min(args.steps, 5), 3, sample_clocks=False)
            w.pop("tensors")
            torch.cuda.empty_cache()
            ws = min(args.steps, 5)
            weak = {"value": B * N * world * ws / (w["ms"] * 1e-3), "unit": "tokens/s", "ms_per_step": w["ms"] / ws,
                    "steps": ws, "global_batch": B * world, "batch_heads_per_gpu": bh_total}
        s = seq_leg(hz, args, WORKLOADS["c5"], 5, 3)
        c5 = {"workload": describe("c5"), "n_gpus": world, "steps": 5, "warmup": 3, "scaling": "strong",
              "ms_per_step": s["ms_per_step"], "tokens_per_s": s["tokens_per_s"], "tokens_per_gpu": s["tokens_per_gpu"],
              "alg_tflops_per_gpu": s["alg_tflops_per_gpu"],
              "ms_outside_library_kernels": s["ms_outside_library_kernels"],
              "parallelism": (f"sequence sharded x{world}: all-gather of per-shard moment totals, all-reduce of "
                              "normalisation statistics") if world > 1 else "one GPU, no exchange",
              "kernels": _kernel_table(s["per"])}

    if rank == 0:
        peaks = load_peaks()
        ff, fq, fkv = alg_flops_per_token_head(D, p)
        lib_version = int(_cabi.lib().fastmax_b200_version())
        line = {
            "metric": "fastmax_fwd_bwd_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": args.scaling, "vs_baseline": None, "dtype": dt, "data": "synthetic",
            "config": {"workload": describe(args.workload), "global_batch": B * (1 if strong else world),
                       "batch_heads_per_gpu": bh,
                       "parallelism": f"batch*head units {'split' if strong else 'replicated'} x{world}, no collective",
                       "l2": l2_note(main["in_bytes"], main["flushed"])},
            "clocks": main["clocks"], "gpu_launches": main["launches"],
            "alg_tflops_per_gpu": (ff + fq + fkv) * bh * N * args.steps / (ms * 1e-3) / 1e12,
            "kernels": _kernel_table(main["per"]),
            "roofline": roofline_of(main["per"], cfg, bh, peaks, lib_version, args.chunk),
            "e2e": None if e2e_ms is None else
                   {"value": tokens_job / (e2e_ms * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": nbytes,
                    "d2h_bytes_per_step": nbytes, "ms_per_step": e2e_ms, "steps": args.steps,
                    "host_numa_node_rank0": numa_node},
        }
        if weak:
            line["weak"] = weak
        if c5:
            line["c5"] = c5
        if world == 1 and not args.no_cpu:
            line["cpu_baseline"] = cpu_arm(args.workload, 2, 1, budget_s=30.0)[0]
        print(json.dumps(line), flush=True)
    hz.close()


def run_seq(hz, args, cfg):
    """`--workload c5` / `c5u`: the long-context configurations as the whole line."""
    B, H, N, D, dt, mask, p, norm = cfg
    world = hz.world
    s = seq_leg(hz, args, cfg, args.steps, args.warmup, sample_clocks=True)
    if hz.rank == 0:
        line = {
            "metric": "fastmax_fwd_bwd_tokens_per_s", "value": s["tokens_per_s"], "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": s["ms_per_step"],
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": dt, "data": "synthetic",
            "config": {"workload": describe(args.workload), "tokens_per_gpu": s["tokens_per_gpu"],
                       "parallelism": f"sequence sharded x{world}; "
                                      + ("all-gather" if mask else "all-reduce") + " of per-shard moment totals, "
                                      "all-reduce of normalisation statistics",
                       "l2": "inputs larger than the 126 MB L2"},
            "clocks": s["clocks"], "gpu_launches": s["launches"],
            "alg_tflops_per_gpu": s["alg_tflops_per_gpu"],
            "ms_outside_library_kernels": s["ms_outside_library_kernels"],
            "kernels": _kernel_table(s["per"]),
        }
        print(json.dumps(line), flush=True)
    hz.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c3", choices=sorted(WORKLOADS))
    ap.add_argument("--profile-case", default=None, choices=sorted(PROFILE_CASES),
                    help="run a reduced shape meant for profiler captures instead of a workload")
    ap.add_argument("--scaling", default="strong", choices=["weak", "strong"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg")
    ap.add_argument("--no-extras", action="store_true", help="skip the weak-scaling and long-context legs of c3")
    ap.add_argument("--family", default="auto", choices=["auto", "dense_ffma", "dense_tc", "moments", "moments_ffma"],
                    help="kernel family to force (default: the library's own choice)")
    ap.add_argument("--chunk", type=int, default=0, help="moment family: tokens per chunk (0 = default)")
    ap.add_argument("--e2e-group", type=int, default=32,
                    help="batch*head units per group of the host-buffer pipeline of the e2e leg")
    args = ap.parse_args()
    if args.profile_case:
        args.workload, args.no_cpu, args.no_extras = args.profile_case, True, True
    if args.warmup < 3 and args.impl == "ours":
        args.warmup = 3
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
