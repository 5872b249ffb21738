"""Generate the golden vectors in this directory from the reference's own code.

Run once, in a checkout that has the reference tree next to it:

    python tests/golden/make_golden.py /path/to/reference

The reference's ``example.py`` cannot be imported (it imports its CUDA extension
and runs a CUDA demo at import time), so its ``fastmax_function`` definition is
lifted out of the source with ``ast`` and executed unmodified against ``torch``
and ``math`` on the CPU.  Nothing of the reference is written into this
repository except the numbers it produced.

Outputs:
  small_cases.npz   every (mask, p, normalize) combination at small shapes, with
                    full inputs, fp32 and fp64 outputs and autograd gradients.
  c1_sampled.npz    the reference's CPU-runnable benchmark configuration
                    (B=2, H=8, N=1024, D=32, unmasked, p=2, normalize) with
                    inputs regenerated from a seed; stores every 16th row of two heads.
"""
from __future__ import annotations

import ast
import math
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def lift_reference(ref_root: str):
    src = open(os.path.join(ref_root, "example.py")).read()
    fn = [n for n in ast.parse(src).body
          if isinstance(n, ast.FunctionDef) and n.name == "fastmax_function"][0]
    ns = {"torch": torch, "math": math}
    exec(compile(ast.Module([fn], []), "reference_example_py", "exec"), ns)
    return ns["fastmax_function"]


def run(ref, q, k, v, go, dtype, **kw):
    q, k, v = [t.to(dtype).clone().requires_grad_(True) for t in (q, k, v)]
    out = ref(q, k, v, **kw)
    out.backward(go.to(out.dtype))
    return [t.detach().numpy() for t in (out, q.grad, k.grad, v.grad)]


# (tag, b, h, n, d, mask, p, normalize, a0, a1, a2, lim, input scale)
SMALL = []
for _mask in (0, 1):
    for _p in (1, 2):
        for _norm in (0, 1):
            SMALL.append((f"m{_mask}p{_p}n{_norm}_a", 2, 2, 19, 8, _mask, _p, _norm, 1.0, 1.0, 0.5, 1.0, 0.5))
            SMALL.append((f"m{_mask}p{_p}n{_norm}_b", 1, 2, 33, 16, _mask, _p, _norm, 0.7, 1.3, 0.4, 1.5, 0.35))
SMALL.append(("m1p2n1_d32", 1, 1, 70, 32, 1, 2, 1, 1.0, 1.0, 0.5, 1.0, 1.0))
SMALL.append(("m0p2n1_d32", 1, 1, 70, 32, 0, 2, 1, 1.0, 1.0, 0.5, 1.0, 1.0))
SMALL.append(("m1p2n1_n1", 1, 1, 1, 8, 1, 2, 1, 1.0, 1.0, 0.5, 1.0, 1.0))
SMALL.append(("m1p2n1_n2", 2, 1, 2, 8, 1, 2, 1, 1.0, 1.0, 0.5, 1.0, 1.0))


def main(ref_root: str):
    ref = lift_reference(ref_root)
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    blob = {}
    names = []
    for i, (tag, b, h, n, d, mask, p, norm, a0, a1, a2, lim, scale) in enumerate(SMALL):
        g = torch.Generator().manual_seed(1000 + i)
        q, k, v, go = [torch.randn(b, h, n, d, generator=g) * s
                       for s in (scale, scale, 1.0, 1.0)]
        kw = dict(mask=mask, dropout_rate=0.0, normalize=norm, temperature=1.0,
                  a0=a0, a1=a1, a2=a2, lim=lim, p=p)
        r32 = run(ref, q, k, v, go, torch.float32, **kw)
        r64 = run(ref, q, k, v, go, torch.float64, **kw)
        names.append(tag)
        blob[f"{tag}/cfg"] = np.array([b, h, n, d, mask, p, norm, a0, a1, a2, lim], dtype=np.float64)
        for nm, t in zip(("q", "k", "v", "go"), (q, k, v, go)):
            blob[f"{tag}/{nm}"] = t.numpy()
        for nm, a32, a64 in zip(("out", "dq", "dk", "dv"), r32, r64):
            blob[f"{tag}/{nm}32"] = a32
            blob[f"{tag}/{nm}64"] = a64
    blob["names"] = np.array(names)
    np.savez_compressed(os.path.join(HERE, "small_cases.npz"), **blob)

    # Benchmark configuration 1 of the reference (CPU-runnable): inputs from a seed.
    b, h, n, d = 2, 8, 1024, 32
    g = torch.Generator().manual_seed(1234)
    q, k, v, go = [torch.randn(b, h, n, d, generator=g) for _ in range(4)]
    kw = dict(mask=0, dropout_rate=0.0, normalize=1, temperature=1.0,
              a0=1.0, a1=1.0, a2=0.5, lim=1.0, p=2)
    r64 = run(ref, q, k, v, go, torch.float64, **kw)
    r32 = run(ref, q, k, v, go, torch.float32, **kw)
    heads = [(0, 0), (1, 5)]
    ROW_STRIDE = 16
    c1 = {"cfg": np.array([b, h, n, d, 0, 2, 1, 1.0, 1.0, 0.5, 1.0], dtype=np.float64),
          "seed": np.array(1234), "heads": np.array(heads), "row_stride": np.array(16),
          "input_checksum": np.array([float(t.double().sum()) for t in (q, k, v, go)])}
    for nm, a32, a64 in zip(("out", "dq", "dk", "dv"), r32, r64):
        c1[f"{nm}32"] = np.stack([a32[bb, hh, ::ROW_STRIDE] for bb, hh in heads])
        c1[f"{nm}64"] = np.stack([a64[bb, hh, ::ROW_STRIDE] for bb, hh in heads])
        c1[f"{nm}64_absmax"] = np.array(np.abs(a64).max())
    np.savez_compressed(os.path.join(HERE, "c1_sampled.npz"), **c1)
    for f in ("small_cases.npz", "c1_sampled.npz"):
        print(f, os.path.getsize(os.path.join(HERE, f)), "bytes")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_golden.py /path/to/reference")
    main(sys.argv[1])
