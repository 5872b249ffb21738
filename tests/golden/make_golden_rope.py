"""Generate ``rope.npz`` from the reference's own rotary-embedding code.

    python tests/golden/make_golden_rope.py /path/to/reference

The reference's ``model.py`` cannot be imported (it needs the ``litgpt`` package),
so its ``apply_rope`` definition is lifted out of the source with ``ast`` and
executed unmodified against ``torch`` on the CPU.  Only the numbers it produced
are stored: seeded inputs x (B, H, T, r), tables cos / sin (T, r), the rotated
output and, for a seeded upstream gradient, the autograd gradient of x.
"""
from __future__ import annotations

import ast
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def lift_apply_rope(ref_root: str):
    src = open(os.path.join(ref_root, "model.py")).read()
    fn = [n for n in ast.parse(src).body if isinstance(n, ast.FunctionDef) and n.name == "apply_rope"][0]
    ns = {"torch": torch}
    exec(compile(ast.Module([fn], []), "reference_model_py", "exec"), ns)
    return ns["apply_rope"]


def main(ref_root: str):
    ref = lift_apply_rope(ref_root)
    out = {}
    for tag, (b, h, t, r) in {"a": (2, 3, 17, 8), "b": (1, 2, 40, 32)}.items():
        g = torch.Generator().manual_seed(1234 + r)
        x = torch.randn(b, h, t, r, generator=g, dtype=torch.float64).requires_grad_(True)
        # tables as a rotary cache builds them (both halves equal) and a generic pair (halves differ)
        ang = torch.outer(torch.arange(t, dtype=torch.float64), 1.0 / (10000 ** (torch.arange(0, r, 2) / r)))
        tables = {"rot": (torch.cos(ang).repeat(1, 2), torch.sin(ang).repeat(1, 2)),
                  "gen": (torch.randn(t, r, generator=g, dtype=torch.float64),
                          torch.randn(t, r, generator=g, dtype=torch.float64))}
        go = torch.randn(b, h, t, r, generator=g, dtype=torch.float64)
        out[f"{tag}_x"], out[f"{tag}_go"] = x.detach().numpy(), go.numpy()
        for name, (c, s) in tables.items():
            y = ref(x, c, s)
            (gx,) = torch.autograd.grad(y, x, go)
            out[f"{tag}_{name}_cos"], out[f"{tag}_{name}_sin"] = c.numpy(), s.numpy()
            out[f"{tag}_{name}_y"], out[f"{tag}_{name}_gx"] = y.detach().numpy(), gx.numpy()
    np.savez_compressed(os.path.join(HERE, "rope.npz"), **out)
    print("wrote rope.npz with", len(out), "arrays")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit(__doc__)
    main(sys.argv[1])
