import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def load_small_cases():
    """The reference-generated small cases as a list of dicts of torch tensors."""
    z = np.load(os.path.join(GOLDEN, "small_cases.npz"))
    cases = []
    for tag in z["names"]:
        tag = str(tag)
        b, h, n, d, mask, p, norm, a0, a1, a2, lim = z[f"{tag}/cfg"]
        c = dict(tag=tag, mask=int(mask), p=int(p), normalize=int(norm),
                 a0=float(a0), a1=float(a1), a2=float(a2), lim=float(lim))
        for nm in ("q", "k", "v", "go"):
            c[nm] = torch.from_numpy(z[f"{tag}/{nm}"])
        for nm in ("out", "dq", "dk", "dv"):
            c[nm + "32"] = torch.from_numpy(z[f"{tag}/{nm}32"])
            c[nm + "64"] = torch.from_numpy(z[f"{tag}/{nm}64"])
        cases.append(c)
    return cases


def case_kwargs(c):
    return dict(mask=c["mask"], normalize=c["normalize"], a0=c["a0"], a1=c["a1"],
                a2=c["a2"], lim=c["lim"], p=c["p"])
