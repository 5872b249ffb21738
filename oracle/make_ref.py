"""Builds ``oracle/_ref/`` from the reference tree -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.

    python oracle/make_ref.py /path/to/reference

The reference's CPU implementation of the hot path is the pure-PyTorch function
``fastmax_function`` in its ``example.py`` (lines 83-212), the path its
``use_custom_gradient=False`` switch selects.  That file cannot be imported (it imports the
reference's CUDA extension and runs a CUDA demo at import time), so this recipe parses it
with ``ast``, takes the one function definition as it stands, compiles it and stores the
*compiled code object* (``marshal``) in ``oracle/_ref/fastmax_function.bin`` together with a
small manifest (Python version, SHA-256 of the source file it came from).  No source text of
the reference is written anywhere; the directory is listed in ``.gitignore`` and therefore
stays out of the history, but travels with the working tree to the machine the benchmark
runs on, the way the built shared libraries do.

``load()`` returns the function (executed against ``torch`` and ``math``) or None when the
directory has not been built or was built by another Python version.  Users: the CPU arm of
``bench.py`` (``--impl reference`` and ``cpu_baseline``), where it is the thing timed, and the
oracle tests, which hold the restatement in ``fastmax_oracle.py`` against it.
"""
from __future__ import annotations

import ast
import hashlib
import json
import marshal
import math
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
BIN = os.path.join(OUT, "fastmax_function.bin")
MANIFEST = os.path.join(OUT, "manifest.json")


def build(ref_root: str) -> str:
    path = os.path.join(ref_root, "example.py")
    raw = open(path, "rb").read()
    fn = [n for n in ast.parse(raw.decode()).body
          if isinstance(n, ast.FunctionDef) and n.name == "fastmax_function"][0]
    code = compile(ast.Module([fn], []), "reference:example.py", "exec")
    os.makedirs(OUT, exist_ok=True)
    with open(BIN, "wb") as f:
        marshal.dump(code, f)
    with open(MANIFEST, "w") as f:
        json.dump({"function": "fastmax_function", "source": "example.py", "lines": [fn.lineno, fn.end_lineno],
                   "sha256": hashlib.sha256(raw).hexdigest(), "python": list(sys.version_info[:3])}, f)
    return BIN


def load():
    """The reference's ``fastmax_function`` from ``oracle/_ref`` or None."""
    if not (os.path.exists(BIN) and os.path.exists(MANIFEST)):
        return None
    try:
        man = json.load(open(MANIFEST))
        if man.get("python", [])[:2] != list(sys.version_info[:2]):
            return None
        import torch
        ns = {"torch": torch, "math": math}
        with open(BIN, "rb") as f:
            exec(marshal.load(f), ns)
        return ns["fastmax_function"]
    except Exception:
        return None


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit(__doc__)
    print(build(sys.argv[1]))
