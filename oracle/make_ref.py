"""Stages the UNMODIFIED reference package next to the oracle, as a second checker and GPU baseline.

TEST INFRASTRUCTURE ONLY.  Nothing in the product package imports what this script produces.

    python oracle/make_ref.py [path to a checkout of fattorib/hawk-pytorch]

copies the checkout's `hawk/*.py` byte for byte into `oracle/_ref/hawk/` (a git-ignored folder: the
reference's sources never enter this repository's history, but the folder travels with the working
tree to wherever the GPU tests and the benchmark run).  Without an argument the checkout is looked
for in $HAWK_REFERENCE_DIR, then in a folder named `reference` beside the repository.

What uses the staged package (only these, and only as the thing compared against):
  tests/test_gpu_reference.py   the reference's own HawkModel on the CUDA kernels through
                                hawk_b200.install, and its Triton scan as a second oracle;
  tests/test_reference_dropin.py  the same drop-in on CPU with oracle stand-ins for the operators;
  bench.py                      `reference_gpu`: the reference's Triton scan, eager conv, compiled
                                cross-entropy and training step timed on the same GPU.
`load()` returns the staged package (or None when it has not been staged).
"""
from __future__ import annotations

import hashlib
import importlib
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(HERE, "_ref")
FILES = ("__init__.py", "cache.py", "external.py", "fused_cross_entropy.py", "hawk.py", "scan_fused.py")


def find_checkout(path: str | None = None) -> str | None:
    cands = [path, os.environ.get("HAWK_REFERENCE_DIR"),
             os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")]
    for c in cands:
        if c and os.path.isfile(os.path.join(c, "hawk", "scan_fused.py")):
            return c
    return None


def stage(path: str | None = None) -> str | None:
    """Copies the reference package; returns the destination, or None when no checkout was found."""
    src = find_checkout(path)
    if src is None:
        return None
    dst = os.path.join(DEST, "hawk")
    os.makedirs(dst, exist_ok=True)
    digest = hashlib.sha256()
    for f in FILES:
        shutil.copyfile(os.path.join(src, "hawk", f), os.path.join(dst, f))
        with open(os.path.join(dst, f), "rb") as fh:
            digest.update(fh.read())
    with open(os.path.join(DEST, "SOURCE.txt"), "w") as fh:
        fh.write(f"fattorib/hawk-pytorch hawk/*.py, unmodified; sha256 of the concatenated files: {digest.hexdigest()}\n")
    return dst


def available() -> bool:
    return all(os.path.isfile(os.path.join(DEST, "hawk", f)) for f in FILES)


def load():
    """The staged reference package `hawk` (imported from oracle/_ref), or None when absent."""
    if not available():
        return None
    mod = sys.modules.get("hawk")
    if mod is not None and os.path.dirname(os.path.dirname(os.path.abspath(mod.__file__))) == DEST:
        return mod
    for m in [m for m in sys.modules if m == "hawk" or m.startswith("hawk.")]:
        del sys.modules[m]
    sys.path.insert(0, DEST)
    try:
        return importlib.import_module("hawk")
    finally:
        sys.path.remove(DEST)


if __name__ == "__main__":
    out = stage(sys.argv[1] if len(sys.argv) > 1 else None)
    if out is None:
        sys.exit("no checkout of the reference found (argument, $HAWK_REFERENCE_DIR, ../reference)")
    print("reference staged in", out)
