"""Place the reference's own pure-Python package under oracle/_ref so that the CPU baseline can time the
reference itself (`layer(x, implementation="reference")`) instead of the oracle port.

    python oracle/build_ref.py [path of the reference checkout; default: REFERENCE_ROOT below, or the
                                environment variable MEMSOLVE_REFERENCE_ROOT]

The package (memsolve/: five Python files) is copied as it lies, unmodified, into oracle/_ref/memsolve.  That
folder is listed in .gitignore: the copy is a build product of this recipe, like a compiled reference library
would be, not source of this repository.  bench.py (`--impl reference` and the `cpu_baseline` leg) uses it when
it is there and falls back to the oracle port otherwise; nothing else imports it.
"""
from __future__ import annotations

import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
TARGET = os.path.join(HERE, "_ref")
REFERENCE_ROOT = os.environ.get("MEMSOLVE_REFERENCE_ROOT", os.path.join(os.sep, "root", "reference"))


def build(reference_root: str = REFERENCE_ROOT) -> bool:
    source = os.path.join(reference_root, "memsolve")
    if not os.path.isdir(source):
        return os.path.isdir(os.path.join(TARGET, "memsolve"))   # keep what an earlier build left
    os.makedirs(TARGET, exist_ok=True)
    destination = os.path.join(TARGET, "memsolve")
    if os.path.isdir(destination):
        shutil.rmtree(destination)
    shutil.copytree(source, destination, ignore=shutil.ignore_patterns("__pycache__", "*.pyc"))
    return True


if __name__ == "__main__":
    ok = build(sys.argv[1] if len(sys.argv) > 1 else REFERENCE_ROOT)
    print("oracle/_ref/memsolve", "ready" if ok else "not available (no reference checkout)")
