"""Compiles the reference's own Python modules for the hot path into ``oracle/_ref/`` (bytecode only).

TEST / BENCHMARK INFRASTRUCTURE. The SparseForge reference is pure Python on PyTorch; its three modules
on this path (``legacy/sparse_modeling.py``, ``legacy/utils.py``, ``legacy/adamw.py``) are compiled with
``py_compile`` from where they lie in a checkout (``$SPARSEFORGE_REFERENCE``) into sourceless ``.pyc``
files under ``oracle/_ref/`` (named ``<module>.bytecode``: tools that ship a source tree tend to drop
``*.pyc``). No source text is copied; ``oracle/_ref/`` is not tracked. The CPU arm of
``bench.py`` (``--impl reference``) imports these modules to time the reference's own code on the host
cores; nothing in ``sparseforge_b200/`` does.

    SPARSEFORGE_REFERENCE=<checkout> python oracle/build_ref.py
"""
from __future__ import annotations

import hashlib
import os
import py_compile
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
MODULES = ("sparse_modeling", "utils", "adamw")


def build(reference_root: str) -> str:
    legacy = os.path.join(reference_root, "legacy")
    if not os.path.isdir(legacy):
        raise SystemExit(f"{reference_root}: no legacy/ directory (set SPARSEFORGE_REFERENCE to a SparseForge checkout)")
    os.makedirs(OUT, exist_ok=True)
    lines = [f"python {sys.version.split()[0]}"]
    for name in MODULES:
        src = os.path.join(legacy, name + ".py")
        py_compile.compile(src, cfile=os.path.join(OUT, name + ".bytecode"), dfile=f"legacy/{name}.py", doraise=True)
        with open(src, "rb") as f:
            lines.append(f"legacy/{name}.py sha256 {hashlib.sha256(f.read()).hexdigest()}")
    with open(os.path.join(OUT, "MANIFEST.txt"), "w") as f:
        f.write("\n".join(lines) + "\n")
    return OUT


if __name__ == "__main__":
    root = os.environ.get("SPARSEFORGE_REFERENCE") or (sys.argv[1] if len(sys.argv) > 1 else "")
    if not root:
        raise SystemExit("set SPARSEFORGE_REFERENCE to a checkout of the SparseForge reference")
    print(build(root))
