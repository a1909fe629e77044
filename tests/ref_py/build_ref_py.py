#!/usr/bin/env python3
"""Compiles the REFERENCE's Python engine (py/*.py) and its own test files (tests/*.py) to bytecode, from where they
lie in the reference tree, so that tests/test_ref_py_gpu.py can run the reference's tests on a machine that has a GPU
but no reference tree. Like the reference's C++ mains (tests/ref_mains/build_ref_mains.py), nothing is copied into the
repository: the outputs are build artefacts under build/ref_py/ (git-ignored; they travel to the GPU box).

    python tests/ref_py/build_ref_py.py --reference <path of the tt-perf tree>   (or TTPERF_REFERENCE=<path>)

Layout of build/ref_py/: src/<module>.mod (the reference's test files import the engine as `src.*` although its
directory is called py/) and tests/<file>.mod. A .mod file is what py_compile writes (a .pyc under another suffix, so
that tools which skip Python caches when they copy a tree leave it alone); it is only valid for the Python version that
wrote it (same image here and on the GPU box)."""
from __future__ import annotations

import argparse
import os
import py_compile
import shutil
import sys
from pathlib import Path

REPO = Path(__file__).resolve().parents[2]
OUT = REPO / "build" / "ref_py"


def default_reference() -> str:
    """$TTPERF_REFERENCE, else a checkout named `reference` beside this repository."""
    return os.environ.get("TTPERF_REFERENCE", str(REPO.parent / "reference"))


def build(reference: str | None = None) -> list[str]:
    """Returns the names of the compiled test files ([] when the reference tree is absent)."""
    ref = Path(reference or default_reference())
    if not (ref / "py" / "engine.py").exists():
        return []
    if OUT.exists():
        shutil.rmtree(OUT)
    (OUT / "src").mkdir(parents=True)
    (OUT / "tests").mkdir(parents=True)
    for src in sorted((ref / "py").glob("*.py")):
        py_compile.compile(str(src), cfile=str(OUT / "src" / (src.stem + ".mod")), dfile=f"py/{src.name}", doraise=True)
    names = []
    for src in sorted((ref / "tests").glob("*.py")):
        py_compile.compile(str(src), cfile=str(OUT / "tests" / (src.stem + ".mod")), dfile=f"tests/{src.name}", doraise=True)
        names.append(src.stem)
    (OUT / "python_version.txt").write_text(sys.version.split()[0] + "\n")
    return names


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=default_reference())
    print("\n".join(build(ap.parse_args().reference)) or "no reference tree: nothing built")
