"""Builds the one program of the reference that compiles on a machine without Tenstorrent hardware: its libtorch
twin of the traced transformer layer, bench/autograd/bench_transformer_torch.cpp (attention + ReLU FFN with residuals,
no LayerNorm, bf16 on the CPU). TEST INFRASTRUCTURE: the binary only serves to pin the numpy oracle
(`matmul_oracle.simple_transformer_layer_forward`) to output of the reference's own C++ code.

The source is compiled where it lies in the reference tree (nothing is copied), with g++ against the headers and
libraries of the installed torch package; the only output is oracle/_ref/bench_transformer_torch.

    python oracle/build_ref.py [/path/to/reference]      # prints the binary's path, or why nothing was built
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT_DIR = HERE / "_ref"
SOURCE = "bench/autograd/bench_transformer_torch.cpp"
BINARY = OUT_DIR / "bench_transformer_torch"


def default_reference() -> Path | None:
    """The reference tree: $TTPERF_REFERENCE, else a checkout named `reference` beside this repository; None when absent."""
    cand = Path(os.environ.get("TTPERF_REFERENCE", str(Path(__file__).resolve().parents[2] / "reference")))
    return cand if (cand / SOURCE).exists() else None


def build(reference: Path | None = None, force: bool = False) -> Path | None:
    """Returns the binary's path, or None (with a message on stderr) when the reference tree, g++ or torch's C++
    headers are not there."""
    reference = reference or default_reference()
    if reference is None:
        print("oracle/build_ref.py: no reference tree; nothing built", file=sys.stderr)
        return None
    src = reference / SOURCE
    gxx = shutil.which("g++")
    try:
        import torch
        from torch.utils import cpp_extension
    except Exception as e:  # pragma: no cover
        print(f"oracle/build_ref.py: torch is not importable ({e}); nothing built", file=sys.stderr)
        return None
    if gxx is None:
        print("oracle/build_ref.py: g++ not found; nothing built", file=sys.stderr)
        return None
    if BINARY.exists() and not force and BINARY.stat().st_mtime > src.stat().st_mtime:
        return BINARY
    OUT_DIR.mkdir(parents=True, exist_ok=True)
    lib_dir = Path(torch.__file__).resolve().parent / "lib"
    includes = [p for p in cpp_extension.include_paths() if "cuda" not in Path(p).name.lower()]
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    cmd = [gxx, "-std=c++17", "-O2", f"-D_GLIBCXX_USE_CXX11_ABI={abi}", *[f"-I{p}" for p in includes], str(src), "-o",
           str(BINARY), f"-L{lib_dir}", f"-Wl,-rpath,{lib_dir}", "-ltorch", "-ltorch_cpu", "-lc10", "-lpthread"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        print(f"oracle/build_ref.py: g++ failed:\n{r.stderr[-2000:]}", file=sys.stderr)
        return None
    return BINARY


def run(batch: int, seq: int, dim: int, heads: int, layers: int, ffn_mult: int = 4, timeout: int = 600) -> dict:
    """Runs the binary on one configuration (the program reads BENCH_* from the environment) and parses what it
    prints for verification: the output shape and the first three output values."""
    import re
    env = dict(os.environ, BENCH_BATCH=str(batch), BENCH_SEQ=str(seq), BENCH_DIM=str(dim), BENCH_HEADS=str(heads),
               BENCH_FFN_MULT=str(ffn_mult), BENCH_LAYERS=str(layers), OMP_NUM_THREADS="4")
    r = subprocess.run([str(BINARY)], capture_output=True, text=True, timeout=timeout, env=env)
    if r.returncode != 0:
        raise RuntimeError(f"{BINARY.name} exited {r.returncode}: {r.stderr[-500:]}")
    shape = [int(v) for v in re.search(r"Output shape: \[(\d+), (\d+), (\d+)\]", r.stdout).groups()]
    first = [float(v) for v in re.search(r"First values: ([^\n]+)", r.stdout).group(1).split(",")]
    return {"batch": batch, "seq": seq, "dim": dim, "heads": heads, "layers": layers, "ffn_mult": ffn_mult,
            "output_shape": shape, "first_values": first}


if __name__ == "__main__":
    ref = Path(sys.argv[1]) if len(sys.argv) > 1 else None
    out = build(ref, force="--force" in sys.argv)
    print(out if out else "not built")
