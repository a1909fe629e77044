#!/usr/bin/env python3
"""Compiles the REFERENCE's own C++ mains, unchanged and from where they lie in the reference tree, against this
repository's TTNN stand-in headers (include/ttnn/...) and links them to libb200ttperf.so.

    python tests/ref_mains/build_ref_mains.py --reference <path of the tt-perf tree>   (or TTPERF_REFERENCE=<path>)

Outputs go to build/ref_mains/ (git-ignored; they travel to the GPU box with the snapshot). No reference source is
copied into the repository. tests/test_ref_mains_gpu.py runs whatever binaries exist.

Two reference files cannot compile against ANY TTNN, this stand-in included, because of rot inside the reference:
examples/train_mlp.cpp and autograd/tests/test_mse_debug.cpp define `MLP` / `mse_loss` that now also exist in the
headers they include (ambiguous under `using namespace autograd`), and autograd/tests/test_static_autograd.cpp includes
a directory that does not exist (`static_autograd/nn.hpp`; the directory is `static/`)."""
from __future__ import annotations

import argparse
import concurrent.futures as cf
import os
import subprocess
import sys
from pathlib import Path

REPO = Path(__file__).resolve().parents[2]
OUT = REPO / "build" / "ref_mains"
LIB_DIR = REPO / "tt-perf_b200" / "lib"

MAINS = [
    "autograd/tests/test_matmul.cpp", "autograd/tests/test_tensor.cpp", "autograd/tests/test_relu.cpp",
    "autograd/tests/test_softmax.cpp", "autograd/tests/test_linear.cpp", "autograd/tests/test_sgd.cpp",
    "autograd/tests/test_attention.cpp", "autograd/tests/test_mean_debug.cpp",
    "examples/train_mlp_traced.cpp", "verify/verify_mlp_traced.cpp", "verify/verify_fidelity.cpp",
    "bench/autograd/bench_mlp.cpp", "bench/autograd/bench_autograd.cpp", "bench/autograd/bench_sweep.cpp",
    "bench/autograd/bench_autograd_sweep.cpp", "bench/autograd/bench_shape_sweep.cpp",
    "bench/autograd/bench_single_shape.cpp", "bench/autograd/bench_fusion.cpp",
    "bench/autograd/bench_fusion_forward.cpp", "bench/autograd/bench_transformer_depth.cpp",
    "bench/autograd/bench_gpt2_small.cpp", "bench/autograd/bench_transformer_train.cpp",
    "bench/autograd/bench_gpt2_full.cpp", "bench/autograd/bench_gpt2_trace.cpp",
    "bench/metal/matmul_sweep.cpp", "bench/metal/simple_matmul.cpp", "bench/metal/bench_fusion.cpp",
    "bench/metal/matmul_2dev.cpp", "bench/metal/matmul_2dev_distributed.cpp", "bench/metal/matmul_tensor_parallel.cpp",
]
# Programs of this repository that run on the reference's executors: built with the same recipe. train_mlp_ce includes
# the reference's dynamic autograd headers (so it needs the reference tree); matmul_mesh_fused needs only the stand-in.
OWN_MAINS = ["examples/train_mlp_ce.cpp", "examples/matmul_mesh_fused.cpp"]
# same base name in two directories: keep both
RENAME = {"bench/metal/bench_fusion.cpp": "metal_bench_fusion"}


def default_reference() -> str:
    """$TTPERF_REFERENCE, else a checkout named `reference` beside this repository."""
    return os.environ.get("TTPERF_REFERENCE", str(Path(__file__).resolve().parents[3] / "reference"))


def build_one(ref: Path, rel: str, own: bool = False) -> tuple[str, bool, str]:
    src = (REPO if own else ref) / rel
    name = RENAME.get(rel, Path(rel).stem)
    exe = OUT / name
    if not src.exists():
        return name, False, "source missing"
    cmd = ["g++", "-std=c++20", "-O2", "-I", str(REPO / "include"), "-I", str(ref / "autograd"), str(src), "-o", str(exe),
           "-L", str(LIB_DIR), "-lb200ttperf", f"-Wl,-rpath,$ORIGIN/../../tt-perf_b200/lib", "-lpthread"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        errs = [l for l in r.stderr.splitlines() if "error" in l][:3]
        return name, False, " | ".join(e[-200:] for e in errs)
    return name, True, ""


def build(reference: str | None = None) -> dict:
    ref = Path(reference or default_reference())
    if not ref.exists():
        return {}
    OUT.mkdir(parents=True, exist_ok=True)
    with cf.ThreadPoolExecutor(max_workers=8) as ex:
        results = list(ex.map(lambda rel: build_one(ref, rel), MAINS))
        results += list(ex.map(lambda rel: build_one(ref, rel, own=True), OWN_MAINS))
    return {name: (ok, msg) for name, ok, msg in results}


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=default_reference())
    res = build(ap.parse_args().reference)
    for name, (ok, msg) in res.items():
        print(f"{'OK  ' if ok else 'FAIL'} {name} {msg}")
    sys.exit(0 if res and all(ok for ok, _ in res.values()) else 1)
