"""Generates tests/golden/bench_transformer_torch.json: what the reference's libtorch program
bench/autograd/bench_transformer_torch.cpp — compiled unchanged by oracle/build_ref.py — prints for verification (the
output shape and the first three output values) on a handful of configurations. The program's inputs are fixed by its
source: input all ones, every weight 0.01, bf16 on the CPU.

    python tests/golden/make_ref_torch_golden.py
"""
import json
import sys
from pathlib import Path

REPO = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(REPO))

from oracle import build_ref  # noqa: E402

# (batch, seq, dim, heads, layers); the last one is the program's default configuration
CONFIGS = [(2, 32, 64, 2, 1), (2, 32, 64, 2, 2), (4, 64, 128, 4, 3), (2, 64, 128, 2, 2), (32, 128, 256, 4, 8)]


def main() -> None:
    if build_ref.build() is None:
        raise SystemExit("the reference program could not be built here")
    cases = [build_ref.run(*cfg) for cfg in CONFIGS]
    out = {"source": "bench/autograd/bench_transformer_torch.cpp (input ones, weights 0.01, bf16 CPU)", "cases": cases}
    (Path(__file__).resolve().parent / "bench_transformer_torch.json").write_text(json.dumps(out, indent=1) + "\n")
    for c in cases:
        print(c)


if __name__ == "__main__":
    main()
