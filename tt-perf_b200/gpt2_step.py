#!/usr/bin/env python3
"""Runs a few eager (untraced) training steps of the GPT-2-shaped model of nn.py on synthetic token ids and prints the
loss of each: the smallest program that exercises every kernel of the training step, used for per-kernel launch lists.

    python tt-perf_b200/gpt2_step.py [--steps 2] [--layers 12] [--d-model 768] [--heads 12] [--seq 1024] [--batch 8]
                                     [--vocab 50257]
"""
from __future__ import annotations

import argparse
import importlib.util
from pathlib import Path

import numpy as np

REPO = Path(__file__).resolve().parent.parent


def main() -> None:
    ap = argparse.ArgumentParser()
    for name, default in (("steps", 2), ("layers", 12), ("d-model", 768), ("heads", 12), ("seq", 1024), ("batch", 8),
                          ("vocab", 50257)):
        ap.add_argument("--" + name, type=int, default=default)
    a = ap.parse_args()
    spec = importlib.util.spec_from_file_location("__graft_entry__", REPO / "__graft_entry__.py")
    entry = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(entry)
    pkg = entry.load_package()
    ctx = pkg.Context(0)
    DT = pkg.DeviceTensor
    model = pkg.nn.GPT2(ctx, layers=a.layers, d_model=a.d_model, heads=a.heads, seq=a.seq, vocab=a.vocab)
    model.init_random(42)
    ids = np.random.default_rng(0).integers(0, a.vocab, (a.batch, a.seq)).astype(np.uint32)
    args = (DT.from_numpy(ctx, ids, pkg.U32), DT.from_numpy(ctx, np.roll(ids, -1, axis=1).ravel(), pkg.U32),
            DT.from_numpy(ctx, np.arange(a.seq, dtype=np.uint32), pkg.U32))
    for step in range(a.steps):
        loss, grads = model.forward_backward(*args)
        model.adam_step(grads)
        ctx.synchronize()
        print(f"step {step}: loss {float(loss.numpy()[0]):.4f}", flush=True)
    ctx.close()


if __name__ == "__main__":
    main()
