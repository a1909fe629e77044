#!/usr/bin/env python3
"""Generates the golden fixtures in this directory from the REFERENCE's own torch-CPU code.

Run where the reference tree is mounted:

    python tests/golden/make_golden.py --reference <path of the tt-perf tree>   (or TTPERF_REFERENCE=<path>)

Nothing here is needed at test time: the tests only read the committed .json / .npz files.

What is produced
  verify_mlp.json          printed trajectory of verify/verify_mlp.py (run unmodified as a subprocess)
  verify_comparison.json   fp32 and bf16 trajectories of verify/verify_comparison.py (unmodified subprocess)
  verify_autograd.json     closed-form expectations printed by verify/verify_autograd.py (unmodified subprocess)
  block_small.npz          forward/backward of verify/compare_grads.py::PyTorchTransformerBlock (imported with a
                           stub `ttnn` module, since that file imports ttnn at the top) on seeded random weights
  block_const.npz          the same class in the script's own setting: constant 0.02 weights, MSE-vs-zeros loss
  tiny_transformer_adam.npz  experiment_torch.py::TorchTinyTransformer, 3 Adam steps with cross-entropy on the
                           answer token (seeded random tokens stand in for the modular-division data set)
  adam_two_step.npz        the `_adam_step_ref` recurrence of tests/adam_optimizer.py:15-22 applied twice
  mlp_ce_784_128_10.npz    the 784-128-10 softmax-cross-entropy MLP (batch 64, SGD lr 0.01, 10 steps, seed 42).
                           The reference has no script for this configuration; it is produced with torch fp32
                           in the same style as verify/verify_mlp.py and is marked as such in the file.
"""
from __future__ import annotations

import argparse
import importlib.util
import json
import os
import re
import subprocess
import sys
import types
from pathlib import Path

import numpy as np
import torch
import torch.nn as nn
import torch.nn.functional as F

HERE = Path(__file__).resolve().parent
DEFAULT_REFERENCE = str(Path(__file__).resolve().parents[3] / "reference")   # a checkout beside this repository


def run_script(ref: Path, rel: str) -> str:
    r = subprocess.run([sys.executable, str(ref / rel)], capture_output=True, text=True, cwd=str(HERE), check=True)
    return r.stdout


def floats(pattern: str, text: str) -> list[float]:
    return [float(x) for x in re.findall(pattern, text)]


def gen_verify_mlp(ref: Path) -> None:
    out = run_script(ref, "verify/verify_mlp.py")
    data = {
        "source": "verify/verify_mlp.py (stdout, unmodified)",
        "config": {"batch": 32, "in": 64, "hidden": 32, "out": 32, "lr": 0.1, "steps": 10, "init": 0.01,
                   "x": 1.0, "target": 0.5, "loss": "mse"},
        "initial_loss": floats(r"Initial loss \(step 0\): ([-\d.eE]+)", out)[0],
        "step1_grads": {
            "dW1_00": floats(r"dW1\[0,0\] = ([-\d.eE]+)", out)[0],
            "dW2_00": floats(r"dW2\[0,0\] = ([-\d.eE]+)", out)[0],
            "db1_0": floats(r"db1\[0\] = ([-\d.eE]+)", out)[0],
            "db2_0": floats(r"db2\[0\] = ([-\d.eE]+)", out)[0],
        },
        "loss_after_step": floats(r"Step \d+: loss = ([-\d.eE]+)", out),
        "W1_00_after_step": floats(r"Step \d+: loss = [-\d.eE]+\n  W1\[0,0\] = ([-\d.eE]+)", out),
        "W2_00_after_step": floats(r"(?<!d)W2\[0,0\] = ([-\d.eE]+)", out)[1:],
    }
    assert len(data["loss_after_step"]) == 10
    (HERE / "verify_mlp.json").write_text(json.dumps(data, indent=1) + "\n")


def gen_verify_comparison(ref: Path) -> None:
    out = run_script(ref, "verify/verify_comparison.py")
    parts = re.split(r"Running with dtype: ", out)[1:]
    data = {"source": "verify/verify_comparison.py (stdout, unmodified)",
            "config": {"batch": 1024, "in": 512, "hidden": 256, "out": 128, "lr": 0.01, "steps": 5, "init": 0.01,
                       "x": 1.0, "target": 0.5, "loss": "mse"}}
    for part in parts:
        name = part.split("\n", 1)[0].strip()
        key = "bf16" if "bf16" in name.lower() or "bfloat" in name.lower() else "fp32"
        data[key] = {
            "dtype_label": name,
            "initial_loss": floats(r"Initial loss: ([-\d.eE]+)", part)[0],
            "loss_before": floats(r"loss_before=([-\d.eE]+)", part),
            "loss_after": floats(r"loss_after=([-\d.eE]+)", part),
            "step0_grads": {
                "dW1_00": floats(r"dW1\[0,0\]: ([-\d.eE]+)", part)[0],
                "dW2_00": floats(r"dW2\[0,0\]: ([-\d.eE]+)", part)[0],
                "db1_0": floats(r"db1\[0\]: ([-\d.eE]+)", part)[0],
                "db2_0": floats(r"db2\[0\]: ([-\d.eE]+)", part)[0],
            },
        }
    assert "fp32" in data and "bf16" in data, list(data)
    (HERE / "verify_comparison.json").write_text(json.dumps(data, indent=1) + "\n")


def gen_verify_autograd(ref: Path) -> None:
    out = run_script(ref, "verify/verify_autograd.py")
    assert "ALL TESTS PASSED" in out
    data = {
        "source": "verify/verify_autograd.py (stdout, unmodified)",
        "all_passed": True,
        "matmul": {"shape_a": [32, 64], "shape_b": [64, 32], "C": floats(r"C\[0,0\] = ([-\d.]+)", out)[0],
                   "dA": floats(r"dA\[0,0\] = ([-\d.]+)", out)[0], "dB": floats(r"dB\[0,0\] = ([-\d.]+)", out)[0]},
        "relu": {"y": floats(r"Forward: y\[0,0\] = ([-\d.]+) \(expected: 1\)", out)[0],
                 "dx": floats(r"dx\[0,0\] = ([-\d.]+) \(expected: 1\)", out)[0]},
        "softmax": {"cols": 64, "y": floats(r"Forward: y\[0,0\] = ([-\d.]+) \(expected: 0\.015625\)", out)[0],
                    "dx": floats(r"dx\[0,0\] = ([-\d.]+) \(expected: 0\)", out)[0]},
        "linear": {"y": floats(r"Forward: y\[0,0\] = ([-\d.]+) \(expected: 6\.4\)", out)[0],
                   "dBias": floats(r"dBias\[0\] = ([-\d.]+)", out)[0]},
        "sgd": {"lr": 0.01, "bias_after_1": floats(r"Bias after step 1: ([-\d.]+)", out)[0],
                "bias_after_2": floats(r"Bias after step 2: ([-\d.]+)", out)[0]},
    }
    (HERE / "verify_autograd.json").write_text(json.dumps(data, indent=1) + "\n")


def import_with_stub_ttnn(ref: Path, rel: str, name: str):
    """Imports a reference file whose only obstacle is `import ttnn` at the top."""
    sys.modules.setdefault("ttnn", types.ModuleType("ttnn"))
    spec = importlib.util.spec_from_file_location(name, ref / rel)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


BLOCK_KEYS = {  # fixture key -> attribute path in PyTorchTransformerBlock
    "ln1_g": "ln1.weight", "ln1_b": "ln1.bias", "wq": "wq.weight", "bq": "wq.bias", "wk": "wk.weight",
    "bk": "wk.bias", "wv": "wv.weight", "bv": "wv.bias", "wo": "wo.weight", "bo": "wo.bias",
    "ln2_g": "ln2.weight", "ln2_b": "ln2.bias", "w1": "w1.weight", "b1": "w1.bias", "w2": "w2.weight",
    "b2": "w2.bias",
}


def _get(mod: nn.Module, path: str) -> torch.Tensor:
    obj = mod
    for p in path.split("."):
        obj = getattr(obj, p)
    return obj


def gen_block(ref: Path) -> None:
    cg = import_with_stub_ttnn(ref, "verify/compare_grads.py", "ref_compare_grads")
    # (1) seeded random weights, upstream gradient given explicitly
    B, S, D, H = 2, 32, 64, 2
    torch.manual_seed(42)
    block = cg.PyTorchTransformerBlock(D, H, 4, S)
    with torch.no_grad():
        for name, p in block.named_parameters():
            if name.startswith("ln") and name.endswith("weight"):
                p.copy_(1.0 + 0.1 * torch.randn_like(p))
            elif name.startswith("ln"):
                p.copy_(0.1 * torch.randn_like(p))
            elif name.endswith("weight"):
                p.copy_(0.02 * torch.randn_like(p) * 5)
            else:
                p.copy_(0.05 * torch.randn_like(p))
    x = (torch.randn(B, S, D) * 0.5).requires_grad_(True)
    d_out = torch.randn(B, S, D) * 0.1
    out = block(x)
    out.backward(d_out)
    arrays = {"x": x.detach().numpy(), "d_out": d_out.numpy(), "out": out.detach().numpy(),
              "d_x": x.grad.numpy(), "heads": np.array(H)}
    for k, path in BLOCK_KEYS.items():
        p = _get(block, path)
        arrays["p_" + k] = p.detach().numpy()
        arrays["g_" + k] = p.grad.numpy()
    np.savez_compressed(HERE / "block_small.npz", **arrays)

    # (2) the script's own setting (run_pytorch_reference): constant weights, MSE against zeros, reduced size
    torch.manual_seed(cg.SEED)
    block = cg.PyTorchTransformerBlock(D, H, 4, S)
    cg.init_weights_uniform(block, 0.02)
    x = (torch.randn(B, S, D) * 0.1).requires_grad_(True)
    out = block(x)
    loss = F.mse_loss(out, torch.zeros(B, S, D))
    loss.backward()
    arrays = {"x": x.detach().numpy(), "out": out.detach().numpy(), "loss": np.array(loss.item()),
              "d_x": x.grad.numpy(), "heads": np.array(H), "init": np.array(0.02)}
    for k, path in BLOCK_KEYS.items():
        arrays["g_" + k] = _get(block, path).grad.numpy()
    np.savez_compressed(HERE / "block_const.npz", **arrays)


def gen_tiny_transformer_adam(ref: Path) -> None:
    spec = importlib.util.spec_from_file_location("ref_experiment_torch", ref / "experiment_torch.py")
    et = importlib.util.module_from_spec(spec)
    sys.path.insert(0, str(ref))
    try:
        spec.loader.exec_module(et)
    finally:
        sys.path.pop(0)
    torch.manual_seed(0)
    vocab, seq, dim, heads = 32, 4, 32, 2
    model = et.TorchTinyTransformer(vocab_size=vocab, seq_len=seq, dim=dim, heads=heads, ffn_mult=2)
    opt = torch.optim.Adam(model.parameters(), lr=1e-3)
    tokens = torch.randint(0, vocab, (16, seq))
    targets = torch.randint(0, vocab, (16,))
    names = [n for n, _ in model.named_parameters()]
    arrays = {"tokens": tokens.numpy(), "targets": targets.numpy(), "names": np.array(names),
              "vocab": np.array(vocab), "seq": np.array(seq), "dim": np.array(dim), "heads": np.array(heads),
              "answer_pos": np.array(seq - 1), "lr": np.array(1e-3)}
    for n, p in model.named_parameters():
        arrays["p0/" + n] = p.detach().numpy().copy()
    losses = []
    for step in range(3):
        logits = model(tokens)
        loss = F.cross_entropy(logits[:, seq - 1, :], targets)
        loss.backward()
        if step == 0:
            arrays["logits0"] = logits.detach().numpy().copy()
            for n, p in model.named_parameters():
                arrays["g0/" + n] = p.grad.numpy().copy()
        opt.step()
        opt.zero_grad()
        losses.append(loss.item())
    arrays["losses"] = np.array(losses)
    for n, p in model.named_parameters():
        arrays["p3/" + n] = p.detach().numpy().copy()
    np.savez_compressed(HERE / "tiny_transformer_adam.npz", **arrays)


def gen_adam_two_step() -> None:
    # tests/adam_optimizer.py:15-22, restated by running the same recurrence in torch fp32
    def ref(weight, grad, lr, betas, eps, step, m, v):
        beta1, beta2 = betas
        m = beta1 * m + (1.0 - beta1) * grad
        v = beta2 * v + (1.0 - beta2) * (grad * grad)
        m_hat = m / (1.0 - (beta1 ** step))
        v_hat = v / (1.0 - (beta2 ** step))
        weight = weight - lr * m_hat / (torch.sqrt(v_hat) + eps)
        return weight, m, v

    torch.manual_seed(31)
    w0 = torch.randn(32, 32) * 0.1
    g1 = torch.randn(32, 32)
    g2 = torch.randn(32, 32)
    m = torch.zeros_like(w0)
    v = torch.zeros_like(w0)
    w1, m1, v1 = ref(w0, g1, 0.1, (0.9, 0.999), 1e-8, 1, m, v)
    w2, m2, v2 = ref(w1, g2, 0.1, (0.9, 0.999), 1e-8, 2, m1, v1)
    # cross-check against torch.optim.Adam itself
    p = nn.Parameter(w0.clone())
    opt = torch.optim.Adam([p], lr=0.1, betas=(0.9, 0.999), eps=1e-8)
    for g in (g1, g2):
        p.grad = g.clone()
        opt.step()
    assert torch.allclose(p.detach(), w2, atol=1e-5), (p.detach() - w2).abs().max()
    np.savez_compressed(HERE / "adam_two_step.npz", w0=w0.numpy(), g1=g1.numpy(), g2=g2.numpy(), w1=w1.numpy(),
                        m1=m1.numpy(), v1=v1.numpy(), w2=w2.numpy(), m2=m2.numpy(), v2=v2.numpy(),
                        lr=np.array(0.1), beta1=np.array(0.9), beta2=np.array(0.999), eps=np.array(1e-8))


def gen_mlp_ce() -> None:
    torch.manual_seed(42)
    g = torch.Generator().manual_seed(42)
    x = torch.randn(64, 784, generator=g)
    labels = torch.randint(0, 10, (64,), generator=g)
    model = nn.Sequential(nn.Linear(784, 128), nn.ReLU(), nn.Linear(128, 10))  # Kaiming-uniform default init
    arrays = {"x": x.numpy(), "labels": labels.numpy().astype(np.int64), "lr": np.array(0.01),
              "w1_0": model[0].weight.detach().numpy().copy(), "b1_0": model[0].bias.detach().numpy().copy(),
              "w2_0": model[2].weight.detach().numpy().copy(), "b2_0": model[2].bias.detach().numpy().copy(),
              "note": np.array("no reference script exists for this configuration; torch fp32, style of "
                               "verify/verify_mlp.py")}
    opt = torch.optim.SGD(model.parameters(), lr=0.01)
    losses = []
    for step in range(10):
        opt.zero_grad()
        loss = F.cross_entropy(model(x), labels)
        loss.backward()
        if step == 0:
            arrays["dw1_0"] = model[0].weight.grad.numpy().copy()
            arrays["db1_0"] = model[0].bias.grad.numpy().copy()
            arrays["dw2_0"] = model[2].weight.grad.numpy().copy()
            arrays["db2_0"] = model[2].bias.grad.numpy().copy()
        opt.step()
        losses.append(loss.item())
    arrays["losses"] = np.array(losses)
    arrays["w1_10"] = model[0].weight.detach().numpy().copy()
    arrays["b1_10"] = model[0].bias.detach().numpy().copy()
    arrays["w2_10"] = model[2].weight.detach().numpy().copy()
    arrays["b2_10"] = model[2].bias.detach().numpy().copy()
    np.savez_compressed(HERE / "mlp_ce_784_128_10.npz", **arrays)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("TTPERF_REFERENCE", DEFAULT_REFERENCE))
    ref = Path(ap.parse_args().reference)
    torch.set_num_threads(1)  # bit-stable reductions
    gen_verify_mlp(ref)
    gen_verify_comparison(ref)
    gen_verify_autograd(ref)
    gen_block(ref)
    gen_tiny_transformer_adam(ref)
    gen_adam_two_step()
    gen_mlp_ce()
    for f in sorted(HERE.glob("*.json")) + sorted(HERE.glob("*.npz")):
        print(f"{f.name:32s} {f.stat().st_size:8d} bytes")


if __name__ == "__main__":
    main()
