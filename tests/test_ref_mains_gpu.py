"""Runs the reference's own C++ programs — compiled UNCHANGED against this repository's TTNN stand-in headers by
tests/ref_mains/build_ref_mains.py — on the GPU. The known-answer tests are assert-based (exit code 0 = every
assertion held); the MLP examples print losses that are compared with the reference's torch-CPU goldens."""
import json
import re
import subprocess

import pytest

from conftest import GOLDEN, REPO

pytestmark = pytest.mark.gpu
BIN = REPO / "build" / "ref_mains"


def run(name, timeout=300, env=None):
    exe = BIN / name
    if not exe.exists():
        pytest.skip(f"{exe} not built (tests/ref_mains/build_ref_mains.py needs the reference tree)")
    r = subprocess.run([str(exe)], capture_output=True, text=True, timeout=timeout, env=env)
    assert r.returncode == 0, f"{name} exited {r.returncode}\n{r.stdout[-1500:]}\n{r.stderr[-1500:]}"
    return r.stdout


@pytest.mark.parametrize("name", ["test_matmul", "test_tensor", "test_relu", "test_softmax", "test_linear", "test_sgd",
                                  "test_attention", "test_mean_debug"])
def test_reference_known_answer_programs(name):
    """autograd/tests/*.cpp: ones[32,64].ones[64,32] = 64 with dA = dB = 32, softmax(ones) = 1/64, SGD bias -0.32 then
    -0.64, attention rows summing to 1, ... — all checked by the programs' own asserts."""
    run(name)


def test_train_mlp_traced_matches_torch_bf16_goldens():
    """examples/train_mlp_traced.cpp prints its losses next to the expected torch-bf16 values 159.390625 -> 0.000244."""
    out = run("train_mlp_traced")
    gold = json.loads((GOLDEN / "verify_comparison.json").read_text())["bf16"]
    initial = float(re.search(r"Initial loss: ([-\d.eE]+)", out).group(1))
    assert abs(initial - gold["initial_loss"]) <= 0.01 * gold["initial_loss"]
    steps = re.findall(r"Step (\d+): loss_before=([-\d.eE]+), loss_after=([-\d.eE]+)", out)
    assert len(steps) == 5
    before = [float(s[1]) for s in steps]
    after = [float(s[2]) for s in steps]
    assert abs(before[0] - gold["loss_before"][0]) <= 0.01 * gold["loss_before"][0]
    assert abs(after[0] - gold["loss_after"][0]) <= 0.1 * gold["loss_after"][0]
    assert all(a < b for a, b in zip(after, before)) and after[-1] < 1e-2
    grads = dict(re.findall(r"(dW1\[0,0\]|dW2\[0,0\]|db1\[0\]|db2\[0\]): ([-\d.eE]+)", out))
    ref = gold["step0_grads"]
    for key, name in (("dW1[0,0]", "dW1_00"), ("dW2[0,0]", "dW2_00"), ("db1[0]", "db1_0"), ("db2[0]", "db2_0")):
        assert abs(float(grads[key]) - ref[name]) <= 0.02 * abs(ref[name]), (key, grads[key], ref[name])


def test_verify_mlp_traced_matches_verify_mlp_py():
    """verify/verify_mlp_traced.cpp is the C++ twin of verify/verify_mlp.py (32x64->32->32, lr 0.1, 10 steps)."""
    out = run("verify_mlp_traced")
    gold = json.loads((GOLDEN / "verify_mlp.json").read_text())
    losses = [float(x) for x in re.findall(r"Step \d+: loss = ([-\d.eE]+)", out)]
    assert len(losses) == 10
    initial = float(re.search(r"Initial loss[^:]*: ([-\d.eE]+)", out).group(1))
    assert abs(initial - gold["initial_loss"]) <= 0.02 * gold["initial_loss"]
    assert abs(losses[0] - gold["loss_after_step"][0]) <= 0.05 * gold["loss_after_step"][0]
    assert all(b < a for a, b in zip(losses, losses[1:]))


def test_bench_autograd_runs_all_executor_variants():
    """bench/autograd/bench_autograd.cpp drives the dynamic, static and traced executors (trace capture + replay)."""
    out = run("bench_autograd", timeout=600)
    assert "ms" in out.lower() or "iter" in out.lower()
