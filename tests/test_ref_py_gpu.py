"""Runs the REFERENCE's own Python tests (its tests/*.py: 12 files, each with its torch-CPU comparison and tolerance)
on the GPU, with the reference's Python engine (py/engine.py, nn.py, optim.py, data.py) unchanged and `import ttnn`
resolved to this repository's stand-in over the C ABI (tt-perf_b200/ttnn_py). Both the engine and the tests are the
bytecode build of tests/ref_py/build_ref_py.py (build/ref_py/): the GPU box has no reference tree.

One test per reference file: every `test_*` function of the file must pass; the outcome per function is printed."""
import importlib
import importlib.machinery
import importlib.util
import sys
import traceback
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
REPO = Path(__file__).resolve().parent.parent
BUILD = REPO / "build" / "ref_py"
FILES = ["adam_optimizer", "causal_attention_single_and_batched", "cross_entropy_loss", "linear_embedding_layers",
         "modular_division_dataset", "multihead_attention", "prime_sequence_dataset", "relu_activation", "sgd_optimizer",
         "softmax_logsoftmax_activations", "tensor_add_mul_matmul_tanh", "transformer_block_forward_backward"]


def _load_sourceless(name: str, path: Path, package_dir: Path | None = None):
    loader = importlib.machinery.SourcelessFileLoader(name, str(path))
    # a file location, so that the module gets the __file__ the reference's tests derive their import root from
    spec = importlib.util.spec_from_file_location(name, str(path), loader=loader,
                                                  submodule_search_locations=[str(package_dir)] if package_dir is not None else None)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    loader.exec_module(mod)
    return mod


@pytest.fixture(scope="module")
def reference_engine():
    """`ttnn` = the stand-in; `src` (and its alias `grad`, which py/optim.py uses) = the reference's engine package."""
    if not (BUILD / "src" / "engine.mod").exists():
        pytest.skip("build/ref_py is missing (tests/ref_py/build_ref_py.py needs the reference tree)")
    if (BUILD / "python_version.txt").read_text().split()[0] != sys.version.split()[0]:
        pytest.skip("build/ref_py was compiled by another Python version")
    stand_in = str(REPO / "tt-perf_b200" / "ttnn_py")
    sys.path.insert(0, stand_in)
    saved = {k: sys.modules.pop(k) for k in list(sys.modules) if k == "ttnn" or k.split(".")[0] in ("src", "grad")}
    try:
        importlib.import_module("ttnn")
        pkg = _load_sourceless("src", BUILD / "src" / "__init__.mod", BUILD / "src")
        for sub in ("engine", "data"):
            setattr(pkg, sub, _load_sourceless(f"src.{sub}", BUILD / "src" / f"{sub}.mod"))
        sys.modules["grad"] = pkg
        sys.modules["grad.engine"] = sys.modules["src.engine"]
        for sub in ("nn", "optim"):
            setattr(pkg, sub, _load_sourceless(f"src.{sub}", BUILD / "src" / f"{sub}.mod"))
        yield pkg
    finally:
        for k in [k for k in sys.modules if k == "ttnn" or k.split(".")[0] in ("src", "grad", "ref_tests")]:
            sys.modules.pop(k, None)
        sys.modules.update(saved)
        sys.path.remove(stand_in)


@pytest.mark.parametrize("name", FILES)
def test_reference_python_test_file(reference_engine, name):
    mod = _load_sourceless(f"ref_tests.{name}", BUILD / "tests" / f"{name}.mod")
    tests = sorted(k for k, v in vars(mod).items() if k.startswith("test_") and callable(v))
    assert tests, f"{name}: no test functions found"
    failed = []
    for t in tests:
        try:
            getattr(mod, t)()
            print(f"PASS {name}::{t}")
        except Exception:
            print(f"FAIL {name}::{t}\n{traceback.format_exc(limit=6)}")
            failed.append(t)
    assert not failed, f"{name}: {len(failed)} of {len(tests)} reference tests failed: {failed}"
