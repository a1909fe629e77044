"""CPU-side checks of the C ABI: the library loads, exports every symbol the header declares, the ctypes
table matches the header, and argument validation rejects bad calls without touching a GPU."""
import ctypes as C
import re
import subprocess

import pytest

from conftest import REPO

HEADER = REPO / "include" / "b200_ttperf.h"


def header_functions():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(b200_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(pkg):
    lib = pkg.lib()
    names = header_functions()
    assert "b200_gemm" in names and "b200_ctx_create" in names
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in the header but not exported"


def test_ctypes_table_covers_the_header(pkg):
    assert sorted(pkg.capi.SIGNATURES) == header_functions()


def test_only_c_abi_symbols_are_exported(pkg):
    out = subprocess.run(["nm", "-D", "--defined-only", str(pkg.lib_path())], capture_output=True, text=True,
                         check=True).stdout
    syms = [line.split()[-1] for line in out.splitlines() if line.strip()]
    assert syms and all(s.startswith("b200_") for s in syms), [s for s in syms if not s.startswith("b200_")][:5]


def test_header_compiles_as_plain_c(tmp_path):
    src = tmp_path / "t.c"
    src.write_text('#include "b200_ttperf.h"\nint main(void){ b200_gemm_desc d; (void)d; return B200_OK; }\n')
    subprocess.run(["gcc", "-std=c99", "-Wall", "-Werror", "-I", str(REPO / "include"), "-c", str(src), "-o",
                    str(tmp_path / "t.o")], check=True)


def test_struct_layout_matches_the_header(pkg, tmp_path):
    src = tmp_path / "sz.c"
    src.write_text('#include <stdio.h>\n#include <stddef.h>\n#include "b200_ttperf.h"\n'
                   'int main(void){ printf("%zu %zu %zu %zu %zu", sizeof(b200_gemm_desc), offsetof(b200_gemm_desc, C),'
                   ' offsetof(b200_gemm_desc, alpha), offsetof(b200_gemm_desc, split_k),'
                   ' offsetof(b200_gemm_desc, ab_dtype)); return 0; }\n')
    exe = tmp_path / "sz"
    subprocess.run(["gcc", "-I", str(REPO / "include"), str(src), "-o", str(exe)], check=True)
    size, off_c, off_alpha, off_split, off_ab = map(int, subprocess.run([str(exe)], capture_output=True, text=True,
                                                                check=True).stdout.split())
    G = pkg.GemmDesc
    assert (C.sizeof(G), G.C.offset, G.alpha.offset, G.split_k.offset, G.ab_dtype.offset) == (
        size, off_c, off_alpha, off_split, off_ab)


def test_abi_version_and_desc_defaults(pkg):
    lib = pkg.lib()
    assert lib.b200_abi_version() == 2
    d = pkg.GemmDesc()
    lib.b200_gemm_desc_init(C.byref(d))
    assert (d.batch, d.alpha, d.c_dtype, d.fidelity, d.algo, d.split_k) == (1, 1.0, pkg.BF16, pkg.HIFI4, 0, 0)
    assert d.ab_dtype == pkg.BF16
    assert d.transpose_a == 0 and d.transpose_b == 0 and d.activation == pkg.ACT_NONE


def test_no_cpu_fallback_context_creation_fails_without_a_gpu(pkg):
    torch = pytest.importorskip("torch")
    if torch.cuda.is_available():
        pytest.skip("a GPU is present; this test pins the behaviour on a GPU-less host")
    with pytest.raises(pkg.B200Error) as e:
        pkg.Context(0)
    assert e.value.code == pkg.capi.ERR_CUDA and "no CPU path" in str(e.value)


def test_null_arguments_are_rejected(pkg):
    lib = pkg.lib()
    assert lib.b200_gemm(None, None, None) == pkg.capi.ERR_INVALID_ARG
    assert b"ctx is NULL" in lib.b200_last_error()
    assert lib.b200_ctx_create(0, None) == pkg.capi.ERR_INVALID_ARG
    assert lib.b200_synchronize(None, None) == pkg.capi.ERR_INVALID_ARG
    assert lib.b200_malloc(None, 16, None) == pkg.capi.ERR_INVALID_ARG
    assert lib.b200_ctx_destroy(None) == pkg.capi.OK  # destroying nothing is not an error


def test_python_ttnn_stand_in_imports_and_serves_the_reference_engine():
    """The Python `ttnn` stand-in exposes every name the reference's Python side uses; when the reference tree is
    present, its py/engine.py, py/nn.py and py/optim.py import against it unchanged (no device is opened)."""
    import importlib
    import importlib.util
    import os
    import sys
    from pathlib import Path
    repo = Path(__file__).resolve().parent.parent
    sys.path.insert(0, str(repo / "tt-perf_b200" / "ttnn_py"))
    try:
        sys.modules.pop("ttnn", None)
        ttnn = importlib.import_module("ttnn")
        for name in ("open_device", "close_device", "from_torch", "to_torch", "Tensor", "bfloat16", "float32", "uint32",
                     "TILE_LAYOUT", "ROW_MAJOR_LAYOUT", "add", "sub", "mul", "div", "matmul", "sum", "softmax", "log", "exp",
                     "tanh", "sqrt", "relu", "gtz", "permute", "reshape", "triu", "embedding", "full_like", "ones_like",
                     "WormholeComputeKernelConfig", "MathFidelity", "ReadDeviceProfiler"):
            assert hasattr(ttnn, name), name
        assert ttnn.MathFidelity.HiFi3 and ttnn.WormholeComputeKernelConfig(math_fidelity=ttnn.MathFidelity.HiFi3)
        spec_b = importlib.util.spec_from_file_location("build_ref_mains", repo / "tests" / "ref_mains" / "build_ref_mains.py")
        brm = importlib.util.module_from_spec(spec_b)
        spec_b.loader.exec_module(brm)
        ref = Path(brm.default_reference())     # TTPERF_REFERENCE, else the default location of the tree
        if (ref / "py" / "engine.py").exists():
            # the reference's files import each other as `src.*` while the directory is called py/: load it under that name
            spec = importlib.util.spec_from_file_location("src", ref / "py" / "__init__.py",
                                                          submodule_search_locations=[str(ref / "py")])
            pkg = importlib.util.module_from_spec(spec)
            sys.modules["src"] = pkg
            try:
                spec.loader.exec_module(pkg)
                importlib.import_module("src.engine")
                sys.modules["grad"] = pkg                      # optim.py says `grad.engine` for the same module
                sys.modules["grad.engine"] = sys.modules["src.engine"]
                for mod in ("src.nn", "src.optim"):
                    importlib.import_module(mod)
                eng = sys.modules["src.engine"]
                assert eng.resolve_tt_dtype(None) is ttnn.bfloat16
                assert eng._DEFAULT_COMPUTE_KERNEL_CONFIG.math_fidelity == ttnn.MathFidelity.HiFi3
            finally:
                for mod in [m for m in sys.modules if m in ("src", "grad") or m.startswith(("src.", "grad."))]:
                    sys.modules.pop(mod, None)
    finally:
        sys.path.remove(str(repo / "tt-perf_b200" / "ttnn_py"))
        sys.modules.pop("ttnn", None)
