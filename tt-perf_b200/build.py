"""Builds the CUDA library (one shared object, C ABI) for sm_100a with nvcc.

    python tt-perf_b200/build.py            # incremental build
    python tt-perf_b200/build.py --force    # rebuild everything

Each .cu file is compiled to an object under build/obj (in parallel) and linked into
tt-perf_b200/lib/libb200ttperf.so. nvcc cross-compiles, so this works on a machine with no GPU.
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
REPO = PKG_DIR.parent
CSRC = PKG_DIR / "csrc"
LIB_DIR = PKG_DIR / "lib"
OBJ_DIR = REPO / "build" / "obj"
LIB_PATH = LIB_DIR / "libb200ttperf.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC,-Wall,-Wno-unknown-pragmas",
    "--expt-relaxed-constexpr",
    "-Xptxas", "-v",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; the library cannot be built")
    return exe


def _sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _headers_mtime() -> float:
    hdrs = list(CSRC.glob("*.cuh")) + list((REPO / "include").glob("*.h"))
    return max((h.stat().st_mtime for h in hdrs), default=0.0)


def _compile(src: Path, force: bool, hdr_mtime: float, obj_dir: Path = OBJ_DIR, extra=()) -> tuple[Path, str]:
    obj = obj_dir / (src.stem + ".o")
    if not force and obj.exists() and obj.stat().st_mtime > max(src.stat().st_mtime, hdr_mtime):
        return obj, ""
    cmd = [_nvcc(), *NVCC_FLAGS, *extra, "-I", str(REPO / "include"), "-c", str(src), "-o", str(obj)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed on {src.name}:\n{r.stdout}\n{r.stderr}")
    return obj, r.stderr


def build(force: bool = False, verbose: bool = False) -> Path:
    obj_dir, lib_path, extra = OBJ_DIR, LIB_PATH, ()
    obj_dir.mkdir(parents=True, exist_ok=True)
    LIB_DIR.mkdir(parents=True, exist_ok=True)
    srcs = _sources()
    hdr_mtime = _headers_mtime()
    logs = []
    with cf.ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        results = list(ex.map(lambda s: _compile(s, force, hdr_mtime, obj_dir, extra), srcs))
    objs = [o for o, _ in results]
    logs = [log for _, log in results if log]
    if verbose:
        for log in logs:
            print(log)
    (REPO / "build" / "ptxas.log").write_text("\n".join(logs))
    newest_obj = max(o.stat().st_mtime for o in objs)
    if force or not lib_path.exists() or lib_path.stat().st_mtime < newest_obj:
        # Export only the C ABI: the version script keeps b200_* global and makes every other
        # symbol local.
        vs = obj_dir / "exports.map"
        vs.write_text("{ global: b200_*; local: *; };\n")
        cmd = [_nvcc(), "-shared", "-o", str(lib_path), *map(str, objs),
               "-Xlinker", f"--version-script={vs}", "-lcudart_static", "-ldl", "-lpthread", "-lrt"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return lib_path


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="-v" in sys.argv or "--verbose" in sys.argv)
    print(path)
