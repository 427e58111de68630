"""Builds ``libtriton_b200.so`` (sm_100a only) in-tree with nvcc.

Usage: ``python -m triton_b200.build [--force] [--verbose]``. Each ``csrc/*.cu`` is compiled
to an object file in ``csrc/build/`` (in parallel), then linked into
``triton_b200/libtriton_b200.so``. nvcc cross-compiles, so no GPU is needed to build.
"""
from __future__ import annotations

import concurrent.futures
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
OBJ_DIR = CSRC / "build"
LIB_PATH = PKG_DIR / "libtriton_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr",
    "-Xcompiler", "-fPIC",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; the CUDA toolkit is required to build triton_b200")
    return exe


def _newest_header_mtime() -> float:
    hdrs = list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + [PKG_DIR.parent / "include" / "triton_b200.h"]
    return max(h.stat().st_mtime for h in hdrs if h.exists())


def _compile_one(src: Path, verbose: bool) -> str:
    obj = OBJ_DIR / (src.stem + ".o")
    cmd = [_nvcc(), *NVCC_FLAGS, "-c", str(src), "-o", str(obj)]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{r.stdout}\n{r.stderr}")
    return f"== {src.name}\n{r.stderr}" if verbose else ""


def build(force: bool = False, verbose: bool = False) -> Path:
    sources = sorted(CSRC.glob("*.cu"))
    if not sources:
        raise RuntimeError(f"no CUDA sources under {CSRC}")
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    hdr_m = _newest_header_mtime()
    todo = []
    for s in sources:
        obj = OBJ_DIR / (s.stem + ".o")
        if force or not obj.exists() or obj.stat().st_mtime < max(s.stat().st_mtime, hdr_m):
            todo.append(s)
    logs = []
    if todo:
        with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(todo))) as ex:
            logs = list(ex.map(lambda s: _compile_one(s, verbose), todo))
    objs = [OBJ_DIR / (s.stem + ".o") for s in sources]
    stale = [o for o in OBJ_DIR.glob("*.o") if o not in objs]
    for o in stale:
        o.unlink()
    if todo or not LIB_PATH.exists():
        cmd = [_nvcc(), "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", str(LIB_PATH),
               *map(str, objs), "-lcudart_static", "-ldl", "-lrt", "-lpthread"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    if verbose:
        print("\n".join(l for l in logs if l))
    return LIB_PATH


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path)
