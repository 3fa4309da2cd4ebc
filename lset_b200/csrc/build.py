"""In-tree build of the native library: every ``.cu`` under ``csrc/`` -> ``lset_b200/_C.so``.

The kernels are plain CUDA C++ with ``extern "C"`` launchers (no torch headers), compiled for
``sm_100a`` only and loaded with ``ctypes``; objects are rebuilt when a source or a header is newer.

Usage:  python -m lset_b200.csrc.build [--force] [--verbose]
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import shutil
import subprocess
import sys
from pathlib import Path

CSRC = Path(__file__).resolve().parent
PKG = CSRC.parent
OBJ_DIR = CSRC / "_build"
LIB_PATH = PKG / "_C.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "--expt-relaxed-constexpr", "--expt-extended-lambda",
    "-Xcompiler", "-fPIC",
]


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found; the native library cannot be built")
    return cand


def sources() -> list[Path]:
    return sorted(p for p in CSRC.rglob("*.cu") if "_build" not in p.parts)


def _headers_mtime() -> float:
    hs = [p.stat().st_mtime for p in CSRC.rglob("*") if p.suffix in (".cuh", ".h")]
    return max(hs) if hs else 0.0


def _compile_one(src: Path, obj: Path, verbose: bool, ptxas_v: bool) -> tuple[Path, str]:
    cmd = [_nvcc(), *NVCC_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
    if ptxas_v:
        cmd += ["-Xptxas", "-v"]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src}:\n{proc.stdout}\n{proc.stderr}")
    return src, proc.stderr if (verbose or ptxas_v) else ""


def build(force: bool = False, verbose: bool = False, ptxas_v: bool = False) -> Path:
    """Compile what is out of date and link ``_C.so``. Returns the library path."""
    OBJ_DIR.mkdir(exist_ok=True)
    hdr_m = _headers_mtime()
    todo, objs = [], []
    for src in sources():
        rel = src.relative_to(CSRC)
        obj = OBJ_DIR / ("_".join(rel.with_suffix("").parts) + ".o")
        objs.append(obj)
        if force or ptxas_v or not obj.exists() or obj.stat().st_mtime < max(src.stat().st_mtime, hdr_m):
            todo.append((src, obj))
    if todo:
        workers = max(1, min(len(todo), os.cpu_count() or 4))
        with cf.ThreadPoolExecutor(workers) as ex:
            for src, log in ex.map(lambda so: _compile_one(so[0], so[1], verbose, ptxas_v), todo):
                if verbose or ptxas_v:
                    print(f"[build] {src.relative_to(CSRC)}\n{log}", file=sys.stderr)
    need_link = bool(todo) or not LIB_PATH.exists() or any(
        o.stat().st_mtime > LIB_PATH.stat().st_mtime for o in objs
    )
    if need_link:
        cmd = [_nvcc(), "-shared", "-o", str(LIB_PATH), *map(str, objs),
               "-gencode", "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC"]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError(f"link failed:\n{proc.stdout}\n{proc.stderr}")
    return LIB_PATH


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv,
                 ptxas_v="--ptxas-v" in sys.argv)
    print(path)
