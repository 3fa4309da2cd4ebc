"""In-tree build of the native library: every ``.cu`` under ``csrc/`` -> ``lset_b200/_C.so``.

The kernels are plain CUDA C++ with ``extern "C"`` launchers (no torch headers), compiled for
``sm_100a`` only and loaded with ``ctypes``; objects are rebuilt when a source or a header is newer.

Usage:  python -m lset_b200.csrc.build [--force] [--verbose]
"""
from __future__ import annotations

import concurrent.futures as cf
import contextlib
import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

CSRC = Path(__file__).resolve().parent
PKG = CSRC.parent
OBJ_DIR = CSRC / "_build"
LIB_PATH = PKG / "_C.so"
MANIFEST_PATH = PKG / "_C.so.manifest"   # digest of the sources the library was built from
LOCK_PATH = PKG / "_C.so.lock"

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


def source_digest() -> str:
    """SHA-256 over every source and header (path and content) and the compiler flags: the
    library is current iff the digest stored next to it equals this one. File times are not used,
    they do not survive a copy of the tree to another machine."""
    h = hashlib.sha256(" ".join(NVCC_FLAGS).encode())
    files = sorted(p for p in CSRC.rglob("*") if p.suffix in (".cu", ".cuh", ".h")
                   and "_build" not in p.parts)
    for f in files:
        h.update(str(f.relative_to(CSRC)).encode())
        h.update(f.read_bytes())
    return h.hexdigest()


def is_current() -> bool:
    try:
        return LIB_PATH.exists() and MANIFEST_PATH.read_text().strip() == source_digest()
    except OSError:
        return False


@contextlib.contextmanager
def build_lock():
    """Exclusive lock for builders on one machine (the ranks of a job start together)."""
    import fcntl

    with open(LOCK_PATH, "w") as fh:
        fcntl.flock(fh, fcntl.LOCK_EX)
        try:
            yield
        finally:
            fcntl.flock(fh, fcntl.LOCK_UN)


def ensure_built(verbose: bool = False) -> Path:
    """Build the library unless the one in the tree was made from the present sources. Safe to
    call from several processes at once: one builds, the others wait and find it current."""
    if is_current():
        return LIB_PATH
    with build_lock():
        if not is_current():
            build(verbose=verbose)
    return LIB_PATH


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
        stale = not obj.exists() or obj.stat().st_mtime < max(src.stat().st_mtime, hdr_m)
        if force or ptxas_v or stale or not MANIFEST_PATH.exists():
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
    digest = source_digest()
    if need_link or not MANIFEST_PATH.exists() or MANIFEST_PATH.read_text().strip() != digest:
        # link under a temporary name and move it into place: a process that loads the library
        # meanwhile sees either the old file or the complete new one
        tmp = LIB_PATH.with_name(f"_C.so.tmp{os.getpid()}")
        cmd = [_nvcc(), "-shared", "-o", str(tmp), *map(str, objs),
               "-gencode", "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC"]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError(f"link failed:\n{proc.stdout}\n{proc.stderr}")
        os.replace(tmp, LIB_PATH)
        MANIFEST_PATH.write_text(digest + "\n")
    return LIB_PATH


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv,
                 ptxas_v="--ptxas-v" in sys.argv)
    print(path)
