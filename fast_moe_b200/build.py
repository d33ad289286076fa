"""In-tree build of libfmoe_b200.so (sm_100a only) with nvcc.

Usage: ``python -m fast_moe_b200.build [--force] [--verbose]``. The library lands in
``fast_moe_b200/lib/`` next to the sources so that it travels with a copy of the tree.
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
LIB_DIR = PKG_DIR / "lib"
LIB_PATH = LIB_DIR / "libfmoe_b200.so"
# (source, object stem, extra flags). The grouped GEMM, by far the longest compile, is built as
# four objects in parallel: host code and one set of kernel instantiations per operand size.
UNITS = [("api.cu", "api", []), ("routing.cu", "routing", []), ("combine.cu", "combine", []), ("quant.cu", "quant", []),
         ("expert_parallel.cu", "expert_parallel", []), ("sg_moe.cu", "sg_moe", []),
         ("backward.cu", "backward", [])]
UNITS += [("grouped_gemm.cu", f"grouped_gemm_p{part}", [f"-DFMOE_GEMM_PART={part}"]) for part in range(4)]
SOURCES = sorted({u[0] for u in UNITS})
HEADERS = [CSRC / "common.cuh", CSRC / "ptx.cuh", PKG_DIR.parent / "include" / "fmoe_b200.h"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found: the CUDA library cannot be built")
    return cand


STAMP_PATH = LIB_DIR / "build_stamp.txt"


def source_digest() -> str:
    """SHA-256 over the CUDA sources, the headers and the compiler flags: what the library on
    disk must have been built from. Independent of file times, which a copy of the tree may not
    preserve."""
    import hashlib

    h = hashlib.sha256()
    for path in [CSRC / s for s in SOURCES] + HEADERS:
        h.update(path.name.encode())
        h.update(path.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def library_is_current() -> bool:
    """True when libfmoe_b200.so exists and its stamp matches the sources next to it."""
    try:
        return LIB_PATH.exists() and STAMP_PATH.read_text().strip() == source_digest()
    except OSError:
        return False


def _stale(target: Path, deps) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(Path(d).stat().st_mtime > t for d in deps)


def build_library(force: bool = False, verbose: bool = False) -> Path:
    """Compiles the CUDA sources when they are newer than the library. Returns the .so path.
    Several processes may call this at once (one per GPU under torchrun): a file lock lets one of
    them build while the others wait and then find the library current."""
    import fcntl

    LIB_DIR.mkdir(exist_ok=True)
    with open(LIB_DIR / ".build.lock", "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if not force and library_is_current():
                return LIB_PATH
            return _build_locked(force, verbose)
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)


def _build_locked(force: bool, verbose: bool) -> Path:
    LIB_DIR.mkdir(exist_ok=True)
    obj_dir = LIB_DIR / "obj"
    obj_dir.mkdir(exist_ok=True)
    nvcc = _nvcc()
    if LIB_PATH.exists() and STAMP_PATH.exists() and not library_is_current():
        force = True      # sources changed under a library whose file times may not show it
    jobs = []
    for src, stem, extra in UNITS:
        s = CSRC / src
        o = obj_dir / (stem + ".o")
        if force or _stale(o, [s, *HEADERS]):
            cmd = [nvcc, *NVCC_FLAGS, *extra, "-c", str(s), "-o", str(o)]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            jobs.append(cmd)

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        return cmd, r

    with ThreadPoolExecutor(max_workers=max(1, min(len(jobs), os.cpu_count() or 1))) as ex:
        for cmd, r in ex.map(run, jobs):
            if verbose or r.returncode != 0:
                sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
            if r.returncode != 0:
                raise RuntimeError(f"nvcc failed on {cmd[-3]} -> {cmd[-1]}")
    objs = [str(obj_dir / (stem + ".o")) for _, stem, _ in UNITS]
    if force or jobs or _stale(LIB_PATH, objs):
        cmd = [nvcc, "-shared", "-o", str(LIB_PATH), *objs, "-gencode", "arch=compute_100a,code=sm_100a"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("linking libfmoe_b200.so failed")
    STAMP_PATH.write_text(source_digest() + "\n")
    return LIB_PATH


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args()
    print(build_library(force=a.force, verbose=a.verbose))
