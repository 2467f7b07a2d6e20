"""Builds the native library (sm_100a only) in-tree with nvcc.

Every ``csrc/*.cu`` file is compiled to an object and linked into
``easy_to_hard_b200/ops/_native/libe2h_b200.so``; the Python side loads it with ctypes
(see ``_lib.py``). nvcc cross-compiles without a GPU, so this also runs on a CPU-only box.

    python -m easy_to_hard_b200.ops.build [--force] [--verbose]
"""
from __future__ import annotations

import argparse
import concurrent.futures as cf
import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
OUT_DIR = HERE / "_native"
LIB_NAME = "libe2h_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found; the native library needs CUDA 12.9+")
    return cand


def _digest(paths) -> str:
    h = hashlib.sha256()
    for p in sorted(paths):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def lib_path() -> Path:
    return OUT_DIR / LIB_NAME


def sources():
    return sorted(CSRC.glob("*.cu"))


def needs_build() -> bool:
    stamp = OUT_DIR / "build.stamp"
    if not lib_path().exists() or not stamp.exists():
        return True
    return stamp.read_text().strip() != _digest(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")))


def build_phase_clock() -> Path:
    """A second library, ``libe2h_b200_phase.so``, with the kernels' phase stamps compiled in
    (``-DE2H_PHASE_CLOCK``, see ``ptx.cuh``); only the GEMM sources that carry stamps are
    built. Used by ``bench/gemm_phase_bench.py``; the regular library is not touched."""
    OUT_DIR.mkdir(parents=True, exist_ok=True)
    out = OUT_DIR / "libe2h_b200_phase.so"
    cmd = [_nvcc(), *NVCC_FLAGS, "-DE2H_PHASE_CLOCK", "-shared", "-I", str(CSRC),
           str(CSRC / "gemm_umma.cu"), "-o", str(out)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed:\n{r.stdout}{r.stderr}")
    return out


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile and link; returns the path of the shared library. Processes that start together
    (one per GPU under torchrun) take a file lock, so one of them builds and the others find the
    finished library."""
    if not force and not needs_build():
        return lib_path()
    OUT_DIR.mkdir(parents=True, exist_ok=True)
    import fcntl
    with open(OUT_DIR / "build.lock", "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if not force and not needs_build():     # another process built it meanwhile
                return lib_path()
            return _build_locked(verbose)
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)


def _build_locked(verbose: bool) -> Path:
    nvcc = _nvcc()
    srcs = sources()
    extra = ["-Xptxas", "-v"] if verbose else []

    def compile_one(src: Path) -> Path:
        obj = OUT_DIR / (src.stem + ".o")
        cmd = [nvcc, *NVCC_FLAGS, *extra, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if verbose or r.returncode != 0:
            sys.stderr.write(f"--- {src.name}\n{r.stdout}{r.stderr}\n")
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src.name}")
        return obj

    with cf.ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        objs = list(ex.map(compile_one, srcs))
    tmp = OUT_DIR / (LIB_NAME + ".tmp")
    cmd = [nvcc, "-shared", "-o", str(tmp), *[str(o) for o in objs],
           "-gencode", "arch=compute_100a,code=sm_100a"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}{r.stderr}")
    os.replace(tmp, lib_path())
    (OUT_DIR / "build.stamp").write_text(
        _digest(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh"))))
    return lib_path()


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--phase-clock", action="store_true",
                    help="also build the library with the kernels' phase stamps compiled in")
    a = ap.parse_args()
    print(build(force=a.force, verbose=a.verbose))
    if a.phase_clock:
        print(build_phase_clock())
