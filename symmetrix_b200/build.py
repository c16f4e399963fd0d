"""Builds ``symmetrix_b200/libsymmetrix_b200.so`` in-tree with nvcc for sm_100a.

``python -m symmetrix_b200.build [--force] [--verbose]``. The library is the whole product:
CUDA kernels plus the extern "C" layer declared in ``include/symmetrix_b200.h``.
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB = PKG / "libsymmetrix_b200.so"
BUILD = PKG / "build"
SOURCES = [CSRC / "evaluator_f64.cu", CSRC / "evaluator_f32.cu", CSRC / "capi.cu", CSRC / "noalloc.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-Xcudafe", "--diag_suppress=177",
]


def find_nvcc() -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(nvcc).exists():
        raise RuntimeError("nvcc not found; the CUDA library cannot be built")
    return nvcc


def needs_build() -> bool:
    if not LIB.exists():
        return True
    newest = max(p.stat().st_mtime for p in _inputs())
    return LIB.stat().st_mtime < newest


def _inputs() -> list[Path]:
    """Every file a translation unit may include (generated code in sub-folders too)."""
    return [p for p in CSRC.rglob("*") if p.is_file()] + [PKG.parent / "include" / "symmetrix_b200.h"]


def _compile(nvcc: str, src: Path, obj: Path, verbose: bool) -> str:
    # SMX_NVCC_FLAGS: extra compiler flags (e.g. -D switches of the kernels' tuning macros) for measurement builds
    cmd = [nvcc, *NVCC_FLAGS, *os.environ.get("SMX_NVCC_FLAGS", "").split(), "-c", str(src), "-o", str(obj)]
    if verbose:
        cmd += ["-Xptxas", "-v"]
        print(" ".join(cmd), flush=True)
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed on {src.name}:\n{r.stdout}\n{r.stderr}")
    return r.stdout + r.stderr


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile the translation units in parallel (one nvcc process each) and link them into the shared library.

    An object file is reused when it is newer than every input, so editing one .cu file recompiles only that file;
    a header change recompiles everything.
    """
    if not force and not needs_build():
        return LIB
    nvcc = find_nvcc()
    BUILD.mkdir(exist_ok=True)
    headers = max(p.stat().st_mtime for p in _inputs() if p.suffix != ".cu")
    jobs = []
    for src in SOURCES:
        obj = BUILD / (src.stem + ".o")
        if force or not obj.exists() or obj.stat().st_mtime < max(headers, src.stat().st_mtime):
            jobs.append((src, obj))
    from concurrent.futures import ThreadPoolExecutor

    with ThreadPoolExecutor(max_workers=max(1, len(jobs))) as pool:
        for out in pool.map(lambda j: _compile(nvcc, j[0], j[1], verbose), jobs):
            if verbose and out:
                print(out)
    cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-Xcompiler", "-fPIC"]
    cmd += [str(BUILD / (s.stem + ".o")) for s in SOURCES] + ["-o", str(LIB)]
    if verbose:
        print(" ".join(cmd))
    subprocess.run(cmd, check=True)
    return LIB


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args()
    print(build(a.force, a.verbose))
