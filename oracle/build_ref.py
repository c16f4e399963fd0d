"""Test infrastructure: build recipe for ``oracle/_ref`` (not part of the product library).

Compiles the reference's own CPU evaluator -- class ``MACE`` with its spline, polynomial,
MLP and ZBL helpers -- from the sources where they lie in the reference checkout, together
with three shims that stand in for its un-vendored submodules:

* ``ref_shims/external/cblas-prototypes/cblas.h`` + ``cblas_naive.c`` (four BLAS routines),
* ``ref_shims/include/sphericart.hpp`` (restatement of sphericart's real harmonics),
* nlohmann/json 3.11.3, found inside the ``cudnn_frontend`` wheel of this image,

and a C wrapper of our own (``ref_shims/ref_capi.cpp``) for ctypes. No reference source is
copied; outputs go only to ``oracle/_ref/``:

* ``libref_parity.so``  -O2, no fast-math, plain-loop BLAS: the deterministic parity oracle.
* ``libref_timed.so``   -O3 -ffast-math (the reference's own flags, libsymmetrix/CMakeLists.txt:51-53,
  except that ``-march=native`` is replaced by ``-march=x86-64-v3`` because the binary is built
  on one machine and timed on another): the CPU baseline.

* ``libref_timed_openblas.so``  the timed build linked against the OpenBLAS that ships inside the image's
  ``opencv_python_headless`` wheel (plain ``cblas_*`` symbols) instead of the plain-loop BLAS, when that library is
  found: the closer stand-in for how the reference is normally deployed. It resolves the library by absolute path, so
  it loads only on machines with the same image.

Usage: ``python oracle/build_ref.py [--reference DIR] [--force]``. Does nothing (returns
False) when the reference checkout is absent.
"""
from __future__ import annotations

import argparse
import os
import subprocess
import sys
import sysconfig
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_ref"
SHIMS = HERE / "ref_shims"
REF_SOURCES = [
    "mace.cpp", "cubic_spline.cpp", "cubic_spline_set.cpp", "multilayer_perceptron.cpp",
    "multivariate_polynomial.cpp", "zbl.cpp", "tools.cpp", "spherical_harmonic.cpp",
]


def _find_json_include() -> Path | None:
    """Directory such that ``#include "nlohmann/json.hpp"`` resolves."""
    candidates = []
    purelib = Path(sysconfig.get_paths()["purelib"])
    candidates.append(purelib / "include" / "cudnn_frontend" / "thirdparty")
    for extra in sys.path:
        if extra:
            candidates.append(Path(extra) / "include" / "cudnn_frontend" / "thirdparty")
    candidates.append(Path("/usr/include"))
    for c in candidates:
        if (c / "nlohmann" / "json.hpp").is_file():
            return c
    return None


def _find_openblas() -> Path | None:
    """An OpenBLAS shared library that exports the plain cblas_* symbols (inside the opencv wheel of this image)."""
    purelib = Path(sysconfig.get_paths()["purelib"])
    hits = sorted((purelib / "opencv_python_headless.libs").glob("libopenblas*.so*"))
    return hits[0] if hits else None


def _default_reference() -> Path:
    """The reference checkout: $SYMMETRIX_REFERENCE, else a `reference` folder beside the repository."""
    env = os.environ.get("SYMMETRIX_REFERENCE")
    return Path(env) if env else HERE.parent.parent / "reference"


def build(reference: str | os.PathLike | None = None, force: bool = False, verbose: bool = True) -> bool:
    ref = Path(reference) if reference else _default_reference()
    src_dir = ref / "libsymmetrix" / "source"
    if not src_dir.is_dir():
        if verbose:
            print(f"[oracle/_ref] reference checkout not found at {ref}; keeping prebuilt files")
        return False
    json_inc = _find_json_include()
    if json_inc is None:
        raise RuntimeError("nlohmann/json.hpp not found; cannot build oracle/_ref")
    OUT.mkdir(exist_ok=True)
    sources = [str(src_dir / s) for s in REF_SOURCES] + [str(SHIMS / "ref_capi.cpp")]
    common = [
        "-std=c++20", "-fPIC", "-shared", "-w",
        f"-I{src_dir}", f"-I{SHIMS / 'source'}", f"-I{SHIMS / 'include'}", f"-I{SHIMS}", f"-I{json_inc}",
    ]
    variants = {
        "libref_parity.so": ["-O2"],
        "libref_timed.so": ["-O3", "-march=x86-64-v3", "-ffast-math"],
    }
    deps = [Path(s) for s in sources] + [SHIMS / "cblas_naive.c", SHIMS / "include" / "sphericart.hpp",
                                         SHIMS / "external" / "cblas-prototypes" / "cblas.h"]
    newest = max(p.stat().st_mtime for p in deps)
    for name, flags in variants.items():
        target = OUT / name
        if target.exists() and not force and target.stat().st_mtime > newest:
            continue
        blas_obj = OUT / (name + ".cblas.o")
        cflags = [f for f in flags if f != "-ffast-math"]
        subprocess.run(["gcc", "-c", "-fPIC", *cflags, f"-I{SHIMS}", str(SHIMS / "cblas_naive.c"),
                        "-o", str(blas_obj)], check=True)
        cmd = ["g++", *common, *flags, *sources, str(blas_obj), "-o", str(target)]
        if verbose:
            print("[oracle/_ref] building", name)
        subprocess.run(cmd, check=True)
        blas_obj.unlink()
    openblas = _find_openblas()
    target = OUT / "libref_timed_openblas.so"
    if openblas is not None and (force or not target.exists() or target.stat().st_mtime <= newest):
        if verbose:
            print("[oracle/_ref] building", target.name, "against", openblas.name)
        cmd = ["g++", *common, *variants["libref_timed.so"], *sources, f"-L{openblas.parent}", f"-l:{openblas.name}",
               f"-Wl,--disable-new-dtags,-rpath,{openblas.parent}", "-o", str(target)]   # DT_RPATH: also for the library's own dependencies
        subprocess.run(cmd, check=True)
    return True


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=None)
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args()
    ok = build(a.reference, a.force)
    sys.exit(0 if ok else 1)
