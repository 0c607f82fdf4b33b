"""Compile the CUDA sources into the in-tree C-ABI shared library (sm_100a only)."""

from __future__ import annotations

import os
import shutil
import subprocess
from pathlib import Path

PACKAGE_DIR = Path(__file__).resolve().parent
CSRC_DIR = PACKAGE_DIR / "csrc"
LIB_DIR = PACKAGE_DIR / "_lib"
LIB_PATH = LIB_DIR / "libternel_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-shared",
]


CHECKED_LIB_PATH = LIB_DIR / "libternel_b200_checked.so"
# The checked build: every global store tests its index first and records a violation instead of writing
# (the record is one device array shared by all source files, hence relocatable device code).
CHECKED_FLAGS = ["-DTQ1_BOUNDS_CHECK", "-rdc=true"]


def sources() -> list[Path]:
    return sorted(CSRC_DIR.glob("*.cu"))


def _nvcc() -> str:
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(found).exists():
        raise RuntimeError("nvcc not found; the library can only be built with the CUDA toolkit")
    return found


def is_stale(target: Path = LIB_PATH) -> bool:
    if not target.exists():
        return True
    built = target.stat().st_mtime
    deps = sources() + list(CSRC_DIR.glob("*.cuh")) + [PACKAGE_DIR.parent / "include" / "ternel_b200.h"]
    return any(p.stat().st_mtime > built for p in deps)


def build_checked(force: bool = False) -> Path:
    """Build ``_lib/libternel_b200_checked.so``, the bounds-checking variant used by tests/test_gpu_bounds.py."""
    return build(force=force, target=CHECKED_LIB_PATH, extra=CHECKED_FLAGS)


def build(force: bool = False, verbose: bool = False, target: Path = LIB_PATH, extra: "list[str] | None" = None) -> Path:
    """Build ``_lib/libternel_b200.so`` (or ``target``) when missing or older than a source file."""
    if not force and not is_stale(target):
        return target
    LIB_DIR.mkdir(exist_ok=True)
    tmp = LIB_DIR / f".{target.stem}.{os.getpid()}.so"
    cmd = [_nvcc(), *NVCC_FLAGS, *(extra or []), *( ["-Xptxas", "-v"] if verbose else [] ),
           "-o", str(tmp), *map(str, sources())]
    done = subprocess.run(cmd, capture_output=True, text=True)
    if done.returncode != 0:
        tmp.unlink(missing_ok=True)
        raise RuntimeError(f"nvcc failed:\n{done.stdout}\n{done.stderr}")
    if verbose:
        print(done.stderr)
    os.replace(tmp, target)
    return target


if __name__ == "__main__":
    print(build(force=True, verbose=True))
