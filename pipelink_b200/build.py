"""Build recipe for the in-tree native libraries.

``build_all()`` compiles every ``csrc/*.cu`` into ``pipelink_b200/_native/libpipelink_b200.so``
for sm_100a with nvcc (cross-compiles on a machine without a GPU). The library is kept
in-tree so that a checkout copied to a GPU machine runs without a compile step there.
Rebuilds only when a source is newer than the library.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
NATIVE = PKG / "_native"
LIB = NATIVE / "libpipelink_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-shared",
    "--expt-relaxed-constexpr",
]


def nvcc_path() -> str:
    for cand in (os.environ.get("PLB_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found; set PLB_NVCC")


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _stale(target: Path, deps: list[Path]) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(d.stat().st_mtime > t for d in deps)


def build_all(force: bool = False, verbose: bool = False) -> Path:
    NATIVE.mkdir(exist_ok=True)
    deps = sources() + sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h")) + \
        [PKG.parent / "include" / "pipelink_b200.h"]
    if force or _stale(LIB, deps):
        cmd = [nvcc_path(), *NVCC_FLAGS]
        if verbose:
            cmd += ["-Xptxas", "-v"]
        cmd += ["-o", str(LIB), *map(str, sources())]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if verbose:
            sys.stderr.write(proc.stderr)
        if proc.returncode != 0:
            raise RuntimeError("nvcc failed:\n" + " ".join(cmd) + "\n" + proc.stdout + proc.stderr)
    return LIB


if __name__ == "__main__":
    print(build_all(force="--force" in sys.argv, verbose="-v" in sys.argv))
