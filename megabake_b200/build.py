"""Build libmegabake_b200.so in-tree with nvcc for sm_100a (cross-compiles without a GPU).

    python -m megabake_b200.build [--force]
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PACKAGE = Path(__file__).resolve().parent
CSRC = PACKAGE / "csrc"
LIBRARY = PACKAGE / "libmegabake_b200.so"
SOURCES = [CSRC / "api.cu", CSRC / "reference_mma_baseline.cu"]


def headers() -> list[Path]:
    """Every header the library is built from: a new .cuh cannot be forgotten."""
    return sorted(CSRC.glob("*.cuh")) + sorted((PACKAGE.parent / "include").glob("*.h"))


NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-shared", "-Xcompiler", "-fPIC", "-Xptxas", "-v",
]


def find_nvcc() -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found; the CUDA toolkit is required to build megabake_b200")
    return nvcc


def is_stale() -> bool:
    if not LIBRARY.exists():
        return True
    built = LIBRARY.stat().st_mtime
    return any(path.stat().st_mtime > built for path in SOURCES + headers())


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile the CUDA library if it is missing or older than its sources."""
    if not force and not is_stale():
        return LIBRARY
    command = [find_nvcc(), *NVCC_FLAGS, "-o", str(LIBRARY), *map(str, SOURCES), "-lcudart"]
    result = subprocess.run(command, capture_output=True, text=True)
    if verbose or result.returncode:
        sys.stderr.write(result.stdout + result.stderr)
    if result.returncode:
        raise RuntimeError(f"nvcc failed with exit code {result.returncode}")
    (PACKAGE / "build_log.txt").write_text(result.stdout + result.stderr)
    return LIBRARY


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True))
