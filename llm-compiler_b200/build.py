"""Builds libb200serve.so (the C-ABI library of sm_100a kernels) in-tree with nvcc.

    python llm-compiler_b200/build.py [--force]

nvcc cross-compiles for sm_100a without a GPU. Objects land in csrc/_build/, the shared
library next to this file. Nothing here falls back to another backend: if nvcc is missing
the build fails.
"""

from __future__ import annotations

import concurrent.futures
import os
import shutil
import subprocess
import sys
from pathlib import Path

PACKAGE_DIR = Path(__file__).resolve().parent
CSRC = PACKAGE_DIR / "csrc"
INCLUDE = PACKAGE_DIR.parent / "include"
BUILD_DIR = CSRC / "_build"
LIBRARY = PACKAGE_DIR / "libb200serve.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-lineinfo", "-std=c++17",
    "-Xcompiler", "-fPIC",
    f"-I{INCLUDE}", f"-I{CSRC}",
]


def _nvcc() -> str:
    candidate = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(candidate):
        raise RuntimeError("nvcc not found: the sm_100a library cannot be built")
    return candidate


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _stale(target: Path, inputs: list[Path]) -> bool:
    if not target.exists():
        return True
    stamp = target.stat().st_mtime
    return any(path.stat().st_mtime > stamp for path in inputs)


def _compile(nvcc: str, source: Path, obj: Path) -> None:
    # B200_NVCC_EXTRA: extra compiler flags, e.g. -DB200_TRACE for the timeline-trace build
    extra = os.environ.get("B200_NVCC_EXTRA", "").split()
    command = [nvcc, *NVCC_FLAGS, *extra, "-c", str(source), "-o", str(obj)]
    result = subprocess.run(command, capture_output=True, text=True)
    if result.returncode != 0:
        raise RuntimeError(f"nvcc failed on {source.name}:\n{result.stdout}\n{result.stderr}")


def build(force: bool = False, verbose: bool = False) -> Path:
    nvcc = _nvcc()
    BUILD_DIR.mkdir(parents=True, exist_ok=True)
    headers = sorted(CSRC.glob("*.cuh")) + sorted(INCLUDE.glob("*.h"))
    jobs = []
    objects = []
    for source in sources():
        obj = BUILD_DIR / (source.stem + ".o")
        objects.append(obj)
        if force or _stale(obj, [source, *headers]):
            jobs.append((source, obj))
    if jobs:
        if verbose:
            print(f"[b200 build] compiling {[s.name for s, _ in jobs]}", file=sys.stderr)
        with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as pool:
            for future in [pool.submit(_compile, nvcc, s, o) for s, o in jobs]:
                future.result()
    if force or jobs or _stale(LIBRARY, objects):
        command = [nvcc, "-shared", "-o", str(LIBRARY), *map(str, objects),
                   "-gencode", "arch=compute_100a,code=sm_100a"]
        result = subprocess.run(command, capture_output=True, text=True)
        if result.returncode != 0:
            raise RuntimeError(f"link failed:\n{result.stdout}\n{result.stderr}")
    return LIBRARY


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True))
