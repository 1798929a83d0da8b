"""Build recipe for libanna_b200_kv.so (hand-written CUDA for sm_100a, no torch headers involved).

``python -m anna_b200.build`` compiles every ``csrc/*.cu`` with nvcc (cross-compiles without a GPU) and links
them into ``anna_b200/libanna_b200_kv.so`` next to this file, so the library travels with the source tree.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
BUILD_DIR = PKG_DIR / "_build"
LIB_PATH = PKG_DIR / "libanna_b200_kv.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "-Xptxas=-v",
]


def _nvcc() -> str:
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(found):
        raise RuntimeError("nvcc not found: libanna_b200_kv.so cannot be built")
    return found


def _stale(target: Path, sources: list[Path]) -> bool:
    if not target.exists():
        return True
    stamp = target.stat().st_mtime
    return any(src.stat().st_mtime > stamp for src in sources)


def build(force: bool = False, verbose: bool = False) -> Path:
    sources = sorted(CSRC.glob("*.cu"))
    headers = sorted(CSRC.glob("*.cuh")) + [PKG_DIR.parent / "include" / "anna_b200_kv.h"]
    BUILD_DIR.mkdir(exist_ok=True)
    nvcc = _nvcc()
    jobs = []
    for src in sources:
        obj = BUILD_DIR / (src.stem + ".o")
        if force or _stale(obj, [src, *headers]):
            jobs.append((src, obj))

    def compile_one(job: tuple[Path, Path]) -> str:
        src, obj = job
        cmd = [nvcc, *NVCC_FLAGS, "-c", str(src), "-o", str(obj)]
        done = subprocess.run(cmd, capture_output=True, text=True)
        if done.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src.name}:\n{done.stderr}")
        return done.stderr

    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as pool:
        logs = list(pool.map(compile_one, jobs))
    if verbose:
        for log in logs:
            sys.stderr.write(log)
    objects = [BUILD_DIR / (src.stem + ".o") for src in sources]
    if force or jobs or _stale(LIB_PATH, objects):
        cmd = [nvcc, "-shared", "-o", str(LIB_PATH), *map(str, objects), "-cudart", "shared"]
        done = subprocess.run(cmd, capture_output=True, text=True)
        if done.returncode != 0:
            raise RuntimeError(f"link failed:\n{done.stderr}")
    return LIB_PATH


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(path)
