"""Build libbdfp4.so in-tree with nvcc for sm_100a.

    python bitdecoding-fp4_b200/build.py [--force] [--verbose]

The library lands in ``bitdecoding-fp4_b200/lib/libbdfp4.so`` and is what
``bdfp4`` loads with ctypes. nvcc cross-compiles without a GPU.
"""

from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
LIB_DIR = ROOT / "lib"
LIB_PATH = LIB_DIR / "libbdfp4.so"
OBJ_DIR = ROOT / "build"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    # IEEE division/sqrt and no flush-to-zero: the quantizer is bit-exact by contract.
    "--fmad=true", "--prec-div=true", "--prec-sqrt=true", "--ftz=false",
]


def _nvcc() -> str:
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(found):
        raise RuntimeError("nvcc not found; libbdfp4.so cannot be built")
    return found


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _stale(target: Path, deps: list[Path]) -> bool:
    if not target.exists():
        return True
    stamp = target.stat().st_mtime
    return any(dep.stat().st_mtime > stamp for dep in deps)


def build_library(force: bool = False, verbose: bool = False) -> Path:
    """Compile every ``csrc/*.cu`` and link ``libbdfp4.so``; returns its path."""
    headers = sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h")) + [ROOT.parent / "include" / "bdfp4.h"]
    OBJ_DIR.mkdir(exist_ok=True)
    LIB_DIR.mkdir(exist_ok=True)
    nvcc = _nvcc()
    jobs = []
    for source in sources():
        obj = OBJ_DIR / (source.stem + ".o")
        if force or _stale(obj, [source, *headers]):
            cmd = [nvcc, *NVCC_FLAGS, "-c", str(source), "-o", str(obj)]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            jobs.append(cmd)

    def run(cmd):
        result = subprocess.run(cmd, capture_output=True, text=True)
        if verbose or result.returncode:
            sys.stderr.write(" ".join(cmd) + "\n" + result.stdout + result.stderr)
        if result.returncode:
            raise RuntimeError(f"nvcc failed on {cmd[-3]}")

    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as pool:
        list(pool.map(run, jobs))
    objects = [OBJ_DIR / (source.stem + ".o") for source in sources()]
    if force or jobs or _stale(LIB_PATH, objects):
        run([nvcc, "-shared", "-o", str(LIB_PATH), *map(str, objects), "-gencode",
             "arch=compute_100a,code=sm_100a", "-lcudart_static", "-ldl", "-lrt", "-lpthread"])
    return LIB_PATH


if __name__ == "__main__":
    parser = argparse.ArgumentParser()
    parser.add_argument("--force", action="store_true")
    parser.add_argument("--verbose", action="store_true")
    args = parser.parse_args()
    print(build_library(force=args.force, verbose=args.verbose))
