"""Builds the native library in-tree: every `csrc/*.cu` is compiled for sm_100a with nvcc and linked into
`cuteafd_b200/_native/libcuteafd_b200.so`.  No GPU is needed (nvcc cross-compiles); objects are rebuilt
only when their source or a header is newer.  `python -m cuteafd_b200.build [--force] [--verbose]`.

The reference builds its native library with CMake (native/CMakeLists.txt); here one small Python driver is
enough because there are no AOT-exported objects to stitch in.
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
OUT = ROOT / "_native"
LIB = OUT / "libcuteafd_b200.so"

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "--use_fast_math=false", "-Xptxas", "-v"]


def nvcc_path() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found")


def _stale(obj: Path, src: Path, headers: list[Path]) -> bool:
    if not obj.exists():
        return True
    t = obj.stat().st_mtime
    return any(p.stat().st_mtime > t for p in [src, *headers])


def build(force: bool = False, verbose: bool = False) -> Path:
    OUT.mkdir(exist_ok=True)
    nvcc = nvcc_path()
    headers = sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h"))
    sources = sorted(CSRC.glob("*.cu"))
    flags = [f for f in NVCC_FLAGS if f != "--use_fast_math=false"]
    jobs = []
    for src in sources:
        obj = OUT / (src.stem + ".o")
        if force or _stale(obj, src, headers):
            jobs.append((src, obj))

    def compile_one(job):
        src, obj = job
        cmd = [nvcc, *flags, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
        r = subprocess.run(cmd, capture_output=True, text=True)
        return src, r

    if jobs:
        with ThreadPoolExecutor(max_workers=min(len(jobs), os.cpu_count() or 4)) as ex:
            for src, r in ex.map(compile_one, jobs):
                if verbose or r.returncode != 0:
                    sys.stderr.write(f"--- {src.name}\n{r.stdout}{r.stderr}\n")
                if r.returncode != 0:
                    raise RuntimeError(f"nvcc failed on {src.name}")
    objs = [OUT / (s.stem + ".o") for s in sources]
    if force or jobs or not LIB.exists():
        cmd = [nvcc, "-shared", "--cudart", "shared", "-o", str(LIB), *map(str, objs)]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("link failed")
    return LIB


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args()
    print(build(a.force, a.verbose))


if __name__ == "__main__":
    main()
