"""Builds eke_hive_b200/libhive_b200.so from csrc/*.cu with nvcc for sm_100a (cross-compiles without a GPU).

    python eke_hive_b200/build.py [--force] [--verbose] [--bounds]      (run as a script: importing the package needs the built library)

Objects are rebuilt only when their source or a header is newer; translation units compile in parallel.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
OUT = HERE / "libhive_b200.so"
OBJ = HERE / "build"

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC,-fvisibility=hidden",
         "--use_fast_math=false", "-ccbin", "/usr/bin/g++" if Path("/usr/bin/g++").exists() else "g++"]
FLAGS = [f for f in FLAGS if f != "--use_fast_math=false"]


def _newest_header() -> float:
    hs = list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + list(CSRC.glob("*.hpp")) + [HERE.parent / "include" / "hive_b200.h"]
    return max(h.stat().st_mtime for h in hs)


def build(force: bool = False, verbose: bool = False, bounds: bool = False) -> Path:
    """bounds=True: the range-checked debug library (every kernel compiled with -DHB_BOUNDS) as libhive_b200_bounds.so, objects in
    build_bounds/; load it with HIVE_B200_LIB=<path> (see _lib.py)."""
    global OUT, OBJ, FLAGS
    if bounds:
        OUT, OBJ = HERE / "libhive_b200_bounds.so", HERE / "build_bounds"
        if "-DHB_BOUNDS" not in FLAGS:
            FLAGS = FLAGS + ["-DHB_BOUNDS"]
    OBJ.mkdir(exist_ok=True)
    srcs = sorted(CSRC.glob("*.cu"))
    hdr = _newest_header()
    jobs = []
    for s in srcs:
        o = OBJ / (s.stem + ".o")
        if force or not o.exists() or o.stat().st_mtime < max(s.stat().st_mtime, hdr):
            jobs.append((s, o))

    def compile_one(so):
        s, o = so
        cmd = [NVCC, *FLAGS, "-c", str(s), "-o", str(o)] + (["-Xptxas", "-v"] if verbose else [])
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {s.name}:\n{r.stdout}\n{r.stderr}")
        if verbose:
            print(r.stderr)
        elif "warning" in r.stderr:
            print(r.stderr, file=sys.stderr)

    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        list(ex.map(compile_one, jobs))
    objs = [OBJ / (s.stem + ".o") for s in srcs]
    if jobs or not OUT.exists() or OUT.stat().st_mtime < max(o.stat().st_mtime for o in objs):
        cmd = [NVCC, "-shared", "-o", str(OUT), *map(str, objs), "-gencode", "arch=compute_100a,code=sm_100a", "-lcudart",
               "-ccbin", "/usr/bin/g++" if Path("/usr/bin/g++").exists() else "g++"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return OUT


if __name__ == "__main__":
    p = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv, bounds="--bounds" in sys.argv)
    print(p)
