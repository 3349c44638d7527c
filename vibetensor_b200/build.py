"""Builds libvbt_b200.so in-tree with nvcc for sm_100a (cross-compiles without a GPU).

    python -m vibetensor_b200.build [--force] [--verbose] [--release]

--release leaves -lineinfo out (a smaller library without the source-line tables profilers use);
objects of the two kinds are cached side by side.

One nvcc process per translation unit, run in parallel; objects are cached under
csrc/_obj and rebuilt when the source or any header is newer.
"""
from __future__ import annotations

import argparse
import concurrent.futures as cf
import glob
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(CSRC, "_obj")
LIB_DIR = os.path.join(HERE, "lib")
LIB = os.path.join(LIB_DIR, "libvbt_b200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++20",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "--default-stream", "legacy",
]


def _nvcc() -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found; libvbt_b200.so cannot be built")
    return nvcc


def _stale(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False, release: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    flags = NVCC_FLAGS + ([] if release else ["-lineinfo"])
    suffix = ".rel.o" if release else ".o"
    os.makedirs(LIB_DIR, exist_ok=True)
    srcs = sorted(glob.glob(os.path.join(CSRC, "*.cu")))
    hdrs = sorted(glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(CSRC, "*.h")) +
                  glob.glob(os.path.join(HERE, "..", "include", "*.h")))
    nvcc = _nvcc()
    jobs = []
    objs = []
    for s in srcs:
        o = os.path.join(OBJ, os.path.basename(s)[:-3] + suffix)
        objs.append(o)
        if force or _stale(o, [s] + hdrs):
            cmd = [nvcc] + flags + (["-Xptxas", "-v"] if verbose else []) + ["-c", s, "-o", o]
            jobs.append(cmd)

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        return cmd, r

    if jobs:
        with cf.ThreadPoolExecutor(max_workers=min(len(jobs), os.cpu_count() or 4)) as ex:
            for cmd, r in ex.map(run, jobs):
                if verbose or r.returncode != 0:
                    sys.stderr.write(" ".join(cmd[-4:]) + "\n" + r.stdout + r.stderr + "\n")
                if r.returncode != 0:
                    raise RuntimeError("nvcc failed for " + cmd[-3])
    marker = os.path.join(OBJ, "linked_release" if release else "linked_lineinfo")
    if force or jobs or _stale(LIB, objs) or not os.path.exists(marker):
        cmd = [nvcc, "-shared", "-o", LIB] + objs + ["-gencode", "arch=compute_100a,code=sm_100a",
                                                      "-cudart", "static"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("link failed:\n" + r.stdout + r.stderr)
        for m in ("linked_release", "linked_lineinfo"):
            if os.path.exists(os.path.join(OBJ, m)):
                os.remove(os.path.join(OBJ, m))
        open(marker, "w").close()
    return LIB


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--release", action="store_true")
    a = ap.parse_args()
    print(build(a.force, a.verbose, a.release))
