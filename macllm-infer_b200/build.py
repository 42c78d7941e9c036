"""Build libmacllm_b200.so (sm_100a) in-tree with nvcc.

Usage: python macllm-infer_b200/build.py [--force]
Objects are cached under macllm-infer_b200/build/ and rebuilt when a source or header is newer.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
BUILD = HERE / "build"
LIB = HERE / "libmacllm_b200.so"

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
COMMON = [
    "-std=c++17", "-O3", "-lineinfo",
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-Xcompiler", "-fPIC,-fopenmp,-Wall,-Wno-unknown-pragmas",
    "-I", str(HERE.parent / "include"),
]


def _newest_header() -> float:
    hs = list(CSRC.glob("*.h")) + list(CSRC.glob("*.cuh")) + list((HERE.parent / "include").glob("*.h"))
    return max(p.stat().st_mtime for p in hs)


def build(force: bool = False, verbose: bool = False) -> Path:
    BUILD.mkdir(exist_ok=True)
    srcs = sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cpp")))
    hdr_time = _newest_header()
    jobs = []
    objs = []
    for s in srcs:
        o = BUILD / (s.name + ".o")
        objs.append(o)
        if force or not o.exists() or o.stat().st_mtime < max(s.stat().st_mtime, hdr_time):
            cmd = [NVCC, *COMMON, "-x", "cu", "-c", str(s), "-o", str(o)]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            jobs.append(cmd)

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed:\n" + " ".join(cmd) + "\n" + r.stdout + r.stderr)
        return r.stderr

    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            for out in ex.map(run, jobs):
                if verbose and out:
                    print(out)
    if jobs or not LIB.exists():
        link = [NVCC, "-shared", "-o", str(LIB), *map(str, objs), "-Xcompiler", "-fopenmp", "-lgomp", "-lcudart_static",
                "-gencode", "arch=compute_100a,code=sm_100a"]
        run(link)
    return LIB


if __name__ == "__main__":
    p = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(p)
