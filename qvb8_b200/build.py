"""Builds ``libqvb8_b200.so`` (the C-ABI kernel library) in-tree with nvcc for sm_100a.

    python -m qvb8_b200.build [--force] [--verbose]

nvcc cross-compiles without a GPU.  Objects are rebuilt only when their source (or a header) is newer.
"""
from __future__ import annotations

import concurrent.futures
import glob
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libqvb8_b200.so")
OBJ_DIR = os.path.join(HERE, "build")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
    "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC,-fvisibility=hidden", "-Xptxas", "-v",
]


def _nvcc() -> str:
    for cand in (os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc"), shutil.which("nvcc")):
        if cand and os.path.isfile(cand):
            return cand
    raise RuntimeError("nvcc not found: the kernel library cannot be built")


def _host_cxx() -> list[str]:
    # a host compiler nvcc accepts; /usr/bin/g++ is the distribution's
    return ["-ccbin", "/usr/bin/g++"] if os.path.isfile("/usr/bin/g++") else []


def sources() -> list[str]:
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")))


def _newest_header() -> float:
    hs = glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(HERE, "..", "include", "*.h"))
    return max((os.path.getmtime(h) for h in hs), default=0.0)


def build(force: bool = False, verbose: bool = False) -> str:
    nvcc = _nvcc()
    os.makedirs(OBJ_DIR, exist_ok=True)
    hdr = _newest_header()
    jobs = []
    objs = []
    for src in sources():
        obj = os.path.join(OBJ_DIR, os.path.basename(src)[:-3] + ".o")
        objs.append(obj)
        stale = force or not os.path.exists(obj) or os.path.getmtime(obj) < max(os.path.getmtime(src), hdr)
        if stale:
            jobs.append((src, obj))

    def compile_one(job):
        src, obj = job
        # QVB8_EXTRA_NVCC_FLAGS: extra -D switches for tuning builds (e.g. -DQVB8_PIPES_NT1=2); build with force=True
        extra = os.environ.get("QVB8_EXTRA_NVCC_FLAGS", "").split()
        cmd = [nvcc, *NVCC_FLAGS, *extra, *_host_cxx(), "-c", src, "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        return src, r

    if jobs:
        with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            for src, r in ex.map(compile_one, jobs):
                log = os.path.join(OBJ_DIR, os.path.basename(src)[:-3] + ".ptxas.log")
                with open(log, "w") as fh:
                    fh.write(r.stderr)
                if verbose:
                    sys.stderr.write(r.stderr)
                if r.returncode != 0:
                    raise RuntimeError(f"nvcc failed on {src}:\n{r.stdout}\n{r.stderr}")
    lib_stale = force or jobs or not os.path.exists(LIB) or any(os.path.getmtime(o) > os.path.getmtime(LIB) for o in objs)
    if lib_stale:
        cmd = [nvcc, "-shared", *_host_cxx(), "-o", LIB, *objs, "-lcudart"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
