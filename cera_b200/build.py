"""Build libcera_cuda.so (sm_100a) from cera_b200/csrc with nvcc.

The library is built in-tree so that it travels with the source tree; nothing
is JIT-compiled at import time.  Run it by path, `python cera_b200/build.py [--force] [-v]`:
importing the package itself requires the library to exist already.
"""
import concurrent.futures
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ_DIR = os.path.join(HERE, "_obj")
LIB = os.path.join(HERE, "libcera_cuda.so")

SOURCES = ["runtime.cu", "weight.cu", "quantize.cu", "gemv.cu", "attention.cu", "glue.cu", "convert.cu", "model.cu"]
# Translation units whose float arithmetic must not be contracted into FMAs.
NO_FMAD = {"convert.cu"}

ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
          "--expt-relaxed-constexpr"]


def nvcc():
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found: the CUDA library cannot be built")
    return exe


def _headers():
    hs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    hs.append(os.path.join(os.path.dirname(HERE), "include", "cera_cuda.h"))
    return hs


def _stale(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def _sources():
    extra = [f for f in sorted(os.listdir(CSRC)) if f.endswith(".cu") and f not in SOURCES]
    return SOURCES + extra


def build(force=False, verbose=False):
    os.makedirs(OBJ_DIR, exist_ok=True)
    hdrs = _headers()
    jobs = []
    objs = []
    for src in _sources():
        s = os.path.join(CSRC, src)
        o = os.path.join(OBJ_DIR, src.replace(".cu", ".o"))
        objs.append(o)
        if force or _stale(o, [s] + hdrs):
            cmd = [nvcc()] + ARCH + COMMON + (["-fmad=false"] if src in NO_FMAD else [])
            if verbose:
                cmd += ["-Xptxas", "-v"]
            cmd += ["-c", s, "-o", o]
            jobs.append(cmd)

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        return cmd, r

    if jobs:
        with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            for cmd, r in ex.map(run, jobs):
                if verbose or r.returncode:
                    sys.stderr.write(" ".join(cmd[-3:]) + "\n" + r.stdout + r.stderr)
                if r.returncode:
                    raise RuntimeError("nvcc failed for " + cmd[-3])
    if jobs or force or _stale(LIB, objs):
        cmd = [nvcc()] + ARCH + ["-shared", "-o", LIB] + objs
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("link failed")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
