"""In-tree build of the native libraries (``python -m tsplit_b200.build``).

* ``lib/libtsplit_kernels.so`` — every ``csrc/kernels/*.cu`` compiled by nvcc for
  ``sm_100a`` only (``-gencode arch=compute_100a,code=sm_100a``); cross-compiles
  without a GPU.
* ``lib/libtsplit_comm.so``    — ``csrc/comm/*.cu`` (peer-memory collectives).
* ``lib/libtsplit_runtime.so`` — ``csrc/runtime/*.cc`` + ``csrc/planner/*.cc``,
  host-only C++17 (g++), no CUDA needed.

Objects are cached under ``build/`` and rebuilt when a source or header is newer.
"""
from __future__ import annotations

import glob
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "lib")
OBJ = os.path.join(os.path.dirname(HERE), "build", "obj")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "--use_fast_math", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=default"]
# extra nvcc flags for developer builds, e.g. TSB_NVCC_EXTRA="-DTSB_CONV_PROF" (role-time counters)
NVCC_FLAGS += os.environ.get("TSB_NVCC_EXTRA", "").split()
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-Wall", "-pthread", "-fopenmp"]


def _nvcc():
    return shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"


def _newer(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def _run(cmd, verbose):
    if verbose:
        print(" ".join(cmd), flush=True)
    res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if res.returncode != 0:
        raise RuntimeError("build step failed:\n%s\n%s" % (" ".join(cmd), res.stdout))
    return res.stdout


def _compile_group(name, sources, headers, compiler, flags, link_flags, verbose):
    if not sources:
        return None
    os.makedirs(OBJ, exist_ok=True)
    os.makedirs(LIB, exist_ok=True)
    objs, jobs = [], []
    for src in sources:
        obj = os.path.join(OBJ, name + "_" + os.path.basename(src) + ".o")
        objs.append(obj)
        if _newer(obj, [src] + headers):
            jobs.append([compiler] + flags + ["-c", src, "-o", obj])
    with ThreadPoolExecutor(max_workers=max(1, min(8, os.cpu_count() or 1))) as pool:
        list(pool.map(lambda c: _run(c, verbose), jobs))
    out = os.path.join(LIB, "lib%s.so" % name)
    if jobs or _newer(out, objs):
        _run([compiler, "-shared", "-o", out] + objs + link_flags, verbose)
    return out


def build_all(verbose=False, cuda=True):
    built = []
    headers = glob.glob(os.path.join(CSRC, "**", "*.cuh"), recursive=True) + \
        glob.glob(os.path.join(CSRC, "**", "*.h"), recursive=True)
    host_src = sorted(glob.glob(os.path.join(CSRC, "runtime", "*.cc")) +
                      glob.glob(os.path.join(CSRC, "planner", "*.cc")) +
                      glob.glob(os.path.join(CSRC, "comm", "*.cc")))
    built.append(_compile_group("tsplit_runtime", host_src, headers, "g++", CXX_FLAGS, ["-pthread", "-fopenmp"],
                                verbose))
    if cuda:
        inc = ["-I", os.path.join(CSRC, "kernels")]
        ksrc = sorted(glob.glob(os.path.join(CSRC, "kernels", "*.cu")))
        built.append(_compile_group("tsplit_kernels", ksrc, headers, _nvcc(), NVCC_FLAGS + inc,
                                    ["-Xcompiler", "-fPIC"], verbose))
        csrc = sorted(glob.glob(os.path.join(CSRC, "comm", "*.cu")))
        built.append(_compile_group("tsplit_comm", csrc, headers, _nvcc(), NVCC_FLAGS + inc,
                                    ["-Xcompiler", "-fPIC"], verbose))
    return [b for b in built if b]


if __name__ == "__main__":
    libs = build_all(verbose="-v" in sys.argv, cuda="--no-cuda" not in sys.argv)
    for lib in libs:
        print("built", lib)
