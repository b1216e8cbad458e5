"""Build libtq_b200.so (CUDA kernels + C ABI) for sm_100a with nvcc, in-tree.

    python transformers-turboquant_b200/build.py [--force] [--verbose] [--trace]

Each csrc/*.cu is compiled to an object in build/ (only when its sources changed) and
the objects are linked into turboquant_b200/libtq_b200.so.  nvcc cross-compiles, so no
GPU is needed.  `-Xptxas -v` output (registers, spills, shared memory per kernel) is
kept in build/ptxas_<file>.log.  `--trace` (implies a full rebuild) adds the diagnostic
instantiations of the attention kernels that tq_trace_enable / tq_trace_read need; the
default product build leaves them out.
"""

from __future__ import annotations

import concurrent.futures as cf
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")
BUILD = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "turboquant_b200", "libtq_b200.so")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
         "-Xcompiler", "-fPIC", "-Xptxas", "-v", "-I", INCLUDE, "-I", CSRC]


def _newest(paths):
    return max(os.path.getmtime(p) for p in paths)


def build(force: bool = False, verbose: bool = False, trace: bool = False) -> str:
    os.makedirs(BUILD, exist_ok=True)
    flags = FLAGS + (["-DTQ_B200_TRACE=1"] if trace else [])
    # a library built with tracing is a different product: switching the option rebuilds everything
    stamp = os.path.join(BUILD, "trace.flag")
    had_trace = os.path.exists(stamp)
    if trace != had_trace:
        force = True
        if trace:
            open(stamp, "w").close()
        else:
            os.remove(stamp)
    sources = sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cuh")]
    headers.append(os.path.join(INCLUDE, "tq_b200.h"))
    hdr_time = _newest(headers)

    def compile_one(src):
        obj = os.path.join(BUILD, src[:-3] + ".o")
        path = os.path.join(CSRC, src)
        if not force and os.path.exists(obj) and os.path.getmtime(obj) > max(os.path.getmtime(path), hdr_time):
            return obj, False
        res = subprocess.run([NVCC, *flags, "-c", path, "-o", obj], capture_output=True, text=True)
        with open(os.path.join(BUILD, f"ptxas_{src[:-3]}.log"), "w") as fh:
            fh.write(res.stderr)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}:\n{res.stdout}\n{res.stderr}")
        if verbose:
            print(res.stderr)
        return obj, True

    with cf.ThreadPoolExecutor(max_workers=min(8, len(sources))) as pool:
        results = list(pool.map(compile_one, sources))
    objs = [o for o, _ in results]
    if force or any(c for _, c in results) or not os.path.exists(LIB):
        res = subprocess.run([NVCC, "-shared", "-o", LIB, *objs, "-gencode", "arch=compute_100a,code=sm_100a",
                              "-lcudart"], capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv, trace="--trace" in sys.argv))
