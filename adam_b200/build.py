"""Builds ``libadam_b200.so`` in-tree from ``adam_b200/csrc/*.cu`` with nvcc for
sm_100a.  ``python -m adam_b200.build [--force] [--verbose]``."""
from __future__ import annotations

import argparse
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libadam_b200.so")
OBJ_DIR = os.path.join(HERE, "build")
TRACE_LIB = os.path.join(HERE, "libadam_b200_trace.so")
TRACE_OBJ_DIR = os.path.join(HERE, "build", "trace")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--use_fast_math=false",
]


def _nvcc() -> str:
    for c in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if c and (os.path.isabs(c) and os.path.exists(c) or not os.path.isabs(c)):
            return c
    raise RuntimeError("nvcc not found")


def sources():
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def _deps_mtime() -> float:
    files = [os.path.join(CSRC, f) for f in os.listdir(CSRC)] + [os.path.join(HERE, "..", "include", "adam_b200.h"), __file__]
    return max(os.path.getmtime(f) for f in files)


def build(force: bool = False, verbose: bool = False, ptxas_info: bool = False, step_trace: bool = False) -> str:
    """Compile and link; returns the library path.  Skips work when the library
    is newer than every source.  ``step_trace`` builds the diagnostics variant ``libadam_b200_trace.so``
    (kernels of the decode step stamp their phase boundaries; select it with ``ADAM_B200_LIB_PATH``)."""
    LIB = TRACE_LIB if step_trace else globals()["LIB"]
    OBJ_DIR = TRACE_OBJ_DIR if step_trace else globals()["OBJ_DIR"]
    if not force and os.path.exists(LIB) and os.path.getmtime(LIB) >= _deps_mtime():
        return LIB
    os.makedirs(OBJ_DIR, exist_ok=True)
    nvcc = _nvcc()
    hdr_time = max(os.path.getmtime(os.path.join(CSRC, f)) for f in os.listdir(CSRC) if not f.endswith(".cu"))
    hdr_time = max(hdr_time, os.path.getmtime(os.path.join(HERE, "..", "include", "adam_b200.h")), os.path.getmtime(__file__))

    def compile_one(src: str) -> str:
        obj = os.path.join(OBJ_DIR, os.path.basename(src)[:-3] + ".o")
        if not force and os.path.exists(obj) and os.path.getmtime(obj) >= max(os.path.getmtime(src), hdr_time):
            return obj
        cmd = [nvcc, *[f for f in NVCC_FLAGS if f != "--use_fast_math=false"], *os.environ.get("ADAM_B200_NVCC_EXTRA", "").split(),
               *(["-DADAM_B200_STEP_TRACE"] if step_trace else []), "-c", src, "-o", obj]
        if ptxas_info:
            cmd[1:1] = ["-Xptxas", "-v"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if verbose or ptxas_info or r.returncode:
            sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
        if r.returncode:
            raise RuntimeError(f"nvcc failed on {src}")
        return obj

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as ex:
        objs = list(ex.map(compile_one, sources()))
    cmd = [nvcc, "-shared", "-o", LIB, *objs, "-lcudart", "-lnccl"] if _want_nccl() else [nvcc, "-shared", "-o", LIB, *objs, "-lcudart"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode:
        sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
        raise RuntimeError("link failed")
    return LIB


def _want_nccl() -> bool:
    return any("nccl" in open(s).read() for s in sources() if os.path.basename(s) == "tp.cu")


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--ptxas", action="store_true", help="print registers / spills / shared memory per kernel")
    ap.add_argument("--step-trace", action="store_true", help="build the diagnostics variant libadam_b200_trace.so (-DADAM_B200_STEP_TRACE)")
    a = ap.parse_args()
    print(build(force=a.force, verbose=a.verbose, ptxas_info=a.ptxas, step_trace=a.step_trace))
