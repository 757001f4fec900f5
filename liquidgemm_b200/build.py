"""Build the C-ABI CUDA library in-tree: ``python -m liquidgemm_b200.build``.

Plain ``nvcc`` for sm_100a, no libtorch and no third-party headers; the result
``liquidgemm_b200/_lq_b200.so`` is what :mod:`liquidgemm_b200._lib` loads
(the reference builds a torch CUDAExtension instead: setup.py:24-53).
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
SOURCES = ["lq_api.cu", "lq_elementwise.cu", "lq_gemv.cu", "lq_gemm_tc.cu", "lq_gemm_tile.cu", "lq_gemv_blob.cu", "lq_decode_tc.cu", "lq_gemm_pair.cu", "lq_i8_pair.cu", "lq_quantize.cu", "lq_host.cu"]
HEADERS = ["lq_common.cuh", "lq_tc_ptx.cuh", "lq_sched.cuh", "lq_pair_common.cuh", os.path.join("..", "..", "include", "liquidgemm_b200.h")]
LIB_PATH = os.path.join(HERE, "_lq_b200.so")
# Measurement-only kernels (building-block rates; nothing in the product calls them): a library of their own,
# built on request with ``python -m liquidgemm_b200.build --debug`` and loaded by liquidgemm_b200.microbench.
DEBUG_SOURCES = ["lq_api.cu", os.path.join("dbg", "lq_debug.cu")]
DEBUG_LIB_PATH = os.path.join(HERE, "_lq_b200_dbg.so")

NVCC_FLAGS = [
    "-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def _stale(lib_path, sources) -> bool:
    if not os.path.exists(lib_path):
        return True
    t = os.path.getmtime(lib_path)
    deps = [os.path.join(CSRC, s) for s in sources + HEADERS] + [os.path.abspath(__file__)]
    return any(os.path.getmtime(d) > t for d in deps)


TRACE_LIB_PATH = os.path.join(HERE, "_lq_b200_trace.so")


def build(force: bool = False, verbose: bool = False, debug: bool = False, trace: bool = False) -> str:
    """Compile every .cu of the product (or, with ``debug``, the measurement kernels) into one shared
    library; returns its path.  ``trace`` builds the product sources with -DLQ_PIPELINE_TRACE (per-CTA cycle
    counters in the decode kernel) into a library of its own, which ``LIQUIDGEMM_B200_TRACE=1`` makes
    :mod:`liquidgemm_b200._lib` load instead."""
    lib_path, sources = (DEBUG_LIB_PATH, DEBUG_SOURCES) if debug else (LIB_PATH, SOURCES)
    if trace:
        lib_path = TRACE_LIB_PATH
    if not force and not _stale(lib_path, sources):
        return lib_path
    nvcc = _nvcc()
    objs = []
    procs = []
    for src in sources:
        obj = os.path.join(CSRC, src.replace(".cu", ".dbg.o" if debug else ".trace.o" if trace else ".o"))
        cmd = [nvcc, *NVCC_FLAGS, "-c", os.path.join(CSRC, src), "-o", obj]
        if trace:
            cmd.insert(1, "-DLQ_PIPELINE_TRACE")
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(obj)
    failed = False
    for src, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0 or verbose:
            sys.stderr.write(f"--- nvcc {src}\n{out}\n")
        failed |= p.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed")
    tmp = lib_path + ".tmp"
    subprocess.check_call([nvcc, "-shared", "-o", tmp, *objs, "-gencode", "arch=compute_100a,code=sm_100a"])
    os.replace(tmp, lib_path)
    return lib_path


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv, debug="--debug" in sys.argv,
                trace="--trace" in sys.argv))
