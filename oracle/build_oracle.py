"""Compile the C restatement of the oracle (``oracle/lqq_oracle.c``) into ``oracle/_build/``.

``python -m oracle.build_oracle``.  Two variants are built so that the library also loads on a
host older than the build machine: ``liblqq_oracle_v3.so`` (x86-64-v3: AVX2/FMA/BMI2) and
``liblqq_oracle_base.so`` (baseline x86-64).  :func:`load` picks by the flags in /proc/cpuinfo.

The reference itself is pure Python on this path, so there is nothing of it to compile
(``oracle/_ref`` stays empty); its outputs are pinned through tests/golden instead.
"""

from __future__ import annotations

import ctypes
import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "lqq_oracle.c")
OUT = os.path.join(HERE, "_build")
VARIANTS = {"v3": ["-march=x86-64-v3"], "base": []}


def lib_path(variant: str) -> str:
    return os.path.join(OUT, f"liblqq_oracle_{variant}.so")


def build(force: bool = False) -> None:
    os.makedirs(OUT, exist_ok=True)
    for name, flags in VARIANTS.items():
        dst = lib_path(name)
        if not force and os.path.exists(dst) and os.path.getmtime(dst) >= os.path.getmtime(SRC):
            continue
        cmd = ["gcc", "-O3", "-fopenmp", "-fPIC", "-shared", "-fno-fast-math", *flags, SRC, "-o", dst, "-lm"]
        subprocess.check_call(cmd)


def _cpu_has_avx2() -> bool:
    try:
        with open("/proc/cpuinfo") as f:
            for line in f:
                if line.startswith("flags"):
                    fl = line.split()
                    return all(x in fl for x in ("avx2", "fma", "bmi2"))
    except OSError:
        pass
    return False


def load() -> ctypes.CDLL:
    """Load the C oracle, building it first if it is missing (gcc only, a second or two)."""
    variant = "v3" if _cpu_has_avx2() else "base"
    if not os.path.exists(lib_path(variant)):
        build()
    lib = ctypes.CDLL(lib_path(variant))
    P, I = ctypes.c_void_p, ctypes.c_int
    lib.lqo_num_threads.restype = I
    lib.lqo_set_num_threads.argtypes = [I]
    lib.lqo_set_num_threads.restype = None
    lib.lqo_dequant_i8.argtypes = [P, P, P, P, I, I, I]
    lib.lqo_dequant_i8_simd.argtypes = [P, P, P, P, I, I, I]
    lib.lqo_int_gemm.argtypes = [P, P, P, I, I, I]
    lib.lqo_scale_f32.argtypes = [P, P, P, P, I, I]
    lib.lqo_quant_per_token.argtypes = [P, P, P, I, I]
    lib.lqo_w4a8_linear.argtypes = [P, P, P, P, P, P, I, I, I, I]
    for fn in ("lqo_dequant_i8", "lqo_dequant_i8_simd", "lqo_int_gemm", "lqo_scale_f32", "lqo_quant_per_token",
               "lqo_w4a8_linear"):
        getattr(lib, fn).restype = None
    return lib


if __name__ == "__main__":
    build(force=True)
    print(lib_path("v3"), lib_path("base"))
