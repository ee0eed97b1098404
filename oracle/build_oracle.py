"""Build recipe for the CPU oracle and for the pieces of the Blaze reference that compile here.

TEST INFRASTRUCTURE ONLY: nothing in the product package imports this module.

Outputs
  oracle/libblaze_oracle.so        the C restatement (blaze_oracle.c), gcc, no FMA contraction
  oracle/pin_formats               host-only program comparing the oracle's number formats with
                                   CUDA's own host conversions (cuda_fp16.h / cuda_bf16.h /
                                   cuda_fp8.h / cuda_fp4.h); built with nvcc, needs no GPU
  oracle/_ref/libblaze_ref_naive.so  Blaze's own tests/test_gemm_naive.cu compiled where it lies
                                   (its main() renamed), exporting gemm_cpu_fp16 and
                                   init_random_fp16; only built when the reference tree is present
  oracle/_ref/test_gemm, bench_gemm  Blaze's tests/test_gemm.cu and benchmarks/bench_gemm.cu compiled
                                   unchanged against this repository's headers and library
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
# The Blaze source tree: BLAZE_REFERENCE_ROOT, else a directory named "reference" beside this repository.
# Absent (e.g. on a GPU box) -> the steps that need it are skipped and the prebuilt files are used.
REF_ROOT = os.environ.get("BLAZE_REFERENCE_ROOT") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")
NVCC = os.environ.get("NVCC", shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc")


def _newer(src: list[str], dst: str) -> bool:
    if not os.path.exists(dst):
        return True
    t = os.path.getmtime(dst)
    return any(os.path.getmtime(s) > t for s in src if os.path.exists(s))


def _run(cmd: list[str]) -> None:
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("build step failed: %s\n%s\n%s" % (" ".join(cmd), r.stdout, r.stderr))


def build_oracle(force: bool = False) -> str:
    src = os.path.join(HERE, "blaze_oracle.c")
    out = os.path.join(HERE, "libblaze_oracle.so")
    if force or _newer([src], out):
        _run(["gcc", "-O2", "-ffp-contract=off", "-fno-fast-math", "-fPIC", "-shared", "-pthread",
              "-o", out, src, "-lm"])
    return out


def build_pin_formats(force: bool = False) -> str | None:
    src = os.path.join(HERE, "pin_formats.cu")
    out = os.path.join(HERE, "pin_formats")
    if not os.path.exists(NVCC):
        return None
    if force or _newer([src, os.path.join(HERE, "blaze_oracle.c")], out):
        obj = os.path.join(HERE, "blaze_oracle_pin.o")
        _run(["gcc", "-O2", "-ffp-contract=off", "-c", "-o", obj, os.path.join(HERE, "blaze_oracle.c")])
        _run([NVCC, "-O2", "-std=c++17", "-o", out, src, obj, "-lpthread"])
    return out


def build_ref(force: bool = False) -> str | None:
    """Compile Blaze's host reference GEMM from its own source file; outputs only into oracle/_ref."""
    src = os.path.join(REF_ROOT, "tests", "test_gemm_naive.cu")
    out_dir = os.path.join(HERE, "_ref")
    out = os.path.join(out_dir, "libblaze_ref_naive.so")
    if not os.path.exists(src):
        return out if os.path.exists(out) else None
    if not os.path.exists(NVCC):
        return out if os.path.exists(out) else None
    os.makedirs(out_dir, exist_ok=True)
    if force or _newer([src], out):
        # The CUDA runtime is linked statically and initialises lazily, so no GPU driver is needed to load it;
        # cuBLAS is referenced only by functions the oracle never calls: load with RTLD_LAZY.
        _run([NVCC, "-O2", "-std=c++17", "-Dmain=blaze_ref_naive_main", "-Xcompiler", "-fPIC", "-shared",
              "-o", out, src])
    return out


def build_ref_programs(force: bool = False) -> list[str]:
    """Blaze's own tests/test_gemm.cu and benchmarks/bench_gemm.cu, compiled unchanged against THIS
    repository's include/gemm headers and linked to blaze_b200/libblaze_b200.so (the drop-in check).
    Outputs only into oracle/_ref; skipped when the reference tree or the library is absent."""
    root = os.path.dirname(HERE)
    lib_dir = os.path.join(root, "blaze_b200")
    lib = os.path.join(lib_dir, "libblaze_b200.so")
    out_dir = os.path.join(HERE, "_ref")
    built = []
    if not os.path.exists(lib) or not os.path.exists(NVCC):
        return built
    for rel, name in (("tests/test_gemm.cu", "test_gemm"), ("benchmarks/bench_gemm.cu", "bench_gemm")):
        src = os.path.join(REF_ROOT, rel)
        out = os.path.join(out_dir, name)
        if not os.path.exists(src):
            if os.path.exists(out):
                built.append(out)
            continue
        os.makedirs(out_dir, exist_ok=True)
        if force or _newer([src, lib], out):
            _run([NVCC, "-gencode", "arch=compute_100a,code=sm_100a", "-O2", "-std=c++17", "-w", "-I", os.path.join(root, "include"), src,
                  "-L", lib_dir, "-lblaze_b200", "-lcublas", "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN/../../blaze_b200", "-o", out])
        built.append(out)
    # Blaze's bring-up test of the raw tcgen05 / TMA helpers: compiled to an object only, against this
    # repository's gemm/tma_utils.cuh and gemm/tmem_utils.cuh (a check that the helper names and
    # signatures are all there).  It is not linked into a program: its kernels are Blaze's own.
    src = os.path.join(REF_ROOT, "tests", "test_sm100_primitives.cu")
    obj = os.path.join(out_dir, "test_sm100_primitives.o")
    if os.path.exists(src):
        os.makedirs(out_dir, exist_ok=True)
        hdrs = [os.path.join(root, "include", "gemm", h) for h in ("tma_utils.cuh", "tmem_utils.cuh")]
        if force or _newer([src] + hdrs, obj):
            _run([NVCC, "-gencode", "arch=compute_100a,code=sm_100a", "-O2", "-std=c++17", "-w", "-I", os.path.join(root, "include"), "-c", src, "-o", obj])
        built.append(obj)
    return built


def build_all(force: bool = False) -> dict:
    res = {"oracle": build_oracle(force)}
    try:
        res["pin_formats"] = build_pin_formats(force)
    except RuntimeError as e:  # nvcc host-only build is optional for the oracle itself
        res["pin_formats_error"] = str(e)
    try:
        res["ref_naive"] = build_ref(force)
    except RuntimeError as e:
        res["ref_naive_error"] = str(e)
    try:
        res["ref_programs"] = build_ref_programs(force)
    except RuntimeError as e:
        res["ref_programs_error"] = str(e)
    return res


if __name__ == "__main__":
    for k, v in build_all("--force" in sys.argv).items():
        print(k, "->", v)
