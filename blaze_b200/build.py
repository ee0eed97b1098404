"""Builds the CUDA library in-tree: blaze_b200/libblaze_b200.so (sm_100a only).

nvcc cross-compiles without a GPU.  The library links the CUDA runtime statically and looks the
one driver entry point it needs up at run time, so it loads on a machine without a GPU driver.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "libblaze_b200.so")
NVCC = os.environ.get("NVCC", shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc")

SOURCES = ["capi.cu", "blaze_compat.cu", "decode_static.cu", "sharded.cu"]
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
         "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=default"]


def _stale() -> bool:
    if not os.path.exists(OUT):
        return True
    t = os.path.getmtime(OUT)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)]
    inc = os.path.join(os.path.dirname(HERE), "include")
    for root, _, files in os.walk(inc):
        deps += [os.path.join(root, f) for f in files]
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not _stale():
        return OUT
    # the translation units compile side by side (the tiled-kernel instances in capi.cu take most of the time)
    jobs = []
    for src in SOURCES:
        obj = os.path.join(CSRC, src.replace(".cu", ".o"))
        cmd = [NVCC, *FLAGS, "-c", "-o", obj, os.path.join(CSRC, src)]
        if verbose:
            cmd.insert(1, "-Xptxas")
            cmd.insert(2, "-v")
        jobs.append((src, obj, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)))
    objs = []
    failed = None
    for src, obj, proc in jobs:
        out, err = proc.communicate()
        if verbose:
            sys.stderr.write(err)
        if proc.returncode != 0 and failed is None:
            failed = "nvcc failed for %s:\n%s\n%s" % (src, out, err)
        objs.append(obj)
    if failed:
        raise RuntimeError(failed)
    r = subprocess.run([NVCC, "-shared", "-o", OUT, *objs, "-ldl"], capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("link failed:\n%s\n%s" % (r.stdout, r.stderr))
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
