"""Developer tool: per-role cycle counters and an event trace of the tiled kernel, from a tuning build.

    python -m blaze_b200.tuning roles KIND M N K [VARIANT]     cycles per tile spent waiting / working, per role
    python -m blaze_b200.tuning trace KIND M N K [VARIANT]     CTA 0: gap between consecutive stage issues of the MMA
                                                                thread, and when the accumulator changed hands

The tuning build is the same sources compiled with -DBLZ_KERNEL_TIMING into
blaze_b200/libblaze_b200_tuning.so (built here on first use; the shipped library carries no counters).
KIND: nvfp4 | fp8 | bf16 | f16; VARIANT as in GemmPlan (default auto).  Needs a B200.
The library's environment switches apply (BLZ_TAIL_SPLIT=1: `roles` then also prints the phases of a K-split unit).
"""
from __future__ import annotations

import ctypes
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
TUNING_LIB = os.path.join(HERE, "libblaze_b200_tuning.so")


def build_tuning_library(force: bool = False) -> str:
    from . import build as b
    deps = [os.path.join(b.CSRC, f) for f in os.listdir(b.CSRC)]
    if not force and os.path.exists(TUNING_LIB) and all(os.path.getmtime(d) <= os.path.getmtime(TUNING_LIB) for d in deps):
        return TUNING_LIB
    objs = []
    for src in b.SOURCES:
        obj = os.path.join(b.CSRC, src.replace(".cu", ".tuning.o"))
        subprocess.run([b.NVCC, *b.FLAGS, "-DBLZ_KERNEL_TIMING", "-c", "-o", obj, os.path.join(b.CSRC, src)], check=True)
        objs.append(obj)
    subprocess.run([b.NVCC, "-shared", "-o", TUNING_LIB, *objs, "-ldl"], check=True)
    for o in objs:
        os.remove(o)
    return TUNING_LIB


def _plan(kind, M, N, K, variant, tail_split=False):
    import torch
    from . import GemmPlan, quantize_fp8, quantize_nvfp4
    dev = torch.device("cuda:0")
    ga, gb = torch.Generator(device=dev).manual_seed(42), torch.Generator(device=dev).manual_seed(123)
    xa, xb = torch.randn((M, K), generator=ga, device=dev), torch.randn((N, K), generator=gb, device=dev)
    if kind == "nvfp4":
        ad, asf, gA = quantize_nvfp4(xa, tiled=True); bd, bsf, gB = quantize_nvfp4(xb, tiled=True)
        kw = dict(A_sf=asf, B_sf=bsf, a_scale=float(gA.item()), b_scale=float(gB.item()), a_sf_layout="tiled", b_sf_layout="tiled")
        A, B = ad, bd
    elif kind == "fp8":
        qa, sa = quantize_fp8(xa); qb, sb = quantize_fp8(xb)
        A, B, kw = qa, qb, dict(a_scale=float(sa[1].item()), b_scale=float(sb[1].item()))
    else:
        dt = torch.bfloat16 if kind == "bf16" else torch.float16
        A, B, kw = xa.to(dt), xb.to(dt), {}
    C = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
    plan = GemmPlan(kind, M, N, K, A, B, out_dtype="bf16", variant=variant, tail_split=tail_split, **kw)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    for _ in range(3):
        flush.fill_(1); plan.execute(C)
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    flush.fill_(1); s.record(); plan.execute(C); e.record(); torch.cuda.synchronize()
    return plan, s.elapsed_time(e), (A, B, C, kw)


def roles(kind, M, N, K, variant="auto"):
    import numpy as np
    from . import _native
    plan, ms, _keep = _plan(kind, M, N, K, variant)
    info = plan.info()
    n = info["grid"] * 16
    buf = (ctypes.c_ulonglong * n)()
    _native.lib().blz_debug_read_timing(buf, n)
    t = np.array(buf[:], dtype=np.float64).reshape(info["grid"], 16)
    lead = t[:, 8] > 0
    tiles = t[lead, 8].mean() if lead.any() else 1
    t = t[lead] if lead.any() else t
    print("%s %dx%dx%d %s: %.4f ms, %.0f TFLOP/s, grid %d, %.2f tiles per CTA group (tile %dx%d, %d stages)" % (
        kind, M, N, K, variant, ms, 2.0 * M * N * K / ms / 1e9, info["grid"], tiles, info["tile_m"], info["tile_n"], info["stages"]))
    for i, nm in enumerate(["producer: wait for a free stage", "producer: total", "MMA thread: wait for a loaded stage", "MMA thread: wait for the accumulator",
                            "MMA thread: total", "epilogue: wait for a full accumulator", "epilogue: work", "epilogue: total"]):
        print("   %-40s %9.0f cycles per tile" % (nm, t[:, i].mean() / max(tiles, 1)))
    if info["tail_tiles"]:
        print("   %d tiles cut along K into %d units each; per unit (CTAs that ran one):" % (info["tail_tiles"], info["tail_split"]))
        for i, nm in ((9, "accumulator -> scratch"), (10, "fence and publish"), (11, "wait for the tile's other units"), (12, "sum, finish, store")):
            col = t[:, i][t[:, i] > 0]
            if len(col):
                print("   %-40s %9.0f cycles (max %.0f)" % (nm, col.mean(), col.max()))
    plan.destroy()


def trace(kind, M, N, K, variant="auto"):
    import numpy as np
    from . import _native
    plan, ms, _keep = _plan(kind, M, N, K, variant)
    buf = (ctypes.c_ulonglong * (4 * 4096))()
    _native.lib().blz_debug_read_trace(buf, 4 * 4096)
    t = np.array(buf[:], dtype=np.int64).reshape(4, 4096)
    row_bytes = K // 2 if kind == "nvfp4" else K if kind == "fp8" else 2 * K
    ks = -(-row_bytes // 128)
    mma = t[0]
    n = int((mma > 0).sum())
    t0 = mma[0]
    print("%s %dx%dx%d %s: %.4f ms; CTA 0 issued %d stages, %d per tile" % (kind, M, N, K, variant, ms, n, ks))
    for ti in range(min(n // ks, 8)):
        st = mma[ti * ks:(ti + 1) * ks] - t0
        print("tile %d: accumulator free seen at %7d, first stage %7d, last stage %7d; cycles between stage issues: %s" % (
            ti, t[1][ti] - t0, st[0], st[-1], " ".join(str(int(x)) for x in np.diff(st))))
        print("        epilogue: accumulator full seen %7d, handed back %7d / %7d (the two warp sets), tile stored %7d" % (
            t[2][8 * ti] - t0, t[3][2 * ti] - t0, t[3][2 * ti + 1] - t0, t[2][8 * ti + 1] - t0))
    plan.destroy()


def main(argv) -> int:
    if len(argv) < 5 or argv[0] not in ("roles", "trace"):
        print(__doc__)
        return 2
    from . import _native
    _native.LIB_PATH, _native._LIB = build_tuning_library(), None        # every call below goes to the tuning build
    fn = roles if argv[0] == "roles" else trace
    fn(argv[1], int(argv[2]), int(argv[3]), int(argv[4]), argv[5] if len(argv) > 5 else "auto")
    return 0


if __name__ == "__main__":
    sys.exit(main(sys.argv[1:]))
