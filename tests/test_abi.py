"""CPU tests of the drop-in boundary: the shared library loads without a GPU, exports every
symbol the header declares (C ABI and the namespace blaze shims), and rejects bad arguments
before touching the device."""
import ctypes
import os
import re
import subprocess

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _header_symbols():
    text = open(os.path.join(ROOT, "include", "blaze_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(blz_[a-z0-9_]+)\s*\(", text)))


def test_exports_every_declared_symbol(native_lib):
    from blaze_b200 import _native
    names = _header_symbols()
    assert len(names) >= 16
    assert set(names) == set(_native.EXPORTS)
    for n in names:
        assert hasattr(native_lib, n), n


def test_blaze_namespace_entry_points_exported(native_lib):
    from blaze_b200 import _native
    out = subprocess.run(["nm", "-D", "--defined-only", _native.LIB_PATH], capture_output=True, text=True).stdout
    for name in ["launch_gemm_fp8", "create_fp8_gemm_plan", "execute_fp8_gemm", "destroy_fp8_gemm_plan",
                 "launch_gemm_fp4", "create_fp4_gemm_plan", "execute_fp4_gemm", "destroy_fp4_gemm_plan",
                 "launch_gemm_fp4_blkscaled", "create_fp4_blkscaled_gemm_plan", "execute_fp4_blkscaled_gemm",
                 "destroy_fp4_blkscaled_gemm_plan", "launch_gemm_fp4_blkscaled_persistent",
                 "create_fp4_blkscaled_persistent_gemm_plan", "execute_fp4_blkscaled_persistent_gemm",
                 "destroy_fp4_blkscaled_persistent_gemm_plan", "launch_gemm_mixed", "launch_fused_gate_up",
                 "create_mixed_gemm_plan", "execute_mixed_gemm", "destroy_mixed_gemm_plan",
                 "launch_gemm_fp16", "create_fp16_gemm_plan", "execute_fp16_gemm", "destroy_fp16_gemm_plan"]:
        assert re.search(r"_ZN5blaze\d+%s[A-Z]" % name, out), name


def test_argument_errors_without_device(native_lib):
    from blaze_b200 import _native as nv
    L = native_lib
    plan = ctypes.c_void_p()
    assert L.blz_gemm_plan_create(None, ctypes.byref(plan)) == nv.ERR_INVALID_ARGUMENT
    d = nv.GemmDesc()
    d.kind = nv.GEMM_FP8; d.M, d.N, d.K = 16, 16, 0
    assert L.blz_gemm_plan_create(ctypes.byref(d), ctypes.byref(plan)) == nv.ERR_INVALID_ARGUMENT
    d.K = 24; d.A = 4096; d.B = 4096                      # K not a multiple of 16 for E4M3 rows
    assert L.blz_gemm_plan_create(ctypes.byref(d), ctypes.byref(plan)) == nv.ERR_INVALID_ARGUMENT
    d.kind = nv.GEMM_NVFP4; d.K = 64                      # block scales missing
    assert L.blz_gemm_plan_create(ctypes.byref(d), ctypes.byref(plan)) == nv.ERR_INVALID_ARGUMENT
    assert L.blz_gemm_execute(None, None, None) == nv.ERR_INVALID_ARGUMENT
    assert L.blz_gemm_plan_destroy(None) == nv.OK          # destroy(nullptr) is a no-op, as in Blaze
    assert L.blz_amax(None, 0, 10, None, None) == nv.ERR_INVALID_ARGUMENT
    assert nv.status_string(nv.ERR_DEVICE_TIMEOUT) == "device-side wait ran out"


def test_tiled_scale_size(native_lib):
    # ceil(rows/128) rounded to 2 row blocks, ceil(K/64) rounded to 4 atoms, 512 bytes each
    assert native_lib.blz_tiled_scales_bytes(16, 4096) == 2 * 64 * 512
    assert native_lib.blz_tiled_scales_bytes(300, 64) == 4 * 4 * 512
    assert native_lib.blz_tiled_scales_bytes(0, 64) == 0


def test_shard_arithmetic_and_sharded_plan_argument_errors_without_device(native_lib):
    """The sharded wrapper's host logic through the C ABI: equal shards of whole 128-column tiles, refusals
    for everything else, and descriptor errors caught before any device call."""
    from blaze_b200 import _native as nv
    L = native_lib
    lo, hi = ctypes.c_int64(), ctypes.c_int64()
    for world, per in ((1, 28672), (2, 14336), (4, 7168), (8, 3584)):
        for rank in range(world):
            assert L.blz_shard_bounds(28672, world, rank, 128, ctypes.byref(lo), ctypes.byref(hi)) == nv.OK
            assert (lo.value, hi.value) == (rank * per, (rank + 1) * per)
    assert L.blz_shard_bounds(28672, 3, 0, 128, ctypes.byref(lo), ctypes.byref(hi)) == nv.ERR_INVALID_ARGUMENT     # not divisible
    assert L.blz_shard_bounds(1024, 16, 0, 128, ctypes.byref(lo), ctypes.byref(hi)) == nv.ERR_INVALID_ARGUMENT     # shards of 64 columns
    assert L.blz_shard_bounds(1024, 2, 2, 128, ctypes.byref(lo), ctypes.byref(hi)) == nv.ERR_INVALID_ARGUMENT      # rank outside the world
    assert L.blz_shard_bounds(1024, 2, 0, 128, None, ctypes.byref(hi)) == nv.ERR_INVALID_ARGUMENT
    plan = ctypes.c_void_p()
    assert L.blz_sharded_plan_create(None, ctypes.byref(plan)) == nv.ERR_INVALID_ARGUMENT
    sd = nv.ShardedDesc()
    sd.gemm.kind = nv.GEMM_FP8; sd.gemm.M, sd.gemm.N, sd.gemm.K = 256, 1024, 512
    sd.gemm.A = 4096; sd.gemm.B = 4096
    sd.world, sd.rank, sd.exchange = 2, 2, nv.EXCHANGE_NONE
    assert L.blz_sharded_plan_create(ctypes.byref(sd), ctypes.byref(plan)) == nv.ERR_INVALID_ARGUMENT              # rank >= world
    sd.rank, sd.exchange = 0, 7
    assert L.blz_sharded_plan_create(ctypes.byref(sd), ctypes.byref(plan)) == nv.ERR_INVALID_ARGUMENT              # no such exchange
    sd.exchange = nv.EXCHANGE_NCCL
    assert L.blz_sharded_plan_create(ctypes.byref(sd), ctypes.byref(plan)) == nv.ERR_INVALID_ARGUMENT              # NCCL without an id
    sd.exchange, sd.world = nv.EXCHANGE_NONE, 3
    assert L.blz_sharded_plan_create(ctypes.byref(sd), ctypes.byref(plan)) == nv.ERR_INVALID_ARGUMENT              # 1024 columns over 3 ranks
    sd.world = 2; sd.gemm.b_layout = nv.B_NMAJOR
    assert L.blz_sharded_plan_create(ctypes.byref(sd), ctypes.byref(plan)) == nv.ERR_UNSUPPORTED                   # shards are rows of K-major weights
    sd.gemm.b_layout = nv.B_KMAJOR; sd.gemm.epilogue = nv.EPI_RESIDUAL_ADD
    assert L.blz_sharded_plan_create(ctypes.byref(sd), ctypes.byref(plan)) == nv.ERR_UNSUPPORTED
    assert L.blz_sharded_plan_execute(None, None, None) == nv.ERR_INVALID_ARGUMENT
    assert L.blz_sharded_plan_destroy(None) == nv.OK
