"""Host-side mirror of Blaze's plan / execute API over the C ABI, for Python callers.

Device memory, streams and process groups come from PyTorch; all arithmetic happens in the CUDA
library.  The functions named like Blaze's (``create_fp8_gemm_plan`` / ``execute_fp8_gemm`` /
``destroy_fp8_gemm_plan`` ... see include/gemm/fp8_gemm_sm100.cuh:84-99 and its siblings in the
Blaze project) take the same arguments with the same meaning: B in Blaze's [K, N] row-major
convention, fp16 output, operands owned by the caller and alive as long as the plan.
``GemmPlan`` exposes everything else the C ABI offers (K-major weights, bf16 / fp32 output,
per-tensor scales, pre-tiled scale factors, kernel variant).
"""
from __future__ import annotations

import ctypes
from typing import Any

from . import _native as nv


def _ptr(t: Any):
    if t is None:
        return None
    if isinstance(t, int):
        return t
    return t.data_ptr()


def _stream(stream=None):
    if stream is not None:
        return stream if isinstance(stream, int) else stream.cuda_stream
    import torch  # noqa: PLC0415
    return torch.cuda.current_stream().cuda_stream


def make_desc(kind: str, M: int, N: int, K: int, A, B, *, A_sf=None, B_sf=None, a_scale: float = 1.0, b_scale: float = 1.0,
              out_dtype: str = "bf16", epilogue: str = "none", bias=None, residual=None, b_layout: str = "kmajor",
              a_sf_layout: str = "rowmajor", b_sf_layout: str = "rowmajor", variant: str = "auto", ldc: int = 0, b_scale2: float = 0.0,
              scheduler: str = "static", static_weights: bool = False, tail_split: bool = False):
    """blz_gemm_desc from keyword arguments (field meanings: include/blaze_b200.h)."""
    d = nv.GemmDesc()
    d.kind = nv.KINDS[kind]
    d.out_dtype = nv.DTYPES[out_dtype]
    d.epilogue = nv.EPILOGUES[epilogue]
    d.variant = nv.VARIANTS[variant]
    d.M, d.N, d.K = int(M), int(N), int(K)
    d.b_layout = nv.B_NMAJOR if b_layout == "nmajor" else nv.B_KMAJOR
    d.a_sf_layout = nv.SF_TILED if a_sf_layout == "tiled" else nv.SF_ROWMAJOR
    d.b_sf_layout = nv.SF_TILED if b_sf_layout == "tiled" else nv.SF_ROWMAJOR
    d.A, d.A_sf, d.B, d.B_sf = _ptr(A), _ptr(A_sf), _ptr(B), _ptr(B_sf)
    d.a_scale, d.b_scale = float(a_scale), float(b_scale)
    d.bias, d.residual = _ptr(bias), _ptr(residual)
    d.ldc = int(ldc)
    d.b_scale2 = float(b_scale2)
    d.flags = ((nv.FLAG_CLC_SCHEDULER if scheduler == "clc" else 0) | (nv.FLAG_STATIC_WEIGHTS if static_weights else 0)
               | (nv.FLAG_TAIL_SPLIT if tail_split else 0))
    return d


class GemmPlan:
    """One planned GEMM: C[M,N] = epilogue(a_scale*b_scale * A[M,K] x B^T) -- see blz_gemm_desc."""

    def __init__(self, kind: str, M: int, N: int, K: int, A, B, *, A_sf=None, B_sf=None, a_scale: float = 1.0,
                 b_scale: float = 1.0, out_dtype: str = "bf16", epilogue: str = "none", bias=None, residual=None,
                 b_layout: str = "kmajor", a_sf_layout: str = "rowmajor", b_sf_layout: str = "rowmajor",
                 variant: str = "auto", ldc: int = 0, b_scale2: float = 0.0, scheduler: str = "static",
                 static_weights: bool = False, tail_split: bool = False):
        L = nv.lib()
        d = make_desc(kind, M, N, K, A, B, A_sf=A_sf, B_sf=B_sf, a_scale=a_scale, b_scale=b_scale, out_dtype=out_dtype, epilogue=epilogue,
                      bias=bias, residual=residual, b_layout=b_layout, a_sf_layout=a_sf_layout, b_sf_layout=b_sf_layout, variant=variant,
                      ldc=ldc, b_scale2=b_scale2, scheduler=scheduler, static_weights=static_weights, tail_split=tail_split)
        self._keep = (A, B, A_sf, B_sf, bias, residual)   # operands must outlive the plan
        self._handle = ctypes.c_void_p()
        self.kind, self.M, self.N, self.K, self.out_dtype = kind, int(M), int(N), int(K), out_dtype
        nv.check("blz_gemm_plan_create", L.blz_gemm_plan_create(ctypes.byref(d), ctypes.byref(self._handle)))

    def execute(self, C, stream=None) -> None:
        nv.check("blz_gemm_execute", nv.lib().blz_gemm_execute(self._handle, _ptr(C), _stream(stream)))

    def execute_gather(self, dst_ptrs, ld_total: int, col_offset: int, stream=None) -> None:
        """Fused GEMM + all-gather: writes this plan's [M, N] block at columns [col_offset, ...) of every
        full-width output in `dst_ptrs` (device pointers, own buffer and peers')."""
        n = len(dst_ptrs)
        arr = (ctypes.c_void_p * n)(*[int(x) for x in dst_ptrs])
        nv.check("blz_gemm_execute_gather", nv.lib().blz_gemm_execute_gather(self._handle, n, arr, int(ld_total), int(col_offset), _stream(stream)))

    def set_a(self, A, A_sf=None, a_scale: float = 0.0) -> None:
        nv.check("blz_gemm_plan_set_a", nv.lib().blz_gemm_plan_set_a(self._handle, _ptr(A), _ptr(A_sf), float(a_scale)))
        self._keep = (A, A_sf) + self._keep[1:]

    def refresh_weights(self, stream=None) -> None:
        """static_weights plans: expand the packed weights again after they changed in place."""
        nv.check("blz_gemm_plan_refresh_weights", nv.lib().blz_gemm_plan_refresh_weights(self._handle, _stream(stream)))

    def check(self, stream=None) -> None:
        """Synchronises the stream and raises if a kernel of this plan gave up on a device-side wait."""
        nv.check("blz_gemm_plan_check", nv.lib().blz_gemm_plan_check(self._handle, _stream(stream)))

    def info(self) -> dict:
        i = nv.PlanInfo()
        nv.check("blz_gemm_plan_info", nv.lib().blz_gemm_plan_info(self._handle, ctypes.byref(i)))
        return {name: getattr(i, name) for name, _ in nv.PlanInfo._fields_}

    def destroy(self) -> None:
        if self._handle:
            nv.lib().blz_gemm_plan_destroy(self._handle)
            self._handle = ctypes.c_void_p()

    def __del__(self):
        try:
            self.destroy()
        except Exception:
            pass


# ---------------------------------------------------------------- Blaze-named mirrors

def create_fp8_gemm_plan(A, B, M, N, K, bias=None, epilogue: str = "none") -> GemmPlan:
    """A [M,K] E4M3, B [K,N] E4M3 (row-major), fp16 output, no scales (Blaze's signature has none)."""
    return GemmPlan("fp8", M, N, K, A, B, out_dtype="f16", epilogue=epilogue, bias=bias, b_layout="nmajor")


def create_fp4_blkscaled_gemm_plan(A: dict, B: dict, M, N, K, bias=None, epilogue: str = "none") -> GemmPlan:
    """A / B are dicts with Blaze's Fp4BlkScaledWeightTensor fields: data, block_scales,
    tensor_scale (A: data [M,K/2], scales [M,K/16]; B: data [K,N/2], scales [K/16,N])."""
    return GemmPlan("nvfp4", M, N, K, A["data"], B["data"], A_sf=A["block_scales"], B_sf=B["block_scales"],
                    a_scale=A["tensor_scale"], b_scale=B["tensor_scale"], out_dtype="f16", epilogue=epilogue, bias=bias,
                    b_layout="nmajor")


create_fp4_gemm_plan = create_fp4_blkscaled_gemm_plan
create_fp4_blkscaled_persistent_gemm_plan = create_fp4_blkscaled_gemm_plan


def create_mixed_gemm_plan(A, B: dict, M, N, K, bias=None, residual=None, epilogue: str = "none") -> GemmPlan:
    """fp16 activations A [M,K] x NVFP4 weights B (Fp4WeightTensor fields, [K,N] convention)."""
    return GemmPlan("w4a16_f16", M, N, K, A, B["data"], B_sf=B["block_scales"], b_scale=B["tensor_scale"], out_dtype="f16",
                    epilogue=epilogue, bias=bias, residual=residual, b_layout="nmajor", static_weights=True)


def interleave_gate_up(gate, up, group_bytes: int, stream=None):
    """Groups of `group_bytes` bytes alternately from two equally sized uint8 tensors (blz_interleave_gate_up):
    the weight layout the "swiglu" epilogue expects."""
    import torch  # noqa: PLC0415
    nbytes = gate.numel() * gate.element_size()
    assert nbytes == up.numel() * up.element_size() and nbytes % group_bytes == 0
    out = torch.empty(2 * nbytes, dtype=torch.uint8, device=gate.device)
    nv.check("blz_interleave_gate_up", nv.lib().blz_interleave_gate_up(gate.data_ptr(), up.data_ptr(), out.data_ptr(), nbytes // group_bytes,
                                                                        int(group_bytes), _stream(stream)))
    return out


def create_fused_gate_up_plan(x, W_gate: dict, W_up: dict, M, N, K) -> GemmPlan:
    """output[M, N] = silu(x W_gate) * (x W_up) in one kernel: fp16 activations x [M, K], two NVFP4
    weights with Blaze's Fp4WeightTensor fields ([K, N] convention), N a multiple of 16.
    Mirrors launch_fused_gate_up (Blaze: include/gemm/mixed_gemm_sm100.cuh:87-109)."""
    data = interleave_gate_up(W_gate["data"], W_up["data"], 8)                    # [K, N/2] bytes: 16 columns per group
    sf = interleave_gate_up(W_gate["block_scales"], W_up["block_scales"], 16)      # [K/16, N] bytes
    return GemmPlan("w4a16_f16", M, 2 * N, K, x, data, B_sf=sf, b_scale=W_gate["tensor_scale"], b_scale2=W_up["tensor_scale"],
                    out_dtype="f16", epilogue="swiglu", b_layout="nmajor")


def create_fp16_gemm_plan(A, B_colmajor, M, N, K) -> GemmPlan:
    """Dense fp16: A row-major, B column-major (stored [N,K]), fp32 output."""
    return GemmPlan("f16", M, N, K, A, B_colmajor, out_dtype="f32")


def _execute(plan: GemmPlan, C, stream=None) -> None:
    plan.execute(C, stream)


def _destroy(plan) -> None:
    if plan is not None:
        plan.destroy()


execute_fp8_gemm = execute_fp4_gemm = execute_fp4_blkscaled_gemm = execute_fp4_blkscaled_persistent_gemm = _execute
execute_mixed_gemm = execute_fp16_gemm = _execute
destroy_fp8_gemm_plan = destroy_fp4_gemm_plan = destroy_fp4_blkscaled_gemm_plan = _destroy
destroy_fp4_blkscaled_persistent_gemm_plan = destroy_mixed_gemm_plan = destroy_fp16_gemm_plan = _destroy


# ---------------------------------------------------------------- operand preparation

def _dtype_code(t) -> int:
    import torch  # noqa: PLC0415
    return {torch.float32: nv.F32, torch.float16: nv.F16, torch.bfloat16: nv.BF16}[t.dtype]


def tiled_scales_bytes(rows: int, K: int) -> int:
    return int(nv.lib().blz_tiled_scales_bytes(int(rows), int(K)))


def amax(x, out=None, stream=None):
    """max |x| as a 1-element fp32 device tensor (combined with `out` when given)."""
    import torch  # noqa: PLC0415
    x = x.contiguous()
    if out is None:
        out = torch.zeros(1, dtype=torch.float32, device=x.device)
    nv.check("blz_amax", nv.lib().blz_amax(x.data_ptr(), _dtype_code(x), x.numel(), out.data_ptr(), _stream(stream)))
    return out


def quantize_fp8(x, stream=None):
    """Per-tensor E4M3: returns (codes uint8 like x, scales fp32[2] = {s, 1/s}) with s = 448/amax."""
    import torch  # noqa: PLC0415
    x = x.contiguous()
    am = amax(x, stream=stream)
    q = torch.empty(x.shape, dtype=torch.uint8, device=x.device)
    scales = torch.empty(2, dtype=torch.float32, device=x.device)
    nv.check("blz_quantize_fp8", nv.lib().blz_quantize_fp8(x.data_ptr(), _dtype_code(x), x.numel(), am.data_ptr(), q.data_ptr(),
                                                             scales.data_ptr(), _stream(stream)))
    return q, scales


def quantize_nvfp4(x, tiled: bool = False, stream=None):
    """Two-level NVFP4 of a [rows, K] matrix: (data uint8 [rows,K/2], sf uint8, g fp32[1]).
    sf is [rows, K/16] row-major, or the flat tiled array when tiled=True."""
    import torch  # noqa: PLC0415
    x = x.contiguous()
    rows, K = x.shape
    am = amax(x, stream=stream)
    data = torch.empty((rows, K // 2), dtype=torch.uint8, device=x.device)
    if tiled:
        sf = torch.empty(tiled_scales_bytes(rows, K), dtype=torch.uint8, device=x.device)
    else:
        sf = torch.empty((rows, K // 16), dtype=torch.uint8, device=x.device)
    g = torch.empty(1, dtype=torch.float32, device=x.device)
    nv.check("blz_quantize_nvfp4", nv.lib().blz_quantize_nvfp4(x.data_ptr(), _dtype_code(x), rows, K, am.data_ptr(), data.data_ptr(),
                                                                 sf.data_ptr(), nv.SF_TILED if tiled else nv.SF_ROWMAJOR, g.data_ptr(),
                                                                 _stream(stream)))
    return data, sf, g


def tile_scales(sf, rows: int, K: int, row_stride: int | None = None, blk_stride: int = 1, stream=None):
    """Row-major E4M3 scales -> the tiled layout (flat uint8 tensor)."""
    import torch  # noqa: PLC0415
    if row_stride is None:
        row_stride = K // 16
    out = torch.empty(tiled_scales_bytes(rows, K), dtype=torch.uint8, device=sf.device)
    nv.check("blz_tile_scales", nv.lib().blz_tile_scales(sf.data_ptr(), rows, K, row_stride, blk_stride, out.data_ptr(), _stream(stream)))
    return out


# ---------------------------------------------------------------- allocation-free decode GEMM

def gemm_nvfp4_decode_static(A, A_sf_tiled, a_scale: float, B, B_sf_tiled, b_scale: float, M: int, N: int, K: int, C,
                             out_dtype: str = "bf16", ldc: int = 0, status=None, stream=None) -> None:
    """blz_gemm_nvfp4_decode_static: the skinny-M NVFP4 GEMM for callers that must not allocate
    device memory (an inference runtime that owns all of HBM through its own arena, a loop that
    cannot take an allocation's synchronisation).  Scales must already be in the tiled layout; the
    split-K workspace is a fixed array inside the library, shared by every call on the device."""
    nv.check("blz_gemm_nvfp4_decode_static", nv.lib().blz_gemm_nvfp4_decode_static(
        _ptr(A), _ptr(A_sf_tiled), float(a_scale), _ptr(B), _ptr(B_sf_tiled), float(b_scale), int(M), int(N), int(K), _ptr(C),
        nv.DTYPES[out_dtype], int(ldc), _ptr(status), _stream(stream)))
