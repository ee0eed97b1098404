"""Small CUDA programs written against Blaze's own names.

Blaze's low-level helper names (gemm/tma_utils.cuh, gemm/tmem_utils.cuh): a one-tile GEMM written
only with those names is compiled here (CPU) and run on the GPU, where it must reproduce the known
answer of Blaze's primitive test (all-ones E4M3 tile = K) and a position-dependent case exactly.
launch_fused_gate_up (namespace blaze, Blaze's Fp4WeightTensor layout): a program with exactly
representable operands is linked against the library and checked against first-principles values."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, "tests", "compat_primitives.cu")


def _nvcc():
    return os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"


def _build(out_dir) -> str:
    exe = os.path.join(str(out_dir), "compat_primitives")
    r = subprocess.run([_nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-O2", "-std=c++17", "-I", os.path.join(ROOT, "include"), SRC, "-o", exe],
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-2000:]
    return exe


def test_helper_name_program_compiles(tmp_path):
    if not os.path.exists(_nvcc()):
        pytest.skip("nvcc not available")
    assert os.path.exists(_build(tmp_path))


@pytest.mark.gpu
def test_helper_name_program_known_answers(tmp_path, cuda_device):
    if not os.path.exists(_nvcc()):
        pytest.skip("nvcc not available")
    exe = _build(tmp_path)
    r = subprocess.run([exe], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0 and "PASS" in r.stdout, (r.stdout + r.stderr)[-2000:]


GATE_UP_SRC = os.path.join(ROOT, "tests", "compat_gate_up.cu")


def _build_gate_up(out_dir, native_lib) -> str:
    exe = os.path.join(str(out_dir), "compat_gate_up")
    lib_dir = os.path.join(ROOT, "blaze_b200")
    r = subprocess.run([_nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-O2", "-std=c++17", "-I", os.path.join(ROOT, "include"), GATE_UP_SRC,
                        "-L", lib_dir, "-lblaze_b200", "-Xlinker", "-rpath", "-Xlinker", lib_dir, "-o", exe], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-2000:]
    return exe


def test_gate_up_program_compiles(tmp_path, native_lib):
    if not os.path.exists(_nvcc()):
        pytest.skip("nvcc not available")
    assert os.path.exists(_build_gate_up(tmp_path, native_lib))


@pytest.mark.gpu
def test_gate_up_program_known_answers(tmp_path, native_lib, cuda_device):
    if not os.path.exists(_nvcc()):
        pytest.skip("nvcc not available")
    exe = _build_gate_up(tmp_path, native_lib)
    r = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "PASS" in r.stdout, (r.stdout + r.stderr)[-2000:]
