"""Generates the golden vectors under tests/golden/ from Blaze's own host functions.

Runs only where the reference tree is present: it loads oracle/_ref/libblaze_ref_naive.so (Blaze's
tests/test_gemm_naive.cu compiled where it lies, see oracle/build_oracle.py) and records what
Blaze's init_random_fp16 (seeds 42 / 123, tests/test_gemm_naive.cu:79-80) and gemm_cpu_fp16
(:38-48) produce.  The parity tests then need neither the reference tree nor that library.

    python tests/golden/make_golden.py
"""
import hashlib
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from oracle import build_oracle  # noqa: E402
from oracle import oracle as O  # noqa: E402


def sha(a: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def main() -> None:
    build_oracle.build_all()
    assert O.ref_available(), "oracle/_ref is not built (reference tree missing?)"
    # small case, everything stored: M, N, K = 48, 80, 96 (ragged against every tile size)
    M, N, K = 48, 80, 96
    A = O.ref_init_random_fp16(M * K, 42).reshape(M, K)
    B = O.ref_init_random_fp16(K * N, 123).reshape(K, N)
    C = O.ref_gemm_cpu_fp16(A, B)
    np.savez_compressed(os.path.join(HERE, "ref_gemm_cpu_fp16_48x80x96.npz"), A=A, B=B, C=C)
    # the 256^3 fp16 configuration: operands are regenerated from the seeds; digests and sampled rows stored
    M = N = K = 256
    A = O.ref_init_random_fp16(M * K, 42).reshape(M, K)
    B = O.ref_init_random_fp16(K * N, 123).reshape(K, N)
    C = O.ref_gemm_cpu_fp16(A, B)
    rows = np.array([0, 1, 37, 127, 128, 200, 255])
    np.savez_compressed(os.path.join(HERE, "ref_gemm_cpu_fp16_256.npz"), rows=rows, C_rows=C[rows],
                        A_head=A.reshape(-1)[:64], B_head=B.reshape(-1)[:64],
                        sha_A=np.array(sha(A)), sha_B=np.array(sha(B)), sha_C=np.array(sha(C)))
    # byte patterns Blaze's tests rely on (tests/test_gemm.cu:193-194, 338-342): decoded by CUDA's
    # own host conversions when pin_formats ran; recorded here as the known answers
    np.savez_compressed(os.path.join(HERE, "known_bytes.npz"),
                        e4m3_codes=np.array([0x38, 0x3C], np.uint8), e4m3_values=np.array([1.0, 1.5], np.float32),
                        e2m1_codes=np.array([0x2, 0x5], np.uint8), e2m1_values=np.array([1.0, 3.0], np.float32))
    print("golden vectors written to", HERE)


if __name__ == "__main__":
    main()
