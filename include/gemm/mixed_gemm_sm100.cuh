// mixed_gemm_sm100.cuh -- kept under this name so programs written against Blaze's include/gemm tree build
// unchanged; every declaration lives in blaze_gemm.cuh.
#pragma once
#include "blaze_gemm.cuh"
