/* hip/hip_fp16.h stand-in for the reference pin builds: CUDA's half type under the same names. */
#pragma once
#include <cuda_fp16.h>
