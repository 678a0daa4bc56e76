/* ref_fp8a8.cu -- libr3d's fp8a8 band file compiled from where it lies in the mounted reference
 * tree (never copied): src/r3d_gemm_fp8a8.hip, through nvcc for sm_100a with oracle/hipstub standing
 * in for the HIP and rocWMMA headers and this repository's rad_*.h stand-ins for radiance's. The
 * reference's own kernels and entries then run on the B200 beside this library's, on the same
 * operands. TEST INFRASTRUCTURE ONLY. */
#include <cuda_runtime.h>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>
#include "hip/hip_runtime.h"
#include "hip/hip_fp16.h"
#include "rocwmma/rocwmma.hpp"
/* The file holds one AMD instruction in inline asm (the f16-pair dot of an arm that an environment
 * lever switches on and that is off by default). nvcc cannot assemble it, so, with every system
 * header above already in, the statement is defined away; that arm is never selected here. */
#define asm(...)
#include "r3d_gemm_fp8a8.hip"
#undef asm

void r3d_dump_begin(R3dDumpSlot* slot, const char*, const void*, const RadArgs*, RadStream) { if (slot) slot->priv = nullptr; }
void r3d_dump_end(R3dDumpSlot*, int) {}

#define REF_API extern "C" __attribute__((visibility("default")))
REF_API int ref_fp8a8_gemm_nt_q(const RadArgs* a, void* stream) { return r3d_rad_gemm_nt_q_fp8(a, (RadStream)stream); }
REF_API int ref_fp8a8_gemm_nt_q_decode(const RadArgs* a, void* stream) { return r3d_rad_gemm_nt_q_fp8_decode(a, (RadStream)stream); }
REF_API int ref_fp8a8_gemm_nt_q_gated(const RadArgs* a, void* stream) { return r3d_rad_gemm_nt_q_gated_fp8(a, (RadStream)stream); }
