/* ref_band.cu -- libr3d's activation-producer file compiled from where it lies in the mounted
 * reference tree (never copied): src/r3d_band.hip, through nvcc with oracle/hipstub standing in
 * for the HIP runtime header and this repository's rad_*.h stand-ins for radiance's. Its pure
 * helpers (the bf16 narrowing, the e4m3 encoder, the sigmoid) are exported for the CPU so that the
 * oracle's restatements can be compared with the reference's own compiled code over every input
 * class. TEST INFRASTRUCTURE ONLY. */
#include <cuda_runtime.h>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include "hip/hip_runtime.h"
#include "ref_host_pass.h"
#include "rad_abi.h"
#include "rad_plugin.h"
/* The file holds one empty `asm volatile("" : "+v"(..))` statement: an AMD vector-register
 * constraint used as a code-motion barrier. It has no instructions; these two definitions
 * (made after every system header above is in) turn it into an empty statement. */
#define asm
#define volatile(...)
/* make the reference's __device__ helpers callable on the host as well */
#undef __device__
#define __device__ __location__(host) __location__(device)
#include "r3d_band.hip"

/* the file wraps its entries in an operand-capture hook (r3d_dump.h); the pin keeps it inert */
void r3d_dump_begin(R3dDumpSlot* slot, const char*, const void*, const RadArgs*, RadStream) { if (slot) slot->priv = nullptr; }
void r3d_dump_end(R3dDumpSlot*, int) {}

#define REF_API extern "C" __attribute__((visibility("default")))
REF_API unsigned char ref_band_f32_to_e4m3(float f) { return r3d_f32_to_e4m3(f); }
REF_API unsigned short ref_band_f32_to_bf16(float f) { return r3d_f32_to_bf16(f); }
REF_API float ref_band_sigmoid(float x) { return r3d_sigmoid(x); }
REF_API void ref_band_f32_to_e4m3_n(const float* x, long long n, unsigned char* out) {
    for (long long i = 0; i < n; ++i) out[i] = r3d_f32_to_e4m3(x[i]);
}
/* The reference's own quantiser rows (kernels and entries compiled above for sm_100a), for a
 * device-executed comparison: same RadArgs the engine would pass. */
REF_API int ref_band_quant_act_fp8(const RadArgs* a, void* stream) { return r3d_rad_quant_act_fp8(a, (RadStream)stream); }
REF_API int ref_band_gated_quant_fp8(const RadArgs* a, void* stream) { return r3d_rad_gated_quant_fp8(a, (RadStream)stream); }
