/* ref_more.cu -- libr3d's r3d_more.hip (the file that holds rmsnorm_quant_fp8) compiled from where
 * it lies in the mounted reference tree (never copied), through nvcc for sm_100a with
 * oracle/hipstub standing in for the HIP runtime header and this repository's rad_*.h stand-ins for
 * radiance's. The reference's own kernel and entry then run on the B200 beside this library's.
 * TEST INFRASTRUCTURE ONLY. */
#include <cuda_runtime.h>
#include <cstdint>
#include "r3d_more.hip"

void r3d_dump_begin(R3dDumpSlot* slot, const char*, const void*, const RadArgs*, RadStream) { if (slot) slot->priv = nullptr; }
void r3d_dump_end(R3dDumpSlot*, int) {}

#define REF_API extern "C" __attribute__((visibility("default")))
REF_API int ref_more_rmsnorm_quant_fp8(const RadArgs* a, void* stream) { return r3d_rad_rmsnorm_quant_fp8(a, (RadStream)stream); }
REF_API int ref_more_row_topk(const RadArgs* a, void* stream) { return r3d_rad_row_topk(a, (RadStream)stream); }
