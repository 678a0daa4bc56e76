/* ref_w2a8_host.cpp -- the host-only part of libr3d's w2a8 file (its three layout hooks), compiled from
 * where it lies in the mounted reference tree (never copied): src/r3d_gemm_w2a8.hip under
 * R3D_W2A8_HOST_GATE, the switch the reference's own tools/gate_w2a8.cpp uses to include just these
 * hooks, with this repository's rad_*.h stand-ins for radiance's headers. TEST INFRASTRUCTURE ONLY. */
#define R3D_W2A8_HOST_GATE 1
#include "r3d_gemm_w2a8.hip"

#define REF_API extern "C" __attribute__((visibility("default")))
REF_API int ref_layout_gemm_w2a8(const RadParam* p, int n_p, int operand, const RadEncoding* enc, const int* sel,
                                 const RadTensor* planes, int n, RadLayout* out) {
    return r3d_layout_gemm_w2a8(p, n_p, operand, enc, sel, planes, n, out);
}
