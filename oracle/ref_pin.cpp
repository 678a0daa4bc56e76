/* ref_pin.cpp -- the one piece of libr3d that is plain C++ and builds with g++ here,
 * compiled from where it lies in the mounted reference tree (never copied):
 * src/r3d_mxfp4_q8x.h (the doubled e2m1 table and the E8M0 decode the q8x arm ships).
 * The Makefile passes -I<reference>/src and neutralises the two HIP qualifiers.
 * TEST INFRASTRUCTURE ONLY: tests compare oracle/r3d_oracle.cpp's tables against these. */
#include "r3d_mxfp4_q8x.h"

extern "C" __attribute__((visibility("default"))) int ref_e2m1_x2(int code) {
    static const int8_t lut[16] = R3D_E2M1_X2;
    return lut[code & 15];
}
extern "C" __attribute__((visibility("default"))) float ref_e8m0_sc(unsigned char x) {
    return r3d_e8m0_sc((uint8_t)x);
}
