/* tc_common.cuh -- device-side helpers shared by the tcgen05 kernels: mbarrier waits with a
 * bounded spin, TMA tile loads, shared-memory matrix descriptors, TMEM loads, cluster access.
 * Every wait gives up after ~1 s of clock64 and records a code in the status word the including
 * file names with R3D_TC_STATUS_WORD (a __device__ int of that translation unit). */
#pragma once
#include <cuda.h>
#include <cuda_fp16.h>
#include <cstdint>
#include "r3d_kernels.h"
#include "r3d_numerics.cuh"

namespace r3d {

namespace tcdev {

constexpr long long kTcSpin = 2000000000LL;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;"
                 ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
/* mbarrier.try_wait may suspend the thread until the phase completes or a hardware time limit
 * passes: a waiting warp then issues a handful of instructions per microsecond instead of
 * spinning on test_wait, which took issue slots from the warps that had work */
__device__ __forceinline__ bool mbar_try(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int code) {
    if (mbar_try(bar, parity)) return true;
    const long long t0 = clock64();
    while (!mbar_try(bar, parity)) {
        if (clock64() - t0 > kTcSpin) { atomicExch(&R3D_TC_STATUS_WORD, code); return false; }
    }
    return true;
}
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile(
        "{\n\t.reg .pred P;\n\t"
        "elect.sync _|P, 0xffffffff;\n\t"
        "selp.u32 %0, 1, 0, P;\n\t}"
        : "=r"(pred));
    return pred != 0;
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y,
                                            uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y) : "memory");
}

/* shared-memory matrix descriptor: K-major operand, 128-byte swizzle, rows of 128 bytes, 8-row
 * swizzle atoms stacked 1024 bytes apart; descriptor version 1 */
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t saddr) {
    return (uint64_t)((saddr >> 4) & 0x3FFFu) | (1ull << 16) | (64ull << 32) | (1ull << 46) |
           (2ull << 61);
}
__device__ __forceinline__ void umma_f8f6f4(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc,
                                            uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
                 ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
/* tcgen05.ld 32x32b: thread i of the warp reads N consecutive 32-bit columns of TMEM lane
 * (lane base + i) */
__device__ __forceinline__ void tmem_ld1(uint32_t taddr, float* v) {
    uint32_t r0;
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x1.b32 {%0}, [%1];" : "=r"(r0) : "r"(taddr) : "memory");
    v[0] = __uint_as_float(r0);
}
__device__ __forceinline__ void tmem_ld2(uint32_t taddr, float* v) {
    uint32_t r0, r1;
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x2.b32 {%0,%1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(taddr) : "memory");
    v[0] = __uint_as_float(r0); v[1] = __uint_as_float(r1);
}
__device__ __forceinline__ void tmem_ld4(uint32_t taddr, float* v) {
    uint32_t r[4];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(taddr) : "memory");
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, float* v) {
    uint32_t r[8];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
                   "=r"(r[7]) : "r"(taddr) : "memory");
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float* v) {
    uint32_t r[16];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15])
        : "r"(taddr) : "memory");
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}
/* the first ML columns (ML = 1, 2, 4, 8 or a multiple of 16) */
template <int ML>
__device__ __forceinline__ void tmem_ld(uint32_t taddr, float* v) {
    if (ML == 1) tmem_ld1(taddr, v);
    else if (ML == 2) tmem_ld2(taddr, v);
    else if (ML == 4) tmem_ld4(taddr, v);
    else if (ML == 8) tmem_ld8(taddr, v);
    else {
#pragma unroll
        for (int h = 0; h < ML / 16; ++h) tmem_ld16(taddr + h * 16, v + h * 16);
    }
}
__device__ __forceinline__ void tmem_ld_wait() {
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
/* tcgen05.ld is asynchronous: its destination registers hold the data only after tcgen05.wait::ld.
 * The wait instruction does not name those registers, so nothing stops the compiler from moving
 * arithmetic on them above it. These empty statements "rewrite" the registers right after the wait
 * (volatile statements keep their order), which pins every use behind it. */
__device__ __forceinline__ void tmem_pin8(float* v) {
    asm volatile("" : "+f"(v[0]), "+f"(v[1]), "+f"(v[2]), "+f"(v[3]), "+f"(v[4]), "+f"(v[5]), "+f"(v[6]), "+f"(v[7]));
}
__device__ __forceinline__ void tmem_pin16(float* v) { tmem_pin8(v); tmem_pin8(v + 8); }
template <int N>
__device__ __forceinline__ void tmem_pin(float* v) {
    if (N == 1) asm volatile("" : "+f"(v[0]));
    else if (N == 2) asm volatile("" : "+f"(v[0]), "+f"(v[1]));
    else if (N == 4) asm volatile("" : "+f"(v[0]), "+f"(v[1]), "+f"(v[2]), "+f"(v[3]));
    else {
#pragma unroll
        for (int i = 0; i < N / 8; ++i) tmem_pin8(v + 8 * i);
    }
}

__device__ __forceinline__ float ld_scale(const uint8_t* base, int64_t idx, int dt) {
    if (dt == RAD_F32) return __ldg((const float*)base + idx);
    if (dt == RAD_F16) return __half2float(__ushort_as_half(__ldg((const unsigned short*)base + idx)));
    return bf16_to_f32(__ldg((const uint16_t*)base + idx));
}
__device__ __forceinline__ int scale_col(int c, int cols, int nchunk) {
    return cols == nchunk ? c : (cols == 1 ? 0 : (int)((int64_t)c * cols / nchunk));
}

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float ld_peer_f32(const float* local, uint32_t rank) {
    uint32_t ra;
    float v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(smem_u32(local)), "r"(rank));
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(ra) : "memory");
    return v;
}

__device__ __forceinline__ void tmem_st1(uint32_t taddr, uint32_t v) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x1.b32 [%0], {%1};" ::"r"(taddr), "r"(v) : "memory");
}
/* kind::mxf8f6f4 with hardware block scaling, one E8M0 scale per operand row per K=32 instruction:
 * the scale words live in tensor memory at sfa / sfb */
__device__ __forceinline__ void umma_mxf8(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                          uint32_t sfa, uint32_t sfb, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %6, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale.scale_vec::1X [%0], %1, %2, %3, [%4], [%5], p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(sfa), "r"(sfb), "r"(accumulate) : "memory");
}
/* Programmatic dependent launch: the next kernel in the stream may start its own prologue as
 * soon as every CTA of this grid has said so; a kernel reads what its predecessor wrote only
 * after dep_wait(), which returns once the predecessor has completed and flushed. */
__device__ __forceinline__ void dep_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void dep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }


/* true unless R3D_NO_PDL is set: kernels are launched with programmatic stream serialisation */
} /* namespace tcdev */

bool tc_pdl_on();

/* host side (kern_tc.cu): cached 2-D tensor maps, box = box0 x box1 elements; an inner box of 128
 * elements gets the 128-byte swizzle, any other none */
const CUtensorMap* tc_tensor_map(const void* ptr, uint64_t d0, uint64_t d1, uint64_t pitch_bytes,
                                 CUtensorMapDataType dt, uint32_t box1, uint32_t box0 = 128u, int promo128 = 0);
/* the current device's ordinal, or -1 (no device, or beyond kTcMaxDevices): function attributes and
 * device properties are remembered per device, one process may drive several GPUs */
constexpr int kTcMaxDevices = 64;
int  tc_device();
bool tc_have_encoder();
int  tc_sm_count();

} /* namespace r3d */
