/* launch.cu -- the thin C ABI between the host-side row entries and the CUDA kernels
 * (declared in r3d_b200.h). Operands arrive validated; this layer only picks an arm.
 * There is no CPU path: when no CUDA device of the right generation is present every call
 * returns RAD_E_UNSUPPORTED, loudly once. */
#include "r3d_kernels.h"
#include "push.cuh"
#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>

namespace r3d {

static std::atomic<long long> g_launches{0};
void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

/* The kernels are compiled for sm_100a only. Checked once per device (the reference's chip gate:
 * src/r3d_gemm_fp8a8.hip:903-913); one process may drive several GPUs. */
bool device_is_sm100() {
    static signed char ok[64] = {};                       /* 0 unknown, 1 yes, -1 no */
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
        static bool said = false;
        if (!said) fprintf(stderr, "libr3d_b200: no usable CUDA device -- every row refuses\n");
        said = true;
        (void)cudaGetLastError();
        return false;
    }
    if (!ok[dev]) {
        int major = 0, minor = 0;
        if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess ||
            cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, dev) != cudaSuccess) {
            fprintf(stderr, "libr3d_b200: device %d cannot be queried -- every row refuses\n", dev);
            (void)cudaGetLastError();
            ok[dev] = -1;
        } else {
            ok[dev] = major == 10 ? 1 : -1;
            if (major != 10)
                fprintf(stderr, "libr3d_b200: device %d is sm_%d%d; this library holds sm_100a code only -- "
                                "every row refuses\n", dev, major, minor);
        }
    }
    return ok[dev] == 1;
}

static void debug_arm(const char* band, const char* arm, int m) {
    /* one line per distinct (band, arm), the reference's R3D_DEBUG_GEMM law
     * (src/r3d_gemm_fp8a8.hip:976-983): a lever that never dispatches must not look live */
    static const bool on = getenv("R3D_DEBUG_GEMM") != nullptr;
    if (!on) return;
    static char seen[16][48];
    static int nseen = 0;
    char key[48];
    snprintf(key, sizeof key, "%s/%s", band, arm);
    for (int i = 0; i < nseen; ++i) if (!strcmp(seen[i], key)) return;
    if (nseen < 16) { strcpy(seen[nseen++], key); }
    fprintf(stderr, "libr3d_b200: %s -> %s arm launched (m=%d)\n", band, arm, m);
}

} /* namespace r3d */

using namespace r3d;

/* AUTO: the tcgen05 arm when the operands meet TMA's alignment rules, else the mma.sync
 * streaming arm, else the oracle-order arm (any shape, any alignment). M above one pass is
 * probed at the pass size. */
/* R3D_NO_GEMM=1 keeps M > 64 on passes of the decode kernels (each pass re-reads the weights) */
static bool no_gemm() {
    static const bool off = [] { const char* e = getenv("R3D_NO_GEMM"); return e && *e && *e != '0'; }();
    return off;
}
static int auto_arm_fp8a8(const R3dGemmQ& q) {
    R3dGemmQ probe = q; if (probe.m > 64) probe.m = 64;
    if (tc_fp8a8_ok(probe)) return R3D_ARM_TILE;
    return stream_fp8a8_ok(probe) ? R3D_ARM_STREAM : R3D_ARM_EXACT;
}
static int auto_arm_mxfp4a8(const R3dGemmQ& q) {
    static const bool pack_off = [] { const char* e = getenv("R3D_NO_PACK"); return e && *e && *e != '0'; }();
    /* measured: above M = 4 the packed kernel's single accumulator buffer loses to the unpacking kernel */
    static const int pack_max = [] { const char* e = getenv("R3D_PACK_MAXM"); const int v = e ? atoi(e) : 0; return v >= 1 && v <= 8 ? v : 4; }();
    if (!pack_off && q.m <= pack_max && tc_mxf4_ok(q)) return R3D_ARM_PACK;
    R3dGemmQ probe = q; if (probe.m > 32) probe.m = 32;
    if (tc_mxfp4a8_ok(probe)) return R3D_ARM_TILE;
    probe = q; if (probe.m > 64) probe.m = 64;
    return stream_mxfp4a8_ok(probe) ? R3D_ARM_STREAM : R3D_ARM_EXACT;
}

extern "C" long long r3d_b200_launch_count(void) { return g_launches.load(); }

extern "C" int r3d_b200_pick_arm_fp8a8(const R3dGemmQ* q) {
    if (!q) return -1;
    if (q->arm != R3D_ARM_AUTO) return q->arm;
    return auto_arm_fp8a8(*q);
}
extern "C" int r3d_b200_pick_arm_mxfp4a8(const R3dGemmQ* q) {
    if (!q) return -1;
    if (q->arm != R3D_ARM_AUTO) return q->arm;
    return auto_arm_mxfp4a8(*q);
}

/* M above the streaming arm's 64 rides it in passes of 64 tokens, each pass re-reading the
 * weights (the reference's own rule for M above its register group,
 * src/r3d_gemm_logits.hip:24-26). */
template <typename OkFn, typename RunFn>
static int gemm_passes(const R3dGemmQ& q, OkFn ok, RunFn run, cudaStream_t st, int step = 64) {
    for (int m0 = 0; m0 < q.m; m0 += step) {
        R3dGemmQ c = q;
        c.m = q.m - m0 < step ? q.m - m0 : step;
        c.a = (const uint8_t*)q.a + (int64_t)m0 * q.a_pitch;
        c.a_scale = q.a_scale + (int64_t)m0 * q.as_pitch;
        c.y = (uint16_t*)q.y + (int64_t)m0 * q.y_pitch;
        if (!ok(c)) return RAD_E_UNSUPPORTED;
        const int rc = run(c, st);
        if (rc != RAD_OK) return rc;
    }
    return RAD_OK;
}

extern "C" int r3d_b200_gemm_fp8a8(const R3dGemmQ* q, void* stream) {
    if (!q || !device_is_sm100()) return RAD_E_UNSUPPORTED;
    cudaStream_t st = (cudaStream_t)stream;
    int arm = q->arm;
    if (arm == R3D_ARM_AUTO) arm = auto_arm_fp8a8(*q);
    if (arm == R3D_ARM_STREAM) {
        debug_arm("fp8a8", "stream", q->m);
        return gemm_passes(*q, stream_fp8a8_ok, stream_fp8a8, st);
    }
    if (arm == R3D_ARM_EXACT) { debug_arm("fp8a8", "exact", q->m); return exact_fp8a8(*q, st); }
    if (arm == R3D_ARM_TILE) {
        if (q->m > 64 && !no_gemm() && tc_gemm_ws_fp8a8_ok(*q)) {
            debug_arm("fp8a8", "tcgen05 pair tile, one accumulation over K", q->m);
            return tc_gemm_ws_fp8a8(*q, st);
        }
        if (q->m > 64 && !no_gemm() && tc_gemm_fp8a8_ok(*q)) {
            debug_arm("fp8a8", "tcgen05 tile", q->m);
            return tc_gemm_fp8a8(*q, st);
        }
        debug_arm("fp8a8", "tcgen05", q->m);
        return gemm_passes(*q, tc_fp8a8_ok, [](const R3dGemmQ& c, cudaStream_t s) { return tc_fp8a8(c, s); }, st, 64);
    }
    return RAD_E_UNSUPPORTED;
}

/* gemm_nt_q_gated @ fp8a8 in one launch: the band with the gated quantiser as its epilogue. q->y is not
 * used. RAD_E_UNSUPPORTED when the shape is not one the fused kernel serves byte-identically to the
 * band followed by r3d_b200_gated_quant_fp8 (the caller then runs that pair). */
extern "C" int r3d_b200_gemm_fp8a8_gated(const R3dGemmQ* q, void* codes, int64_t q_pitch, float* scale,
                                         int64_t s_pitch, void* ob, int32_t ob_dtype, int64_t ob_pitch,
                                         int32_t silu, void* stream) {
    if (!q || !codes || !scale || !device_is_sm100()) return RAD_E_UNSUPPORTED;
    if (ob && ob_dtype != RAD_BF16 && ob_dtype != RAD_F32) return RAD_E_DTYPE;
    static const bool off = [] { const char* e = getenv("R3D_GATED_COMPOSED"); return e && *e && *e != '0'; }();
    if (off || q->m > 64 || (q->arm != R3D_ARM_AUTO && q->arm != R3D_ARM_TILE) || !tc_fp8a8_gated_ok(*q))
        return RAD_E_UNSUPPORTED;
    debug_arm("fp8a8", "tcgen05 with the gated quantiser as its epilogue", q->m);
    const GatedOut g{codes, q_pitch, scale, s_pitch, ob, ob_dtype, ob_pitch, silu};
    return tc_fp8a8_gated(*q, g, (cudaStream_t)stream);
}

extern "C" int r3d_b200_gemm_mxfp4a8(const R3dGemmQ* q, void* stream) {
    if (!q || !device_is_sm100()) return RAD_E_UNSUPPORTED;
    cudaStream_t st = (cudaStream_t)stream;
    int arm = q->arm;
    if (arm == R3D_ARM_AUTO) arm = auto_arm_mxfp4a8(*q);
    if (arm == R3D_ARM_STREAM) {
        debug_arm("mxfp4a8", "stream", q->m);
        return gemm_passes(*q, stream_mxfp4a8_ok, stream_mxfp4a8, st);
    }
    if (arm == R3D_ARM_EXACT) { debug_arm("mxfp4a8", "exact", q->m); return exact_mxfp4a8(*q, st); }
    if (arm == R3D_ARM_TILE) {
        if (q->m > 64 && !no_gemm() && tc_gemm_mxfp4a8_ok(*q)) {
            debug_arm("mxfp4a8", "tcgen05 tile", q->m);
            return tc_gemm_mxfp4a8(*q, st);
        }
        debug_arm("mxfp4a8", "tcgen05", q->m);
        return gemm_passes(*q, tc_mxfp4a8_ok, [](const R3dGemmQ& c, cudaStream_t s) { return tc_mxfp4a8(c, s); }, st, 32);
    }
    if (arm == R3D_ARM_PACK) {
        if (!tc_mxf4_ok(*q)) return RAD_E_UNSUPPORTED;
        debug_arm("mxfp4a8", "tcgen05 packed", q->m);
        return tc_mxf4(*q, st);
    }
    return RAD_E_UNSUPPORTED;
}

/* gemm_nt_q @ mxfp4mx8: e2m1 weights and e4m3 activations, each with E8M0 scales per 32 of K.
 * AUTO: the CTA-pair tcgen05 kernel for M > 64 when TMA's alignment rules are met, else the
 * oracle-order kernel (any shape). */
extern "C" int r3d_b200_gemm_mxfp4mx8(const R3dGemmQ* q, void* stream) {
    if (!q || !device_is_sm100()) return RAD_E_UNSUPPORTED;
    cudaStream_t st = (cudaStream_t)stream;
    if (q->arm != R3D_ARM_AUTO && q->arm != R3D_ARM_TILE && q->arm != R3D_ARM_EXACT) return RAD_E_UNSUPPORTED;
    if (q->arm != R3D_ARM_EXACT && q->m > 64 && !no_gemm() && tc_gemm_mx_ok(*q)) {
        debug_arm("mxfp4mx8", "tcgen05 pair tile, hardware scales on both operands", q->m);
        return tc_gemm_mx(*q, st);
    }
    if (q->arm == R3D_ARM_TILE) return RAD_E_UNSUPPORTED;
    debug_arm("mxfp4mx8", "exact", q->m);
    return exact_mxfp4mx8(*q, st);
}

extern "C" int r3d_b200_gemm_w2a8(const R3dW2A8* q, void* stream) {
    if (!q || !device_is_sm100()) return RAD_E_UNSUPPORTED;
    debug_arm("w2a8", "integer mma tiles or dp4a row walk", q->m);
    return launch_gemm_w2a8(*q, (cudaStream_t)stream);
}

namespace r3d {
int q8x_run(const R3dGemmQ& q, int8_t* x8, float* sg, int walk, cudaStream_t st) {
    if (tc_q8x_ok(q)) {
        debug_arm("mxfp4a8", walk ? "q8x lane-map on tcgen05" : "q8x dot4 on tcgen05", q.m);
        return tc_q8x(q, x8, sg, walk, st);
    }
    const int rc = q8x_requant(q, x8, sg, st);
    if (rc != RAD_OK) return rc;
    debug_arm("mxfp4a8", walk ? "q8x lane-map" : "q8x dot4", q.m);
    return q8x_gemv(q, x8, sg, walk, st);
}
} /* namespace r3d */

extern "C" int r3d_b200_q8x_on_tensor_core(const R3dGemmQ* q) {
    return q && q->m >= 1 && q->m <= 8 && tc_q8x_ok(*q) ? 1 : 0;
}

extern "C" int r3d_b200_gemm_mxfp4a8_q8x(const R3dGemmQ* q, int8_t* x8, float* sg, int walk,
                                         void* stream) {
    if (!q || !x8 || !sg || !device_is_sm100()) return RAD_E_UNSUPPORTED;
    if (q->m < 1 || q->m > 8 || (q->k & 255) || q->k > (1 << 20)) return RAD_E_UNSUPPORTED;   /* the kernels' 32-bit offsets */
    return q8x_run(*q, x8, sg, walk ? 1 : 0, (cudaStream_t)stream);
}

extern "C" int r3d_b200_logits(const R3dLogits* l, void* stream) {
    if (!l || !device_is_sm100()) return RAD_E_UNSUPPORTED;
    cudaStream_t st = (cudaStream_t)stream;
    int arm = l->arm;
    if (arm == R3D_ARM_AUTO) {
        const int tile_step = l->head_fmt == 1 ? 16 : 32;
        R3dLogits probe = *l; if (probe.m > tile_step) probe.m = tile_step;
        if (tc_logits_ok(probe)) arm = R3D_ARM_TILE;
        else {
            probe = *l; if (probe.m > 64) probe.m = 64;
            arm = stream_logits_ok(probe) ? R3D_ARM_STREAM : R3D_ARM_EXACT;
        }
    }
    if (arm == R3D_ARM_EXACT) { debug_arm("logits", "exact", l->m); return exact_logits(*l, st); }
    if (arm != R3D_ARM_STREAM && arm != R3D_ARM_TILE) return RAD_E_UNSUPPORTED;
    const bool tile = arm == R3D_ARM_TILE;
    debug_arm("logits", tile ? "tcgen05" : "stream", l->m);
    const int ysz = l->y_dtype == RAD_F32 ? 4 : 2;
    const int step = tile ? (l->head_fmt == 1 ? 16 : 32) : 64;
    for (int m0 = 0; m0 < l->m; m0 += step) {
        R3dLogits c = *l;
        c.m = l->m - m0 < step ? l->m - m0 : step;
        c.x = (const uint16_t*)l->x + (int64_t)m0 * l->x_pitch;
        c.y = (uint8_t*)l->y + (int64_t)m0 * l->y_pitch * ysz;
        if (!(tile ? tc_logits_ok(c) : stream_logits_ok(c))) return RAD_E_UNSUPPORTED;
        const int rc = tile ? tc_logits(c, st) : stream_logits(c, st);
        if (rc != RAD_OK) return rc;
    }
    return RAD_OK;
}

/* ---- column-sharded calls with the all-gather fused into the epilogue. The output goes to
 * the gathered [M, world * n_pad] buffer of slot `slot` on every rank (column offset rank * n_pad);
 * kernels that cannot push themselves (exact and streaming arms, multi-pass M) compute into
 * the caller's y and a copy kernel pushes it. */
extern "C" int r3d_b200_gemm_mxfp4a8_push(const R3dGemmQ* q, void* gather, int slot, int64_t n_pad, void* stream) {
    if (!q || !gather || !device_is_sm100()) return RAD_E_UNSUPPORTED;
    if (n_pad < q->n) return RAD_E_SHAPE;
    PushCfg cfg;
    if (!gather_push_cfg((const Gather*)gather, slot, n_pad, q->m, 2, &cfg)) return RAD_E_INVAL;
    cudaStream_t st = (cudaStream_t)stream;
    if (q->arm == R3D_ARM_AUTO || q->arm == R3D_ARM_PACK || q->arm == R3D_ARM_TILE) {
        if (q->arm != R3D_ARM_TILE && (q->m <= 4 || q->arm == R3D_ARM_PACK) && tc_mxf4_ok(*q)) { debug_arm("mxfp4a8", "tcgen05 packed + push", q->m); return tc_mxf4(*q, st, &cfg); }
        if (q->m <= 32 && tc_mxfp4a8_ok(*q)) { debug_arm("mxfp4a8", "tcgen05 + push", q->m); return tc_mxfp4a8(*q, st, &cfg); }
    }
    if (!q->y) return RAD_E_INVAL;
    const int rc = r3d_b200_gemm_mxfp4a8(q, stream);
    return rc != RAD_OK ? rc : push_copy(q->y, q->y_pitch, q->m, q->n, 2, cfg, st);
}

extern "C" int r3d_b200_gemm_fp8a8_push(const R3dGemmQ* q, void* gather, int slot, int64_t n_pad, void* stream) {
    if (!q || !gather || !device_is_sm100()) return RAD_E_UNSUPPORTED;
    if (n_pad < q->n) return RAD_E_SHAPE;
    PushCfg cfg;
    if (!gather_push_cfg((const Gather*)gather, slot, n_pad, q->m, 2, &cfg)) return RAD_E_INVAL;
    cudaStream_t st = (cudaStream_t)stream;
    if ((q->arm == R3D_ARM_AUTO || q->arm == R3D_ARM_TILE) && q->m <= 64 && tc_fp8a8_ok(*q)) {
        debug_arm("fp8a8", "tcgen05 + push", q->m);
        return tc_fp8a8(*q, st, &cfg);
    }
    if (!q->y) return RAD_E_INVAL;
    const int rc = r3d_b200_gemm_fp8a8(q, stream);
    return rc != RAD_OK ? rc : push_copy(q->y, q->y_pitch, q->m, q->n, 2, cfg, st);
}

extern "C" int r3d_b200_logits_push(const R3dLogits* l, void* gather, int slot, int64_t n_pad, void* stream) {
    if (!l || !gather || !device_is_sm100()) return RAD_E_UNSUPPORTED;
    if (n_pad < l->n) return RAD_E_SHAPE;
    const int ysz = l->y_dtype == RAD_F32 ? 4 : 2;
    PushCfg cfg;
    if (!gather_push_cfg((const Gather*)gather, slot, n_pad, l->m, ysz, &cfg)) return RAD_E_INVAL;
    cudaStream_t st = (cudaStream_t)stream;
    if ((l->arm == R3D_ARM_AUTO || l->arm == R3D_ARM_TILE) && tc_logits_ok(*l)) {
        debug_arm("logits", "tcgen05 + push", l->m);
        return tc_logits(*l, st, &cfg);
    }
    if (!l->y) return RAD_E_INVAL;
    const int rc = r3d_b200_logits(l, stream);
    return rc != RAD_OK ? rc : push_copy(l->y, l->y_pitch, l->m, l->n, ysz, cfg, st);
}

extern "C" int r3d_b200_quant_act_fp8(const void* x, int32_t x_dtype, int64_t x_pitch, void* q,
                                      int64_t q_pitch, float* scale, int64_t s_pitch,
                                      int32_t rows, int32_t n, int32_t group, void* stream) {
    if (!x || !q || !scale || rows <= 0 || n <= 0) return RAD_E_INVAL;
    if (x_dtype != RAD_BF16 && x_dtype != RAD_F32) return RAD_E_DTYPE;
    if (!device_is_sm100()) return RAD_E_UNSUPPORTED;
    return launch_quant_act_fp8(x, x_dtype, x_pitch, q, q_pitch, scale, s_pitch, rows, n, group,
                                (cudaStream_t)stream);
}

/* gate_up bf16 [rows, 2n] (pitch in elements) -> e4m3 codes [rows, n], f32 scale per (row, group of g),
 * optional gated product `ob` (bf16 or f32): the quantiser that closes gemm_nt_q_gated. */
extern "C" int r3d_b200_gated_quant_fp8(const void* gu, int64_t gu_pitch, void* q, int64_t q_pitch,
                                        float* scale, int64_t s_pitch, void* ob, int32_t ob_dtype,
                                        int64_t ob_pitch, int32_t rows, int32_t n, int32_t group, int32_t silu,
                                        void* stream) {
    if (!gu || !q || !scale || rows <= 0 || n <= 0) return RAD_E_INVAL;
    if (ob && ob_dtype != RAD_BF16 && ob_dtype != RAD_F32) return RAD_E_DTYPE;
    if (!device_is_sm100()) return RAD_E_UNSUPPORTED;
    return launch_gated_quant_fp8(gu, gu_pitch, q, q_pitch, scale, s_pitch, ob, ob_dtype, ob_pitch, rows, n,
                                  group, silu, (cudaStream_t)stream);
}
