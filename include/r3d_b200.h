/* r3d_b200.h -- the C ABI of libr3d_b200.so, a B200 (sm_100a) drop-in for libr3d's
 * quantised-matmul bands. Two layers, both extern "C", plain pointers and sizes only:
 *
 *  (1) The radiance kernel-plugin surface, exactly what the engine's loader binds in
 *      libr3d (rad_abi.h declares rad_plugin_abi_version / rad_plugin_info /
 *      rad_kernel_schema_* / rad_kernel_*), plus the row entry symbols below, which the
 *      reference's dlopen harnesses also bind by name.
 *  (2) A thin launch layer under the entries (r3d_b200_*): one call per kernel family,
 *      operands already validated. The entries are host C++; this layer is the only
 *      place host code crosses into CUDA.
 *
 * Every launch is asynchronous on the caller's stream and returns RAD_OK once enqueued.
 * Citations name the libr3d interface each symbol replaces (path within that project).
 */
#ifndef R3D_B200_H
#define R3D_B200_H

#include "rad_abi.h"
#ifndef __cplusplus
#include <stdbool.h>
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* ------------------------------------------------------------------ (1) row entries */

/* gemm_nt_q @ fp8a8, any M. Replaces r3d_rad_gemm_nt_q_fp8
 * (src/r3d_gemm_fp8a8.hip:1055-1085). */
int r3d_rad_gemm_nt_q_fp8(const RadArgs* a, RadStream s);
/* gemm_nt_q @ fp8a8, decode band M <= 8. Replaces r3d_rad_gemm_nt_q_fp8_decode
 * (src/r3d_gemm_fp8a8.hip:1098-1130). */
int r3d_rad_gemm_nt_q_fp8_decode(const RadArgs* a, RadStream s);
/* gemm_nt_q_gated @ fp8a8, M <= 64: the fp8a8 band into the launch scratch plus the gated
 * activation quantiser. Replaces r3d_rad_gemm_nt_q_gated_fp8 and its scratch hook
 * (src/r3d_gemm_fp8a8.hip:1167-1253). */
int r3d_rad_gemm_nt_q_gated_fp8(const RadArgs* a, RadStream s);
int64_t r3d_rad_gemm_nt_q_gated_fp8_scratch(const RadArgs* a);
/* The activation producers in front of the bands, as rows of their own.
 * quant_act_fp8 (x, q, scale): replaces r3d_rad_quant_act_fp8 (src/r3d_band.hip:459-489).
 * gated_quant_fp8 (gate_up, q, scale, out_bf16?): replaces r3d_rad_gated_quant_fp8
 * (src/r3d_band.hip:491-548). rmsnorm_quant_fp8 (x, residual?, w, q, scale, out_bf16?): replaces
 * r3d_rad_rmsnorm_quant_fp8 (src/r3d_more.hip:480-541); its sum of squares keeps the reference
 * kernel's order, so codes, scales and the norm output carry the same bits. */
int r3d_rad_quant_act_fp8(const RadArgs* a, RadStream s);
int r3d_rad_gated_quant_fp8(const RadArgs* a, RadStream s);
int r3d_rad_rmsnorm_quant_fp8(const RadArgs* a, RadStream s);
/* row_topk (x, idx, val, pairs?): exact per-row top-R, R <= 32, value descending and ties to the
 * lower column; `vocab_off` is added to every reported column and `pairs` is the [M, R, 2]
 * (int32 id, f32 value) plane a sharded head gathers instead of its logits. Replaces
 * r3d_rad_row_topk (src/r3d_more.hip:179-236, :438-476). */
int r3d_rad_row_topk(const RadArgs* a, RadStream s);
/* scratch hooks of row_topk and sample_argmax (no reference counterpart: the reference's rows re-read the row
 * from one block and need no arena): bytes of the tournament's two survivor planes. With the arena in
 * RadArgs.scratch the rows allocate nothing; without one they fall back to planes of their own. */
int64_t r3d_rad_row_topk_scratch(const RadArgs* a);
int64_t r3d_rad_sample_argmax_scratch(const RadArgs* a);
/* sample_argmax (logits, params, token): greedy decode over f32 logits, ties to the lower token
 * id; `params` is not read. Replaces r3d_rad_sample_argmax (src/r3d_sample.hip:166-173, :607-623). */
int r3d_rad_sample_argmax(const RadArgs* a, RadStream s);
/* gemm_nt_q @ mxfp4a8, any M. Replaces r3d_rad_gemm_nt_q
 * (src/r3d_gemm_mxfp4.hip:1587-1691). */
int r3d_rad_gemm_nt_q(const RadArgs* a, RadStream s);
/* gemm_nt_q @ mxfp4mx8, any M (row gemm_nt_q_mxfp4mx8): a_scale is an E8M0 plane [M, K/32]. No
 * counterpart in the reference; see r3d_b200_gemm_mxfp4mx8. */
int r3d_rad_gemm_nt_q_mx8(const RadArgs* a, RadStream s);
/* gemm_nt_q @ w2a8, the draft head's decode band (M <= 16), and its layout hooks: operand 3 (b_scale) is
 * the canonical rad.planes join of the f16 scale and the u8 / u4 zero plane, operand 2 (the codes) is
 * stored as it is. Replace r3d_rad_gemm_nt_q_w2a8_decode, r3d_layout_gemm_w2a8, r3d_relayout_gemm_w2a8,
 * r3d_unrelayout_gemm_w2a8 (src/r3d_gemm_w2a8.hip:1317-1349, :1362-1436). */
int r3d_rad_gemm_nt_q_w2a8_decode(const RadArgs* a, RadStream s);
int r3d_layout_gemm_w2a8(const RadParam* p, int n_p, int operand, const RadEncoding* enc, const int* sel,
                         const RadTensor* planes, int n, RadLayout* out);
int r3d_relayout_gemm_w2a8(const RadParam* p, int n_p, int operand, const RadEncoding* enc, const int* sel,
                           const RadTensor* planes, int n, void* dst, int64_t dst_bytes);
int r3d_unrelayout_gemm_w2a8(const RadParam* p, int n_p, int operand, const RadEncoding* enc, const int* sel,
                             const void* src, int64_t src_bytes, const RadTensor* planes, int n);
/* gemm_nt_q @ mxfp4a8, decode band M <= 8, fp32 walk. Replaces
 * r3d_rad_gemm_nt_q_mxfp4_decode (src/r3d_gemm_mxfp4.hip:1715-1716). */
int r3d_rad_gemm_nt_q_mxfp4_decode(const RadArgs* a, RadStream s);
/* gemm_nt_q @ mxfp4a8, decode band, int8-per-32 activation arm. Replaces
 * r3d_rad_gemm_nt_q_mxfp4_decode_q8x (src/r3d_gemm_mxfp4.hip:1717-1718). */
int r3d_rad_gemm_nt_q_mxfp4_decode_q8x(const RadArgs* a, RadStream s);
/* The q8x OFF lever (R3D_MXFP4_Q8X=0). Replaces r3d_mxfp4_q8x_off
 * (src/r3d_gemm_mxfp4.hip:1724-1730). */
bool r3d_mxfp4_q8x_off(void);
/* logits_gemm over the joined e4m3 + block-scale head, f32 logits. Replaces
 * r3d_rad_logits_gemm_e4m3 (src/r3d_gemm_logits.hip:145-226). */
int r3d_rad_logits_gemm_e4m3(const RadArgs* a, RadStream s);
/* logit_rerank over the same joined head: R <= 32 candidate ids a row rescored by a double-precision
 * chain in ascending k and re-sorted (larger value, ties to the lower id, pads last). Replaces
 * r3d_rad_logit_rerank_e4m3 (src/r3d_logit_rerank_e4m3.hip:146-345). */
int r3d_rad_logit_rerank_e4m3(const RadArgs* a, RadStream s);
/* Forget the remembered header of a head blob (the rows above copy a device-resident blob's
 * rad.planes header to the host on first sight of its address): call it when the blob's memory is
 * released or rewritten. No counterpart in the reference, which reads the header through the
 * operand pointer on every call. */
void r3d_b200_forget_head(const void* blob);
/* Layout hooks of that row. Replace r3d_layout_head / r3d_relayout_head /
 * r3d_unrelayout_head (src/r3d_gemm_logits.hip:233-272). */
int r3d_layout_head(const RadParam* p, int n_p, int operand, const RadEncoding* enc,
                    const int* sel, const RadTensor* planes, int n, RadLayout* out);
int r3d_relayout_head(const RadParam* p, int n_p, int operand, const RadEncoding* enc,
                      const int* sel, const RadTensor* planes, int n, void* dst,
                      int64_t dst_bytes);
int r3d_unrelayout_head(const RadParam* p, int n_p, int operand, const RadEncoding* enc,
                        const int* sel, const void* src, int64_t src_bytes,
                        const RadTensor* planes, int n);

/* ------------------------------------------------------------------ (2) launch layer */

/* Which kernel serves a call. AUTO picks by shape and alignment the way the entries do.
 *
 * The tcgen05 arms are launched with programmatic stream serialisation: a call's kernel may begin
 * while the previous kernel of the stream is still running, prefetches WEIGHT tiles and weight
 * scales at once and touches everything else (activations, activation scales, outputs) only after
 * griddepcontrol.wait. Weight planes must therefore be complete before the kernel that precedes
 * the call starts (they are written when a model is loaded and not again: the reference's plane
 * cache relies on the same, src/r3d_gemm_mxfp4.hip:1879-1880). R3D_NO_PDL=1 disables the early start.
 * Some arms keep activation pieces in device arrays owned by the library: calls on one device
 * must be ordered on one stream (one dispatch thread, as in the reference). */
enum {
    R3D_ARM_AUTO   = 0,
    R3D_ARM_EXACT  = 1,   /* oracle-order walk: bit-identical to the CPU restatement */
    R3D_ARM_STREAM = 2,   /* weight-streaming tensor-core walk, M <= 64 */
    R3D_ARM_TILE   = 3,   /* tcgen05 + TMA + TMEM walk (swap-AB), one CTA (or cluster) per row tile */
    R3D_ARM_PACK   = 4    /* mxfp4a8 only, M <= 8: tcgen05 kind::mxf4 on packed nibbles, hardware group scales */
};

/* Operands of one gemm_nt_q call. Pitches are in elements of the tensor they belong to,
 * except b_pitch of a packed e2m1 weight, which is in bytes (K/2). */
typedef struct R3dGemmQ {
    const void*  a;         /* e4m3 codes [M, K] */
    const float* a_scale;   /* f32 [M, as_cols] */
    const void*  b;         /* e4m3 codes [N, K]   |  e2m1 nibbles [N, K/2 bytes] */
    const void*  b_scale;   /* bf16|f32 [N/rblk, bs_cols]  |  E8M0 bytes [N, K/32] */
    void*        y;         /* bf16 [M, N] */
    int32_t      m, n, k;
    int32_t      as_cols, bs_cols;
    int32_t      rblk;      /* fp8a8: weight rows one scale row covers (1 or 128) */
    int32_t      bs_dtype;  /* fp8a8: RAD_BF16 or RAD_F32 */
    int64_t      a_pitch, b_pitch, y_pitch, as_pitch, bs_pitch;
    int32_t      arm;
    int32_t      reserved;
} R3dGemmQ;

/* Replaces the kernel dispatch inside f8_launch_tile (src/r3d_gemm_fp8a8.hip:926-1050). */
int r3d_b200_gemm_fp8a8(const R3dGemmQ* q, void* stream);
/* Replaces the kernel dispatch of r3d_gemm_nt_q_impl and the fp32 decode walk
 * (src/r3d_gemm_mxfp4.hip:1613-1690, :2125-2169). */
int r3d_b200_gemm_mxfp4a8(const R3dGemmQ* q, void* stream);
/* gemm_nt_q @ mxfp4mx8 -- a dtype spelling the reference does not have (its mxfp4 band takes e4m3
 * activations with an f32 scale per 128 of K): e2m1 weights [N, K/2 bytes] + E8M0 [N, K/32] and e4m3
 * activations [M, K] + E8M0 [M, K/32], the OCP-MX pair whose scales the tensor core applies itself.
 * `a_scale` carries the activations' E8M0 bytes (as_cols = K/32, as_pitch in bytes). Rule (fixed by
 * this library's CPU checker, no reference pin): per 32 of K  acc += (sum a*w * 2^(xa-127)) * 2^(xw-127).
 * Arms: AUTO / TILE (M > 64: CTA-pair tcgen05 kernel, one accumulation over K) and EXACT. */
int r3d_b200_gemm_mxfp4mx8(const R3dGemmQ* q, void* stream);
/* The int8-per-32 arm: requantise the activation into x8/sg (caller-owned scratch,
 * x8 >= m*k bytes, sg >= m*k/32 floats), then the dot. walk 0 = per-256 tree, 1 = lane
 * map. Replaces m4_act_i8_kernel + gemm_nt_mxfp4_gemv_q8x[_lm]_kernel
 * (src/r3d_gemm_mxfp4.hip:1150-1166, :1217-1458); needs no repacked weight plane. The exact
 * integer dots run on the tensor core (tcgen05.mma kind::mxf4 over e2m1 digit rows of the int8
 * activation, which live in a device array owned by the library: order calls on one stream) when
 * K <= 32768, the weight and scale planes are 16-byte aligned with pitches that are multiples of
 * 16 bytes; otherwise on dp4a. Both give the reference arm's bits. */
int r3d_b200_gemm_mxfp4a8_q8x(const R3dGemmQ* q, int8_t* x8, float* sg, int walk,
                              void* stream);
/* 1 when the call above would run its dots on the tensor core, 0 when on dp4a (no launch): for
 * tests and debug prints, like r3d_b200_pick_arm_*. No counterpart in the reference. */
int r3d_b200_q8x_on_tensor_core(const R3dGemmQ* q);

/* The same arm with no allocation anywhere: the requantised-activation scratch is a fixed
 * array inside the library (288 KiB per GPU, held until the process exits) instead of
 * caller memory. For callers that cannot call cudaMalloc -- a launch issued while a pass is
 * being recorded, or once the engine has given all device memory to weights and KV cache.
 * Serves M <= 8 and K <= 32768 (K % 256 == 0); anything larger returns RAD_E_SHAPE. All
 * calls on a device share the array: calls that overlap in time race, so keep them on one
 * stream. The first call on a device resolves the array's address; make it before any
 * stream capture. This entry point has no counterpart in the reference. */
int r3d_b200_gemm_mxfp4a8_q8x_static(const R3dGemmQ* q, int walk, void* stream);

/* Operands of one gemm_nt_q @ w2a8 call (the draft head's decode band, M <= 16). */
typedef struct R3dW2A8 {
    const void*  a;         /* i8 codes [M, K] in quant_act_i8's step order (column k at index k with bits 2 and 3 swapped) */
    const float* a_scale;   /* f32, one a row */
    const void*  b;         /* u2 codes [N, K/4 bytes], code k of a row in byte k>>2 at bit 2*(k&3) */
    const void*  scale;     /* f16 [N, K/128] */
    const void*  zero;      /* u8 [N, K/128], or u4 (two a byte, low nibble first) when zero_u4 */
    const float* a_sum;     /* f32 [K/128, mpad], group-major: the row's code sums per 128 of K */
    void*        y;         /* bf16 [M, N] */
    int32_t      m, n, k, mpad, zero_u4;
    int32_t      arm;       /* R3D_ARM_AUTO, or R3D_ARM_EXACT: the one-thread-per-row kernel whatever the alignment */
    int64_t      a_pitch, as_pitch, y_pitch;   /* elements */
    int64_t      b_pitch, zp_pitch;            /* bytes */
    int64_t      sc_pitch;                     /* f16 elements */
} R3dW2A8;

/* gemm_nt_q_gated @ fp8a8 as one launch (replaces the fused kernels of src/r3d_gemm_fp8a8.hip:700-825 and
 * their dispatch :1167-1253): the decode band over the [2n, K] gate_up weight with the gated quantiser
 * (silu or sigmoid of the gate times up -> bf16 -> group amax -> e4m3) as the kernel's epilogue; q->n = 2n,
 * q->y unused; codes e4m3 [M, n], scale f32 [M, n/128], ob optional gated product (bf16 | f32).
 * Returns RAD_E_UNSUPPORTED for shapes it does not serve byte-identically to r3d_b200_gemm_fp8a8 followed by
 * r3d_b200_gated_quant_fp8 (M > 64, n not a multiple of 128, projections narrow enough that K is split). */
int r3d_b200_gemm_fp8a8_gated(const R3dGemmQ* q, void* codes, int64_t q_pitch, float* scale, int64_t s_pitch,
                              void* ob, int32_t ob_dtype, int64_t ob_pitch, int32_t silu, void* stream);

/* Replaces the kernel dispatch of w2_launch (src/r3d_gemm_w2a8.hip:1058-1315). 16-byte aligned operands
 * (K >= 512): persistent CTAs stream 256-row tiles by TMA and form the exact group sums with integer
 * mma.sync over byte-quads cut from the 2-bit plane; anything else: one thread per weight row with dp4a.
 * Both apply the oracle's flush per 128 of K; exact, bit-identical to each other. */
int r3d_b200_gemm_w2a8(const R3dW2A8* q, void* stream);

typedef struct R3dLogits {
    const void* x;          /* bf16 [M, K] */
    const void* codes;      /* e4m3 [N, K] dense   |  e2m1 nibbles (head_fmt 1) */
    const void* scale;      /* bf16|f16|f32 [ceil(N/br), ceil(K/128)]  |  E8M0 [N, K/32] */
    void*       y;          /* f32 [M, N] (y_dtype RAD_F32) or bf16 (RAD_BF16) */
    int32_t     m, n, k;
    int32_t     br;         /* weight rows per scale row: 1 or 128 */
    int32_t     scale_dtype;
    int32_t     y_dtype;
    int32_t     head_fmt;   /* 0 = e4m3 + block scale (the reference head), 1 = mxfp4 */
    int32_t     arm;
    int64_t     x_pitch, code_pitch, y_pitch, scale_pitch;
} R3dLogits;

/* Replaces the launch of logits_e4m3_kernel (src/r3d_gemm_logits.hip:196-221). */
int r3d_b200_logits(const R3dLogits* l, void* stream);

/* Activation producer: per (row, group) amax/448 scale and RTNE-saturating e4m3 codes.
 * x_dtype RAD_BF16 or RAD_F32. Replaces quant_act_fp8_kernel (src/r3d_band.hip:119-153). */
int r3d_b200_quant_act_fp8(const void* x, int32_t x_dtype, int64_t x_pitch, void* q,
                           int64_t q_pitch, float* scale, int64_t s_pitch, int32_t rows,
                           int32_t n, int32_t group, void* stream);

/* Which arm AUTO would pick for this call (no launch): for tests and debug prints, the
 * role R3D_DEBUG_GEMM's "which arm launched" lines play in the reference
 * (src/r3d_gemm_fp8a8.hip:976-983). */
int r3d_b200_pick_arm_fp8a8(const R3dGemmQ* q);
int r3d_b200_pick_arm_mxfp4a8(const R3dGemmQ* q);

/* 0 when no bounded device-side wait of the streaming arm has ever expired in this process;
 * otherwise the code of the wait that gave up (1 producer, 2 consumer). The affected launch
 * stored nothing. No counterpart in the reference (its kernels have no device-side waits). */
/* The gated activation quantiser on its own (the reference's gated_quant_fp8 arithmetic,
 * src/r3d_band.hip:167-235, over a bf16 gate_up plane [rows, 2n], pitches in elements). */
int r3d_b200_gated_quant_fp8(const void* gu, int64_t gu_pitch, void* q, int64_t q_pitch, float* scale,
                             int64_t s_pitch, void* ob, int32_t ob_dtype, int64_t ob_pitch, int32_t rows,
                             int32_t n, int32_t group, int32_t silu, void* stream);
int r3d_b200_stream_status(void);

/* The tensor pipe's issue rate, the denominator of the prefill band's fraction: one launch in which
 * every CTA pair issues `iters` stages of four K=32 cta_group::2 MMAs from operand tiles resident in
 * shared memory (kind 0: e4m3 x e4m3, 256 x 256 per instruction; kind 1: block-scaled e2m1 x e4m3,
 * 256 x 192). Returns the FLOPs of the launch for the caller to divide by its event time, negative
 * on failure. No counterpart in the reference. */
double r3d_b200_mma_peak(int kind, int iters, void* stream);

/* Kernels this library launched since load (all arms): bench bookkeeping. */
long long r3d_b200_launch_count(void);

/* ------------------------------------------------------------------ (3) column-sharded calls
 * No reference counterpart: the reference is single-rank (src/r3d_rows.cpp:281-284 of libr3d keeps
 * vocab_off at 0). One process per GPU; every rank holds a contiguous slab of weight rows
 * (= output columns) and the all-gather of the outputs is fused into the GEMV's epilogue: each
 * rank's kernel stores its columns into the gathered [M, world * n_pad] buffer of every rank
 * through CUDA IPC peer mappings (plain stores over NVLink), and the last CTA raises a flag.
 *
 *   r3d_b200_gather_create   allocate this rank's exchange buffer (slots x slot_bytes, use two
 *                            slots alternately so a peer's next push never overwrites a result
 *                            still being read) and export its 64-byte IPC handle
 *   r3d_b200_gather_connect  map the peers' buffers from their handles (world x 64 bytes, rank-major;
 *                            the caller moves handles between processes)
 *   r3d_b200_*_push          the sharded call; output only in the gathered buffers. y of the operand
 *                            struct is used as scratch when the serving kernel cannot push itself
 *                            (may be NULL when the tcgen05 arms are eligible)
 *   r3d_b200_gather_wait     enqueue the wait for every rank's push of the same call; bounded (~1 s),
 *                            after which r3d_b200_gather_status() != 0
 *   r3d_b200_gather_buffer   this rank's gathered buffer of a slot
 * Ranks must issue the same sequence of push calls. */
int   r3d_b200_gather_create(int world, int rank, int64_t slot_bytes, int slots, void** out,
                             unsigned char handle[64]);
int   r3d_b200_gather_connect(void* gather, const unsigned char* handles);
/* same-process peers: the peer's r3d_b200_gather_base() instead of an IPC handle */
int   r3d_b200_gather_connect_ptr(void* gather, int peer, void* base);
void* r3d_b200_gather_base(void* gather);
void* r3d_b200_gather_buffer(void* gather, int slot);
int   r3d_b200_gather_wait(void* gather, void* stream);
int   r3d_b200_gather_status(void* gather);
void  r3d_b200_gather_destroy(void* gather);
int   r3d_b200_gemm_mxfp4a8_push(const R3dGemmQ* q, void* gather, int slot, int64_t n_pad, void* stream);
int   r3d_b200_gemm_fp8a8_push(const R3dGemmQ* q, void* gather, int slot, int64_t n_pad, void* stream);
int   r3d_b200_logits_push(const R3dLogits* l, void* gather, int slot, int64_t n_pad, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* R3D_B200_H */
