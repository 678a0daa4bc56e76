/* r3d_kernels.h -- internal declarations shared by the translation units of libr3d_b200.so:
 * one launcher per (band, arm). Host C++ only sees these; the CUDA lives behind them. */
#pragma once
#include <cstdint>
#include <cuda_runtime.h>
#include "r3d_b200.h"

namespace r3d {

struct PushCfg;                        /* push.cuh: fused all-gather destination, or nullptr */
struct Gather;
bool gather_push_cfg(const Gather* g, int slot, int64_t n_pad, int m, int elem_bytes, PushCfg* out);
int  push_copy(const void* y, int64_t y_pitch, int m, int n, int elem_bytes, const PushCfg& g, cudaStream_t st);

void count_launch(int n = 1);          /* bookkeeping behind r3d_b200_launch_count() */
bool device_is_sm100();                /* chip gate: these kernels are built for sm_100a only */

/* oracle-order arm (kern_exact.cu) */
int exact_fp8a8(const R3dGemmQ& p, cudaStream_t st);
int exact_mxfp4a8(const R3dGemmQ& p, cudaStream_t st);
int exact_mxfp4mx8(const R3dGemmQ& p, cudaStream_t st);   /* a_scale = E8M0 bytes [M, K/32] */
int exact_logits(const R3dLogits& p, cudaStream_t st);
int launch_quant_act_fp8(const void* x, int x_dtype, int64_t x_pitch, void* q, int64_t q_pitch,
                         float* scale, int64_t s_pitch, int rows, int n, int group,
                         cudaStream_t st);

int launch_gated_quant_fp8(const void* gu, int64_t gu_pitch, void* q, int64_t q_pitch, float* scale,
                           int64_t s_pitch, void* ob, int ob_dtype, int64_t ob_pitch, int rows, int n, int g,
                           int silu, cudaStream_t st, int gu_dtype = RAD_BF16);
/* RMS norm + group quantiser, one block per row; pitches in elements; res/ob may be null */
int launch_rmsnorm_quant_fp8(const void* x, int64_t x_pitch, void* res, int64_t r_pitch, const void* w, int w_dtype,
                             void* q, int64_t q_pitch, float* scale, int64_t s_pitch, void* ob, int ob_dtype,
                             int64_t ob_pitch, int rows, int n, int g, float eps, float wadd, cudaStream_t st);

/* exact per-row top-R (kern_topk.cu); pitches in elements (pairs: floats); val and pairs may be null */
int launch_row_topk(const void* x, int x_dtype, int64_t x_pitch, int32_t* idx, int64_t idx_pitch, float* val,
                    int64_t val_pitch, float* pairs, int64_t pairs_pitch, int M, int N, int R, int64_t off,
                    cudaStream_t st, void* scratch = nullptr, int64_t scratch_bytes = 0);
int64_t row_topk_scratch_bytes(int64_t M, int64_t N, int64_t R);

/* logit_rerank over the joined e4m3 head (kern_rerank.cu): pitches in elements; pairs may be null */
int launch_logit_rerank_e4m3(const void* x, int xdt, int64_t x_rs, const void* codes, int64_t code_rs,
                             const void* scale, int64_t scale_rs, int br, int sdt, const int32_t* in, int64_t in_rs,
                             int32_t* idx, int64_t idx_rs, float* val, int64_t val_rs, float* pairs, int M, int R,
                             int K, int64_t NV, int64_t voff, cudaStream_t st);

/* gemm_nt_q @ w2a8 (kern_w2a8.cu) */
int launch_gemm_w2a8(const R3dW2A8& q, cudaStream_t st);

/* weight-streaming tensor-core arm (kern_stream.cu); *_ok say whether the arm can take
 * the call's shape and alignment */
bool stream_fp8a8_ok(const R3dGemmQ& p);
bool stream_mxfp4a8_ok(const R3dGemmQ& p);
bool stream_logits_ok(const R3dLogits& p);
int  stream_fp8a8(const R3dGemmQ& p, cudaStream_t st);
int  stream_mxfp4a8(const R3dGemmQ& p, cudaStream_t st);
int  stream_logits(const R3dLogits& p, cudaStream_t st);

/* tcgen05 arm (kern_tc.cu): TMA tensor maps + TMEM accumulators, swap-AB, M <= 64 (fp8a8) /
 * M <= 32 (mxfp4a8) per pass */
bool tc_fp8a8_ok(const R3dGemmQ& p);
bool tc_mxfp4a8_ok(const R3dGemmQ& p);
int  tc_fp8a8(const R3dGemmQ& p, cudaStream_t st, const PushCfg* push = nullptr);
int  tc_mxfp4a8(const R3dGemmQ& p, cudaStream_t st, const PushCfg* push = nullptr);
bool tc_logits_ok(const R3dLogits& l);    /* e4m3 head, M <= 32 per pass, K <= 16384 */
int  tc_logits(const R3dLogits& l, cudaStream_t st, const PushCfg* push = nullptr);
/* packed-fp4 tcgen05 walk (kern_tc_mxf4.cu): kind::mxf4 with hardware group scales, M <= 8,
 * K a multiple of 256 */
bool tc_mxf4_ok(const R3dGemmQ& p);
int  tc_mxf4(const R3dGemmQ& p, cudaStream_t st, const PushCfg* push = nullptr);
/* prefill tile kernel (kern_tc_gemm.cu): [128 weight rows x 192 tokens] per CTA, M > 64 */
bool tc_gemm_fp8a8_ok(const R3dGemmQ& p);
bool tc_gemm_mxfp4a8_ok(const R3dGemmQ& p);
int  tc_gemm_fp8a8(const R3dGemmQ& p, cudaStream_t st);
int  tc_gemm_mxfp4a8(const R3dGemmQ& p, cudaStream_t st);
/* prefill kernel for scales that are constant along K (kern_tc_gemm2.cu): CTA pairs on
 * tcgen05 cta_group::2, [256 weight rows x 256 tokens] per pair, persistent, one accumulation over K */
bool tc_gemm_ws_fp8a8_ok(const R3dGemmQ& p);
int  tc_gemm_ws_fp8a8(const R3dGemmQ& p, cudaStream_t st);
/* ... and for mxfp4 weights x mxfp8 activations (both E8M0 scale sets applied by the tensor core),
 * [256 x 192] per pair */
bool tc_gemm_mx_ok(const R3dGemmQ& p);
int  tc_gemm_mx(const R3dGemmQ& p, cudaStream_t st);
/* outputs of the gated quantiser when it runs as the epilogue of the fp8a8 decode kernel */
struct GatedOut { void* q; int64_t q_pitch; float* scale; int64_t s_pitch; void* ob; int ob_dtype; int64_t ob_pitch; int silu; };
bool tc_fp8a8_gated_ok(const R3dGemmQ& p);
int  tc_fp8a8_gated(const R3dGemmQ& p, const GatedOut& g, cudaStream_t st);
int  tc_gemm2_status();
int  tc_status();                      /* 0, or the code of a bounded wait that expired */

/* int8-per-32 activation arm (kern_q8x.cu) */
int q8x_requant(const R3dGemmQ& p, int8_t* x8, float* sg, cudaStream_t st);
int q8x_gemv(const R3dGemmQ& p, const int8_t* x8, const float* sg, int walk, cudaStream_t st);
/* the same arm on the tensor core (kern_tc_q8x.cu): packed nibbles by TMA, the exact integer dots by
 * tcgen05.mma kind::mxf4 over e2m1 digit rows of the int8 activation, the float chain in the epilogue;
 * writes x8 and sg like q8x_requant does */
bool tc_q8x_ok(const R3dGemmQ& p);
int  tc_q8x(const R3dGemmQ& p, int8_t* x8, float* sg, int walk, cudaStream_t st);
int  tc_q8x_status();
int  tc_w2a8_status();
int  rerank_status();
/* requantise + dot, on the tensor core when the operands allow it, else the dp4a kernels */
int  q8x_run(const R3dGemmQ& p, int8_t* x8, float* sg, int walk, cudaStream_t st);

} /* namespace r3d */
