/* rows_table.cpp -- what the engine's loader sees: plugin identity, the op schemas of the
 * quantised-matmul bands, the kernel rows with their constraints and priorities, and the
 * registration gate where the environment kill switches act.
 *
 * Row names, ops, constraint tables, priorities and lever names are those of libr3d
 * (src/r3d_rows.cpp:1042-1091, :1167-1177, :1588-1718, :2216-2278), so a resolver query
 * lands on the same row name it would there. Schemas list parameters and operands in the
 * same order with the same kinds (src/r3d_rows.cpp:190-245): a loader that compares a
 * second declarer's schema entry for entry accepts them. Prose fields describe this
 * library's B200 kernels. Pure host C++.
 *
 * Kill switches act HERE, by not enumerating a row, because the engine picks a row when a
 * band is declared: a row that refuses at launch time is an abort, not a re-resolve
 * (src/r3d_rows.cpp:2197-2200). The entries repeat the check only as a backstop.
 */
#include <cstdlib>
#include <cstring>
#include "rad_abi.h"
#include "r3d_b200.h"

#define COUNT_OF(x) ((int)(sizeof(x) / sizeof((x)[0])))

namespace {

/* ------------------------------------------------------------------ schemas */
const RadParamSpec kGemmQParams[] = {
    { "M", RAD_P_INT, RAD_REQUIRED, 0 },     { "N", RAD_P_INT, RAD_REQUIRED, 0 },
    { "K", RAD_P_INT, RAD_REQUIRED, 0 },     { "group", RAD_P_INT, RAD_REQUIRED, 0 },
    { "dtype", RAD_P_STR, RAD_REQUIRED, 0 }, { "pb1", RAD_P_INT, RAD_OPTIONAL, 0 },
    { "pb2", RAD_P_INT, RAD_OPTIONAL, 0 },
    { "split_n", RAD_P_INT, RAD_OPTIONAL, 0 },   /* a K-split hint: accepted, ignored */
};
const RadOperandSpec kGemmQOperands[] = {
    { "a", RAD_OPD_IN, 0 },        { "a_scale", RAD_OPD_IN, 1 },
    { "b", RAD_OPD_WEIGHT, 0 },    { "b_scale", RAD_OPD_WEIGHT, 0 },
    { "y", RAD_OPD_OUT, 0 },       { "a_sum", RAD_OPD_IN, 1 },
    { "b_ref", RAD_OPD_WEIGHT, 1 },
};

const RadParamSpec kGemmQGatedParams[] = {
    { "M", RAD_P_INT, RAD_REQUIRED, 0 },     { "N", RAD_P_INT, RAD_REQUIRED, 0 },
    { "K", RAD_P_INT, RAD_REQUIRED, 0 },     { "group", RAD_P_INT, RAD_REQUIRED, 0 },
    { "dtype", RAD_P_STR, RAD_REQUIRED, 0 }, { "act", RAD_P_STR, RAD_REQUIRED, 0 },
};
const RadOperandSpec kGemmQGatedOperands[] = {
    { "a", RAD_OPD_IN, 0 },        { "a_scale", RAD_OPD_IN, 0 },
    { "b", RAD_OPD_WEIGHT, 0 },    { "b_scale", RAD_OPD_WEIGHT, 0 },
    { "q", RAD_OPD_OUT, 0 },       { "scale", RAD_OPD_OUT, 0 },
    { "out_bf16", RAD_OPD_OUT, 1 },
};

const RadParamSpec kLogitsParams[] = {
    { "M", RAD_P_INT, RAD_REQUIRED, 0 },      { "n_vocab", RAD_P_INT, RAD_REQUIRED, 0 },
    { "n_embd", RAD_P_INT, RAD_REQUIRED, 0 }, { "dtype", RAD_P_STR, RAD_REQUIRED, 0 },
};
const RadOperandSpec kLogitsOperands[] = {
    { "x", RAD_OPD_IN, 0 }, { "lm_head", RAD_OPD_WEIGHT, 0 }, { "logits", RAD_OPD_OUT, 0 },
};

/* the activation producers: src/r3d_rows.cpp:615-638 (quant_act_fp8, gated_quant_fp8),
 * :700-716 (rmsnorm_quant_fp8) */
const RadParamSpec kQuantActParams[] = {
    { "M", RAD_P_INT, RAD_REQUIRED, 0 },     { "n", RAD_P_INT, RAD_REQUIRED, 0 },
    { "group", RAD_P_INT, RAD_REQUIRED, 0 }, { "dtype", RAD_P_STR, RAD_REQUIRED, 0 },
};
const RadOperandSpec kQuantActOperands[] = {
    { "x", RAD_OPD_IN, 0 }, { "q", RAD_OPD_OUT, 0 }, { "scale", RAD_OPD_OUT, 0 },
};
const RadParamSpec kGatedQuantParams[] = {
    { "M", RAD_P_INT, RAD_REQUIRED, 0 },     { "n", RAD_P_INT, RAD_REQUIRED, 0 },
    { "group", RAD_P_INT, RAD_REQUIRED, 0 }, { "dtype", RAD_P_STR, RAD_REQUIRED, 0 },
    { "act", RAD_P_STR, RAD_OPTIONAL, 0 },
};
const RadOperandSpec kGatedQuantOperands[] = {
    { "gate_up", RAD_OPD_IN, 0 }, { "q", RAD_OPD_OUT, 0 }, { "scale", RAD_OPD_OUT, 0 },
    { "out_bf16", RAD_OPD_OUT, 1 },
};
const RadParamSpec kRmsQuantParams[] = {
    { "M", RAD_P_INT, RAD_REQUIRED, 0 },     { "n", RAD_P_INT, RAD_REQUIRED, 0 },
    { "eps", RAD_P_F64, RAD_REQUIRED, 0 },   { "group", RAD_P_INT, RAD_REQUIRED, 0 },
    { "dtype", RAD_P_STR, RAD_REQUIRED, 0 }, { "wadd", RAD_P_F64, RAD_OPTIONAL, 0 },
};
const RadOperandSpec kRmsQuantOperands[] = {
    { "x", RAD_OPD_IN, 0 },      { "residual", RAD_OPD_INOUT, 1 }, { "w", RAD_OPD_WEIGHT, 0 },
    { "q", RAD_OPD_OUT, 0 },     { "scale", RAD_OPD_OUT, 0 },      { "out_bf16", RAD_OPD_OUT, 1 },
};

/* row_topk: src/r3d_rows.cpp:686-699 */
const RadParamSpec kRowTopkParams[] = {
    { "M", RAD_P_INT, RAD_REQUIRED, 0 },         { "N", RAD_P_INT, RAD_REQUIRED, 0 },
    { "R", RAD_P_INT, RAD_REQUIRED, 0 },         { "vocab_off", RAD_P_INT, RAD_OPTIONAL, 0 },
    { "dtype", RAD_P_STR, RAD_REQUIRED, 0 },
};
const RadOperandSpec kRowTopkOperands[] = {
    { "x", RAD_OPD_IN, 0 }, { "idx", RAD_OPD_OUT, 0 }, { "val", RAD_OPD_OUT, 0 }, { "pairs", RAD_OPD_OUT, 1 },
};

/* logit_rerank: src/r3d_rows.cpp:768-791, :1022-1030 */
const RadParamSpec kRerankParams[] = {
    { "M", RAD_P_INT, RAD_REQUIRED, 0 },         { "R", RAD_P_INT, RAD_REQUIRED, 0 },
    { "n_vocab", RAD_P_INT, RAD_REQUIRED, 0 },   { "n_embd", RAD_P_INT, RAD_REQUIRED, 0 },
    { "vocab_off", RAD_P_INT, RAD_OPTIONAL, 0 }, { "dtype", RAD_P_STR, RAD_REQUIRED, 0 },
};
const RadOperandSpec kRerankOperands[] = {
    { "x", RAD_OPD_IN, 0 },    { "head", RAD_OPD_WEIGHT, 0 }, { "idx_in", RAD_OPD_IN, 0 },
    { "idx", RAD_OPD_OUT, 0 }, { "val", RAD_OPD_OUT, 0 },     { "pairs", RAD_OPD_OUT, 1 },
};

/* sample_argmax: src/r3d_rows.cpp:285-288, :655-659 */
const RadParamSpec kArgmaxParams[] = {
    { "M", RAD_P_INT, RAD_REQUIRED, 0 }, { "n_vocab", RAD_P_INT, RAD_REQUIRED, 0 },
};
const RadOperandSpec kArgmaxOperands[] = {
    { "logits", RAD_OPD_IN, 0 }, { "params", RAD_OPD_IN, 0 }, { "token", RAD_OPD_OUT, 0 },
};

const RadOpSchema kSchemas[] = {
    { "logit_rerank", kRerankParams, COUNT_OF(kRerankParams), kRerankOperands, COUNT_OF(kRerankOperands),
      "R candidate ids a row rescored exactly against the full-precision head and re-sorted on those "
      "values; `idx_in` carries global ids as row_topk reports them, `vocab_off` is this rank's first "
      "column, an id outside its rows becomes a pad; ties break on the lower id." },
    { "sample_argmax", kArgmaxParams, COUNT_OF(kArgmaxParams), kArgmaxOperands, COUNT_OF(kArgmaxOperands),
      "greedy: the token of the largest logit, ties to the lower token id." },
    { "row_topk", kRowTopkParams, COUNT_OF(kRowTopkParams), kRowTopkOperands, COUNT_OF(kRowTopkOperands),
      "exact per-row top-R, descending, ties to the lower column; `vocab_off` shifts the reported "
      "columns to global ids and `pairs` is the [M, R, 2] (int32 id, f32 value) plane a sharded "
      "head gathers; an unfillable slot reports id -1." },
    { "quant_act_fp8", kQuantActParams, COUNT_OF(kQuantActParams), kQuantActOperands,
      COUNT_OF(kQuantActOperands),
      "symmetric e4m3 quantisation of a token-major activation per (row, `group` columns), plain "
      "row-major; scale = amax/448, a dequantisation multiplier." },
    { "gated_quant_fp8", kGatedQuantParams, COUNT_OF(kGatedQuantParams), kGatedQuantOperands,
      COUNT_OF(kGatedQuantOperands),
      "silu(gate)*up or sigmoid(gate)*up over a [M, 2n] gate_up plane, then the same quantiser." },
    { "rmsnorm_quant_fp8", kRmsQuantParams, COUNT_OF(kRmsQuantParams), kRmsQuantOperands,
      COUNT_OF(kRmsQuantOperands),
      "RMS norm (optionally after a residual add that is stored back) and the e4m3 group "
      "quantiser in one pass; the codes are taken over the bf16 norm output." },
    { "logits_gemm", kLogitsParams, COUNT_OF(kLogitsParams), kLogitsOperands,
      COUNT_OF(kLogitsOperands),
      "LM-head projection: logits[M, n_vocab] = x[M, n_embd] @ head^T, one row per sampled "
      "position." },
    { "gemm_nt_q", kGemmQParams, COUNT_OF(kGemmQParams), kGemmQOperands,
      COUNT_OF(kGemmQOperands),
      "y[M,N] = a[M,K] @ dequant(b)[N,K]^T; `dtype` names the operand-format combination." },
    { "gemm_nt_q_gated", kGemmQGatedParams, COUNT_OF(kGemmQGatedParams), kGemmQGatedOperands,
      COUNT_OF(kGemmQGatedOperands),
      "gemm_nt_q over a [2n, K] gate_up plane with the gated activation quantiser folded into "
      "the epilogue; outputs are [M, N/2]." },
};

/* ------------------------------------------------------------------ constraints */
const RadConstraint kCLogits[] = {
    { "n_vocab", RAD_C_GE, 1, nullptr }, { "n_embd", RAD_C_GE, 128, nullptr },
    { "dtype", RAD_C_IN, 0, "bf16" },
};
const RadConstraint kCMxfp4[] = { { "dtype", RAD_C_IN, 0, "mxfp4a8" } };
/* src/r3d_rows.cpp:1101-1112: no M and no N constraint (the drafter's op carries no N at issue; the entry
 * re-checks M <= 16 and N % 16) */
const RadConstraint kCW2A8[] = {
    { "dtype", RAD_C_IN, 0, "w2a8" }, { "K", RAD_C_DIV, 128, nullptr }, { "group", RAD_C_EQ, 128, nullptr },
};
const RadConstraint kCMxfp4Mx8[] = { { "dtype", RAD_C_IN, 0, "mxfp4mx8" }, { "K", RAD_C_DIV, 32, nullptr } };
const RadConstraint kCFp8[] = {
    { "dtype", RAD_C_IN, 0, "fp8a8" }, { "K", RAD_C_DIV, 128, nullptr },
    { "group", RAD_C_EQ, 128, nullptr },
};
const RadConstraint kCFp8Decode[] = {
    { "dtype", RAD_C_IN, 0, "fp8a8" }, { "M", RAD_C_LE, 8, nullptr },
    { "K", RAD_C_DIV, 128, nullptr },  { "group", RAD_C_EQ, 128, nullptr },
};
/* no constraint on N anywhere: the engine's gemm ops may omit N at issue and a constraint
 * on a key the query lacks never holds (src/r3d_rows.cpp:1105-1110) */
const RadConstraint kCMxfp4Decode[] = {
    { "dtype", RAD_C_IN, 0, "mxfp4a8" }, { "M", RAD_C_LE, 8, nullptr },
    { "K", RAD_C_DIV, 128, nullptr },
};

/* src/r3d_rows.cpp:1114-1124: the composed row's arena is sized at M = 64, so the band stops there */
const RadConstraint kCFp8Gated[] = {
    { "dtype", RAD_C_IN, 0, "fp8a8" }, { "M", RAD_C_LE, 64, nullptr },
    { "K", RAD_C_DIV, 128, nullptr },  { "group", RAD_C_EQ, 128, nullptr },
    { "act", RAD_C_IN, 0, "silu sigmoid" },
};

/* src/r3d_rows.cpp:1262-1265, :1419-1423 */
const RadConstraint kCBand[] = {
    { "n", RAD_C_GE, 1, nullptr }, { "dtype", RAD_C_IN, 0, "f32 bf16" },
};
const RadConstraint kCRmsQuant[] = {
    { "n", RAD_C_DIV, 4, nullptr }, { "group", RAD_C_EQ, 128, nullptr },
    { "dtype", RAD_C_IN, 0, "bf16" },
};

/* src/r3d_rows.cpp:784-791 */
const RadConstraint kCRerank[] = {
    { "M", RAD_C_GE, 1, nullptr },       { "R", RAD_C_GE, 1, nullptr },      { "R", RAD_C_LE, 32, nullptr },
    { "n_vocab", RAD_C_GE, 1, nullptr }, { "n_embd", RAD_C_GE, 1, nullptr }, { "dtype", RAD_C_IN, 0, "bf16" },
};
/* src/r3d_rows.cpp:1255 */
const RadConstraint kCArgmax[] = { { "n_vocab", RAD_C_GE, 1, nullptr } };
/* src/r3d_rows.cpp:1412-1418 */
const RadConstraint kCRowTopk[] = {
    { "N", RAD_C_DIV, 8, nullptr }, { "M", RAD_C_GE, 1, nullptr }, { "R", RAD_C_GE, 1, nullptr },
    { "R", RAD_C_LE, 32, nullptr }, { "dtype", RAD_C_IN, 0, "bf16" },
};

enum { kPrioPlain = 1000, kPrioDecode = 1100, kPrioQ8x = 1200 };

#define ROW(name, op, family, summary, shapes, dtypes, prio, cons, launch)               \
    { name, op, family, summary, shapes, dtypes, RAD_DOMAIN_DEVICE, prio, cons,          \
      COUNT_OF(cons), nullptr, 0, nullptr, nullptr, nullptr, launch, nullptr, nullptr,    \
      nullptr, nullptr, nullptr, nullptr }
/* the same with a scratch hook (the launch arena the engine provides) */
#define ROW_S(name, op, family, summary, shapes, dtypes, prio, cons, launch, scratch)    \
    { name, op, family, summary, shapes, dtypes, RAD_DOMAIN_DEVICE, prio, cons,          \
      COUNT_OF(cons), nullptr, 0, nullptr, nullptr, nullptr, launch, scratch, nullptr,    \
      nullptr, nullptr, nullptr, nullptr }

const RadKernelInfo kRows[] = {
    { "logits_gemm_e4m3", "logits_gemm", "vocab",
      "weight-streaming GEMV over the joined LM head on tcgen05: e4m3 codes feed the tensor core "
      "untouched, each bf16 activation travels as two exact e4m3 pieces, the block scale is "
      "applied to each 128-column partial in f32",
      "codes [n_vocab, n_embd] e4m3 dense, scale per (1 or 128 rows, 128 cols); M from "
      "numel(logits)/n_vocab, passes of 32 rows",
      "bf16 x, joined e4m3 + bf16/f16/f32 head, f32 logits",
      RAD_DOMAIN_DEVICE, kPrioPlain, kCLogits, COUNT_OF(kCLogits), nullptr, 0, nullptr,
      nullptr, nullptr, r3d_rad_logits_gemm_e4m3, nullptr, r3d_layout_head,
      r3d_relayout_head, nullptr, r3d_unrelayout_head, nullptr },

    /* src/r3d_rows.cpp:2145-2162: the joined-e4m3 sibling of the plain-head rerank row, with the head's hooks */
    { "logit_rerank_e4m3", "logit_rerank", "select",
      "R candidates a row rescored exactly against the joined e4m3 lm_head: a double-precision chain in "
      "ascending k per candidate (four candidates per warp, the products formed in parallel, the adds "
      "in the oracle's order), then the oracle's selection sort",
      "any M, R <= 32; the joined e4m3 head r3d_layout_head admits; M derives from numel(x)/n_embd; "
      "idx_in/idx/val at their own row pitches, pairs only densely packed",
      "bf16/f32 x, joined e4m3 + bf16/f16/f32 head, f32 values + i32 ids out, optional f32 pairs plane",
      RAD_DOMAIN_DEVICE, kPrioPlain, kCRerank, COUNT_OF(kCRerank), nullptr, 0, nullptr,
      nullptr, nullptr, r3d_rad_logit_rerank_e4m3, nullptr, r3d_layout_head,
      r3d_relayout_head, nullptr, r3d_unrelayout_head, nullptr },

    ROW("gemm_nt_q_mxfp4", "gemm_nt_q", "gemm",
        "mxfp4a8, any M: e2m1 nibbles go to tcgen05 packed (M <= 4, hardware E8M0 group scales) or "
        "unpacked by the tensor map; a_scale applied per 128 of K; M > 64 on 128x192 tiles",
        "b:32 / a:128 scale grids; nibble rows byte-packed; M from numel(y)/N",
        "e4m3 a + f32 a_scale, e2m1 b + E8M0 b_scale, bf16 y; b_ref ignored; a_sum refused",
        kPrioPlain, kCMxfp4, r3d_rad_gemm_nt_q),

    /* src/r3d_rows.cpp:1677-1703 */
    { "gemm_nt_q_w2a8_decode", "gemm_nt_q", "gemm",
      "w2a8 decode-band GEMV (the draft head): one thread per weight row walks the 2-bit plane 64 bytes at a "
      "time, byte-quads cut from each dword meet the int8 activation (de-permuted from step order in "
      "shared memory) in dp4a, each group flushes as (sub * a_scale) * b_scale with sub = is - zero * a_sum "
      "in the oracle's order: every value before the scales is an exact integer, so the row is bit-exact",
      "M <= 16; K a multiple of 128; N a multiple of 16; group exactly 128; M derives from numel(y)/N",
      "int8 a with an f32 per-row scale (quant_act_i8's step order), u2 b (stored as it is) with an f16 scale "
      "and a u8/u4 zero per 128 K in the canonical rad.planes join, f32 a_sum [K/128][Mpad] (required), bf16 y; "
      "b_ref refused; pb1/pb2 refused; an encoding transform declines at declare",
      RAD_DOMAIN_DEVICE, kPrioDecode, kCW2A8, COUNT_OF(kCW2A8), nullptr, 0, nullptr,
      nullptr, nullptr, r3d_rad_gemm_nt_q_w2a8_decode, nullptr, r3d_layout_gemm_w2a8,
      r3d_relayout_gemm_w2a8, nullptr, r3d_unrelayout_gemm_w2a8, nullptr },

    /* not a reference row: the OCP-MX activation spelling of the mxfp4 band (weights as above) */
    ROW("gemm_nt_q_mxfp4mx8", "gemm_nt_q", "gemm",
        "mxfp4 weights x mxfp8 activations, any M: both E8M0 scale sets are applied by the tensor core "
        "(kind::mxf8f6f4 block scaling); M > 64 on CTA-pair 256x192 tiles with one accumulation over K",
        "b:32 / a:32 scale grids; nibble rows byte-packed; M from numel(y)/N",
        "e4m3 a + E8M0 a_scale, e2m1 b + E8M0 b_scale, bf16 y; b_ref ignored; a_sum refused",
        kPrioPlain, kCMxfp4Mx8, r3d_rad_gemm_nt_q_mx8),

    ROW("gemm_nt_q_fp8a8", "gemm_nt_q", "gemm",
        "fp8a8, any M: e4m3 codes feed tcgen05 untouched (swap-AB weight streaming up to M = 64, "
        "128x192 tiles above); each 128-of-K partial is flushed with a_scale and b_scale",
        "K a multiple of 128; any N; b_scale per 128x128 block or per row; M from numel(y)/N",
        "e4m3 a + f32 a_scale, e4m3 b + bf16 b_scale, bf16 y; a_sum and b_ref refused",
        kPrioPlain, kCFp8, r3d_rad_gemm_nt_q_fp8),

    ROW("gemm_nt_q_fp8a8_decode", "gemm_nt_q", "gemm",
        "fp8a8 decode band: the same weight-streaming walk, every weight byte read once",
        "M <= 8; K a multiple of 128; any N; a weight plane off the 4-byte grid resolves past "
        "this row",
        "as gemm_nt_q_fp8a8",
        kPrioDecode, kCFp8Decode, r3d_rad_gemm_nt_q_fp8_decode),

    ROW("gemm_nt_q_mxfp4_decode", "gemm_nt_q", "gemm",
        "mxfp4a8 decode band, fp32 walk: per-32 group partials scaled by 2^(e8m0-127)",
        "M <= 8; K a multiple of 128; any N",
        "as gemm_nt_q_mxfp4",
        kPrioDecode, kCMxfp4Decode, r3d_rad_gemm_nt_q_mxfp4_decode),

    ROW("gemm_nt_q_mxfp4_decode_q8x", "gemm_nt_q", "gemm",
        "mxfp4a8 decode band, int8-per-32 activation arm: activations requantised per "
        "dispatch, exact integer dots per group, the arm's own flush chain; reads the nibble "
        "plane as it is (no repacked plane). K % 256 != 0 rides the fp32 walk in place",
        "M <= 8; K a multiple of 128; any N",
        "as gemm_nt_q_mxfp4; R3D_MXFP4_Q8X=0 withdraws this row at registration",
        kPrioQ8x, kCMxfp4Decode, r3d_rad_gemm_nt_q_mxfp4_decode_q8x),

    { "gemm_nt_q_gated_fp8a8", "gemm_nt_q_gated", "gemm",
      "the fp8a8 band writing its bf16 gate_up plane into the launch scratch, closed by the gated "
      "activation quantiser in the same call: byte-identical to gemm_nt_q followed by "
      "gated_quant_fp8; no [M, 2n] tensor reaches the caller",
      "M <= 64 (the scratch is sized at the band's bound); K a multiple of 128; N = 2n; M derives "
      "from numel(q)/n",
      "e4m3 a + f32 a_scale per (row, 128 K), e4m3 b + bf16 scale per 128x128 tile, e4m3 q + f32 scale "
      "out, optional bf16/f32 product; act silu or sigmoid; a_sum refused",
      RAD_DOMAIN_DEVICE, kPrioPlain, kCFp8Gated, COUNT_OF(kCFp8Gated), nullptr, 0, nullptr,
      nullptr, nullptr, r3d_rad_gemm_nt_q_gated_fp8, r3d_rad_gemm_nt_q_gated_fp8_scratch, nullptr,
      nullptr, nullptr, nullptr, nullptr },

    /* the activation producers in front of the bands (src/r3d_rows.cpp:1892-1907, :2093-2101) */
    ROW("quant_act_fp8_act", "quant_act_fp8", "band",
        "per-group symmetric e4m3 quantisation of an activation, plain row-major: one block per "
        "(row, group)",
        "f32/bf16 input; group clamped to n; scale = amax/448 (1 for an all-zero group)",
        "activation in, e4m3 codes and f32 group scales out",
        kPrioPlain, kCBand, r3d_rad_quant_act_fp8),

    ROW("gated_quant_fp8_act", "gated_quant_fp8", "band",
        "silu(gate)*up (or sigmoid(gate)*up) and the same quantiser in one pass; the gated value "
        "narrows to bf16 once and the quantiser sees that value",
        "f32/bf16 gate_up [M, 2n], gate half first; group clamped to n",
        "gate_up in, e4m3 codes, f32 scales, optional bf16/f32 gated output",
        kPrioPlain, kCBand, r3d_rad_gated_quant_fp8),

    ROW("rmsnorm_quant_fp8", "rmsnorm_quant_fp8", "quant",
        "RMS norm and the e4m3 group quantiser in one pass over the row; with a residual the "
        "bf16-narrowed sum is stored before the variance reads it; the codes are taken over the "
        "bf16 norm output",
        "n a multiple of 4 and at most 30720, group 128; one block per row, the row staged in "
        "shared memory",
        "bf16 x (+ bf16 residual), f32/bf16 w, e4m3 codes with f32 per-group scales, optional "
        "bf16/f32 norm output",
        kPrioPlain, kCRmsQuant, r3d_rad_rmsnorm_quant_fp8),

    /* the consumer behind the column-sharded LM head (src/r3d_rows.cpp:2084-2091) */
    ROW_S("rowtopk_bf16", "row_topk", "select",
        "exact per-row top-R of a bf16 matrix, descending, ties to the lower column: a tournament "
        "of 512-item warp tiles held in registers, repeated over the survivors",
        "any M, N a multiple of 8, R <= 32",
        "bf16 in, f32 values + i32 columns out, optional f32 pairs plane",
        kPrioPlain, kCRowTopk, r3d_rad_row_topk, r3d_rad_row_topk_scratch),

    /* greedy decode directly behind logits_gemm's f32 logits (src/r3d_rows.cpp:1791-1798) */
    ROW_S("sample_argmax_f32", "sample_argmax", "sample",
        "greedy, ties to the lower token id: the top-1 of the (value descending, id ascending) "
        "tournament that row_topk runs, so greedy and top-1 agree",
        "any vocabulary",
        "f32 logits, i32 token; the parameter blob is not read",
        kPrioPlain, kCArgmax, r3d_rad_sample_argmax, r3d_rad_sample_argmax_scratch),
};

/* ------------------------------------------------------------------ registration gate */
bool row_hidden(const RadKernelInfo& k) {
    static const bool no_fp8 = getenv("R3D_NO_FP8A8") != nullptr;
    static const bool no_fp8_dec = getenv("R3D_NO_FP8_DEC") != nullptr;
    static const bool no_mx = getenv("R3D_NO_MXFP4") != nullptr;
    static const bool no_mx_dec = getenv("R3D_NO_FP4_DEC") != nullptr;
    static const bool q8x_off = r3d_mxfp4_q8x_off();
    static const bool no_df = getenv("R3D_NO_DFLASH") != nullptr;      /* the drafter family's lever, src/r3d_rows.cpp:2224-2227 */
    if (no_df && (!strcmp(k.op, "logit_rerank") || !strcmp(k.name, "gemm_nt_q_w2a8_decode"))) return true;
    if (!strcmp(k.name, "gemm_nt_q_fp8a8")) return no_fp8;
    if (!strcmp(k.name, "gemm_nt_q_fp8a8_decode")) return no_fp8 || no_fp8_dec;
    if (!strcmp(k.name, "gemm_nt_q_gated_fp8a8")) return no_fp8;       /* src/r3d_rows.cpp:2235 */
    if (!strcmp(k.name, "gemm_nt_q_mxfp4")) return no_mx;
    if (!strcmp(k.name, "gemm_nt_q_mxfp4mx8")) return no_mx;
    if (!strcmp(k.name, "gemm_nt_q_mxfp4_decode")) return no_mx || no_mx_dec;
    /* the q8x sibling rides every lever of its band, plus its own */
    if (!strcmp(k.name, "gemm_nt_q_mxfp4_decode_q8x")) return no_mx || no_mx_dec || q8x_off;
    return false;
}

} /* namespace */

extern "C" {

uint32_t rad_plugin_abi_version(void) { return RAD_ABI_VERSION; }

const RadPluginInfo* rad_plugin_info(void) {
    static const RadPluginInfo info = {
        RAD_PLUGIN_KERNEL, "libr3d_b200", "0.1.0",
        "radiance kernel library for NVIDIA B200: quantised-matmul bands (fp8a8, mxfp4a8, "
        "e4m3 LM head)",
        "sm_100a",
    };
    return &info;
}

int rad_kernel_schema_count(void) { return COUNT_OF(kSchemas); }
const RadOpSchema* rad_kernel_schema_at(int i) {
    return (i >= 0 && i < COUNT_OF(kSchemas)) ? &kSchemas[i] : nullptr;
}

int rad_kernel_count(void) {
    int n = 0;
    for (const RadKernelInfo& k : kRows) if (!row_hidden(k)) ++n;
    return n;
}
const RadKernelInfo* rad_kernel_at(int i) {
    if (i < 0) return nullptr;
    for (const RadKernelInfo& k : kRows)
        if (!row_hidden(k) && i-- == 0) return &k;
    return nullptr;
}

} /* extern "C" */
