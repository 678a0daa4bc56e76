"""Host side of the plugin, no GPU needed: the loader surface, the row tables and band
resolution, the registration-gate kill switches, the entries' refusal codes (every case here
is refused before any device work), and the LM-head layout hooks."""
import ctypes as C
import os
import re
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

from libr3d_b200 import abi
from libr3d_b200.plugin import EXPORTS, ArgPack, Plugin, planes_blob, tensor_desc

ROOT = Path(__file__).resolve().parent.parent


def test_exports_every_declared_symbol(plug):
    for name in EXPORTS:
        assert hasattr(plug.lib, name), name
    # and the list above covers every function the two headers declare
    declared = set()
    for h in ("rad_abi.h", "r3d_b200.h"):
        text = (ROOT / "include" / h).read_text()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        declared |= set(re.findall(r"\b((?:rad|r3d)_[a-z0-9_]+)\s*\(", text))
    declared -= {"rad_arg_in"}
    assert declared <= set(EXPORTS), declared - set(EXPORTS)


def test_identity_and_abi_pin(plug):
    assert plug.lib.rad_plugin_abi_version() == 26            # README.md:10 of the reference
    info = plug.info()
    assert info["kind"] == 1 and info["targets"] == "sm_100a"


def test_schemas_entry_for_entry(plug):
    s = plug.schemas()
    I, S = 0, 2
    R, O = 0, 1
    assert s["gemm_nt_q"]["params"] == [("M", I, R), ("N", I, R), ("K", I, R), ("group", I, R),
                                        ("dtype", S, R), ("pb1", I, O), ("pb2", I, O),
                                        ("split_n", I, O)]
    IN, OUT, W = 0, 1, 3
    assert s["gemm_nt_q"]["operands"] == [("a", IN, 0), ("a_scale", IN, 1), ("b", W, 0),
                                          ("b_scale", W, 0), ("y", OUT, 0), ("a_sum", IN, 1),
                                          ("b_ref", W, 1)]
    assert s["logits_gemm"]["params"] == [("M", I, R), ("n_vocab", I, R), ("n_embd", I, R),
                                          ("dtype", S, R)]
    assert s["logits_gemm"]["operands"] == [("x", IN, 0), ("lm_head", W, 0), ("logits", OUT, 0)]
    assert [p[0] for p in s["gemm_nt_q_gated"]["params"]] == ["M", "N", "K", "group", "dtype", "act"]
    assert [o[0] for o in s["gemm_nt_q_gated"]["operands"]] == ["a", "a_scale", "b", "b_scale", "q",
                                                                 "scale", "out_bf16"]
    F = 1
    INOUT = 2
    assert s["quant_act_fp8"]["params"] == [("M", I, R), ("n", I, R), ("group", I, R), ("dtype", S, R)]
    assert s["quant_act_fp8"]["operands"] == [("x", IN, 0), ("q", OUT, 0), ("scale", OUT, 0)]
    assert s["gated_quant_fp8"]["params"] == [("M", I, R), ("n", I, R), ("group", I, R), ("dtype", S, R),
                                              ("act", S, O)]
    assert s["gated_quant_fp8"]["operands"] == [("gate_up", IN, 0), ("q", OUT, 0), ("scale", OUT, 0),
                                                ("out_bf16", OUT, 1)]
    assert s["rmsnorm_quant_fp8"]["params"] == [("M", I, R), ("n", I, R), ("eps", F, R), ("group", I, R),
                                                ("dtype", S, R), ("wadd", F, O)]
    assert s["rmsnorm_quant_fp8"]["operands"] == [("x", IN, 0), ("residual", INOUT, 1), ("w", W, 0),
                                                  ("q", OUT, 0), ("scale", OUT, 0), ("out_bf16", OUT, 1)]
    assert s["row_topk"]["params"] == [("M", I, R), ("N", I, R), ("R", I, R), ("vocab_off", I, O), ("dtype", S, R)]
    assert s["logit_rerank"]["params"] == [("M", I, R), ("R", I, R), ("n_vocab", I, R), ("n_embd", I, R),
                                           ("vocab_off", I, O), ("dtype", S, R)]
    assert s["logit_rerank"]["operands"] == [("x", IN, 0), ("head", W, 0), ("idx_in", IN, 0), ("idx", OUT, 0),
                                             ("val", OUT, 0), ("pairs", OUT, 1)]
    assert s["sample_argmax"]["params"] == [("M", I, R), ("n_vocab", I, R)]
    assert s["sample_argmax"]["operands"] == [("logits", IN, 0), ("params", IN, 0), ("token", OUT, 0)]
    assert s["row_topk"]["operands"] == [("x", IN, 0), ("idx", OUT, 0), ("val", OUT, 0), ("pairs", OUT, 1)]
    assert plug.lib.rad_kernel_schema_at(-1) is None or not plug.lib.rad_kernel_schema_at(-1)
    assert not plug.lib.rad_kernel_schema_at(99)


def test_rows_names_priorities_constraints(plug):
    rows = {r.name: r for r in plug.rows()}
    want = {"logits_gemm_e4m3": 1000, "logit_rerank_e4m3": 1000, "gemm_nt_q_w2a8_decode": 1100, "gemm_nt_q_mxfp4": 1000, "gemm_nt_q_mxfp4mx8": 1000, "gemm_nt_q_fp8a8": 1000,
            "gemm_nt_q_fp8a8_decode": 1100, "gemm_nt_q_mxfp4_decode": 1100,
            "gemm_nt_q_mxfp4_decode_q8x": 1200, "gemm_nt_q_gated_fp8a8": 1000,
            "quant_act_fp8_act": 1000, "gated_quant_fp8_act": 1000, "rmsnorm_quant_fp8": 1000,
            "rowtopk_bf16": 1000, "sample_argmax_f32": 1000}
    assert {k: v.priority for k, v in rows.items()} == want
    assert all(r.domain == abi.RAD_DOMAIN_DEVICE and r.launch for r in rows.values())
    assert rows["logits_gemm_e4m3"].has_layout
    assert ("M", abi.RAD_C_LE, 8, None) in rows["gemm_nt_q_fp8a8_decode"].constraints
    assert ("group", abi.RAD_C_EQ, 128, None) in rows["gemm_nt_q_fp8a8"].constraints
    assert ("K", abi.RAD_C_DIV, 128, None) in rows["gemm_nt_q_mxfp4_decode"].constraints
    # never constrain N: the engine may omit it and an absent key fails its constraint
    assert not any(c[0] == "N" for r in rows.values() for c in r.constraints if r.op == "gemm_nt_q")
    assert not plug.lib.rad_kernel_at(len(rows)) and not plug.lib.rad_kernel_at(-1)


def test_band_resolution(plug):
    q = dict(N=27648, K=5120)
    name = lambda **kw: plug.resolve("gemm_nt_q", {**q, **kw}).name
    assert name(M=1, group=32, dtype="mxfp4a8") == "gemm_nt_q_mxfp4_decode_q8x"
    assert name(M=8, group=32, dtype="mxfp4a8") == "gemm_nt_q_mxfp4_decode_q8x"
    assert name(M=16, group=32, dtype="mxfp4a8") == "gemm_nt_q_mxfp4"
    assert name(M=8192, group=32, dtype="mxfp4mx8") == "gemm_nt_q_mxfp4mx8"
    assert plug.resolve("gemm_nt_q", dict(M=14, K=5120, group=128, dtype="w2a8")).name == "gemm_nt_q_w2a8_decode"   # no N at issue
    assert name(M=1, group=32, dtype="mxfp4mx8") == "gemm_nt_q_mxfp4mx8"
    assert name(M=4, group=128, dtype="fp8a8") == "gemm_nt_q_fp8a8_decode"
    assert name(M=9, group=128, dtype="fp8a8") == "gemm_nt_q_fp8a8"
    assert plug.resolve("gemm_nt_q", dict(M=1, N=8, K=200, group=128, dtype="fp8a8")) is None
    assert plug.resolve("gemm_nt_q", dict(M=1, N=8, K=256, group=64, dtype="fp8a8")) is None
    assert plug.resolve("gemm_nt_q", dict(M=1, N=8, K=256, group=128, dtype="w4a16")) is None
    # a query without M cannot satisfy the decode rows' M <= 8
    assert plug.resolve("gemm_nt_q", dict(N=8, K=256, group=128, dtype="fp8a8")).name == "gemm_nt_q_fp8a8"
    assert plug.resolve("logits_gemm", dict(M=1, n_vocab=151936, n_embd=5120, dtype="bf16")).name == \
        "logits_gemm_e4m3"
    assert plug.resolve("logits_gemm", dict(M=1, n_vocab=10, n_embd=64, dtype="bf16")) is None
    # the fused gate_up row: act is required, the band stops at the arena's M = 64
    gq = dict(N=512, K=256, group=128, dtype="fp8a8")
    assert plug.resolve("gemm_nt_q_gated", dict(M=64, act="silu", **gq)).name == "gemm_nt_q_gated_fp8a8"
    assert plug.resolve("gemm_nt_q_gated", dict(M=3, act="sigmoid", **gq)).name == "gemm_nt_q_gated_fp8a8"
    assert plug.resolve("gemm_nt_q_gated", dict(M=65, act="silu", **gq)) is None
    assert plug.resolve("gemm_nt_q_gated", dict(M=4, **gq)) is None
    assert plug.resolve("gemm_nt_q_gated", dict(M=4, act="gelu", **gq)) is None
    # the activation producers: one row per op (src/r3d_rows.cpp:1892-1907, :2093-2101 of libr3d)
    assert plug.resolve("quant_act_fp8", dict(M=4, n=5120, group=128, dtype="bf16")).name == "quant_act_fp8_act"
    assert plug.resolve("quant_act_fp8", dict(M=4, n=5120, group=128, dtype="f16")) is None
    assert plug.resolve("gated_quant_fp8", dict(M=4, n=13824, group=128, dtype="f32")).name == "gated_quant_fp8_act"
    rq = dict(M=4, eps=1e-6, dtype="bf16")
    assert plug.resolve("rmsnorm_quant_fp8", dict(n=5120, group=128, **rq)).name == "rmsnorm_quant_fp8"
    assert plug.resolve("rmsnorm_quant_fp8", dict(n=5122, group=128, **rq)) is None
    assert plug.resolve("rmsnorm_quant_fp8", dict(n=5120, group=64, **rq)) is None
    assert plug.resolve("row_topk", dict(M=4, N=19072, R=32, dtype="bf16")).name == "rowtopk_bf16"
    assert plug.resolve("row_topk", dict(M=4, N=19072, R=33, dtype="bf16")) is None
    assert plug.resolve("row_topk", dict(M=4, N=19071, R=8, dtype="bf16")) is None


_DUMP = r"""
import sys
sys.path.insert(0, %r)
from libr3d_b200.plugin import Plugin
p = Plugin()
print(",".join(sorted(r.name for r in p.rows())))
r = p.resolve("gemm_nt_q", dict(M=1, N=64, K=256, group=32, dtype="mxfp4a8"))
print(r.name if r else "-")
r = p.resolve("gemm_nt_q", dict(M=1, N=64, K=256, group=128, dtype="fp8a8"))
print(r.name if r else "-")
""" % str(ROOT)


def _rows_under(env):
    e = {k: v for k, v in os.environ.items() if not k.startswith("R3D_")}
    e.update(env)
    out = subprocess.run([sys.executable, "-c", _DUMP], env=e, capture_output=True, text=True,
                         check=True).stdout.split()
    return set(out[0].split(",")), out[1], out[2]


ALL = {"logits_gemm_e4m3", "logit_rerank_e4m3", "gemm_nt_q_w2a8_decode", "gemm_nt_q_mxfp4", "gemm_nt_q_mxfp4mx8", "gemm_nt_q_fp8a8", "gemm_nt_q_fp8a8_decode",
       "gemm_nt_q_mxfp4_decode", "gemm_nt_q_mxfp4_decode_q8x", "gemm_nt_q_gated_fp8a8",
       "quant_act_fp8_act", "gated_quant_fp8_act", "rmsnorm_quant_fp8", "rowtopk_bf16", "sample_argmax_f32"}


@pytest.mark.parametrize("env,hidden,mx_row,f8_row", [
    ({}, set(), "gemm_nt_q_mxfp4_decode_q8x", "gemm_nt_q_fp8a8_decode"),
    ({"R3D_MXFP4_Q8X": "0"}, {"gemm_nt_q_mxfp4_decode_q8x"}, "gemm_nt_q_mxfp4_decode", "gemm_nt_q_fp8a8_decode"),
    ({"R3D_MXFP4_Q8X": "1"}, set(), "gemm_nt_q_mxfp4_decode_q8x", "gemm_nt_q_fp8a8_decode"),
    ({"R3D_NO_FP4_DEC": "1"}, {"gemm_nt_q_mxfp4_decode", "gemm_nt_q_mxfp4_decode_q8x"}, "gemm_nt_q_mxfp4", "gemm_nt_q_fp8a8_decode"),
    ({"R3D_NO_MXFP4": ""}, {"gemm_nt_q_mxfp4", "gemm_nt_q_mxfp4mx8", "gemm_nt_q_mxfp4_decode", "gemm_nt_q_mxfp4_decode_q8x"}, "-", "gemm_nt_q_fp8a8_decode"),
    ({"R3D_NO_FP8_DEC": "1"}, {"gemm_nt_q_fp8a8_decode"}, "gemm_nt_q_mxfp4_decode_q8x", "gemm_nt_q_fp8a8"),
    ({"R3D_NO_FP8A8": "1"}, {"gemm_nt_q_fp8a8", "gemm_nt_q_fp8a8_decode", "gemm_nt_q_gated_fp8a8"}, "gemm_nt_q_mxfp4_decode_q8x", "-"),
    ({"R3D_NO_DFLASH": "1"}, {"logit_rerank_e4m3", "gemm_nt_q_w2a8_decode"}, "gemm_nt_q_mxfp4_decode_q8x", "gemm_nt_q_fp8a8_decode"),
])
def test_kill_switch_matrix(env, hidden, mx_row, f8_row):
    # levers act at registration: a hidden row is not enumerated and the band re-resolves
    # (src/r3d_rows.cpp:2216-2236 of the reference); presence levers fire on any value, the
    # q8x lever only on the literal "0"
    rows, mx, f8 = _rows_under(env)
    assert rows == ALL - hidden and mx == mx_row and f8 == f8_row


# ------------------------------------------------------------------ refusal matrix
def _fp8_args(M=2, N=256, K=256, drop=(), **over):
    z = np.zeros(16, np.uint8).ctypes.data          # a live host pointer: refusals precede any use
    t = dict(a=tensor_desc(z, abi.RAD_F8E4M3, [M, K]), a_scale=tensor_desc(z, abi.RAD_F32, [M, K // 128]),
             b=tensor_desc(z, abi.RAD_F8E4M3, [N, K]),
             b_scale=tensor_desc(z, abi.RAD_BF16, [(N + 127) // 128, K // 128]),
             y=tensor_desc(z, abi.RAD_BF16, [M, N]), a_sum=tensor_desc(None, abi.RAD_F32, []),
             b_ref=tensor_desc(None, abi.RAD_BF16, []))
    p = dict(dtype="fp8a8", M=64, N=N, K=K, group=128)
    for k, v in over.items():
        if k in t:
            t[k] = v
        else:
            p[k] = v
    for k in drop:
        p.pop(k)
    return ArgPack(list(t.values()), p), z


def _mx_args(M=2, N=64, K=256, drop=(), **over):
    z = np.zeros(16, np.uint8).ctypes.data
    t = dict(a=tensor_desc(z, abi.RAD_F8E4M3, [M, K]), a_scale=tensor_desc(z, abi.RAD_F32, [M, K // 128]),
             b=tensor_desc(z, abi.RAD_FP4E2M1, [N, K]), b_scale=tensor_desc(z, abi.RAD_E8M0, [N, K // 32]),
             y=tensor_desc(z, abi.RAD_BF16, [M, N]), a_sum=tensor_desc(None, abi.RAD_F32, []),
             b_ref=tensor_desc(None, abi.RAD_BF16, []))
    p = dict(dtype="mxfp4a8", M=64, N=N, K=K, group=32)
    for k, v in over.items():
        if k in t:
            t[k] = v
        else:
            p[k] = v
    for k in drop:
        p.pop(k)
    return ArgPack(list(t.values()), p), z


def _both(plug, sym, lib, ref_sym, pack):
    """This library's entry and, where it was built, the reference's own compiled entry on the same
    operands: the status must be the same; returns it."""
    from oracle import oracle as orc
    rc = plug.entry(sym)(C.byref(pack.args), None)
    R = orc.ref_band() if lib == "band" else orc.ref_more()
    if R is not None:
        assert getattr(R, ref_sym)(C.byref(pack.args), None) == rc, (sym, rc)
    return rc


def _ref_entries(which):
    """The reference's band file compiled by oracle/Makefile, or None where it was not built."""
    from oracle import oracle as orc
    return orc.ref_gemm(which)


Z = np.zeros(16, np.uint8)
U, SH, ST = abi.RAD_E_UNSUPPORTED, abi.RAD_E_SHAPE, abi.RAD_E_STRIDE


@pytest.mark.parametrize("over,code", [
    (dict(dtype="mxfp4a8"), U), (dict(pb1=1), U), (dict(K=200), U), (dict(drop=("N",)), SH),
    (dict(N=7, y=tensor_desc(Z.ctypes.data, abi.RAD_BF16, [2, 256])), SH),                                               # numel(y) % N
    (dict(a_sum=tensor_desc(Z.ctypes.data, abi.RAD_F32, [2])), U),
    (dict(b_ref=tensor_desc(Z.ctypes.data, abi.RAD_BF16, [2])), U),
    (dict(y=tensor_desc(Z.ctypes.data, abi.RAD_F32, [2, 256])), U),
    (dict(a=tensor_desc(Z.ctypes.data, abi.RAD_BF16, [2, 256])), U),
    (dict(b_scale=tensor_desc(Z.ctypes.data, abi.RAD_F16, [2, 2])), U),
    (dict(b_scale=tensor_desc(Z.ctypes.data, abi.RAD_BF16, [2, 4])), U),      # grid is 64 of K
    (dict(b_scale=tensor_desc(Z.ctypes.data, abi.RAD_BF16, [3, 2])), U),      # rows: neither N nor N/128
    (dict(b_scale=tensor_desc(Z.ctypes.data, abi.RAD_BF16, [300, 2])), SH),   # more rows than N
    (dict(a_scale=tensor_desc(Z.ctypes.data, abi.RAD_F32, [1, 2])), U),       # fewer rows than M
    (dict(group=64), SH),
    (dict(a=tensor_desc(Z.ctypes.data, abi.RAD_F8E4M3, [2, 256], [512, 2])), ST),
    (dict(y=tensor_desc(Z.ctypes.data, abi.RAD_BF16, [2, 256], [512, 2])), ST),
    (dict(a=tensor_desc(Z.ctypes.data, abi.RAD_F8E4M3, [1, 256])), SH),       # numel(a) < M*K
    (dict(b=tensor_desc(None, abi.RAD_F8E4M3, [256, 256])), U),               # absent operand
])
def test_fp8_entry_refusals(plug, over, code):
    pack, _ = _fp8_args(**over)
    for sym in ("r3d_rad_gemm_nt_q_fp8", "r3d_rad_gemm_nt_q_fp8_decode"):
        assert plug.entry(sym)(C.byref(pack.args), None) == code, sym
    # the reference's own entries (src/r3d_gemm_fp8a8.hip of libr3d, compiled where it lay) refuse the
    # same operands with the same status: every case here stops before any device work
    R = _ref_entries("fp8a8")
    if R is not None:
        for sym in ("ref_fp8a8_gemm_nt_q", "ref_fp8a8_gemm_nt_q_decode"):
            assert getattr(R, sym)(C.byref(pack.args), None) == code, sym


def test_activation_producer_refusals(plug):
    """Status codes and their precedence as in libr3d's entries (src/r3d_band.hip:459-548,
    src/r3d_more.hip:480-541): absent operand, dtype, shape, stride -- all before any device use."""
    z = np.zeros(16, np.uint8).ctypes.data
    T = tensor_desc
    IV, DT = abi.RAD_E_INVAL, abi.RAD_E_DTYPE

    def quant(x=None, q=None, sc=None, **p):
        ts = [x or T(z, abi.RAD_BF16, [2, 256]), q or T(z, abi.RAD_F8E4M3, [2, 256]), sc or T(z, abi.RAD_F32, [2, 2])]
        return _both(plug, "r3d_rad_quant_act_fp8", "band", "ref_band_quant_act_fp8", ArgPack(ts, dict(dict(M=2, n=256, group=128, dtype="bf16"), **p)))
    assert quant(x=T(None, abi.RAD_BF16, [2, 256])) == IV
    assert quant(x=T(z, abi.RAD_F16, [2, 256])) == DT
    assert quant(q=T(z, abi.RAD_U8, [2, 256])) == DT
    assert quant(sc=T(z, abi.RAD_BF16, [2, 2])) == DT
    assert quant(n=0) == SH
    assert quant(q=T(z, abi.RAD_F8E4M3, [1, 256])) == SH
    assert quant(sc=T(z, abi.RAD_F32, [2, 1])) == SH
    assert quant(x=T(z, abi.RAD_BF16, [2, 256], [512, 2])) == ST

    def gated(gu=None, ob=None, **p):
        ts = [gu or T(z, abi.RAD_BF16, [2, 512]), T(z, abi.RAD_F8E4M3, [2, 256]), T(z, abi.RAD_F32, [2, 2]),
              ob or T(None, abi.RAD_BF16, [])]
        return _both(plug, "r3d_rad_gated_quant_fp8", "band", "ref_band_gated_quant_fp8", ArgPack(ts, dict(dict(M=2, n=256, group=128, dtype="bf16"), **p)))
    assert gated(gu=T(z, abi.RAD_F16, [2, 512])) == DT
    assert gated(ob=T(z, abi.RAD_F16, [2, 256])) == DT
    assert gated(ob=T(z, abi.RAD_BF16, [1, 256])) == SH
    assert gated(gu=T(z, abi.RAD_BF16, [1, 2, 512], [2048, 1024, 1])) == ST     # a hole between the rows

    def rms(x=None, res=None, w=None, n_t=6, **p):
        ts = [x or T(z, abi.RAD_BF16, [2, 256]), res or T(None, abi.RAD_BF16, []), w or T(z, abi.RAD_BF16, [256]),
              T(z, abi.RAD_F8E4M3, [2, 256]), T(z, abi.RAD_F32, [2, 2]), T(None, abi.RAD_BF16, [])][:n_t]
        return _both(plug, "r3d_rad_rmsnorm_quant_fp8", "more", "ref_more_rmsnorm_quant_fp8", ArgPack(ts, dict(dict(M=2, n=256, eps=1e-6, group=128, dtype="bf16"), **p)))
    assert rms(n_t=4) == IV
    assert rms(x=T(z, abi.RAD_F32, [2, 256])) == DT                             # the published row is bf16
    assert rms(res=T(z, abi.RAD_F32, [2, 256])) == DT
    assert rms(w=T(z, abi.RAD_F16, [256])) == DT
    assert rms(n=30724) == SH                                                   # the row must fit shared memory
    assert rms(res=T(z, abi.RAD_BF16, [1, 256])) == SH
    assert rms(w=T(z, abi.RAD_BF16, [1, 256])) == ST                            # w is a rank-1 vector

    def topk(x=None, idx=None, val=None, pairs=None, **p):
        ts = [x or T(z, abi.RAD_BF16, [2, 256]), idx or T(z, abi.RAD_I32, [2, 4]), val or T(z, abi.RAD_F32, [2, 4]),
              pairs or T(None, abi.RAD_F32, [])]
        return _both(plug, "r3d_rad_row_topk", "more", "ref_more_row_topk", ArgPack(ts, dict(dict(M=2, N=256, R=4, dtype="bf16"), **p)))
    def argmax(lg=None, tok=None, **p):
        ts = [lg or T(z, abi.RAD_F32, [2, 256]), T(None, abi.RAD_U8, []), tok or T(z, abi.RAD_I32, [2])]
        return plug.entry("r3d_rad_sample_argmax")(C.byref(ArgPack(ts, dict(dict(M=2, n_vocab=256), **p)).args), None)
    assert argmax(tok=T(None, abi.RAD_I32, [2])) == IV
    assert argmax(lg=T(z, abi.RAD_BF16, [2, 256])) == DT
    assert argmax(tok=T(z, abi.RAD_F32, [2])) == DT
    assert argmax(tok=T(z, abi.RAD_I32, [1])) == SH and argmax(tok=T(z, abi.RAD_I32, [2, 1])) == SH
    assert argmax(lg=T(z, abi.RAD_F32, [512])) == ST                            # logits are a rank-2 plane
    assert argmax(lg=T(z, abi.RAD_F32, [2, 256], [512, 2])) == ST
    assert plug.resolve("sample_argmax", dict(M=2, n_vocab=151936)).name == "sample_argmax_f32"
    assert topk(val=T(None, abi.RAD_F32, [2, 4])) == IV
    assert topk(x=T(z, abi.RAD_F16, [2, 256])) == DT
    assert topk(idx=T(z, abi.RAD_F32, [2, 4])) == DT
    assert topk(pairs=T(z, abi.RAD_BF16, [2, 4, 2])) == DT
    assert topk(R=33) == SH and topk(R=0) == SH
    assert topk(idx=T(z, abi.RAD_I32, [1, 4])) == SH
    assert topk(pairs=T(z, abi.RAD_F32, [2, 2, 2])) == SH
    assert topk(pairs=T(z, abi.RAD_F32, [2, 4, 2], [16, 4, 1])) == ST           # not the dense [M, R, 2] plane


def test_fp8_decode_row_band_bound_and_alignment(plug):
    pack, _ = _fp8_args(M=9)
    assert plug.entry("r3d_rad_gemm_nt_q_fp8_decode")(C.byref(pack.args), None) == U
    # M comes from numel(y)/N, never from the M parameter (here 64)
    pack, _ = _fp8_args(M=2, b=tensor_desc(Z.ctypes.data + 1, abi.RAD_F8E4M3, [256, 256]))
    assert plug.entry("r3d_rad_gemm_nt_q_fp8_decode")(C.byref(pack.args), None) == U


@pytest.mark.parametrize("over,code", [
    (dict(dtype="fp8a8"), U), (dict(pb2=3), U), (dict(drop=("K",)), SH), (dict(drop=("N",)), SH),
    (dict(a_sum=tensor_desc(Z.ctypes.data, abi.RAD_F32, [2])), U),
    (dict(b=tensor_desc(Z.ctypes.data, abi.RAD_F8E4M3, [64, 256])), U),
    (dict(b_scale=tensor_desc(Z.ctypes.data, abi.RAD_BF16, [64, 8])), U),
    (dict(b_scale=tensor_desc(Z.ctypes.data, abi.RAD_E8M0, [64, 4])), U),     # grid 64, not 32
    (dict(b_scale=tensor_desc(Z.ctypes.data, abi.RAD_E8M0, [32, 8])), U),     # fewer rows than N
    (dict(a_scale=tensor_desc(Z.ctypes.data, abi.RAD_F32, [2, 1])), U),       # grid 256, not 128
    (dict(b=tensor_desc(Z.ctypes.data, abi.RAD_FP4E2M1, [64, 256], [512, 1])), ST),  # rows not packed
    (dict(y=tensor_desc(Z.ctypes.data, abi.RAD_BF16, [2, 64], [128, 2])), ST),
])
def test_mxfp4_entry_refusals(plug, over, code):
    pack, _ = _mx_args(**over)
    for sym in ("r3d_rad_gemm_nt_q", "r3d_rad_gemm_nt_q_mxfp4_decode", "r3d_rad_gemm_nt_q_mxfp4_decode_q8x"):
        assert plug.entry(sym)(C.byref(pack.args), None) == code, sym
    R = _ref_entries("mxfp4")                      # src/r3d_gemm_mxfp4.hip's own entries: same status
    if R is not None:
        for sym in ("ref_mxfp4_gemm_nt_q", "ref_mxfp4_gemm_nt_q_decode", "ref_mxfp4_gemm_nt_q_decode_q8x"):
            assert getattr(R, sym)(C.byref(pack.args), None) == code, sym


def test_mxfp4_b_ref_is_accepted_and_ignored(plug):
    # refused only later, by the chip gate (no device here) or served on a GPU box -- never for b_ref
    pack, _ = _mx_args(b_ref=tensor_desc(Z.ctypes.data, abi.RAD_BF16, [64]), K=96,
                       a=tensor_desc(Z.ctypes.data, abi.RAD_F8E4M3, [2, 96]),
                       a_scale=tensor_desc(Z.ctypes.data, abi.RAD_F32, [2, 1]),
                       b=tensor_desc(Z.ctypes.data, abi.RAD_FP4E2M1, [64, 96]),
                       b_scale=tensor_desc(Z.ctypes.data, abi.RAD_E8M0, [64, 3]))
    # K = 96 passes the plan of the plain row but fails the decode rows' K % 128 gate
    assert plug.entry("r3d_rad_gemm_nt_q_mxfp4_decode")(C.byref(pack.args), None) == U


def test_mxfp4_decode_rows_band_bound(plug):
    pack, _ = _mx_args(M=9)
    for sym in ("r3d_rad_gemm_nt_q_mxfp4_decode", "r3d_rad_gemm_nt_q_mxfp4_decode_q8x"):
        assert plug.entry(sym)(C.byref(pack.args), None) == U


# ------------------------------------------------------------------ LM head: blob + hooks
def _head(N=256, K=512, br=128, sdt=abi.RAD_BF16):
    codes = np.arange(N * K, dtype=np.uint32).astype(np.uint8).reshape(N, K)
    srows, scols = (N + br - 1) // br, (K + 127) // 128
    scale = (np.arange(srows * scols, dtype=np.uint16) + 0x3C00).reshape(srows, scols)
    if sdt == abi.RAD_F32:
        scale = scale.astype(np.float32)
    return codes, scale


def _logits_args(blob, M=2, N=256, K=512, **over):
    x = np.zeros(M * K, np.uint16)
    y = np.zeros(M * N, np.float32)
    t = dict(x=tensor_desc(x.ctypes.data, abi.RAD_BF16, [M, K]),
             lm_head=tensor_desc(blob.ctypes.data, abi.RAD_U8, [blob.size]),
             logits=tensor_desc(y.ctypes.data, abi.RAD_F32, [M, N]))
    p = dict(M=M, n_vocab=N, n_embd=K, dtype="bf16")
    for k, v in over.items():
        if k in t:
            t[k] = v
        elif v is None:
            p.pop(k)
        else:
            p[k] = v
    return ArgPack(list(t.values()), p), (x, y)


def test_logits_entry_refusals(plug):
    codes, scale = _head()
    good = np.frombuffer(planes_blob([("codes", abi.RAD_F8E4M3, (1, 1), codes),
                                      ("scale", abi.RAD_BF16, (128, 128), scale)]), np.uint8).copy()
    f = plug.entry("r3d_rad_logits_gemm_e4m3")
    D = abi.RAD_E_DTYPE

    from oracle import oracle as orc
    Rl = orc.ref_logits()                      # the reference's own entry (src/r3d_gemm_logits.hip), where built

    def rc(blob=good, **over):
        pack, keep = _logits_args(blob, **over)
        got = f(C.byref(pack.args), None)
        if Rl is not None:
            assert Rl.ref_logits_gemm_e4m3(C.byref(pack.args), None) == got, over
        return got

    assert rc(dtype="f16") == U and rc(n_vocab=None) == SH and rc(n_vocab=7) == SH
    assert rc(n_embd=510, x=tensor_desc(Z.ctypes.data, abi.RAD_BF16, [2, 510])) == U    # K % 4
    assert rc(logits=tensor_desc(Z.ctypes.data, abi.RAD_BF16, [2, 256])) == U            # f32 logits only
    assert rc(x=tensor_desc(Z.ctypes.data, abi.RAD_BF16, [2, 512], [1024, 2])) == ST
    assert rc(x=tensor_desc(Z.ctypes.data, abi.RAD_BF16, [2, 512], [256, 1])) == ST      # pitch < K
    bad = good.copy(); bad[0] ^= 0xFF
    assert rc(blob=bad) == D                                                              # no magic
    one = np.frombuffer(planes_blob([("codes", abi.RAD_F8E4M3, (1, 1), codes)]), np.uint8).copy()
    assert rc(blob=one) == D                                                              # one plane
    i8 = np.frombuffer(planes_blob([("codes", abi.RAD_I8, (1, 1), codes),
                                    ("scale", abi.RAD_BF16, (128, 128), scale)]), np.uint8).copy()
    assert rc(blob=i8) == SH                                                              # int8 head
    g64 = np.frombuffer(planes_blob([("codes", abi.RAD_F8E4M3, (1, 1), codes),
                                     ("scale", abi.RAD_BF16, (128, 64), scale)]), np.uint8).copy()
    assert rc(blob=g64) == U                                                              # 64-col scale grid
    wrongn = np.frombuffer(planes_blob([("codes", abi.RAD_F8E4M3, (1, 1), codes[:200]),
                                        ("scale", abi.RAD_BF16, (128, 128), scale)]), np.uint8).copy()
    assert rc(blob=wrongn) == SH


def test_logit_rerank_entry_refusals(plug):
    """every refusal of the rerank entry, status for status against the reference's own compiled entry
    (src/r3d_logit_rerank_e4m3.hip:226-345), which reads the head's header on the host like this one"""
    codes, scale = _head()
    N, K = codes.shape
    good = np.frombuffer(planes_blob([("codes", abi.RAD_F8E4M3, (1, 1), codes),
                                      ("scale", abi.RAD_BF16, (128, 128), scale)]), np.uint8).copy()
    f = plug.entry("r3d_rad_logit_rerank_e4m3")
    from oracle import oracle as orc
    Rr = orc.ref_rerank()
    M, R = 2, 4
    buf = np.zeros(1 << 16, np.uint8)
    IV, D = abi.RAD_E_INVAL, abi.RAD_E_DTYPE

    def rc(blob=good, drop=None, **over):
        t = dict(x=tensor_desc(buf.ctypes.data, abi.RAD_BF16, [M, K]),
                 head=tensor_desc(blob.ctypes.data, abi.RAD_U8, [blob.size]),
                 idx_in=tensor_desc(buf.ctypes.data, abi.RAD_I32, [M, R]),
                 idx=tensor_desc(buf.ctypes.data, abi.RAD_I32, [M, R]),
                 val=tensor_desc(buf.ctypes.data, abi.RAD_F32, [M, R]),
                 pairs=tensor_desc(buf.ctypes.data, abi.RAD_F32, [M, R, 2]))
        p = dict(M=M, R=R, n_vocab=N, n_embd=K, vocab_off=0, dtype="bf16")
        for k, v in over.items():
            if k in t:
                t[k] = v
            elif v is None:
                p.pop(k)
            else:
                p[k] = v
        ts = list(t.values())
        if drop is not None:
            ts = ts[:drop]
        pack = ArgPack(ts, p)
        got = f(C.byref(pack.args), None)
        if Rr is not None:
            assert Rr.ref_logit_rerank_e4m3(C.byref(pack.args), None) == got, (over, drop)
        return got

    assert rc(drop=4) == IV                                                               # fewer than five operands
    assert rc(val=tensor_desc(None, abi.RAD_F32, [])) == IV
    assert rc(n_vocab=None) == SH and rc(n_embd=None) == SH and rc(R=0) == SH
    assert rc(R=33, idx_in=tensor_desc(buf.ctypes.data, abi.RAD_I32, [M, 33]), idx=tensor_desc(buf.ctypes.data, abi.RAD_I32, [M, 33]),
              val=tensor_desc(buf.ctypes.data, abi.RAD_F32, [M, 33])) == U                 # R beyond the band
    assert rc(idx=tensor_desc(buf.ctypes.data, abi.RAD_I32, [M, 3])) == SH
    assert rc(x=tensor_desc(buf.ctypes.data, abi.RAD_F16, [M, K])) == D
    assert rc(idx_in=tensor_desc(buf.ctypes.data, abi.RAD_F32, [M, R])) == D
    bad = good.copy(); bad[0] ^= 0xFF
    assert rc(blob=bad) == U                                                              # a plain head: not this row's
    one = np.frombuffer(planes_blob([("codes", abi.RAD_F8E4M3, (1, 1), codes)]), np.uint8).copy()
    assert rc(blob=one) == D
    i8 = np.frombuffer(planes_blob([("codes", abi.RAD_I8, (1, 1), codes),
                                    ("scale", abi.RAD_BF16, (128, 128), scale)]), np.uint8).copy()
    assert rc(blob=i8) == SH
    g64 = np.frombuffer(planes_blob([("codes", abi.RAD_F8E4M3, (1, 1), codes),
                                     ("scale", abi.RAD_BF16, (128, 64), scale)]), np.uint8).copy()
    assert rc(blob=g64) == D
    assert rc(pairs=tensor_desc(buf.ctypes.data, abi.RAD_F32, [M, R])) == SH              # too small
    assert rc(pairs=tensor_desc(buf.ctypes.data, abi.RAD_F32, [M, R, 2], [4 * R, 2, 1])) == ST   # not densely packed
    assert rc(x=tensor_desc(buf.ctypes.data, abi.RAD_BF16, [M, K], [2 * K, 2])) == ST


def _enc(roles=("codes", "scale"), dtypes=(abi.RAD_F8E4M3, abi.RAD_BF16), scheme=b"affine",
         blocks=((1, 1), (128, 128)), transform=b""):
    e = abi.RadEncoding()
    e.scheme, e.n_planes, e.transform = scheme, len(roles), transform
    for i, (r, d, b) in enumerate(zip(roles, dtypes, blocks)):
        e.plane[i].role, e.plane[i].kind, e.plane[i].dtype = r.encode(), abi.RAD_PLANE_TILED, d
        e.plane[i].block[0], e.plane[i].block[1] = b
    return e


def test_layout_hooks_roundtrip_and_gates(plug):
    L = plug.lib
    codes, scale = _head(N=130, K=300)
    planes = (abi.RadTensor * 2)(tensor_desc(codes.ctypes.data, abi.RAD_F8E4M3, codes.shape),
                                 tensor_desc(scale.ctypes.data, abi.RAD_BF16, scale.shape))
    sel = (C.c_int * 2)(0, 1)
    lay = abi.RadLayout()
    enc = _enc()
    args = (None, 0, 1, C.byref(enc), sel, planes, 2)
    assert L.r3d_layout_head(*args, C.byref(lay)) == abi.RAD_OK and lay.bytes > codes.nbytes
    dst = np.zeros(lay.bytes, np.uint8)
    assert L.r3d_relayout_head(*args, C.c_void_p(dst.ctypes.data), C.c_int64(dst.size)) == abi.RAD_OK
    want = np.frombuffer(planes_blob([("codes", abi.RAD_F8E4M3, (1, 1), codes),
                                      ("scale", abi.RAD_BF16, (128, 128), scale)]), np.uint8)
    assert np.array_equal(dst, want)                     # the hook writes the documented blob
    c2, s2 = np.zeros_like(codes), np.zeros_like(scale)
    back = (abi.RadTensor * 2)(tensor_desc(c2.ctypes.data, abi.RAD_F8E4M3, c2.shape),
                               tensor_desc(s2.ctypes.data, abi.RAD_BF16, s2.shape))
    assert L.r3d_unrelayout_head(None, 0, 1, C.byref(enc), sel, C.c_void_p(dst.ctypes.data),
                                 C.c_int64(dst.size), back, 2) == abi.RAD_OK
    assert np.array_equal(c2, codes) and np.array_equal(s2, scale)
    # gates (src/r3d_gemm_logits.hip:233-254 of the reference)
    D = abi.RAD_E_DTYPE
    assert L.r3d_layout_head(None, 0, 0, C.byref(enc), sel, planes, 2, C.byref(lay)) == U   # operand
    assert L.r3d_layout_head(None, 0, 1, C.byref(enc), sel, planes, 1, C.byref(lay)) == U
    for bad in (_enc(dtypes=(abi.RAD_I8, abi.RAD_BF16)), _enc(scheme=b"lattice"),
                _enc(roles=("scale", "codes")), _enc(transform=b"givens"),
                _enc(dtypes=(abi.RAD_F8E4M3, abi.RAD_U8)), _enc(blocks=((1, 2), (128, 128)))):
        assert L.r3d_layout_head(None, 0, 1, C.byref(bad), sel, planes, 2, C.byref(lay)) == D


def _w2_enc(zero_dt=abi.RAD_U8, scale_dt=abi.RAD_F16, codes_dt=abi.RAD_U2, scheme=b"affine", transform=b"",
            roles=("codes", "scale", "zero"), group=128):
    return _enc(roles=roles, dtypes=(codes_dt, scale_dt, zero_dt), scheme=scheme, transform=transform,
                blocks=((1, 1), (1, group), (1, group)))


def test_w2a8_layout_hooks_roundtrip_and_gates(plug):
    """the w2a8 row's hooks (operand 3 = the joined scale + zero planes) against the reference's own hook
    compiled host-only from src/r3d_gemm_w2a8.hip:1362-1401, gate for gate"""
    from oracle import oracle as orc
    L = plug.lib
    Rw = orc.ref_w2a8_host()
    N, K = 32, 512
    G = K // 128
    rng = np.random.default_rng(2)
    scale = rng.integers(0, 0x3C00, (N, G)).astype(np.uint16)
    zero = rng.integers(0, 256, (N, G), dtype=np.uint8)
    planes = (abi.RadTensor * 2)(tensor_desc(scale.ctypes.data, abi.RAD_F16, scale.shape),
                                 tensor_desc(zero.ctypes.data, abi.RAD_U8, zero.shape))
    sel = (C.c_int * 2)(1, 2)
    lay = abi.RadLayout()

    def params(**kw):
        items = [abi.RadParam(k.encode(), abi.RAD_PK_INT, v, 0, None, 0.0) for k, v in kw.items()]
        return (abi.RadParam * max(1, len(items)))(*items), len(items)

    def rc(enc, operand=3, n=2, pl=planes, se=sel, **kw):
        kw = {**dict(N=N, K=K, group=128), **kw}
        pa, npar = params(**{k: v for k, v in kw.items() if v is not None})
        lay2 = abi.RadLayout()
        got = L.r3d_layout_gemm_w2a8(pa, npar, operand, C.byref(enc), se, pl, n, C.byref(lay))
        if Rw is not None:
            assert Rw.ref_layout_gemm_w2a8(pa, npar, operand, C.byref(enc), se, pl, n, C.byref(lay2)) == got
            if got == abi.RAD_OK:
                assert lay2.bytes == lay.bytes
        return got

    enc = _w2_enc()
    assert rc(enc) == abi.RAD_OK and lay.bytes > scale.nbytes + zero.nbytes
    pa, npar = params(N=N, K=K, group=128)
    dst = np.zeros(lay.bytes, np.uint8)
    assert L.r3d_relayout_gemm_w2a8(pa, npar, 3, C.byref(enc), sel, planes, 2, C.c_void_p(dst.ctypes.data),
                                    C.c_int64(dst.size)) == abi.RAD_OK
    want = np.frombuffer(planes_blob([("scale", abi.RAD_F16, (1, 128), scale), ("zero", abi.RAD_U8, (1, 128), zero)]), np.uint8)
    assert np.array_equal(dst, want)
    s2, z2 = np.zeros_like(scale), np.zeros_like(zero)
    back = (abi.RadTensor * 2)(tensor_desc(s2.ctypes.data, abi.RAD_F16, s2.shape), tensor_desc(z2.ctypes.data, abi.RAD_U8, z2.shape))
    assert L.r3d_unrelayout_gemm_w2a8(pa, npar, 3, C.byref(enc), sel, C.c_void_p(dst.ctypes.data), C.c_int64(dst.size),
                                      back, 2) == abi.RAD_OK
    assert np.array_equal(s2, scale) and np.array_equal(z2, zero)
    D = abi.RAD_E_DTYPE
    assert rc(enc, operand=2) == U and rc(enc, n=1) == U                    # the codes are stored as they are
    for bad in (_w2_enc(scheme=b"lattice"), _w2_enc(transform=b"givens"), _w2_enc(codes_dt=abi.RAD_U4),
                _w2_enc(scale_dt=abi.RAD_BF16), _w2_enc(zero_dt=abi.RAD_U2), _w2_enc(group=64),
                _w2_enc(roles=("codes", "zero", "scale"))):
        assert rc(bad) == D
    assert rc(_w2_enc(zero_dt=abi.RAD_U4)) == abi.RAD_OK
    assert rc(enc, group=64) == D and rc(enc, K=500) == SH and rc(enc, N=None) == SH
    assert rc(enc, N=N + 1) == SH                                           # planes of another geometry
    two = _enc(roles=("scale", "zero"), dtypes=(abi.RAD_F16, abi.RAD_U8), blocks=((1, 128), (1, 128)))
    assert rc(two, se=(C.c_int * 2)(0, 1)) == D                             # no codes plane in the encoding


def test_w2a8_entry_refusals(plug):
    """every refusal of the w2a8 row entry in the reference's order (src/r3d_gemm_w2a8.hip:964-1028, :1320-1342)"""
    N, K, M = 32, 512, 3
    G = K // 128
    buf = np.zeros(1 << 16, np.uint8)
    scale = np.zeros((N, G), np.uint16); zero = np.zeros((N, G), np.uint8)
    good = np.frombuffer(planes_blob([("scale", abi.RAD_F16, (1, 128), scale), ("zero", abi.RAD_U8, (1, 128), zero)]), np.uint8).copy()
    f = plug.entry("r3d_rad_gemm_nt_q_w2a8_decode")
    D = abi.RAD_E_DTYPE

    def rc(blob=good, **over):
        t = dict(a=tensor_desc(buf.ctypes.data, abi.RAD_I8, [M, K]), a_scale=tensor_desc(buf.ctypes.data, abi.RAD_F32, [M, 1]),
                 b=tensor_desc(buf.ctypes.data, abi.RAD_U2, [N, K]), b_scale=tensor_desc(blob.ctypes.data, abi.RAD_U8, [blob.size]),
                 y=tensor_desc(buf.ctypes.data, abi.RAD_BF16, [M, N]), a_sum=tensor_desc(buf.ctypes.data, abi.RAD_F32, [G, 16]),
                 b_ref=tensor_desc(None, abi.RAD_BF16, []))
        p = dict(M=M, N=N, K=K, group=128, dtype="w2a8")
        for k, v in over.items():
            if k in t:
                t[k] = v
            elif v is None:
                p.pop(k)
            else:
                p[k] = v
        return f(C.byref(ArgPack(list(t.values()), p).args), None)

    assert rc(a_sum=tensor_desc(None, abi.RAD_F32, [])) == U                     # the zero point needs the group sums
    assert rc(b_ref=tensor_desc(buf.ctypes.data, abi.RAD_BF16, [N, K])) == U
    assert rc(N=None) == SH and rc(y=tensor_desc(buf.ctypes.data, abi.RAD_BF16, [M, N - 1])) == SH
    assert rc(dtype="mxfp4a8") == U and rc(pb1=1) == U
    assert rc(group=64) == SH and rc(group=None) == SH and rc(K=None) == SH
    assert rc(K=500, a=tensor_desc(buf.ctypes.data, abi.RAD_I8, [M, 500]), b=tensor_desc(buf.ctypes.data, abi.RAD_U2, [N, 500])) == U
    assert rc(y=tensor_desc(buf.ctypes.data, abi.RAD_BF16, [17, N]), a=tensor_desc(buf.ctypes.data, abi.RAD_I8, [17, K])) == U   # M > 16
    assert rc(N=40, y=tensor_desc(buf.ctypes.data, abi.RAD_BF16, [M, 40]), b=tensor_desc(buf.ctypes.data, abi.RAD_U2, [40, K])) == U   # N % 16
    assert rc(a=tensor_desc(buf.ctypes.data, abi.RAD_U8, [M, K])) == U
    assert rc(a=tensor_desc(buf.ctypes.data, abi.RAD_I8, [M - 1, K])) == SH
    assert rc(a=tensor_desc(buf.ctypes.data, abi.RAD_I8, [M, K], [2 * K, 2])) == ST
    assert rc(b=tensor_desc(buf.ctypes.data + 2, abi.RAD_U2, [N, K])) == U       # breaks the dword walk
    assert rc(a_sum=tensor_desc(buf.ctypes.data, abi.RAD_F32, [G, 8])) == SH     # smaller than G x mpad
    bad = good.copy(); bad[0] ^= 0xFF
    assert rc(blob=bad) == D
    bf = np.frombuffer(planes_blob([("scale", abi.RAD_BF16, (1, 128), scale), ("zero", abi.RAD_U8, (1, 128), zero)]), np.uint8).copy()
    assert rc(blob=bf) == U
    z2 = np.frombuffer(planes_blob([("scale", abi.RAD_F16, (1, 128), scale), ("zero", abi.RAD_U2, (1, 128), zero)]), np.uint8).copy()
    assert rc(blob=z2) == U
    g64 = np.frombuffer(planes_blob([("scale", abi.RAD_F16, (1, 64), scale), ("zero", abi.RAD_U8, (1, 128), zero)]), np.uint8).copy()
    assert rc(blob=g64) == SH
    wrongn = np.frombuffer(planes_blob([("scale", abi.RAD_F16, (1, 128), scale[:16]), ("zero", abi.RAD_U8, (1, 128), zero)]), np.uint8).copy()
    assert rc(blob=wrongn) == SH


def test_no_product_code_touches_the_oracle():
    """The CPU checker is test infrastructure: nothing the package ships may import, load,
    link or run it."""
    pat = re.compile(r"liboracle|import\s+oracle|from\s+oracle|oracle[/.]")
    for f in list((ROOT / "libr3d_b200").rglob("*")):
        if f.is_file() and f.suffix in (".py", ".cu", ".cpp", ".h", ".cuh"):
            assert not pat.search(f.read_text()), f


def test_topk_rows_declare_a_launch_arena(plug):
    """row_topk and sample_argmax carry a scratch hook: two survivor planes of M * ceil(N / 4096) * R 64-bit keys
    (nothing when the row fits one block of the selection kernel), computed from the query when the operands are not there yet"""
    rows = {r.name: r for r in plug.rows()}
    assert rows["rowtopk_bf16"].has_scratch and rows["sample_argmax_f32"].has_scratch
    q = ArgPack([], dict(M=4, N=151936, R=32, dtype="bf16"))
    assert plug.lib.r3d_rad_row_topk_scratch(q.args) == 2 * 4 * 38 * 32 * 8
    assert plug.lib.r3d_rad_row_topk_scratch(ArgPack([], dict(M=4, N=4096, R=8, dtype="bf16")).args) == 0
    assert plug.lib.r3d_rad_sample_argmax_scratch(ArgPack([], dict(M=2, n_vocab=151936)).args) == 2 * 2 * 38 * 8
