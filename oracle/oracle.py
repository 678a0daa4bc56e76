"""ctypes loader for the CPU checker (oracle/liboracle.so) and the reference pin.

TEST INFRASTRUCTURE ONLY: imported by tests/, by __graft_entry__.smoke() and by bench.py's
CPU-baseline legs. Nothing under libr3d_b200/ may import this module.
"""
from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
_lib = None
_ref = None


def build() -> None:
    subprocess.run(["make", "-C", str(HERE)], check=True, capture_output=True)


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        so = HERE / "liboracle.so"
        if not so.exists():
            build()
        L = C.CDLL(str(so))
        L.orc_e4m3_to_f32.restype = C.c_float
        L.orc_e4m3_to_f32.argtypes = [C.c_uint8]
        L.orc_f32_to_e4m3.restype = C.c_uint8
        L.orc_f32_to_e4m3.argtypes = [C.c_float]
        L.orc_e2m1_to_f32.restype = C.c_float
        L.orc_e2m1_to_f32.argtypes = [C.c_uint8]
        L.orc_e2m1_x2.restype = C.c_int
        L.orc_e2m1_x2.argtypes = [C.c_uint8]
        L.orc_e8m0_to_f32.restype = C.c_float
        L.orc_e8m0_to_f32.argtypes = [C.c_uint8]
        L.orc_f32_to_bf16.restype = C.c_uint16
        L.orc_f32_to_bf16.argtypes = [C.c_float]
        L.orc_bf16_to_f32.restype = C.c_float
        L.orc_bf16_to_f32.argtypes = [C.c_uint16]
        L.orc_f16_to_f32.restype = C.c_float
        L.orc_f16_to_f32.argtypes = [C.c_uint16]
        L.orc_num_threads.restype = C.c_int
        L.orc_set_threads.argtypes = [C.c_int]
        L.orc_set_threads.restype = None
        _lib = L
    return _lib


def ref_pin() -> C.CDLL | None:
    """The reference's own header compiled as it lies (oracle/_ref/libref_pin.so), or None."""
    global _ref
    if _ref is None:
        so = HERE / "_ref" / "libref_pin.so"
        if not so.exists():
            return None
        R = C.CDLL(str(so))
        R.ref_e2m1_x2.restype = C.c_int
        R.ref_e2m1_x2.argtypes = [C.c_int]
        R.ref_e8m0_sc.restype = C.c_float
        R.ref_e8m0_sc.argtypes = [C.c_ubyte]
        _ref = R
    return _ref


_ref_band = None


def ref_band() -> C.CDLL | None:
    """The reference's activation-producer file (src/r3d_band.hip of libr3d) compiled as it lies by
    nvcc through oracle/hipstub (oracle/_ref/libref_band.so), or None when it was not built.
    Loading it needs the CUDA runtime library but no GPU for the CPU helpers."""
    global _ref_band
    if _ref_band is None:
        so = HERE / "_ref" / "libref_band.so"
        if not so.exists():
            return None
        try:
            R = C.CDLL(str(so))
        except OSError:
            return None
        R.ref_band_f32_to_e4m3.restype = C.c_ubyte
        R.ref_band_f32_to_e4m3.argtypes = [C.c_float]
        R.ref_band_f32_to_bf16.restype = C.c_ushort
        R.ref_band_f32_to_bf16.argtypes = [C.c_float]
        R.ref_band_sigmoid.restype = C.c_float
        R.ref_band_sigmoid.argtypes = [C.c_float]
        R.ref_band_f32_to_e4m3_n.argtypes = [C.c_void_p, C.c_longlong, C.c_void_p]
        R.ref_band_quant_act_fp8.argtypes = [C.c_void_p, C.c_void_p]
        R.ref_band_gated_quant_fp8.argtypes = [C.c_void_p, C.c_void_p]
        _ref_band = R
    return _ref_band


_ref_logits = None


def ref_logits() -> C.CDLL | None:
    """The reference's LM-head file (src/r3d_gemm_logits.hip of libr3d) compiled as it lies for
    sm_100a (oracle/_ref/libref_logits.so), or None when it was not built."""
    global _ref_logits
    if _ref_logits is None:
        so = HERE / "_ref" / "libref_logits.so"
        if not so.exists():
            return None
        try:
            R = C.CDLL(str(so))
        except OSError:
            return None
        R.ref_logits_gemm_e4m3.argtypes = [C.c_void_p, C.c_void_p]
        R.ref_logits_alloc.restype = C.c_void_p
        R.ref_logits_alloc.argtypes = [C.c_longlong]
        R.ref_logits_free.argtypes = [C.c_void_p]
        R.ref_logits_free.restype = None
        _ref_logits = R
    return _ref_logits


_ref_w2a8: list = []


def ref_w2a8_host() -> C.CDLL | None:
    """The host-only layout hook of src/r3d_gemm_w2a8.hip of libr3d compiled as it lies
    (oracle/_ref/libref_w2a8_host.so): ref_layout_gemm_w2a8 with the hook's own signature. None when
    the library was not built."""
    if not _ref_w2a8:
        so, R = HERE / "_ref" / "libref_w2a8_host.so", None
        if so.exists():
            try:
                R = C.CDLL(str(so))
            except OSError:
                R = None
        _ref_w2a8.append(R)
    return _ref_w2a8[0]


_ref_rerank: list = []


def ref_rerank() -> C.CDLL | None:
    """src/r3d_logit_rerank_e4m3.hip of libr3d compiled as it lies for sm_100a
    (oracle/_ref/libref_rerank.so): entry ref_logit_rerank_e4m3(const RadArgs*, stream) plus a managed
    allocator for the head blob. None when the library was not built."""
    if not _ref_rerank:
        so, R = HERE / "_ref" / "libref_rerank.so", None
        if so.exists():
            try:
                R = C.CDLL(str(so))
                R.ref_logit_rerank_e4m3.argtypes = [C.c_void_p, C.c_void_p]
                R.ref_rerank_alloc.restype = C.c_void_p
                R.ref_rerank_alloc.argtypes = [C.c_longlong]
                R.ref_rerank_free.argtypes = [C.c_void_p]
                R.ref_rerank_free.restype = None
            except OSError:
                R = None
        _ref_rerank.append(R)
    return _ref_rerank[0]


_ref_gemm: dict = {}


_ref_more: list = []


def ref_more() -> C.CDLL | None:
    """src/r3d_more.hip of libr3d compiled as it lies for sm_100a (oracle/_ref/libref_more.so): entry
    ref_more_rmsnorm_quant_fp8 and ref_more_row_topk, each (const RadArgs*, stream). None when the library was not built."""
    if not _ref_more:
        so, R = HERE / "_ref" / "libref_more.so", None
        if so.exists():
            try:
                R = C.CDLL(str(so))
                R.ref_more_rmsnorm_quant_fp8.argtypes = [C.c_void_p, C.c_void_p]
                R.ref_more_row_topk.argtypes = [C.c_void_p, C.c_void_p]
            except OSError:
                R = None
        _ref_more.append(R)
    return _ref_more[0]


def ref_gemm(which: str) -> C.CDLL | None:
    """The reference's band files compiled as they lie for sm_100a: which = "fp8a8"
    (src/r3d_gemm_fp8a8.hip -> oracle/_ref/libref_fp8a8.so; entries ref_fp8a8_gemm_nt_q, _decode, _gated)
    or "mxfp4" (src/r3d_gemm_mxfp4.hip -> libref_mxfp4.so; ref_mxfp4_gemm_nt_q, _decode, _decode_q8x).
    Every entry takes (const RadArgs*, stream). None when the library was not built."""
    if which not in _ref_gemm:
        so = HERE / "_ref" / f"libref_{which}.so"
        R = None
        if so.exists():
            try:
                R = C.CDLL(str(so))
                for name in (("ref_fp8a8_gemm_nt_q", "ref_fp8a8_gemm_nt_q_decode", "ref_fp8a8_gemm_nt_q_gated")
                             if which == "fp8a8" else
                             ("ref_mxfp4_gemm_nt_q", "ref_mxfp4_gemm_nt_q_decode", "ref_mxfp4_gemm_nt_q_decode_q8x")):
                    getattr(R, name).argtypes = [C.c_void_p, C.c_void_p]
            except OSError:
                R = None
        _ref_gemm[which] = R
    return _ref_gemm[which]


def _p(a: np.ndarray | None):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _c(a, dt):
    a = np.ascontiguousarray(a, dtype=dt)
    return a


I64 = C.c_int64


def encode_e4m3(x: np.ndarray) -> np.ndarray:
    """element-wise clamp(+-448) + RTNE-saturating e4m3 encode"""
    x = _c(x, np.float32)
    q = np.empty(x.shape, np.uint8)
    lib().orc_f32_to_e4m3_n(_p(x), I64(x.size), _p(q))
    return q


def quant_act_fp8(x: np.ndarray, group: int = 128):
    x = _c(x, np.float32)
    M, n = x.shape
    ngrp = (n + group - 1) // group
    q = np.empty((M, n), np.uint8)
    s = np.empty((M, ngrp), np.float32)
    lib().orc_quant_act_fp8(_p(x), I64(M), I64(n), I64(group), _p(q), _p(s))
    return q, s


def gated_quant_fp8(gu_bits: np.ndarray, group: int = 128, silu: bool = True, want_ob: bool = False):
    """bf16 gate_up bits [M, 2n] -> (e4m3 codes [M, n], f32 scales [M, n/group][, bf16 product bits])."""
    gu = _c(gu_bits, np.uint16)
    M, N2 = gu.shape
    n = N2 // 2
    g = min(group, n) if group > 0 else n
    ngrp = (n + g - 1) // g
    q = np.empty((M, n), np.uint8)
    s = np.empty((M, ngrp), np.float32)
    ob = np.empty((M, n), np.uint16) if want_ob else None
    lib().orc_gated_quant_fp8(_p(gu), I64(M), I64(n), I64(g), C.c_int(1 if silu else 0), _p(q), _p(s),
                              _p(ob) if ob is not None else None)
    return (q, s, ob) if want_ob else (q, s)


def rmsnorm_quant_fp8(x_bits: np.ndarray, w: np.ndarray, eps: float, group: int = 128, wadd: float = 0.0,
                      res_bits: np.ndarray | None = None):
    """bf16 bits x [M, n] (+ optional bf16 residual, updated in a copy), w as bf16 bits (uint16) or f32 ->
    dict(q e4m3 [M, n], scale f32 [M, n/group], ob bf16 bits [M, n], res updated bf16 bits or None)."""
    x = _c(x_bits, np.uint16)
    M, n = x.shape
    g = min(group, n) if group > 0 else n
    ngrp = (n + g - 1) // g
    res = _c(res_bits, np.uint16).copy() if res_bits is not None else None
    wb = _c(w, np.uint16) if w.dtype == np.uint16 else None
    wf = _c(w, np.float32) if wb is None else None
    q = np.empty((M, n), np.uint8)
    s = np.empty((M, ngrp), np.float32)
    ob = np.empty((M, n), np.uint16)
    lib().orc_rmsnorm_quant_fp8(_p(x), _p(res) if res is not None else None, _p(wb) if wb is not None else None,
                                _p(wf) if wf is not None else None, I64(M), I64(n), I64(g), C.c_float(eps),
                                C.c_float(wadd), _p(q), _p(s), _p(ob))
    return dict(q=q, scale=s, ob=ob, res=res)


def row_topk(x_bits: np.ndarray, R: int, vocab_off: int = 0):
    """bf16 bits x [M, N] -> (idx int32 [M, R], val f32 [M, R]): exact top-R per row, descending, ties to
    the lower column; unfillable slots are (-1, -inf)."""
    x = _c(x_bits, np.uint16)
    M, N = x.shape
    idx = np.empty((M, R), np.int32)
    val = np.empty((M, R), np.float32)
    lib().orc_row_topk(_p(x), I64(M), I64(N), I64(R), I64(vocab_off), _p(idx), _p(val))
    return idx, val


def sample_argmax(logits: np.ndarray) -> np.ndarray:
    """f32 logits [M, n_vocab] -> int32 token [M]: the largest logit, ties to the lower token id."""
    lg = _c(logits, np.float32)
    M, nv = lg.shape
    tok = np.empty(M, np.int32)
    lib().orc_sample_argmax(_p(lg), I64(M), I64(nv), _p(tok))
    return tok


def quant_act_mx8(x: np.ndarray):
    x = _c(x, np.float32)
    M, n = x.shape
    q = np.empty((M, n), np.uint8)
    e = np.empty((M, (n + 31) // 32), np.uint8)
    lib().orc_quant_act_mx8(_p(x), I64(M), I64(n), _p(q), _p(e))
    return q, e


def q8x_requant(A: np.ndarray):
    A = _c(A, np.uint8)
    M, K = A.shape
    x8 = np.empty((M, K), np.int8)
    sg = np.empty((M, K // 32), np.float32)
    lib().orc_q8x_requant(_p(A), I64(M), I64(K), I64(K), _p(x8), _p(sg))
    return x8, sg


def gemm_fp8a8(A, AS, B, BS, rblk: int, want_acc: bool = False):
    """BS: uint16 (bf16 bits) or float32 array [N/rblk, cols]."""
    A, B, AS = _c(A, np.uint8), _c(B, np.uint8), _c(AS, np.float32)
    is_f32 = BS.dtype == np.float32
    BS = _c(BS, np.float32 if is_f32 else np.uint16)
    M, K = A.shape
    N = B.shape[0]
    Y = np.empty((M, N), np.uint16)
    acc = np.empty((M, N), np.float32) if want_acc else None
    lib().orc_gemm_fp8a8(_p(A), _p(AS), _p(B), _p(BS), C.c_int(int(is_f32)), I64(M), I64(N), I64(K),
                         I64(AS.shape[1]), I64(BS.shape[1]), I64(rblk), _p(Y), _p(acc))
    return (Y, acc) if want_acc else Y


def gemm_mxfp4a8(A, AS, B, BS, want_acc: bool = False):
    A, B, AS, BS = _c(A, np.uint8), _c(B, np.uint8), _c(AS, np.float32), _c(BS, np.uint8)
    M, K = A.shape
    N = B.shape[0]
    Y = np.empty((M, N), np.uint16)
    acc = np.empty((M, N), np.float32) if want_acc else None
    lib().orc_gemm_mxfp4a8(_p(A), _p(AS), _p(B), _p(BS), I64(M), I64(N), I64(K), I64(AS.shape[1]),
                           _p(Y), _p(acc))
    return (Y, acc) if want_acc else Y


def gemm_mxfp4_q8x(A, AS, B, BS, walk: int):
    """Full arm: requantise A (e4m3 codes) then the int8 chain."""
    x8, sg = q8x_requant(A)
    AS, B, BS = _c(AS, np.float32), _c(B, np.uint8), _c(BS, np.uint8)
    M, K = x8.shape
    N = B.shape[0]
    Y = np.empty((M, N), np.uint16)
    lib().orc_gemm_mxfp4_q8x(_p(x8), _p(sg), _p(AS), _p(B), _p(BS), I64(M), I64(N), I64(K),
                             I64(AS.shape[1]), C.c_int(walk), _p(Y), None)
    return Y


def logits_e4m3(X, codes, scale, sdt: int, br: int):
    """X uint16 bf16 bits [M,K]; scale uint16 (bf16 sdt 0 / f16 sdt 1) or float32 (sdt 2)."""
    X, codes = _c(X, np.uint16), _c(codes, np.uint8)
    scale = np.ascontiguousarray(scale)
    M, K = X.shape
    N = codes.shape[0]
    Y = np.empty((M, N), np.float32)
    lib().orc_logits_e4m3(_p(X), _p(codes), _p(scale), C.c_int(sdt), I64(br), I64(M), I64(N),
                          I64(K), _p(Y))
    return Y


def logits_mxfp4(X, B, BS):
    X, B, BS = _c(X, np.uint16), _c(B, np.uint8), _c(BS, np.uint8)
    M, K = X.shape
    N = B.shape[0]
    Y = np.empty((M, N), np.float32)
    lib().orc_logits_mxfp4(_p(X), _p(B), _p(BS), I64(M), I64(N), I64(K), _p(Y))
    return Y


def truth_fp8a8(A, AS, B, BS, rblk: int):
    A, B, AS = _c(A, np.uint8), _c(B, np.uint8), _c(AS, np.float32)
    is_f32 = BS.dtype == np.float32
    BS = _c(BS, np.float32 if is_f32 else np.uint16)
    M, K = A.shape
    N = B.shape[0]
    Yt = np.empty((M, N), np.float64)
    Ya = np.empty((M, N), np.float64)
    lib().orc_truth_fp8a8(_p(A), _p(AS), _p(B), _p(BS), C.c_int(int(is_f32)), I64(M), I64(N),
                          I64(K), I64(AS.shape[1]), I64(BS.shape[1]), I64(rblk), _p(Yt), _p(Ya))
    return Yt, Ya


def truth_mxfp4a8(A, AS, B, BS):
    A, B, AS, BS = _c(A, np.uint8), _c(B, np.uint8), _c(AS, np.float32), _c(BS, np.uint8)
    M, K = A.shape
    N = B.shape[0]
    Yt = np.empty((M, N), np.float64)
    Ya = np.empty((M, N), np.float64)
    lib().orc_truth_mxfp4a8(_p(A), _p(AS), _p(B), _p(BS), I64(M), I64(N), I64(K),
                            I64(AS.shape[1]), _p(Yt), _p(Ya))
    return Yt, Ya


def gemm_w2a8(A, AS, B, SC, ZP, ASUM, zp_u4: bool = False, want_acc: bool = False):
    """gemm_nt_q @ w2a8: A int8 [M,K] in quant_act_i8's step order, AS f32 [M], B u2 codes [N, K/4] bytes,
    SC f16 bits [N, K/128], ZP u8 [N, K/128] (or u4 [N, ceil(K/256)] bytes), ASUM f32 [K/128, mpad]."""
    A, AS, B = _c(A, np.int8), _c(AS, np.float32), _c(B, np.uint8)
    SC, ZP, ASUM = _c(SC, np.uint16), _c(ZP, np.uint8), _c(ASUM, np.float32)
    M, K = A.shape
    N = B.shape[0]
    Y = np.empty((M, N), np.uint16)
    acc = np.empty((M, N), np.float32) if want_acc else None
    lib().orc_gemm_w2a8(_p(A), _p(AS), _p(B), _p(SC), _p(ZP), C.c_int(1 if zp_u4 else 0), _p(ASUM), I64(M), I64(N),
                        I64(K), _p(Y), _p(acc) if want_acc else None)
    return (Y, acc) if want_acc else Y


def w2a8_group_sums(A):
    A = _c(A, np.int8)
    M, K = A.shape
    out = np.empty((K // 128, (M + 15) // 16 * 16), np.float32)
    lib().orc_w2a8_group_sums(_p(A), I64(M), I64(K), _p(out))
    return out


def logit_rerank_e4m3(X_bits, codes, scale, sdt: int, br: int, idx_in, vocab_off: int = 0):
    """X_bits: bf16 bit patterns [M,K] (or float32 values); scale in its stored dtype (sdt 0 bf16 bits,
    1 f16 bits, 2 f32). Returns (idx int32 [M,R], val f32 [M,R], pairs f32 [M,R,2])."""
    X = X_bits if X_bits.dtype == np.float32 else bf16_bits_to_f32(X_bits)
    X = _c(X, np.float32)
    if sdt == 0:
        sc = bf16_bits_to_f32(scale)
    elif sdt == 1:
        sc = scale.view(np.float16).astype(np.float32)
    else:
        sc = scale
    sc, codes, idx_in = _c(sc, np.float32), _c(codes, np.uint8), _c(idx_in, np.int32)
    M, K = X.shape
    R = idx_in.shape[1]
    NV = codes.shape[0]
    idx = np.empty((M, R), np.int32); val = np.empty((M, R), np.float32); pairs = np.empty((M, R, 2), np.float32)
    lib().orc_logit_rerank_e4m3(_p(X), _p(codes), _p(sc), I64(sc.shape[1]), C.c_int(br), _p(idx_in), I64(M), I64(R),
                                I64(K), I64(NV), I64(vocab_off), _p(idx), _p(val), _p(pairs))
    return idx, val, pairs


def gemm_mxfp4mx8(A, AE, B, BS, want_acc: bool = False):
    """mxfp4 weights x mxfp8 activations (A e4m3 [M,K], AE E8M0 [M,K/32]); parity unpinned."""
    A, B, AE, BS = _c(A, np.uint8), _c(B, np.uint8), _c(AE, np.uint8), _c(BS, np.uint8)
    M, K = A.shape
    N = B.shape[0]
    Y = np.empty((M, N), np.uint16)
    acc = np.empty((M, N), np.float32) if want_acc else None
    lib().orc_gemm_mxfp4mx8(_p(A), _p(AE), _p(B), _p(BS), I64(M), I64(N), I64(K), _p(Y),
                            _p(acc) if want_acc else None)
    return (Y, acc) if want_acc else Y


def truth_mxfp4mx8(A, AE, B, BS):
    A, B, AE, BS = _c(A, np.uint8), _c(B, np.uint8), _c(AE, np.uint8), _c(BS, np.uint8)
    M, K = A.shape
    N = B.shape[0]
    Yt = np.empty((M, N), np.float64)
    Ya = np.empty((M, N), np.float64)
    lib().orc_truth_mxfp4mx8(_p(A), _p(AE), _p(B), _p(BS), I64(M), I64(N), I64(K), _p(Yt), _p(Ya))
    return Yt, Ya


# ---- numpy helpers shared by the graders ----
def bf16_bits_to_f32(h: np.ndarray) -> np.ndarray:
    return (h.astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16_bits(f: np.ndarray) -> np.ndarray:
    u = np.ascontiguousarray(f, np.float32).view(np.uint32).astype(np.uint64)
    nan = (u & 0x7FFFFFFF) > 0x7F800000
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    r[nan] = ((u[nan] >> 16) | 0x40).astype(np.uint16)
    return r


def bf16_ulp_distance(a_bits: np.ndarray, b_bits: np.ndarray) -> np.ndarray:
    """Distance in bf16 ulps between two bf16 bit arrays (sign-magnitude mapped to a line)."""
    def line(h):
        h = h.astype(np.int32)
        return np.where(h & 0x8000, -(h & 0x7FFF), h & 0x7FFF)
    return np.abs(line(a_bits) - line(b_bits))
