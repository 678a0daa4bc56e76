"""Device-side plumbing for the GPU tests: uploads, guard-banded outputs, launch-layer calls
with a forced arm, and the graders. torch is used for device memory only."""
from __future__ import annotations

import ctypes as C

import numpy as np
import torch

from libr3d_b200 import abi, ops
from oracle import oracle as orc

GUARD = 4096          # poisoned bytes on each side of every output
POISON = 0xEE


def dev(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


class GuardedOut:
    """An output buffer with poisoned bands before and after it; `check()` asserts that the
    kernel wrote nothing outside [0, nbytes) (the reference's red-zone practice,
    tools/probe_m4_entry.cpp:46 of libr3d)."""

    def __init__(self, shape, np_dtype):
        self.shape, self.np_dtype = shape, np.dtype(np_dtype)
        self.nbytes = int(np.prod(shape)) * self.np_dtype.itemsize
        self.raw = torch.full((GUARD + self.nbytes + GUARD,), POISON, dtype=torch.uint8, device="cuda")

    @property
    def ptr(self) -> int:
        return self.raw.data_ptr() + GUARD

    def view(self) -> torch.Tensor:
        tdt = {2: torch.uint16, 4: torch.float32}[self.np_dtype.itemsize]
        return self.raw[GUARD:GUARD + self.nbytes].view(tdt).view(*self.shape)

    def get(self) -> np.ndarray:
        torch.cuda.synchronize()
        h = self.raw.cpu().numpy()
        assert (h[:GUARD] == POISON).all() and (h[GUARD + self.nbytes:] == POISON).all(), \
            "kernel wrote outside its output"
        return h[GUARD:GUARD + self.nbytes].view(self.np_dtype).reshape(self.shape).copy()


def gemm_launch(kind: str, case: dict, arm: int, a_dev=None) -> np.ndarray:
    """Call the launch layer (r3d_b200_gemm_*) with a forced arm. Returns bf16 bits [M,N]."""
    P = ops.plugin()
    A, AS, B, BS = dev(case["A"]), dev(case["AS"]), dev(case["B"]), dev(case["BS"])
    M, K = case["A"].shape
    N = case["B"].shape[0]
    out = GuardedOut((M, N), np.uint16)
    q = abi.R3dGemmQ()
    q.a, q.a_scale, q.b, q.b_scale, q.y = A.data_ptr(), AS.data_ptr(), B.data_ptr(), BS.data_ptr(), out.ptr
    q.m, q.n, q.k = M, N, K
    q.as_cols, q.bs_cols = case["AS"].shape[1], case["BS"].shape[1]
    q.a_pitch, q.y_pitch, q.as_pitch, q.bs_pitch = K, N, q.as_cols, q.bs_cols
    q.arm = arm
    if kind == "fp8a8":
        q.rblk = case["rblk"]
        q.bs_dtype = abi.RAD_F32 if case["BS"].dtype == np.float32 else abi.RAD_BF16
        q.b_pitch = K
        rc = P.lib.r3d_b200_gemm_fp8a8(C.byref(q), None)
    else:
        q.rblk, q.bs_dtype, q.b_pitch = 1, abi.RAD_E8M0, K // 2
        rc = P.lib.r3d_b200_gemm_mxfp4a8(C.byref(q), None)
    assert rc == abi.RAD_OK, abi.STATUS_NAMES[rc]
    return out.get()


def mx8_launch(case: dict, arm: int) -> np.ndarray:
    """gemm_nt_q @ mxfp4mx8 through the launch layer: case has A (e4m3), AE (E8M0 [M, K/32]), B, BS."""
    P = ops.plugin()
    A, AE, B, BS = dev(case["A"]), dev(case["AE"]), dev(case["B"]), dev(case["BS"])
    M, K = case["A"].shape
    N = case["B"].shape[0]
    out = GuardedOut((M, N), np.uint16)
    q = abi.R3dGemmQ()
    q.a, q.a_scale, q.b, q.b_scale, q.y = A.data_ptr(), AE.data_ptr(), B.data_ptr(), BS.data_ptr(), out.ptr
    q.m, q.n, q.k = M, N, K
    q.as_cols, q.bs_cols = K // 32, K // 32
    q.a_pitch, q.b_pitch, q.y_pitch, q.as_pitch, q.bs_pitch = K, K // 2, N, K // 32, K // 32
    q.rblk, q.bs_dtype, q.arm = 1, abi.RAD_E8M0, arm
    rc = P.lib.r3d_b200_gemm_mxfp4mx8(C.byref(q), None)
    assert rc == abi.RAD_OK, abi.STATUS_NAMES[rc]
    y = out.get()
    assert P.lib.r3d_b200_stream_status() == 0
    return y


def q8x_launch(case: dict, walk: int, want_tc: bool | None = None):
    """The int8 arm through the launch layer with caller scratch; returns (Y bits, x8, sg).
    want_tc: assert that the dots run on the tensor core (True) or on dp4a (False)."""
    P = ops.plugin()
    A, AS, B, BS = dev(case["A"]), dev(case["AS"]), dev(case["B"]), dev(case["BS"])
    M, K = case["A"].shape
    N = case["B"].shape[0]
    out = GuardedOut((M, N), np.uint16)
    x8 = torch.zeros((M, K), dtype=torch.int8, device="cuda")
    sg = torch.zeros((M, K // 32), dtype=torch.float32, device="cuda")
    q = abi.R3dGemmQ()
    q.a, q.a_scale, q.b, q.b_scale, q.y = A.data_ptr(), AS.data_ptr(), B.data_ptr(), BS.data_ptr(), out.ptr
    q.m, q.n, q.k = M, N, K
    q.as_cols, q.bs_cols = K // 128, K // 32
    q.a_pitch, q.b_pitch, q.y_pitch, q.as_pitch, q.bs_pitch = K, K // 2, N, K // 128, K // 32
    q.rblk, q.bs_dtype = 1, abi.RAD_E8M0
    if want_tc is not None:
        assert bool(P.lib.r3d_b200_q8x_on_tensor_core(C.byref(q))) == want_tc
    rc = P.lib.r3d_b200_gemm_mxfp4a8_q8x(C.byref(q), x8.data_ptr(), sg.data_ptr(), walk, None)
    assert rc == abi.RAD_OK, abi.STATUS_NAMES[rc]
    y = out.get()
    assert P.lib.r3d_b200_stream_status() == 0
    return y, x8.cpu().numpy(), sg.cpu().numpy()


def logits_launch(case: dict, arm: int, y_dtype: int = abi.RAD_F32) -> np.ndarray:
    P = ops.plugin()
    X, codes, scale = dev(case["X"]), dev(case["codes"]), dev(case["scale"])
    M, K = case["X"].shape
    N = case["codes"].shape[0]
    out = GuardedOut((M, N), np.float32 if y_dtype == abi.RAD_F32 else np.uint16)
    l = abi.R3dLogits()
    l.x, l.codes, l.scale, l.y = X.data_ptr(), codes.data_ptr(), scale.data_ptr(), out.ptr
    l.m, l.n, l.k, l.br = M, N, K, case["br"]
    l.scale_dtype = {0: abi.RAD_BF16, 1: abi.RAD_F16, 2: abi.RAD_F32}[case["sdt"]]
    l.y_dtype, l.head_fmt, l.arm = y_dtype, 0, arm
    l.x_pitch, l.code_pitch, l.y_pitch, l.scale_pitch = K, K, N, case["scale"].shape[1]
    rc = P.lib.r3d_b200_logits(C.byref(l), None)
    assert rc == abi.RAD_OK, abi.STATUS_NAMES[rc]
    return out.get()


# ------------------------------------------------------------------ graders
def same_bits_or_both_nan(got: np.ndarray, want: np.ndarray) -> np.ndarray:
    """bf16 bit arrays: equal, or both NaN (NaN payloads are not part of the contract)."""
    nan_g = (got & 0x7FFF) > 0x7F80
    nan_w = (want & 0x7FFF) > 0x7F80
    return (got == want) | (nan_g & nan_w)


def grade_bf16(got_bits: np.ndarray, acc32: np.ndarray, absum: np.ndarray | None = None) -> dict:
    """bf16 output vs the fp32-accumulated oracle value `acc32`.
    strict: ulp distance between got and bf16(acc32).
    floored: misses forgiven when |got - acc32| is below 2 ulp of the cancellation floor
    (sum|terms| * 2^-16): an output that is the small difference of large terms carries the
    rounding of those terms whatever the summation order."""
    want = orc.f32_to_bf16_bits(acc32)
    nan = np.isnan(acc32)
    d = orc.bf16_ulp_distance(got_bits, want).astype(np.int64)
    d[nan] = np.where(((got_bits[nan] & 0x7FFF) > 0x7F80), 0, 1 << 20)
    res = dict(max_ulp=int(d.max()), frac_le2=float((d <= 2).mean()), nonzero=int(np.count_nonzero(got_bits & 0x7FFF)))
    if absum is not None:
        g = orc.bf16_bits_to_f32(got_bits).astype(np.float64)
        floor = absum * 2.0 ** -16
        ulp = np.maximum(np.abs(acc32.astype(np.float64)), floor) * 2.0 ** -7
        bad = (d > 2) & ~nan & (np.abs(g - acc32) > 2 * ulp)
        res["floored_bad"] = int(bad.sum())
    got = orc.bf16_bits_to_f32(got_bits).astype(np.float64)
    ref = orc.bf16_bits_to_f32(want).astype(np.float64)
    ok = ~nan
    den = float(np.sqrt((ref[ok] ** 2).sum()))
    res["rel_l2"] = float(np.sqrt(((got[ok] - ref[ok]) ** 2).sum()) / den) if den > 0 else 0.0
    return res
