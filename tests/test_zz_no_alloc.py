"""The allocation-free q8x entry point (r3d_b200_gemm_mxfp4a8_q8x_static).

Some callers of this library cannot allocate device memory at launch time: an engine that
is recording a pass for replay (an allocation would synchronise the device mid-recording),
or one that has already committed all device memory to weights and KV cache (the allocation
would fail). For them the int8 arm exists in a form whose scratch is a fixed array inside
the library. This test calls that form through the C ABI, twice in a row with different
operands (the array is shared and keeps the previous call's bytes), and requires the output
to be bit-identical to the ordinary entry point's, which takes caller scratch.

Collected last on purpose (file name), so a run that stops at the first failure has already
run every other test. Runs the same alone in a fresh process.
"""
import ctypes as C

import numpy as np
import pytest

import gen
import gpu_util as gu
from libr3d_b200 import abi, ops

pytestmark = pytest.mark.gpu


def _call_static(case, walk):
    P = ops.plugin()
    A, AS, B, BS = map(gu.dev, (case["A"], case["AS"], case["B"], case["BS"]))
    M, K = case["A"].shape
    N = case["B"].shape[0]
    out = gu.GuardedOut((M, N), np.uint16)
    q = abi.R3dGemmQ()
    q.a, q.a_scale, q.b, q.b_scale, q.y = A.data_ptr(), AS.data_ptr(), B.data_ptr(), BS.data_ptr(), out.ptr
    q.m, q.n, q.k = M, N, K
    q.as_cols, q.bs_cols = K // 128, K // 32
    q.a_pitch, q.b_pitch, q.y_pitch, q.as_pitch, q.bs_pitch = K, K // 2, N, K // 128, K // 32
    q.rblk, q.bs_dtype = 1, abi.RAD_E8M0
    rc = P.lib.r3d_b200_gemm_mxfp4a8_q8x_static(C.byref(q), walk, None)
    return rc, out


def test_static_scratch_entry_matches_caller_scratch_entry_twice():
    # first a large call that fills the shared array, then a smaller one with other operands:
    # stale bytes of the first must not reach the second
    for seed, M, N, K, walk in [(71, 8, 333, 2048, 1), (72, 3, 200, 768, 0)]:
        case = gen.case_mxfp4(seed, M, N, K)
        rc, out = _call_static(case, walk)
        assert rc == abi.RAD_OK, abi.STATUS_NAMES[rc]
        got = out.get()
        want, _, _ = gu.q8x_launch(case, walk)
        assert np.array_equal(got, want)
        assert np.count_nonzero(got & 0x7FFF) > got.size * 0.9


def test_static_scratch_entry_refuses_oversize():
    case = gen.case_mxfp4(73, 1, 8, 256)
    case9 = dict(case, A=np.repeat(case["A"], 9, axis=0), AS=np.repeat(case["AS"], 9, axis=0))
    rc, _ = _call_static(case9, 0)
    assert rc == abi.RAD_E_SHAPE                      # M = 9 > 8
    big = gen.case_mxfp4(74, 1, 4, 32768 + 256)
    rc, _ = _call_static(big, 0)
    assert rc == abi.RAD_E_SHAPE                      # K beyond the built-in array
