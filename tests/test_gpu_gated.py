"""gemm_nt_q_gated @ fp8a8 on the GPU: the gated activation quantiser bit for bit against the oracle,
and the fused row byte-identical to gemm_nt_q followed by the quantiser."""
import ctypes as C

import numpy as np
import pytest
import torch

import gen
import gpu_util as gu
from libr3d_b200 import abi, ops
from oracle import oracle as orc

pytestmark = pytest.mark.gpu


def _gated_on_device(gu_bits, group, silu, ob_dtype=None):
    P = ops.plugin()
    M, N2 = gu_bits.shape
    n = N2 // 2
    g = n if group <= 0 else min(group, n)
    ngrp = (n + g - 1) // g
    d = gu.dev(gu_bits)
    q = gu.GuardedOut((M, n), np.uint8)
    s = gu.GuardedOut((M, ngrp), np.float32)
    ob = None if ob_dtype is None else gu.GuardedOut((M, n), np.float32 if ob_dtype == abi.RAD_F32 else np.uint16)
    rc = P.lib.r3d_b200_gated_quant_fp8(d.data_ptr(), N2, q.ptr, n, s.ptr, ngrp, ob.ptr if ob else None,
                                        ob_dtype or abi.RAD_BF16, n, M, n, group, 1 if silu else 0, None)
    assert rc == 0
    return q.get(), s.get(), (ob.get() if ob else None)


@pytest.mark.parametrize("silu", [True, False])
@pytest.mark.parametrize("M,n,group", [(1, 128, 128), (5, 300, 128), (64, 1024, 128), (3, 200, 0)])
def test_gated_quantiser_bit_identical_to_oracle(M, n, group, silu):
    rng = np.random.default_rng(M * 1000 + n)
    bits = gen.f32_to_bf16_bits((rng.standard_normal((M, 2 * n)) * 4).astype(np.float32))
    bits[0, :4] = [0x0000, 0x8000, 0x7F80, 0xFF80]
    want_q, want_s, want_ob = orc.gated_quant_fp8(bits, group, silu, want_ob=True)
    q, s, ob = _gated_on_device(bits, group, silu, abi.RAD_BF16)
    assert np.array_equal(s.view(np.uint32), want_s.view(np.uint32))
    assert gu.same_bits_or_both_nan(ob, want_ob).all()          # NaN sign/payload is not part of the contract
    assert np.array_equal(q & 0x7F, want_q & 0x7F) and np.array_equal((q & 0x80)[(q & 0x7F) != 0x7F], (want_q & 0x80)[(want_q & 0x7F) != 0x7F])
    _, _, obf = _gated_on_device(bits, group, silu, abi.RAD_F32)
    assert gu.same_bits_or_both_nan(gen.f32_to_bf16_bits(obf), want_ob).all()


@pytest.mark.parametrize("M,N,K,act", [(1, 512, 256, "silu"), (7, 768, 512, "silu"), (16, 1024, 1024, "sigmoid"),
                                       (64, 512, 384, "silu")])
def test_fused_row_is_the_unfused_pair_byte_for_byte(M, N, K, act):
    case = gen.case_fp8(600 + M, M, N, K, "ref128")
    t = {k: gu.dev(case[k]) for k in ("A", "AS", "B", "BS")}
    n = N // 2
    # the unfused pair: the plain row, then the quantiser over its bf16 plane
    y = torch.zeros((M, N), dtype=torch.bfloat16, device="cuda")
    ops.gemm_nt_q(t["A"], t["AS"], t["B"], t["BS"].view(torch.bfloat16), y, dtype="fp8a8", N=N, K=K)
    torch.cuda.synchronize()
    ybits = y.view(torch.int16).cpu().numpy().view(np.uint16)
    want_q, want_s, want_ob = orc.gated_quant_fp8(ybits, 128, act == "silu", want_ob=True)
    # the fused row
    q = torch.zeros((M, n), dtype=torch.uint8, device="cuda")
    s = torch.zeros((M, n // 128), dtype=torch.float32, device="cuda")
    ob = torch.zeros((M, n), dtype=torch.bfloat16, device="cuda")
    r = ops.gemm_nt_q_gated(t["A"], t["AS"], t["B"], t["BS"].view(torch.bfloat16), q, s, N=N, K=K, act=act, out=ob)
    assert r.name == "gemm_nt_q_gated_fp8a8"
    torch.cuda.synchronize()
    assert np.array_equal(q.cpu().numpy(), want_q)
    assert np.array_equal(s.cpu().numpy().view(np.uint32), want_s.view(np.uint32))
    assert np.array_equal(ob.view(torch.int16).cpu().numpy().view(np.uint16), want_ob)
    assert np.count_nonzero(want_q & 0x7F) > want_q.size // 2


def test_fused_row_refusals():
    from libr3d_b200.ops import RowRefused
    M, N, K = 4, 512, 256
    case = gen.case_fp8(1, M, N, K, "ref128")
    t = {k: gu.dev(case[k]) for k in ("A", "AS", "B", "BS")}
    q = torch.zeros((M, N // 2), dtype=torch.uint8, device="cuda")
    s = torch.zeros((M, N // 256), dtype=torch.float32, device="cuda")
    small = torch.empty(M * N * 2 - 2, dtype=torch.uint8, device="cuda")     # an arena one element short
    with pytest.raises(RowRefused) as e:
        ops.gemm_nt_q_gated(t["A"], t["AS"], t["B"], t["BS"].view(torch.bfloat16), q, s, N=N, K=K, scratch=small)
    assert e.value.rc == abi.RAD_E_UNSUPPORTED
    exact = torch.empty(M * N * 2, dtype=torch.uint8, device="cuda")
    ops.gemm_nt_q_gated(t["A"], t["AS"], t["B"], t["BS"].view(torch.bfloat16), q, s, N=N, K=K, scratch=exact)
    torch.cuda.synchronize()
    assert int(torch.count_nonzero(q)) > 0


def _q_struct(t, M, N, K, y_ptr=0):
    q = abi.R3dGemmQ()
    q.a, q.a_scale, q.b, q.b_scale, q.y = t["A"].data_ptr(), t["AS"].data_ptr(), t["B"].data_ptr(), t["BS"].data_ptr(), y_ptr
    q.m, q.n, q.k, q.as_cols = M, N, K, K // 128
    q.a_pitch, q.y_pitch, q.as_pitch, q.arm = K, N, K // 128, abi.R3D_ARM_AUTO
    q.bs_cols, q.rblk, q.bs_dtype, q.b_pitch, q.bs_pitch = K // 128, 128, abi.RAD_BF16, K, K // 128
    return q


@pytest.mark.parametrize("M,N,K,act", [(1, 19200, 512, "silu"), (2, 27648, 1024, "silu"), (4, 19200, 640, "sigmoid"),
                                       (5, 27648, 640, "sigmoid"), (8, 19200, 256, "silu"), (16, 27648, 5120, "silu"),
                                       (33, 19200, 1024, "silu"), (64, 19200, 384, "sigmoid")])
def test_wide_projections_run_as_one_launch_with_the_pair_s_bytes(M, N, K, act):
    """Projections wide enough that the band does not split K are served by the decode kernel with the gated
    quantiser as its epilogue (a gate tile and its up tile in a cluster of two): the launch-layer entry takes
    the call, and codes, scales and the gated product are the bytes of the band followed by the quantiser."""
    case = gen.case_fp8(900 + M, M, N, K, "ref128")
    t = {k: gu.dev(case[k]) for k in ("A", "AS", "B", "BS")}
    n = N // 2
    y = torch.zeros((M, N), dtype=torch.bfloat16, device="cuda")
    ops.gemm_nt_q(t["A"], t["AS"], t["B"], t["BS"].view(torch.bfloat16), y, dtype="fp8a8", N=N, K=K)
    torch.cuda.synchronize()
    ybits = y.view(torch.int16).cpu().numpy().view(np.uint16)
    want_q, want_s, want_ob = orc.gated_quant_fp8(ybits, 128, act == "silu", want_ob=True)
    # the row
    q = torch.zeros((M, n), dtype=torch.uint8, device="cuda")
    s = torch.zeros((M, n // 128), dtype=torch.float32, device="cuda")
    ob = torch.zeros((M, n), dtype=torch.bfloat16, device="cuda")
    ops.gemm_nt_q_gated(t["A"], t["AS"], t["B"], t["BS"].view(torch.bfloat16), q, s, N=N, K=K, act=act, out=ob)
    torch.cuda.synchronize()
    assert np.array_equal(q.cpu().numpy(), want_q)
    assert np.array_equal(s.cpu().numpy().view(np.uint32), want_s.view(np.uint32))
    assert np.array_equal(ob.view(torch.int16).cpu().numpy().view(np.uint16), want_ob)
    # the one-launch entry itself, guard bands around its outputs, f32 product
    P = ops.plugin()
    gq, gs, gob = gu.GuardedOut((M, n), np.uint8), gu.GuardedOut((M, n // 128), np.float32), gu.GuardedOut((M, n), np.float32)
    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    qs = _q_struct(t, M, N, K)
    rc = P.lib.r3d_b200_gemm_fp8a8_gated(C.byref(qs), C.c_void_p(gq.ptr), C.c_int64(n), C.c_void_p(gs.ptr), C.c_int64(n // 128),
                                         C.c_void_p(gob.ptr), C.c_int32(abi.RAD_F32), C.c_int64(n), C.c_int32(act == "silu"), st)
    assert rc == abi.RAD_OK
    assert np.array_equal(gq.get(), want_q)
    assert np.array_equal(gs.get().view(np.uint32), want_s.view(np.uint32))
    assert np.array_equal(gen.f32_to_bf16_bits(gob.get()), want_ob)
    assert P.lib.r3d_b200_stream_status() == 0


def test_narrow_projections_stay_on_the_pair():
    """where the band splits K between the CTAs of a cluster the one-launch entry declines (its accumulation
    would differ from the band's) and the row runs the pair"""
    M, N, K = 4, 1024, 512
    case = gen.case_fp8(2, M, N, K, "ref128")
    t = {k: gu.dev(case[k]) for k in ("A", "AS", "B", "BS")}
    P = ops.plugin()
    n = N // 2
    gq, gs = gu.GuardedOut((M, n), np.uint8), gu.GuardedOut((M, n // 128), np.float32)
    qs = _q_struct(t, M, N, K)
    rc = P.lib.r3d_b200_gemm_fp8a8_gated(C.byref(qs), C.c_void_p(gq.ptr), C.c_int64(n), C.c_void_p(gs.ptr), C.c_int64(n // 128),
                                         None, C.c_int32(abi.RAD_BF16), C.c_int64(0), C.c_int32(1), None)
    assert rc == abi.RAD_E_UNSUPPORTED
