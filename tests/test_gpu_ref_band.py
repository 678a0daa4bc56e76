"""The reference's own activation-producer kernels, compiled for sm_100a from the reference file
where it lay (src/r3d_band.hip of libr3d -> oracle/_ref/libref_band.so), executed on the GPU beside
this library's kernels on the same operands: quant_act_fp8 and gated_quant_fp8 must agree byte for
byte (NaN sign and payload excepted), and both with the CPU oracle."""
import ctypes as C

import numpy as np
import pytest
import torch

import gen
import gpu_util as gu
from libr3d_b200 import abi, ops
from libr3d_b200.plugin import ArgPack, tensor_desc
from oracle import oracle as orc

pytestmark = pytest.mark.gpu


def _ref():
    R = orc.ref_band()
    if R is None:
        pytest.skip("oracle/_ref/libref_band.so not present")
    return R


def _desc(t, dt):
    return tensor_desc(t.data_ptr(), dt, list(t.shape))


@pytest.mark.parametrize("rows,n,group,f32", [(1, 5120, 128, False), (7, 1000, 128, False), (64, 512, 512, True),
                                              (3, 300, 0, False)])
def test_quant_act_fp8_matches_the_reference_kernel(rows, n, group, f32):
    R = _ref()
    rng = np.random.default_rng(rows * 31 + n)
    xf = (rng.standard_normal((rows, n)) * np.exp(rng.uniform(-6, 6, (rows, 1)))).astype(np.float32)
    xf[0, :3] = [0.0, -0.0, 1e-30]
    x = torch.from_numpy(xf).cuda() if f32 else torch.from_numpy(gen.f32_to_bf16_bits(xf).view(np.int16)).cuda().view(torch.bfloat16)
    g = n if group <= 0 else group
    ngrp = (n + g - 1) // g
    q_ref = torch.zeros((rows, n), dtype=torch.uint8, device="cuda"); s_ref = torch.zeros((rows, ngrp), dtype=torch.float32, device="cuda")
    pack = ArgPack([_desc(x, abi.RAD_F32 if f32 else abi.RAD_BF16), _desc(q_ref, abi.RAD_F8E4M3), _desc(s_ref, abi.RAD_F32)],
                   dict(n=n, group=g))
    assert R.ref_band_quant_act_fp8(C.byref(pack.args), None) == 0
    q, s = ops.quant_act_fp8(x, g)
    torch.cuda.synchronize()
    assert torch.equal(q, q_ref) and torch.equal(s.view(torch.int32), s_ref.view(torch.int32))
    xin = xf if f32 else orc.bf16_bits_to_f32(gen.f32_to_bf16_bits(xf))
    want_q, want_s = orc.quant_act_fp8(xin, g)
    assert np.array_equal(q_ref.cpu().numpy(), want_q) and np.array_equal(s_ref.cpu().numpy().view(np.uint32), want_s.view(np.uint32))


@pytest.mark.parametrize("act", ["silu", "sigmoid"])
@pytest.mark.parametrize("rows,n,group", [(1, 128, 128), (5, 300, 128), (16, 13824, 128), (3, 200, 0)])
def test_gated_quant_fp8_matches_the_reference_kernel(rows, n, group, act):
    R = _ref()
    P = ops.plugin()
    rng = np.random.default_rng(rows * 17 + n)
    bits = gen.f32_to_bf16_bits((rng.standard_normal((rows, 2 * n)) * 4).astype(np.float32))
    gu_t = torch.from_numpy(bits.view(np.int16)).cuda().view(torch.bfloat16)
    g = n if group <= 0 else group
    ngrp = (n + g - 1) // g
    mk = lambda: (torch.zeros((rows, n), dtype=torch.uint8, device="cuda"), torch.zeros((rows, ngrp), dtype=torch.float32, device="cuda"),
                  torch.zeros((rows, n), dtype=torch.bfloat16, device="cuda"))
    q_ref, s_ref, o_ref = mk()
    pack = ArgPack([_desc(gu_t, abi.RAD_BF16), _desc(q_ref, abi.RAD_F8E4M3), _desc(s_ref, abi.RAD_F32), _desc(o_ref, abi.RAD_BF16)],
                   dict(n=n, group=g, act=act))
    assert R.ref_band_gated_quant_fp8(C.byref(pack.args), None) == 0
    q, s, o = mk()
    assert P.lib.r3d_b200_gated_quant_fp8(gu_t.data_ptr(), 2 * n, q.data_ptr(), n, s.data_ptr(), ngrp, o.data_ptr(), abi.RAD_BF16, n,
                                          rows, n, g, 1 if act == "silu" else 0, None) == 0
    torch.cuda.synchronize()
    assert torch.equal(s.view(torch.int32), s_ref.view(torch.int32))
    assert torch.equal(q, q_ref)
    assert gu.same_bits_or_both_nan(o.view(torch.int16).cpu().numpy().view(np.uint16), o_ref.view(torch.int16).cpu().numpy().view(np.uint16)).all()
    want_q, want_s = orc.gated_quant_fp8(bits, g, act == "silu")
    assert np.array_equal(q_ref.cpu().numpy(), want_q) and np.array_equal(s_ref.cpu().numpy().view(np.uint32), want_s.view(np.uint32))


@pytest.mark.parametrize("N,K,M,br,sdt", [(256, 512, 1, 128, 0), (136, 300, 5, 128, 0), (200, 512, 2, 1, 0),
                                          (256, 384, 4, 128, 1), (256, 512, 8, 128, 2), (1000, 1024, 16, 128, 0),
                                          (4096, 5120, 4, 128, 0)])
def test_logits_kernels_against_the_reference_kernel(N, K, M, br, sdt):
    """The reference's own logits_e4m3 kernel and entry (src/r3d_gemm_logits.hip of libr3d, compiled
    for sm_100a into oracle/_ref/libref_logits.so) on the same head and activations: it re-associates
    K across 32 lanes, so it is graded against the oracle at its own unit test's 1e-4, and this
    library's arms are graded against IT at the same bound. N is kept a multiple of 8 here: in a
    partial last block of 8 head rows the reference kernel's out-of-range warps return before the
    block stages its activation tile (src/r3d_gemm_logits.hip:83 and :108-111), so under this build
    the surviving warps read unstaged shared memory; this library and the oracle have no such case."""
    from libr3d_b200.plugin import planes_blob
    R = orc.ref_logits()
    if R is None:
        pytest.skip("oracle/_ref/libref_logits.so not present")
    c = gen.case_logits(5 * N + K + M, M, N, K, br, sdt)
    sdts = {0: abi.RAD_BF16, 1: abi.RAD_F16, 2: abi.RAD_F32}[sdt]
    blob = planes_blob([("codes", abi.RAD_F8E4M3, (1, 1), c["codes"]), ("scale", sdts, (br, 128), c["scale"])])
    mem = R.ref_logits_alloc(len(blob))                 # managed: the reference entry reads the header on the host
    assert mem
    try:
        C.memmove(mem, blob, len(blob))
        x = gu.dev(c["X"]).view(torch.bfloat16)
        y_ref = torch.zeros((M, N), dtype=torch.float32, device="cuda")
        pack = ArgPack([_desc(x, abi.RAD_BF16), tensor_desc(mem, abi.RAD_U8, [len(blob)]), _desc(y_ref, abi.RAD_F32)],
                       dict(M=M, n_vocab=N, n_embd=K, dtype="bf16"))
        assert R.ref_logits_gemm_e4m3(C.byref(pack.args), None) == 0
        torch.cuda.synchronize()
        ref = y_ref.cpu().numpy().astype(np.float64)
        want = orc.logits_e4m3(c["X"], c["codes"], c["scale"], sdt, br).astype(np.float64)
        rel = lambda a, b: np.abs(a - b).max() / max(np.abs(b).max(), 1e-6)
        assert rel(ref, want) < 1e-4                    # the reference kernel against the oracle
        arms = [abi.R3D_ARM_EXACT] + ([abi.R3D_ARM_STREAM] if K % 64 == 0 else []) + ([abi.R3D_ARM_TILE] if K % 128 == 0 else [])
        for arm in arms:
            got = gu.logits_launch(c, arm).astype(np.float64)
            assert rel(got, ref) < 1e-4, arm            # this library against the reference kernel
    finally:
        torch.cuda.synchronize()
        R.ref_logits_free(mem)


# ------------------------------------------------------------------ the reference's own GEMM kernels
def _gemm_pack(t, kind, M, N, K, y):
    bdesc = (_desc(t["B"], abi.RAD_F8E4M3) if kind == "fp8a8"
             else tensor_desc(t["B"].data_ptr(), abi.RAD_FP4E2M1, [N, K], [K, 1]))
    sdt = abi.RAD_BF16 if kind == "fp8a8" else abi.RAD_E8M0
    tensors = [_desc(t["A"], abi.RAD_F8E4M3), _desc(t["AS"], abi.RAD_F32), bdesc, _desc(t["BS"], sdt),
               _desc(y, abi.RAD_BF16), tensor_desc(None, abi.RAD_F32, []), tensor_desc(None, abi.RAD_BF16, [])]
    return ArgPack(tensors, dict(M=M, N=N, K=K, group=128 if kind == "fp8a8" else 32, dtype=kind))


@pytest.mark.parametrize("kind,entry,M,N,K", [
    ("fp8a8", "ref_fp8a8_gemm_nt_q_decode", 1, 512, 1024), ("fp8a8", "ref_fp8a8_gemm_nt_q_decode", 2, 384, 2560),
    ("fp8a8", "ref_fp8a8_gemm_nt_q_decode", 3, 1000, 512), ("fp8a8", "ref_fp8a8_gemm_nt_q", 2, 512, 1024),
    ("fp8a8", "ref_fp8a8_gemm_nt_q", 1, 4096, 4096),
    ("mxfp4a8", "ref_mxfp4_gemm_nt_q_decode", 1, 512, 1024), ("mxfp4a8", "ref_mxfp4_gemm_nt_q_decode", 4, 384, 2560),
    ("mxfp4a8", "ref_mxfp4_gemm_nt_q_decode", 8, 1000, 512), ("mxfp4a8", "ref_mxfp4_gemm_nt_q_decode", 2, 27648, 5120)])
def test_gemm_arms_against_the_reference_kernels(kind, entry, M, N, K):
    """The reference's own band kernels and entries (src/r3d_gemm_fp8a8.hip, src/r3d_gemm_mxfp4.hip of
    libr3d, compiled for sm_100a through the HIP / rocWMMA stand-ins) on the same operands. Graded
    like everything else at 2 bf16 ulp: the reference against the fp32-accumulated oracle, and this
    library's tensor-core arms against the reference's output.
    Only the reference's GEMV kernels are run (fp8a8 at M < 4: from M = 4 its dispatch hands the call
    to the skinny WMMA kernel; mxfp4a8 decode rows at M <= 8). Its 64-row tile kernel hands rocWMMA
    a leading dimension of 20 elements, which nvcuda::wmma (multiples of 8 elements, 32-byte aligned
    tiles) does not allow, so the WMMA kernels are compiled but never launched here."""
    R = orc.ref_gemm("fp8a8" if kind == "fp8a8" else "mxfp4")
    if R is None:
        pytest.skip("reference band library not present")
    case = gen.case_fp8(7000 + M, M, N, K, "ref128") if kind == "fp8a8" else gen.case_mxfp4(7000 + M, M, N, K)
    t = {k: gu.dev(case[k]) for k in ("A", "AS", "B", "BS")}
    y_ref = torch.zeros((M, N), dtype=torch.bfloat16, device="cuda")
    pack = _gemm_pack(t, kind, M, N, K, y_ref)
    assert getattr(R, entry)(C.byref(pack.args), None) == 0
    torch.cuda.synchronize()
    ref = y_ref.view(torch.int16).cpu().numpy().view(np.uint16)
    if kind == "fp8a8":
        _, acc = orc.gemm_fp8a8(case["A"], case["AS"], case["B"], case["BS"], case["rblk"], want_acc=True)
    else:
        _, acc = orc.gemm_mxfp4a8(**case, want_acc=True)
    g = gu.grade_bf16(ref, acc)
    assert g["frac_le2"] > 0.999 and g["rel_l2"] < 5e-3, ("reference vs oracle", g)
    got = gu.gemm_launch(kind, case, abi.R3D_ARM_AUTO)
    d = orc.bf16_ulp_distance(got, ref)
    assert (d <= 2).mean() > 0.999, ("this library vs reference", float((d <= 2).mean()), int(d.max()))


_IMMORTAL_WEIGHTS: list = []


@pytest.mark.parametrize("M", [1, 2, 4, 8])
def test_q8x_arm_against_the_reference_q8x_row(M):
    """The reference's int8-per-32 decode row (its repacked plane, requantiser and dot4 / lane-map
    kernels, all its own code) against this library's q8x arm, which reads the nibble plane as it
    is: the arm's chain is integer-exact inside a group, so the outputs must be identical bits."""
    R = orc.ref_gemm("mxfp4")
    if R is None:
        pytest.skip("reference band library not present")
    N, K = 640, 2048
    case = gen.case_mxfp4(7100 + M, M, N, K)
    t = {k: gu.dev(case[k]) for k in ("A", "AS", "B", "BS")}
    # The reference row remembers the int8 plane it repacked by the weight's device address and treats
    # weights as immortal (src/r3d_gemm_mxfp4.hip:1879-1880): a weight freed here could hand its address to
    # the next case's weight, which the reference would then serve with this case's plane.
    _IMMORTAL_WEIGHTS.append((t["B"], t["BS"]))
    y_ref = torch.zeros((M, N), dtype=torch.bfloat16, device="cuda")
    pack = _gemm_pack(t, "mxfp4a8", M, N, K, y_ref)
    assert R.ref_mxfp4_gemm_nt_q_decode_q8x(C.byref(pack.args), None) == 0
    torch.cuda.synchronize()
    ref = y_ref.view(torch.int16).cpu().numpy().view(np.uint16)
    y = torch.zeros((M, N), dtype=torch.bfloat16, device="cuda")
    r = ops.gemm_nt_q(t["A"], t["AS"], t["B"], t["BS"], y, dtype="mxfp4a8", N=N, K=K, row="gemm_nt_q_mxfp4_decode_q8x")
    torch.cuda.synchronize()
    got = y.view(torch.int16).cpu().numpy().view(np.uint16)
    assert r.name == "gemm_nt_q_mxfp4_decode_q8x"
    assert np.array_equal(got, ref)
