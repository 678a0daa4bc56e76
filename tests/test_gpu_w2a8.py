"""gemm_nt_q at the w2a8 encoding (the draft head's decode band) on the GPU, through the row table:
bit for bit against the CPU oracle, which follows the reference's own transcription of the rule
(src/r3d_gemm_w2a8.hip:32-51 of libr3d). Every value before the scales is an exact integer, so the
row has no tolerance class: the bf16 bits must be equal. The reference's own kernels of this band are
AMD-intrinsic-heavy (DPP folds, v_dot4_i32_iu8, rocWMMA i8 tiles) and are not run here."""
import numpy as np
import pytest
import torch

import gpu_util as gu
from libr3d_b200 import abi, ops
from libr3d_b200.plugin import planes_blob
from oracle import oracle as orc

pytestmark = pytest.mark.gpu


def _case(seed, M, N, K, u4=False, wide=False):
    rng = np.random.default_rng(seed)
    G = K // 128
    A = rng.integers(-127, 128, (M, K), dtype=np.int8) if wide else rng.integers(-4, 4, (M, K)).astype(np.int8)
    AS = (0.01 + 0.001 * rng.integers(0, 16, M)).astype(np.float32)
    B = rng.integers(0, 256, (N, K // 4), dtype=np.uint8)
    SC = (0.0030 + 0.000125 * rng.integers(0, 32, (N, G))).astype(np.float16).view(np.uint16)
    if u4:
        z = rng.integers(0, 16, (N, G), dtype=np.uint8)
        zp = np.zeros((N, (G + 1) // 2), np.uint8)
        zp[:, : (G + 1) // 2] = z[:, 0::2]
        zp[:, : G // 2] |= z[:, 1::2] << 4
    else:
        zp = rng.integers(0, 256 if wide else 3, (N, G), dtype=np.uint8)
    ASUM = orc.w2a8_group_sums(A)
    return dict(A=A, AS=AS, B=B, SC=SC, ZP=zp, ASUM=ASUM, u4=u4)


def _run(c, N, K, M_param=None):
    M = c["A"].shape[0]
    G = K // 128
    blob = np.frombuffer(planes_blob([("scale", abi.RAD_F16, (1, 128), c["SC"]),
                                      ("zero", abi.RAD_U4 if c["u4"] else abi.RAD_U8, (1, 128), c["ZP"], G)]), np.uint8)
    out = gu.GuardedOut((M, N), np.uint16)
    r = ops.gemm_w2a8(gu.dev(c["A"]), gu.dev(c["AS"]), gu.dev(c["B"]), gu.dev(blob), out.view(), gu.dev(c["ASUM"]),
                      N=N, K=K, M_param=M_param)
    assert r.name == "gemm_nt_q_w2a8_decode"
    return out.get()


@pytest.mark.parametrize("M,N,K,u4,wide", [(1, 256, 1024, False, False), (2, 1024, 5120, False, True), (3, 48, 640, False, True),
                                           (4, 4096, 5120, False, False), (7, 272, 2048, False, True), (8, 512, 1152, False, True),
                                           (14, 1024, 5120, False, True), (16, 64, 128, False, True), (5, 160, 1024, True, True),
                                           (16, 2048, 3200, True, True)])
def test_w2a8_row_bit_identical_to_oracle(M, N, K, u4, wide):
    """M over every row bucket (1, 2, 4, 8, 16 and the ragged counts between), K with and without whole
    blocks of eight groups, u8 and u4 zero planes, small and full-range int8 activations."""
    c = _case(9000 + M + N, M, N, K, u4, wide)
    want = orc.gemm_w2a8(c["A"], c["AS"], c["B"], c["SC"], c["ZP"], c["ASUM"], zp_u4=u4)
    got = _run(c, N, K)
    assert np.array_equal(got, want)
    assert np.count_nonzero(got & 0x7FFF) > got.size * 0.9
    # M is numel(y)/N: an arena-capacity M parameter must not change a byte
    assert np.array_equal(_run(c, N, K, M_param=16), want)


def test_w2a8_draft_head_size_sampled():
    """N = 248320 rows x K = 5120 (the draft head), M = 4: every output written, a row sample against the oracle."""
    M, N, K = 4, 248320, 5120
    c = _case(77, M, N, K)
    got = _run(c, N, K)
    rows = np.sort(np.random.default_rng(3).choice(N, 512, replace=False))
    want = orc.gemm_w2a8(c["A"], c["AS"], c["B"][rows], c["SC"][rows], c["ZP"][rows], c["ASUM"])
    assert np.array_equal(got[:, rows], want)
    assert np.count_nonzero(got & 0x7FFF) > got.size * 0.9


def _direct(c, N, K, arm, u4=False):
    """the launch layer's entry itself (plain pointers and pitches), so that the kernel can be named"""
    import ctypes as C
    M = c["A"].shape[0]
    G = K // 128
    keep = [gu.dev(c[k]) for k in ("A", "AS", "B", "SC", "ZP", "ASUM")]
    out = gu.GuardedOut((M, N), np.uint16)
    q = abi.R3dW2A8()
    q.a, q.a_scale, q.b, q.scale, q.zero, q.a_sum = (t.data_ptr() for t in keep)
    q.y = out.ptr
    q.m, q.n, q.k, q.mpad, q.zero_u4, q.arm = M, N, K, (M + 15) // 16 * 16, int(u4), arm
    q.a_pitch, q.as_pitch, q.y_pitch = K, 1, N
    q.b_pitch, q.zp_pitch, q.sc_pitch = K // 4, c["ZP"].shape[1], G
    P = ops.plugin()
    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert P.lib.r3d_b200_gemm_w2a8(C.byref(q), st) == abi.RAD_OK
    torch.cuda.synchronize()
    assert P.lib.r3d_b200_stream_status() == 0
    return out.get()


@pytest.mark.parametrize("M,N,K,u4", [(1, 300, 5120, False), (6, 1000, 640, False), (8, 4097, 2560, True),
                                      (9, 777, 5120, False), (16, 8192 + 40, 1024, True)])
def test_w2a8_tile_kernel_and_row_kernel_agree_with_the_oracle(M, N, K, u4):
    """The persistent tensor-core kernel (several 256-row tiles a CTA would need N > 37888; here ragged last
    tiles, partial last stages (K / 128 not a multiple of four), eight and sixteen token columns) and the
    one-thread-per-row kernel both give the oracle's bits."""
    c = _case(4000 + M + N, M, N, K, u4, True)
    want = orc.gemm_w2a8(c["A"], c["AS"], c["B"], c["SC"], c["ZP"], c["ASUM"], zp_u4=u4)
    assert np.array_equal(_direct(c, N, K, abi.R3D_ARM_AUTO, u4), want)
    assert np.array_equal(_direct(c, N, K, abi.R3D_ARM_EXACT, u4), want)


def test_w2a8_tile_kernel_walks_several_tiles_a_cta():
    """N = 148 * 256 * 2 + 100 rows: every CTA walks at least two tiles and the ring wraps between them;
    the two kernels must agree on every output, and a row sample with the oracle."""
    M, N, K = 5, 148 * 512 + 100, 1536
    c = _case(31, M, N, K, False, True)
    a = _direct(c, N, K, abi.R3D_ARM_AUTO)
    b = _direct(c, N, K, abi.R3D_ARM_EXACT)
    assert np.array_equal(a, b)
    rows = np.sort(np.random.default_rng(5).choice(N, 256, replace=False))
    want = orc.gemm_w2a8(c["A"], c["AS"], c["B"][rows], c["SC"][rows], c["ZP"][rows], c["ASUM"])
    assert np.array_equal(a[:, rows], want)


@pytest.mark.parametrize("M,z", [(8, 0), (16, 1), (3, 2)])
def test_w2a8_small_integer_outputs_show_every_misplaced_code(M, z):
    """bf16 outputs of ordinary magnitude hide an integer error of a few units. Here the scales are one,
    the zeros a constant and the activations a sparse +-1 pattern, so every output is an integer below 256
    in magnitude, which bf16 holds exactly: one code or activation byte met by the wrong partner changes
    an output. Several tiles a CTA (the ring wraps between tiles), both kernels, and the closed form."""
    N, K = 148 * 256 + 300, 5120
    G = K // 128
    rng = np.random.default_rng(50 + M)
    A = np.zeros((M, K), np.int8)
    for m in range(M):
        pos = rng.choice(K, 40, replace=False)
        A[m, pos] = rng.choice(np.array([-1, 1], np.int8), 40)
    B = rng.integers(0, 256, (N, K // 4), dtype=np.uint8)
    c = dict(A=A, AS=np.ones(M, np.float32), B=B, SC=np.full((N, G), 0x3C00, np.uint16),
             ZP=np.full((N, G), z, np.uint8), ASUM=orc.w2a8_group_sums(A), u4=False)
    got = _direct(c, N, K, abi.R3D_ARM_AUTO)
    assert np.array_equal(got, _direct(c, N, K, abi.R3D_ARM_EXACT))
    # closed form: the stored activation column p holds logical column step(p); y = sum_k A[k] (q[k] - z)
    k = np.arange(K)
    step = (k & ~12) | ((k & 4) << 1) | ((k & 8) >> 1)
    Alog = A[:, step].astype(np.int32)
    rows = np.sort(rng.choice(N, 2048, replace=False))
    q = ((B[rows][:, :, None] >> (2 * np.arange(4))) & 3).reshape(len(rows), K).astype(np.int32) - z
    want = (Alog @ q.T).astype(np.float32)
    assert np.abs(want).max() < 256
    assert np.array_equal(gu.bf16_to_f32(got[:, rows]) if hasattr(gu, "bf16_to_f32") else
                          (got[:, rows].astype(np.uint32) << 16).view(np.float32), want)
