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
