"""GPU parity of logits_gemm over the joined e4m3 + block-scale head."""
import ctypes as C

import numpy as np
import pytest
import torch

import gen
import gpu_util as gu
from libr3d_b200 import abi, ops
from libr3d_b200.plugin import planes_blob
from oracle import oracle as orc

pytestmark = pytest.mark.gpu
EX, STREAM, TILE = abi.R3D_ARM_EXACT, abi.R3D_ARM_STREAM, abi.R3D_ARM_TILE

CASES = [(256, 512, 1, 128, 0), (256, 512, 3, 128, 0), (130, 300, 5, 128, 0), (256, 512, 9, 128, 0),
         (200, 512, 2, 1, 0), (256, 384, 4, 128, 1), (256, 512, 8, 128, 2), (8, 4, 1, 128, 0)]


def _rel(y, want):
    return np.abs(y.astype(np.float64) - want).max() / max(np.abs(want).max(), 1e-6)


@pytest.mark.parametrize("N,K,M,br,sdt", CASES)
def test_reference_unit_geometries_exact_arm_bitwise(N, K, M, br, sdt):
    # the eight cases of tools/test_logits_e4m3.cpp:155-164
    c = gen.case_logits(N + K + M, M, N, K, br, sdt)
    want = orc.logits_e4m3(c["X"], c["codes"], c["scale"], sdt, br)
    got = gu.logits_launch(c, EX)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("N,K,M,br,sdt", [c for c in CASES if c[1] % 64 == 0] +
                         [(1000, 1024, 16, 128, 0), (333, 640, 33, 1, 2), (512, 5120, 4, 128, 0)])
def test_stream_arm_within_reference_tolerance(N, K, M, br, sdt):
    # graded like the reference's own unit test: 1e-4 relative (its kernel also re-associates)
    c = gen.case_logits(7 * N + K + M, M, N, K, br, sdt)
    want = orc.logits_e4m3(c["X"], c["codes"], c["scale"], sdt, br)
    got = gu.logits_launch(c, STREAM)
    assert _rel(got, want.astype(np.float64)) < 1e-4
    assert np.count_nonzero(got) > got.size * 0.9


@pytest.mark.parametrize("N,K,M,br,sdt", [c for c in CASES if c[1] % 128 == 0] +
                         [(1000, 1024, 16, 128, 0), (333, 640, 33, 1, 2), (512, 5120, 4, 128, 0),
                          (700, 2048, 32, 128, 1), (129, 128, 17, 1, 0), (4096, 16384, 2, 128, 0)])
def test_tcgen05_arm_within_reference_tolerance(N, K, M, br, sdt):
    # bf16 activations enter as two e4m3 pieces on a power-of-two grid (exact for all but
    # elements 2^13 below their block's amax); the grade is the reference unit test's 1e-4
    c = gen.case_logits(11 * N + K + M, M, N, K, br, sdt)
    want = orc.logits_e4m3(c["X"], c["codes"], c["scale"], sdt, br)
    got = gu.logits_launch(c, TILE)
    assert _rel(got, want.astype(np.float64)) < 2e-5
    assert np.count_nonzero(got) > got.size * 0.9


def test_tcgen05_arm_wide_dynamic_range_activations():
    """activations spanning 2^-20 .. 2^20 inside one 128-column block, zeros and denormal-small
    blocks: the split must stay within the grade and produce no NaN."""
    N, K, M = 384, 1024, 3
    c = gen.case_logits(4242, M, N, K, 128, 0)
    rng = np.random.default_rng(8)
    x = rng.standard_normal((M, K)).astype(np.float32) * np.exp2(rng.integers(-20, 21, (M, K))).astype(np.float32)
    x[0, 128:256] = 0.0
    x[1, 256:384] *= np.float32(2.0 ** -120)
    x[2, 512:640] *= np.float32(2.0 ** 60)
    c["X"] = gen.f32_to_bf16_bits(x)
    want = orc.logits_e4m3(c["X"], c["codes"], c["scale"], 0, 128)
    got = gu.logits_launch(c, TILE)
    assert np.isfinite(got).all()
    assert _rel(got, want.astype(np.float64)) < 2e-5


def test_stream_arm_dequant_exact_incl_subnormal_and_nan_codes():
    """one-hot x = 1.0 picks each code times a power-of-two scale: results must be exact."""
    K, N = 128, 256
    codes = np.zeros((N, K), np.uint8); codes[:, 7] = np.arange(256)
    X = np.zeros((1, K), np.uint16); X[0, 7] = 0x3F80
    c = dict(X=X, codes=codes, scale=np.full((2, 1), 0x3E80, np.uint16), sdt=0, br=128)   # 0.25
    want = orc.logits_e4m3(X, codes, c["scale"], 0, 128)
    for arm in (EX, STREAM, TILE):
        got = gu.logits_launch(c, arm)
        nan = np.isnan(want)
        assert nan.sum() == 2 and np.array_equal(np.isnan(got), nan)
        assert np.array_equal(got[~nan], want[~nan]), arm


def test_row_entry_with_joined_blob():
    N, K, M = 1024, 1024, 5
    c = gen.case_logits(99, M, N, K, 128, 0)
    blob = np.frombuffer(planes_blob([("codes", abi.RAD_F8E4M3, (1, 1), c["codes"]),
                                      ("scale", abi.RAD_BF16, (128, 128), c["scale"])]), np.uint8)
    out = gu.GuardedOut((M, N), np.float32)
    x = gu.dev(c["X"]).view(torch.bfloat16)
    r = ops.logits_gemm(x, gu.dev(blob), out.view(), n_vocab=N, n_embd=K)
    assert r.name == "logits_gemm_e4m3"
    want = orc.logits_e4m3(c["X"], c["codes"], c["scale"], 0, 128)
    assert _rel(out.get(), want.astype(np.float64)) < 1e-4


@pytest.fixture(scope="module")
def vocab_head():
    """N = 151936, K = 5120: the LM head of the benchmark, e4m3 codes + a bf16 scale per 128x128"""
    N, K = 151936, 5120
    rng = np.random.default_rng(5)
    codes = rng.integers(0, 256, (N, K), dtype=np.uint8)
    codes[(codes & 0x7F) == 0x7F] &= 0x7E
    scale = gen.f32_to_bf16_bits(np.exp(rng.uniform(-6, -4, ((N + 127) // 128, K // 128))).astype(np.float32))
    return codes, scale


@pytest.mark.parametrize("M", [1, 4, 16])
def test_vocab_size_head_sampled_rows(vocab_head, M):
    """The full-size head at M = 1, 4 and 16 (one pass of 32 piece rows): both tensor-core arms vs
    the oracle on a sample of rows (first, random, last), nothing left unwritten."""
    codes, scale = vocab_head
    N, K = codes.shape
    rng = np.random.default_rng(50 + M)
    X = gen.f32_to_bf16_bits(rng.standard_normal((M, K)).astype(np.float32))
    c = dict(X=X, codes=codes, scale=scale, sdt=0, br=128)
    rows = np.concatenate([np.arange(0, 256), rng.choice(N, 256, replace=False), np.arange(N - 64, N)])
    want = orc.logits_e4m3(X, codes[rows], np.repeat(scale, 128, axis=0)[rows], 0, 1)
    for arm, tol in ((STREAM, 1e-4), (TILE, 2e-5)):
        got = gu.logits_launch(c, arm)
        assert _rel(got[:, rows], want.astype(np.float64)) < tol, arm
        assert np.count_nonzero(got) > got.size * 0.99


def _mxfp4_head_launch(Xb, B, BS, arm, y_dtype=abi.RAD_F32):
    P = ops.plugin()
    X, codes, scale = gu.dev(Xb), gu.dev(B), gu.dev(BS)
    M, K = Xb.shape
    N = B.shape[0]
    out = gu.GuardedOut((M, N), np.float32 if y_dtype == abi.RAD_F32 else np.uint16)
    l = abi.R3dLogits()
    l.x, l.codes, l.scale, l.y = X.data_ptr(), codes.data_ptr(), scale.data_ptr(), out.ptr
    l.m, l.n, l.k, l.br = M, N, K, 1
    l.scale_dtype, l.y_dtype, l.head_fmt, l.arm = abi.RAD_E8M0, y_dtype, 1, arm
    l.x_pitch, l.code_pitch, l.y_pitch, l.scale_pitch = K, K // 2, N, K // 32
    rc = P.lib.r3d_b200_logits(C.byref(l), None)
    assert rc == abi.RAD_OK, abi.STATUS_NAMES[rc]
    return out.get()


def test_mxfp4_head_vocab_size_sampled_rows():
    """The mxfp4 head at N = 151936, K = 5120, M = 4: the tcgen05 arm vs the oracle on a row sample."""
    N, K, M = 151936, 5120, 4
    rng = np.random.default_rng(6)
    B = rng.integers(0, 256, (N, K // 2), dtype=np.uint8)
    BS = rng.integers(119, 124, (N, K // 32), dtype=np.uint8)
    Xb = gen.f32_to_bf16_bits(rng.standard_normal((M, K)).astype(np.float32))
    rows = np.concatenate([np.arange(0, 256), rng.choice(N, 256, replace=False), np.arange(N - 64, N)])
    want = orc.logits_mxfp4(Xb, np.ascontiguousarray(B[rows]), np.ascontiguousarray(BS[rows])).astype(np.float64)
    got = _mxfp4_head_launch(Xb, B, BS, abi.R3D_ARM_AUTO).astype(np.float64)
    assert np.abs(got[:, rows] - want).max() / np.abs(want).max() < 2e-5
    assert np.count_nonzero(got) > got.size * 0.99


@pytest.mark.parametrize("M,N,K", [(1, 512, 1024), (4, 1000, 5120), (16, 384, 2560), (20, 256, 512)])
def test_mxfp4_head_tcgen05_arm_against_oracle_and_exact_arm(M, N, K):
    """The mxfp4 LM head (e2m1 nibbles, one E8M0 byte per 32 columns; not a reference format: the
    oracle fixes y = sum f32(x) * (e2m1 * 2^(s-127)) as one fp32 fma chain). The exact arm must match
    the oracle bit for bit; the tcgen05 arm (hardware group scales, two exact e4m3 pieces per bf16
    activation) within the logits tolerance. M = 20 takes two passes of 16."""
    c = gen.case_mxfp4(4400 + M, 1, N, K)
    rng = np.random.default_rng(M + N)
    Xb = gen.f32_to_bf16_bits(rng.uniform(-2, 2, (M, K)).astype(np.float32))
    want = orc.logits_mxfp4(Xb, c["B"], c["BS"]).astype(np.float64)
    exact = _mxfp4_head_launch(Xb, c["B"], c["BS"], abi.R3D_ARM_EXACT)
    assert np.array_equal(exact.view(np.uint32), orc.logits_mxfp4(Xb, c["B"], c["BS"]).view(np.uint32))
    rel = lambda a, b: np.abs(a - b).max() / max(np.abs(b).max(), 1e-6)
    for arm in (abi.R3D_ARM_TILE, abi.R3D_ARM_AUTO):
        got = _mxfp4_head_launch(Xb, c["B"], c["BS"], arm).astype(np.float64)
        assert rel(got, want) < 2e-5, (arm, rel(got, want))
    gb = _mxfp4_head_launch(Xb, c["B"], c["BS"], abi.R3D_ARM_TILE, abi.RAD_BF16)
    d = orc.bf16_ulp_distance(gb, orc.f32_to_bf16_bits(want.astype(np.float32)))
    assert (d <= 2).mean() > 0.999
