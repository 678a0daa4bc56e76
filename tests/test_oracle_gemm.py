"""The oracle's matmul rules: known-answer fixtures the reference's tools hold, independent
numpy re-derivations on small shapes, and the committed golden vectors."""
import math
from pathlib import Path

import numpy as np
import pytest

import gen
from oracle import oracle as orc

GOLD = Path(__file__).resolve().parent / "golden"


def test_fp8_unit_fixture_is_analytic():
    # tools/bench_fp8_skinny.cpp:595-624: every output must equal K * (1 + r % 3) exactly
    for (M, K, N) in [(1, 128, 7), (14, 512, 130), (3, 2048, 64)]:
        case, expect = gen.fixture_fp8_unit(M, K, N)
        Y, acc = orc.gemm_fp8a8(case["A"], case["AS"], case["B"], case["BS"], 1, want_acc=True)
        assert np.array_equal(acc, expect)
        assert np.array_equal(Y, orc.f32_to_bf16_bits(expect.astype(np.float32)))


def _numpy_fp8(case):
    """independent restatement: same order, written with numpy scalars"""
    lut = gen.e4m3_decode_table()
    A, B, AS, BS, rblk = case["A"], case["B"], case["AS"], case["BS"], case["rblk"]
    sb = BS if BS.dtype == np.float32 else orc.bf16_bits_to_f32(BS)
    M, K = A.shape
    N = B.shape[0]
    out = np.zeros((M, N), np.float32)
    for m in range(M):
        for n in range(N):
            acc = np.float32(0)
            for g in range(K // 128):
                part = np.float32(0)
                for k in range(g * 128, g * 128 + 128):
                    part = np.float32(part + np.float32(lut[A[m, k]] * lut[B[n, k]]))
                ca = g if AS.shape[1] > 1 else 0
                cb = g if sb.shape[1] > 1 else 0
                acc = np.float32(acc + np.float32(np.float32(part * AS[m, ca]) * sb[n // rblk, cb]))
            out[m, n] = acc
    return out


@pytest.mark.parametrize("grid", ["ref128", "row", "channel"])
def test_fp8_oracle_matches_numpy_walk(grid):
    case = gen.case_fp8(3, 2, 9 if grid != "ref128" else 130, 256, grid)
    if grid == "ref128":
        case = {k: (v[:, :] if hasattr(v, "shape") else v) for k, v in case.items()}
    want = _numpy_fp8(case)
    Y, acc = orc.gemm_fp8a8(case["A"], case["AS"], case["B"], case["BS"], case["rblk"], want_acc=True)
    assert np.array_equal(acc.view(np.uint32), want.view(np.uint32))


def _numpy_mxfp4(case):
    lut = gen.e4m3_decode_table()
    mag = np.array([0, .5, 1, 1.5, 2, 3, 4, 6], np.float32)
    A, B, AS, BS = case["A"], case["B"], case["AS"], case["BS"]
    M, K = A.shape
    N = B.shape[0]
    out = np.zeros((M, N), np.float32)
    for m in range(M):
        for n in range(N):
            acc = np.float32(0)
            for g in range(K // 32):
                s = np.float32(0)
                for k in range(g * 32, g * 32 + 32):
                    byte = B[n, k >> 1]
                    nib = (byte >> 4) if (k & 1) else (byte & 15)
                    w = -mag[nib & 7] if nib & 8 else mag[nib & 7]
                    s = np.float32(s + np.float32(lut[A[m, k]] * w))
                x = int(BS[n, g])
                sc = np.float32("nan") if x == 255 else np.float32(math.ldexp(1.0, x - 127))
                with np.errstate(invalid="ignore"):
                    acc = np.float32(acc + np.float32(np.float32(s * AS[m, g >> 2]) * sc))
            out[m, n] = acc
    return out


def test_mxfp4_oracle_matches_probe_walk_on_probe_fixture():
    # the walk of tools/probe_m4_entry.cpp:72-91 over that tool's own srand(777) fixture
    case = gen.fixture_probe_m4(2, 256, 12)
    want = _numpy_mxfp4(case)
    Y, acc = orc.gemm_mxfp4a8(case["A"], case["AS"], case["B"], case["BS"], want_acc=True)
    assert np.array_equal(acc.view(np.uint32), want.view(np.uint32))
    assert np.count_nonzero(acc) > acc.size // 2              # not a fixture of zeros


def test_mxfp4_scale_byte_torture():
    case = gen.case_mxfp4(4, 1, 8, 128)
    case["BS"][:] = 127
    case["BS"][0, 1] = 255            # NaN scale poisons the row even if the group sums to 0
    case["B"][0, 16:32] = 0
    case["BS"][1, :] = 0              # 2^-127 everywhere: tiny but not zero
    Y, acc = orc.gemm_mxfp4a8(case["A"], case["AS"], case["B"], case["BS"], want_acc=True)
    assert math.isnan(acc[0, 0]) and not np.isnan(acc[0, 1:]).any()
    base = case["BS"].copy(); base[1, :] = 127
    _, acc1 = orc.gemm_mxfp4a8(case["A"], case["AS"], case["B"], base, want_acc=True)
    assert acc[0, 1] != 0 and abs(acc[0, 1] / acc1[0, 1] - 2.0 ** -127) < 1e-6 * 2.0 ** -127


def test_q8x_chain_integer_exact_witness():
    # With activations that requantise exactly (all |e| in a group equal) and unit scales the
    # int8 arm's chain must reproduce the fp32 oracle bit for bit.
    rng = np.random.default_rng(9)
    M, N, K = 2, 16, 512
    A = np.where(rng.integers(0, 2, (M, K)) > 0, 0x38, 0xB8).astype(np.uint8)      # +-1.0
    AS = np.full((M, K // 128), 127.0, np.float32)
    B = rng.integers(0, 256, (N, K // 2), dtype=np.uint8)
    BS = np.full((N, K // 32), 127, np.uint8)
    y_ref = orc.gemm_mxfp4a8(A, AS, B, BS)
    for walk in (0, 1):
        assert np.array_equal(orc.gemm_mxfp4_q8x(A, AS, B, BS, walk), y_ref)


def test_q8x_close_to_fp32_walk_on_random_data():
    case = gen.case_mxfp4(11, 4, 64, 1024)
    y = orc.bf16_bits_to_f32(orc.gemm_mxfp4a8(**case))
    for walk in (0, 1):
        yq = orc.bf16_bits_to_f32(orc.gemm_mxfp4_q8x(case["A"], case["AS"], case["B"], case["BS"], walk))
        rel = np.linalg.norm(yq - y) / np.linalg.norm(y)
        assert rel < 3e-2                     # the op's tolerance; the arm grades ~1e-3..7e-3


@pytest.mark.parametrize("N,K,M,br,sdt", [
    (256, 512, 1, 128, 0), (256, 512, 3, 128, 0), (130, 300, 5, 128, 0), (256, 512, 9, 128, 0),
    (200, 512, 2, 1, 0), (256, 384, 4, 128, 1), (256, 512, 8, 128, 2), (8, 4, 1, 128, 0)])
def test_logits_oracle_on_reference_case_geometries(N, K, M, br, sdt):
    # the eight geometries of tools/test_logits_e4m3.cpp:155-164, graded against float64
    c = gen.case_logits(N * 31 + K * 7 + M, M, N, K, br, sdt)
    y = orc.logits_e4m3(c["X"], c["codes"], c["scale"], sdt, br)
    lut = gen.e4m3_decode_table().astype(np.float64)
    sv = (c["scale"] if sdt == 2 else
          c["scale"].view(np.float16).astype(np.float32) if sdt == 1 else
          orc.bf16_bits_to_f32(c["scale"])).astype(np.float64)
    w = lut[c["codes"]] * np.repeat(np.repeat(sv, br, axis=0)[:N], 128, axis=1)[:, :K]
    want = orc.bf16_bits_to_f32(c["X"]).astype(np.float64) @ w.T
    den = np.maximum(np.abs(lut[c["codes"]] * 1.0).max() * np.abs(want).max() * 1e-3, 1e-6)
    assert np.abs(y - want).max() / max(np.abs(want).max(), den) < 1e-5


def test_golden_vectors():
    files = sorted(GOLD.glob("*.npz"))
    assert files, "golden fixtures missing: run tests/golden/make_golden.py"
    for f in files:
        g = np.load(f)
        kind = str(g["kind"])
        if kind == "fp8a8":
            y = orc.gemm_fp8a8(g["A"], g["AS"], g["B"], g["BS"], int(g["rblk"]))
        elif kind == "mxfp4a8":
            y = orc.gemm_mxfp4a8(g["A"], g["AS"], g["B"], g["BS"])
        elif kind == "mxfp4a8_q8x":
            y = orc.gemm_mxfp4_q8x(g["A"], g["AS"], g["B"], g["BS"], int(g["walk"]))
        elif kind == "logits_e4m3":
            y = orc.logits_e4m3(g["X"], g["codes"], g["scale"], int(g["sdt"]), int(g["br"]))
        else:
            raise AssertionError(kind)
        a, b = np.ascontiguousarray(y), g["Y"]
        assert a.dtype == b.dtype and np.array_equal(a.view(np.uint8), b.view(np.uint8)), f.name


def test_gated_quant_matches_independent_numpy_walk():
    """orc_gated_quant_fp8 (src/r3d_gemm_fp8a8.hip:700-825 of libr3d) against a numpy restatement
    written from the rule: h = bf16((silu ? g*sig(g) : sig(g)) * up), sig through double exp,
    amax/448 scale per group, saturating RTNE codes."""
    rng = np.random.default_rng(11)
    M, n = 5, 300                                        # a ragged last group
    gu = gen.f32_to_bf16_bits((rng.standard_normal((M, 2 * n)) * 3).astype(np.float32))
    gu[0, :4] = [0x0000, 0x8000, 0x7F80, 0xFF80]         # zeros and infinities in the gate
    gu[1, n:n + 128] = 0                                 # an all-zero group: scale 1
    gf = orc.bf16_bits_to_f32(gu)
    for silu in (True, False):
        q, s, ob = orc.gated_quant_fp8(gu, 128, silu, want_ob=True)
        gt, up = gf[:, :n], gf[:, n:]
        with np.errstate(over="ignore", invalid="ignore"):
            sg = (np.float32(1) / (np.float32(1) + np.exp(-gt.astype(np.float64)).astype(np.float32))).astype(np.float32)
            a = (gt * sg).astype(np.float32) if silu else sg
            h = orc.bf16_bits_to_f32(gen.f32_to_bf16_bits((a * up).astype(np.float32)))
        assert np.array_equal(ob, gen.f32_to_bf16_bits(h))
        for gi in range(3):
            blk = h[:, gi * 128:min(gi * 128 + 128, n)]
            am = np.zeros(M, np.float32)
            for k in range(blk.shape[1]):                # strict >: NaN never wins
                m = np.abs(blk[:, k]); am = np.where(m > am, m, am)
            sc = np.where(am > 0, (am * np.float32(1 / 448)).astype(np.float32), np.float32(1))
            assert np.array_equal(s[:, gi].view(np.uint32), sc.astype(np.float32).view(np.uint32))
            c = np.clip((blk * (np.float32(1) / sc)[:, None]).astype(np.float32), -448, 448)
            assert np.array_equal(q[:, gi * 128:gi * 128 + blk.shape[1]], orc.encode_e4m3(c))
        assert s[1, 0] == 1.0 and (q[1, :128] & 0x7F).max() == 0


def test_rmsnorm_quant_matches_independent_numpy_walk():
    """orc_rmsnorm_quant_fp8 (the kernel of src/r3d_more.hip:248-330 of libr3d) against a numpy
    restatement written from the rule: 256 strided partial sums of squares, a shuffle-down tree per
    group of 32 partials, the eight results added ascending, rs = 1/sqrt(ss/n + eps),
    h = bf16(src * rs * (w + wadd)), then the group quantiser; with a residual the bf16 sum is stored
    first and is what gets squared and normed."""
    rng = np.random.default_rng(12)
    M, n, eps, wadd = 3, 1000, np.float32(1e-6), np.float32(1.0)
    x = gen.f32_to_bf16_bits((rng.standard_normal((M, n)) * 2).astype(np.float32))
    res = gen.f32_to_bf16_bits((rng.standard_normal((M, n)) * 5).astype(np.float32))
    w = gen.f32_to_bf16_bits((0.1 * rng.standard_normal(n)).astype(np.float32))
    for with_res in (False, True):
        out = orc.rmsnorm_quant_fp8(x, w, float(eps), 128, float(wadd), res if with_res else None)
        src = orc.bf16_bits_to_f32(x)
        if with_res:
            sb = gen.f32_to_bf16_bits((orc.bf16_bits_to_f32(res) + src).astype(np.float32))
            assert np.array_equal(out["res"], sb)
            src = orc.bf16_bits_to_f32(sb)
        sq = (src * src).astype(np.float32)
        for r in range(M):
            part = np.zeros(256, np.float32)
            for i in range(n):                              # thread i % 256 adds its elements ascending
                part[i % 256] = np.float32(part[i % 256] + sq[r, i])
            tot = None
            for wp in range(8):
                lane = part[wp * 32:(wp + 1) * 32].copy()
                for off in (16, 8, 4, 2, 1):
                    lane[:32 - off] = (lane[:32 - off] + lane[off:]).astype(np.float32)
                tot = lane[0] if tot is None else np.float32(tot + lane[0])
            rs = np.float32(1) / np.sqrt(np.float32(np.float32(tot / np.float32(n)) + eps), dtype=np.float32)
            wv = (orc.bf16_bits_to_f32(w) + wadd).astype(np.float32)
            h = gen.f32_to_bf16_bits(((src[r] * rs).astype(np.float32) * wv).astype(np.float32))
            assert np.array_equal(out["ob"][r], h)
            hf = orc.bf16_bits_to_f32(h)
            for gi in range((n + 127) // 128):
                blk = hf[gi * 128:gi * 128 + 128]
                am = np.abs(blk).max()
                sc = np.float32(am * np.float32(1 / 448)) if am > 0 else np.float32(1)
                assert out["scale"][r, gi] == sc
                c = np.clip((blk * (np.float32(1) / sc)).astype(np.float32), -448, 448)
                assert np.array_equal(out["q"][r, gi * 128:gi * 128 + len(blk)], orc.encode_e4m3(c))


def test_row_topk_matches_a_sort():
    """orc_row_topk (src/r3d_more.hip:179-236 of libr3d: R rounds of argmax, each after the previous
    pick) against a plain sort by (value descending, column ascending); unfillable slots are (-1, -inf)."""
    rng = np.random.default_rng(13)
    M, N, R, off = 4, 40, 32, 1000
    x = gen.f32_to_bf16_bits(np.round(rng.standard_normal((M, N)) * 4).astype(np.float32) / 2)
    x[0, :3] = [0x7F80, 0xFF80, 0x8000]
    xf = orc.bf16_bits_to_f32(x)
    idx, val = orc.row_topk(x, R, off)
    for m in range(M):
        order = np.lexsort((np.arange(N), -xf[m]))
        assert np.array_equal(idx[m], order[:R] + off) and np.array_equal(val[m], xf[m][order[:R]])
    idx, val = orc.row_topk(x[:, :8], R, 0)
    assert (idx[:, 8:] == -1).all() and np.isneginf(val[:, 8:]).all() and (idx[:, :8] >= 0).all()
