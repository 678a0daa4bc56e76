"""The oracle's number formats against the reference's own statements of them.

Pins, in order of strength:
  * oracle/_ref/libref_pin.so -- libr3d's src/r3d_mxfp4_q8x.h compiled as it lies: the doubled
    e2m1 table and the E8M0 decode, all codes;
  * constant tables written in libr3d's sources (cited per test);
  * spec identities (round trips, ties, saturation) for the encoder of src/r3d_band.hip:61-87.
"""
import math
import struct

import numpy as np
import pytest

from oracle import oracle as orc

L = orc.lib()


def bits(f):
    return struct.unpack("<I", struct.pack("<f", f))[0]


def test_ref_pin_e2m1_x2_all_codes():
    R = orc.ref_pin()
    if R is None:
        pytest.skip("reference pin not built (reference tree was not mounted at build time)")
    assert [L.orc_e2m1_x2(c) for c in range(16)] == [R.ref_e2m1_x2(c) for c in range(16)]


def test_ref_pin_e8m0_all_bytes():
    R = orc.ref_pin()
    if R is None:
        pytest.skip("reference pin not built")
    for x in range(256):
        a, b = L.orc_e8m0_to_f32(x), R.ref_e8m0_sc(x)
        assert (math.isnan(a) and math.isnan(b)) or bits(a) == bits(b), x


def test_e2m1_table_src_r3d_mxfp4_q8x_h_22():
    # R3D_E2M1_X2 as written at src/r3d_mxfp4_q8x.h:22; codes 7/15 are numbers (+-6 -> +-12)
    want = [0, 1, 2, 3, 4, 6, 8, 12, 0, -1, -2, -3, -4, -6, -8, -12]
    assert [L.orc_e2m1_x2(c) for c in range(16)] == want
    assert [L.orc_e2m1_to_f32(c) * 2 for c in range(16)] == [float(v) for v in want]
    assert bits(L.orc_e2m1_to_f32(8)) == 0x80000000          # code 8 is -0


def test_e2m1_bf16_patterns_src_r3d_gemm_mxfp4_hip_168():
    # kE2M1 bf16 bit patterns at src/r3d_gemm_mxfp4.hip:168-171
    want = [0x0000, 0x3F00, 0x3F80, 0x3FC0, 0x4000, 0x4040, 0x4080, 0x40C0,
            0x8000, 0xBF00, 0xBF80, 0xBFC0, 0xC000, 0xC040, 0xC080, 0xC0C0]
    assert [L.orc_f32_to_bf16(L.orc_e2m1_to_f32(c)) for c in range(16)] == want


def test_e8m0_rules_src_r3d_mxfp4_q8x_h_29():
    assert L.orc_e8m0_to_f32(127) == 1.0
    assert bits(L.orc_e8m0_to_f32(0)) == 0x00400000          # 2^-127 subnormal, not zero
    assert math.isnan(L.orc_e8m0_to_f32(255))
    assert L.orc_e8m0_to_f32(254) == 2.0 ** 127
    for x in range(1, 255):
        assert L.orc_e8m0_to_f32(x) == math.ldexp(1.0, x - 127)


def test_e4m3_decode_against_spec_walk():
    # independent field walk in the form of tools/test_logits_e4m3.cpp:26-32
    for b in range(256):
        s, e, m = (b >> 7) & 1, (b >> 3) & 0xF, b & 7
        got = L.orc_e4m3_to_f32(b)
        if e == 0xF and m == 7:
            assert math.isnan(got)
            continue
        want = (m / 8.0) * 2.0 ** -6 if e == 0 else (1 + m / 8.0) * 2.0 ** (e - 7)
        want = -want if s else want
        assert got == want and (math.copysign(1, got) < 0) == bool(s), b
    # the unit codes of tools/bench_fp8_skinny.cpp:497 and the format's extremes
    assert [L.orc_e4m3_to_f32(c) for c in (0x38, 0x40, 0x44)] == [1.0, 2.0, 3.0]
    assert L.orc_e4m3_to_f32(0x7E) == 448.0 and L.orc_e4m3_to_f32(0x01) == 2.0 ** -9


def test_e4m3_encode_roundtrip_and_saturation():
    for b in range(256):
        if (b & 0x7F) == 0x7F:
            continue
        assert L.orc_f32_to_e4m3(L.orc_e4m3_to_f32(b)) == b, b
    assert L.orc_f32_to_e4m3(float("nan")) & 0x7F == 0x7F
    assert L.orc_f32_to_e4m3(448.0) == 0x7E and L.orc_f32_to_e4m3(1e9) == 0x7E
    assert L.orc_f32_to_e4m3(-1e9) == 0xFE and L.orc_f32_to_e4m3(float("inf")) == 0x7E
    assert L.orc_f32_to_e4m3(465.0) == 0x7E                 # rounds past 448: re-saturates
    assert L.orc_f32_to_e4m3(2.0 ** -11) == 0x00             # below half the smallest subnormal
    assert L.orc_f32_to_e4m3(2.0 ** -10) == 0x00             # tie to even (0)
    assert L.orc_f32_to_e4m3(3 * 2.0 ** -10) == 0x02         # tie 1.5 ulp -> even (2)
    assert L.orc_f32_to_e4m3(2.0 ** -10 * 1.0001) == 0x01


def test_e4m3_encode_is_nearest_even_everywhere():
    tab = np.array([L.orc_e4m3_to_f32(b) for b in range(0x7F)], np.float64)   # ascending, >= 0
    rng = np.random.default_rng(5)
    xs = np.concatenate([rng.uniform(0, 460, 20000), rng.uniform(0, 0.05, 20000),
                         (tab[:-1] + tab[1:]) / 2])          # midpoints: the tie cases
    for x in xs.astype(np.float32):
        c = L.orc_f32_to_e4m3(float(x))
        d = np.abs(tab - float(x))
        best = d.min()
        assert abs(tab[c] - float(x)) == best or float(x) >= 448, x
        ties = np.nonzero(d == best)[0]
        if len(ties) == 2 and float(x) < 448:
            assert c % 2 == 0, (x, c)                        # tie -> even mantissa


def test_bf16_narrowing_rules():
    assert L.orc_f32_to_bf16(1.0) == 0x3F80
    assert L.orc_f32_to_bf16(struct.unpack("<f", struct.pack("<I", 0x3F808000))[0]) == 0x3F80
    assert L.orc_f32_to_bf16(struct.unpack("<f", struct.pack("<I", 0x3F818000))[0]) == 0x3F82
    assert L.orc_f32_to_bf16(struct.unpack("<f", struct.pack("<I", 0x7FA00001))[0]) == 0x7FE0
    x = np.random.default_rng(1).standard_normal(1000).astype(np.float32)
    assert np.array_equal(orc.f32_to_bf16_bits(x),
                          np.array([L.orc_f32_to_bf16(float(v)) for v in x], np.uint16))


def test_f16_decode():
    h = np.arange(0, 65536, 7, dtype=np.uint16)
    want = h.view(np.float16).astype(np.float32)
    for hv, w in zip(h, want):
        g = L.orc_f16_to_f32(int(hv))
        assert (math.isnan(g) and math.isnan(w)) or g == w


def test_quant_act_fp8_rule():
    # src/r3d_band.hip:119-153: scale = amax/448 (a dequant multiplier), all-zero group -> 1
    x = np.zeros((2, 256), np.float32)
    x[0, :128] = np.linspace(-3, 3, 128)
    x[1, 130] = float("nan")
    q, s = orc.quant_act_fp8(x, 128)
    assert s[0, 0] == np.float32(3.0) * np.float32(1.0 / 448.0) and s[0, 1] == 1.0
    assert q[0, 0] == 0xFE and q[0, 127] == 0x7E and not q[0, 128:].any()
    assert s[1, 1] == 1.0 and q[1, 130] & 0x7F == 0x7F       # NaN never wins amax; encodes NaN


def test_q8x_requant_rule():
    # src/r3d_gemm_mxfp4.hip:1150-1166
    A = np.zeros((1, 64), np.uint8)
    A[0, :32] = 0x38
    A[0, 5] = 0x7E
    x8, sg = orc.q8x_requant(A)
    assert sg[0, 0] == np.float32(448.0) / np.float32(127.0) and sg[0, 1] == 1.0
    assert x8[0, 5] == 127 and x8[0, 0] == 0 and not x8[0, 32:].any()


def test_mx8_quantiser_rule():
    x = np.zeros((1, 64), np.float32)
    x[0, 0], x[0, 1] = 300.0, 0.75
    q, e = orc.quant_act_mx8(x)
    assert e[0, 0] == 127 + 8 - 8 and e[0, 1] == 127      # floor(log2 300) = 8
    assert L.orc_e4m3_to_f32(int(q[0, 0])) == 288.0 and L.orc_e4m3_to_f32(int(q[0, 1])) == 0.75


def test_encoder_against_the_reference_file_compiled_as_it_lies():
    """src/r3d_band.hip of libr3d, compiled where it lies (oracle/_ref/libref_band.so): its e4m3
    encoder, bf16 narrowing and sigmoid against the oracle's restatements over every bf16-exact
    float, every rounding midpoint of e4m3, a million random bit patterns and the specials."""
    R = orc.ref_band()
    if R is None:
        pytest.skip("oracle/_ref/libref_band.so not built (reference tree or nvcc absent)")
    rng = np.random.default_rng(0)
    bits = np.concatenate([
        (np.arange(1 << 16, dtype=np.uint32) << 16),                       # every bf16-exact float
        rng.integers(0, 1 << 32, 1_000_000, dtype=np.uint64).astype(np.uint32),
        np.array([0x7F800000, 0xFF800000, 0x7FC00000, 0xFFC00001, 0x43E00000, 0x43DFFFFF, 0x43E00001,
                  0x3A800000, 0x3A7FFFFF, 0x3A000000, 0x39FFFFFF, 0x00000001, 0x80000001], np.uint32)])
    x = bits.view(np.float32)
    # every midpoint between neighbouring e4m3 values, and one ulp either side
    vals = np.array([orc.lib().orc_e4m3_to_f32(c) for c in range(0x7F)], np.float32)
    mid = ((vals[:-1].astype(np.float64) + vals[1:]) / 2).astype(np.float32)
    x = np.concatenate([x, mid, -mid, np.nextafter(mid, np.float32(np.inf)), np.nextafter(mid, np.float32(-np.inf))])
    want = np.empty(x.size, np.uint8)
    R.ref_band_f32_to_e4m3_n(x.ctypes.data_as(orc.C.c_void_p), x.size, want.ctypes.data_as(orc.C.c_void_p))
    got = np.empty(x.size, np.uint8)
    orc.lib().orc_f32_to_e4m3_n(x.ctypes.data_as(orc.C.c_void_p), orc.I64(x.size), got.ctypes.data_as(orc.C.c_void_p))
    assert np.array_equal(got, want)
    some = x[::97]
    assert all(orc.lib().orc_f32_to_bf16(float(v)) == R.ref_band_f32_to_bf16(float(v)) for v in some[np.isfinite(some)][:20000])
    for v in (-1e9, -88.0, -10.5, -1.0, -1e-8, 0.0, 1e-8, 0.3, 1.0, 17.25, 88.0, 1e9):
        e = np.float32(1) / (np.float32(1) + np.float32(np.exp(-np.float64(np.float32(v)))))
        assert np.float32(R.ref_band_sigmoid(v)).view(np.uint32) == np.float32(e).view(np.uint32)
