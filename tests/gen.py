"""Seeded synthetic operands for the quantised-matmul path (numpy, host side).

Two families:
  * the benchmark configurations (value distributions of the 27B-class layer shapes), and
  * re-statements of the reference's own self-generating fixtures, so a case here is the
    case libr3d's tools run: tools/probe_m4_entry.cpp:36-40 (glibc srand(777)/rand()),
    tools/bench_fp8_skinny.cpp:467-509 (xorshift32 seeded 0x13579bdf, unit codes).
"""
from __future__ import annotations

import ctypes
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

from oracle import oracle as orc  # noqa: E402  (tests are the oracle's only importers)


# ------------------------------------------------------------------ small codecs (numpy)
def e4m3_decode_table() -> np.ndarray:
    return np.array([orc.lib().orc_e4m3_to_f32(i) for i in range(256)], np.float32)


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    return orc.f32_to_bf16_bits(x)


def bf16_round(x: np.ndarray) -> np.ndarray:
    return orc.bf16_bits_to_f32(orc.f32_to_bf16_bits(x))


def quant_weights_e4m3_per_row(w: np.ndarray):
    """per-output-channel fp32 scale max|w|/448 and RTNE-saturating e4m3 codes (config C1):
    the reference quantiser's rule with one group spanning the row."""
    return orc.quant_act_fp8(w, group=w.shape[1])


def quant_weights_e4m3_block(w: np.ndarray, rblk: int):
    """bf16 scale per (rblk rows, 128 cols) block: the checkpoint grid of the reference."""
    N, K = w.shape
    nr, nc = (N + rblk - 1) // rblk, K // 128
    pad = nr * rblk - N
    wp = np.pad(np.abs(w), ((0, pad), (0, 0)))
    amax = wp.reshape(nr, rblk, nc, 128).max(axis=(1, 3))
    s = bf16_round((np.maximum(amax, 1e-30) / np.float32(448.0)).astype(np.float32))
    full = np.repeat(np.repeat(s, rblk, axis=0)[:N], 128, axis=1)
    q = orc.encode_e4m3((w / full).astype(np.float32))
    return q, f32_to_bf16_bits(s)


# ------------------------------------------------------------------ benchmark configs
def act_bf16(rng: np.random.Generator, M: int, K: int) -> np.ndarray:
    """bf16 N(0,1) activations, returned as float32 holding bf16-exact values."""
    return bf16_round(rng.standard_normal((M, K), dtype=np.float32))


def case_fp8(seed: int, M: int, N: int, K: int, grid: str = "ref128"):
    """fp8 W8A8. grid: 'ref128' (bf16 scale per 128x128 block, act scale per 128 of K),
    'row' (bf16 scale per row x 128), 'channel' (config C1: fp32 per output channel, fp32
    per token)."""
    rng = np.random.default_rng(seed)
    w = (rng.standard_normal((N, K), dtype=np.float32) * np.float32(0.02))
    x = act_bf16(rng, M, K)
    if grid == "channel":
        B, BS = quant_weights_e4m3_per_row(w)
        A, AS = orc.quant_act_fp8(x, group=K)
        return dict(A=A, AS=AS, B=B, BS=BS.astype(np.float32), rblk=1)
    A, AS = orc.quant_act_fp8(x, group=128)
    rblk = 128 if grid == "ref128" else 1
    B, BS = quant_weights_e4m3_block(w, rblk)
    return dict(A=A, AS=AS, B=B, BS=BS, rblk=rblk)


def case_mxfp4(seed: int, M: int, N: int, K: int, scale_lo: int = 119, scale_hi: int = 123):
    """mxfp4: codes uniform over the 16 e2m1 codes, E8M0 bytes uniform in [lo, hi];
    activations bf16 N(0,1) through quant_act_fp8 (group 128)."""
    rng = np.random.default_rng(seed)
    B = rng.integers(0, 256, size=(N, K // 2), dtype=np.uint8)
    BS = rng.integers(scale_lo, scale_hi + 1, size=(N, K // 32), dtype=np.uint8)
    A, AS = orc.quant_act_fp8(act_bf16(rng, M, K), group=128)
    return dict(A=A, AS=AS, B=B, BS=BS)


def case_mxfp4mx8(seed: int, M: int, N: int, K: int, spread: int = 0):
    """mxfp4 weights as in case_mxfp4; activations bf16 N(0,1) (optionally with per-block magnitudes
    spread over 2^+-spread) through the OCP-MX quantiser of the CPU checker: e4m3 codes A and one
    E8M0 byte per 32 columns AE. Parity unpinned (the reference has no such activation format)."""
    w = case_mxfp4(seed, 1, N, K)
    rng = np.random.default_rng(seed + 7)
    x = act_bf16(rng, M, K)
    if spread:
        x = bf16_round(x * np.exp2(rng.integers(-spread, spread + 1, (M, K // 32))).repeat(32, axis=1).astype(np.float32))
    A, AE = orc.quant_act_mx8(x)
    return dict(A=A, AE=AE, B=w["B"], BS=w["BS"])


def case_logits(seed: int, M: int, N: int, K: int, br: int, sdt: int):
    """LM head in the reference test's distributions (tools/test_logits_e4m3.cpp:55-95):
    random e4m3 bytes (NaN codes excluded here), x uniform(-2,2) in bf16, scales exp(U(-2,2))
    stored as bf16 (sdt 0), f16 (1) or f32 (2)."""
    rng = np.random.default_rng(seed)
    codes = rng.integers(0, 256, size=(N, K), dtype=np.uint8)
    codes[(codes & 0x7F) == 0x7F] &= 0x7E
    x = f32_to_bf16_bits(rng.uniform(-2, 2, size=(M, K)).astype(np.float32))
    srows, scols = (N + br - 1) // br, (K + 127) // 128
    sv = np.exp(rng.uniform(-2, 2, size=(srows, scols))).astype(np.float32)
    if sdt == 0:
        scale = f32_to_bf16_bits(sv)
    elif sdt == 1:
        scale = sv.astype(np.float16).view(np.uint16)
    else:
        scale = sv
    return dict(X=x, codes=codes, scale=scale, sdt=sdt, br=br)


# ------------------------------------------------------------------ reference fixtures
class GlibcRand:
    """glibc srand/rand: the generator behind tools/probe_m4_entry.cpp's fixture."""

    def __init__(self, seed: int):
        self.libc = ctypes.CDLL("libc.so.6")
        self.libc.srand(ctypes.c_uint(seed))

    def draw(self, n: int) -> np.ndarray:
        r = self.libc.rand
        return np.fromiter((r() for _ in range(n)), dtype=np.int64, count=n)


def fixture_probe_m4(M: int, K: int, N: int):
    """tools/probe_m4_entry.cpp:36-40, draw for draw: A = (rand()%224)&0x7e, B = rand() byte,
    BS = 115 + rand()%25, AS = 0.001 + 0.01*(rand()%1000)/1000."""
    g = GlibcRand(777)
    as_cols, bs_cols = (K + 127) // 128, (K + 31) // 32
    A = ((g.draw(M * K) % 224).astype(np.uint8) & 0x7E).reshape(M, K)
    B = (g.draw(N * (K // 2)) & 0xFF).astype(np.uint8).reshape(N, K // 2)
    BS = (115 + g.draw(N * bs_cols) % 25).astype(np.uint8).reshape(N, bs_cols)
    r = g.draw(M * as_cols)
    AS = (np.float32(0.001) + np.float32(0.01) * (r % 1000).astype(np.float32) / np.float32(1000.0))
    return dict(A=A, AS=AS.astype(np.float32).reshape(M, as_cols), B=B, BS=BS)


def xorshift32_stream(n: int, state: int = 0x13579BDF):
    out = np.empty(n, np.uint32)
    s = state
    for i in range(n):
        s ^= (s << 13) & 0xFFFFFFFF
        s ^= s >> 17
        s ^= (s << 5) & 0xFFFFFFFF
        out[i] = s
    return out, s


def fixture_fp8_unit(M: int, K: int, N: int):
    """The analytic mode of tools/bench_fp8_skinny.cpp:475-509, :595-624: activation codes all
    0x38 (1.0), weight row r all kUnitCodes[r % 3] (1.0, 2.0, 3.0), every scale 1.0. Each
    output is then exactly K * (1 + r % 3)."""
    A = np.full((M, K), 0x38, np.uint8)
    B = np.empty((N, K), np.uint8)
    for r in range(N):
        B[r, :] = (0x38, 0x40, 0x44)[r % 3]
    AS = np.ones((M, K // 128), np.float32)
    BS = np.full((N, K // 128), 0x3F80, np.uint16)
    expect = (np.float32(K) * (1 + (np.arange(N) % 3))).astype(np.float32)
    return dict(A=A, AS=AS, B=B, BS=BS, rblk=1), np.broadcast_to(expect, (M, N))
