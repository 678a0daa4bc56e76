"""logit_rerank over the joined e4m3 LM head on the GPU, through the row table: bit for bit against the
CPU oracle (the reference's statement of the rule: a double-precision chain in ascending k per
candidate, one f32 rounding for code * scale, then its selection sort) and bit for bit against the
reference's own kernel and entry (src/r3d_logit_rerank_e4m3.hip of libr3d, compiled where it lay for
sm_100a into oracle/_ref/libref_rerank.so)."""
import ctypes as C

import numpy as np
import pytest
import torch

import gen
import gpu_util as gu
from libr3d_b200 import abi, ops
from libr3d_b200.plugin import ArgPack, planes_blob, tensor_desc
from oracle import oracle as orc

pytestmark = pytest.mark.gpu

SDT = {0: abi.RAD_BF16, 1: abi.RAD_F16, 2: abi.RAD_F32}


def _case(seed, M, N, K, R, br, sdt, off=0, pads=True, ties=False):
    c = gen.case_logits(seed, M, N, K, br, sdt)
    rng = np.random.default_rng(seed + 1)
    ids = np.stack([rng.choice(N, R, replace=False) for _ in range(M)]).astype(np.int32) + off
    if pads and R >= 4:
        ids[:, 1] = -1                       # an explicit pad
        ids[:, 2] = off - 1                  # below this rank's columns
        ids[:, 3] = off + N                  # past them
    if ties and R >= 6:
        # two candidates with identical head rows tie exactly: the lower id must come first
        c["codes"][ids[0, 5] - off] = c["codes"][ids[0, 4] - off]
        if br == 128 and (ids[0, 5] - off) // 128 != (ids[0, 4] - off) // 128:
            ids[0, 5] = ids[0, 4]
    return c, ids


def _run(c, ids, N, K, off, with_pairs=True, x_f32=False):
    M, R = ids.shape
    blob = np.frombuffer(planes_blob([("codes", abi.RAD_F8E4M3, (1, 1), c["codes"]),
                                      ("scale", SDT[c["sdt"]], (c["br"], 128), c["scale"])]), np.uint8)
    x = gu.dev(orc.bf16_bits_to_f32(c["X"])) if x_f32 else gu.dev(c["X"]).view(torch.bfloat16)
    idx = torch.full((M, R), -7, dtype=torch.int32, device="cuda")
    val = torch.zeros((M, R), dtype=torch.float32, device="cuda")
    pairs = torch.zeros((M, R, 2), dtype=torch.float32, device="cuda") if with_pairs else None
    r = ops.logit_rerank(x, gu.dev(blob), gu.dev(ids), idx, val, pairs, n_vocab=N, n_embd=K, vocab_off=off)
    torch.cuda.synchronize()
    assert r.name == "logit_rerank_e4m3"
    return idx.cpu().numpy(), val.cpu().numpy(), (pairs.cpu().numpy() if with_pairs else None)


@pytest.mark.parametrize("M,N,K,R,br,sdt,off", [(1, 512, 1024, 32, 128, 0, 0), (4, 1000, 5120, 32, 128, 0, 0),
                                               (3, 300, 640, 8, 1, 2, 1000), (16, 2048, 2560, 17, 128, 1, 4096),
                                               (2, 130, 300, 5, 1, 0, 7), (5, 256, 16384, 32, 128, 0, 0)])
def test_logit_rerank_bit_identical_to_oracle(M, N, K, R, br, sdt, off):
    c, ids = _case(31 * M + N + K, M, N, K, R, br, sdt, off, ties=True)
    want_i, want_v, want_p = orc.logit_rerank_e4m3(c["X"], c["codes"], c["scale"], sdt, br, ids, off)
    for x_f32 in (False, True):
        got_i, got_v, got_p = _run(c, ids, N, K, off, x_f32=x_f32)
        assert np.array_equal(got_i, want_i)
        assert np.array_equal(got_v.view(np.uint32), want_v.view(np.uint32))
        assert np.array_equal(got_p.view(np.uint32), want_p.view(np.uint32))
    assert (want_i[:, -1] == -1).all() or R < 4       # the pads sort last


def test_logit_rerank_vocab_size_head():
    """N = 151936, K = 5120, R = 32, M = 8: the drafter's rescoring band at the benchmark's head."""
    N, K, M, R = 151936, 5120, 8, 32
    rng = np.random.default_rng(9)
    codes = rng.integers(0, 256, (N, K), dtype=np.uint8)
    codes[(codes & 0x7F) == 0x7F] &= 0x7E
    scale = gen.f32_to_bf16_bits(np.exp(rng.uniform(-6, -4, ((N + 127) // 128, K // 128))).astype(np.float32))
    X = gen.f32_to_bf16_bits(rng.standard_normal((M, K)).astype(np.float32))
    c = dict(X=X, codes=codes, scale=scale, sdt=0, br=128)
    ids = np.stack([rng.choice(N, R, replace=False) for _ in range(M)]).astype(np.int32)
    want_i, want_v, _ = orc.logit_rerank_e4m3(X, codes, scale, 0, 128, ids, 0)
    got_i, got_v, _ = _run(c, ids, N, K, 0, with_pairs=False)
    assert np.array_equal(got_i, want_i) and np.array_equal(got_v.view(np.uint32), want_v.view(np.uint32))


@pytest.mark.parametrize("M,N,K,R,br,sdt,off", [(4, 1000, 5120, 32, 128, 0, 0), (3, 300, 640, 8, 1, 2, 1000),
                                               (16, 2048, 2560, 17, 128, 1, 4096)])
def test_logit_rerank_against_the_reference_kernel(M, N, K, R, br, sdt, off):
    Rf = orc.ref_rerank()
    if Rf is None:
        pytest.skip("oracle/_ref/libref_rerank.so not present")
    c, ids = _case(77 * M + N + K, M, N, K, R, br, sdt, off, ties=True)
    got_i, got_v, got_p = _run(c, ids, N, K, off)
    blob = planes_blob([("codes", abi.RAD_F8E4M3, (1, 1), c["codes"]), ("scale", SDT[sdt], (br, 128), c["scale"])])
    mem = Rf.ref_rerank_alloc(len(blob))                # managed: the reference entry reads the header on the host
    assert mem
    try:
        C.memmove(mem, blob, len(blob))
        x = gu.dev(c["X"]).view(torch.bfloat16)
        idx = torch.full((M, R), -7, dtype=torch.int32, device="cuda")
        val = torch.zeros((M, R), dtype=torch.float32, device="cuda")
        pairs = torch.zeros((M, R, 2), dtype=torch.float32, device="cuda")
        d = lambda t, dt: tensor_desc(t.data_ptr(), dt, list(t.shape), list(t.stride()))
        pack = ArgPack([d(x, abi.RAD_BF16), tensor_desc(mem, abi.RAD_U8, [len(blob)]), d(gu.dev(ids), abi.RAD_I32),
                        d(idx, abi.RAD_I32), d(val, abi.RAD_F32), d(pairs, abi.RAD_F32)],
                       dict(M=M, R=R, n_vocab=N, n_embd=K, vocab_off=off, dtype="bf16"))
        assert Rf.ref_logit_rerank_e4m3(C.byref(pack.args), None) == 0
        torch.cuda.synchronize()
        assert np.array_equal(got_i, idx.cpu().numpy())
        assert np.array_equal(got_v.view(np.uint32), val.cpu().numpy().view(np.uint32))
        assert np.array_equal(got_p.view(np.uint32), pairs.cpu().numpy().view(np.uint32))
    finally:
        torch.cuda.synchronize()
        Rf.ref_rerank_free(mem)


@pytest.mark.parametrize("nan", [False, True])
def test_logit_rerank_duplicate_ids_and_nan_scores(nan):
    """The same id twice in a row's list (equal value, equal id: the earlier slot is picked first) and, in the
    second case, a head row holding a NaN code: its score is NaN and the selection's comparisons with it are
    all false, which makes the outcome depend on the slot order exactly as the reference's loop does."""
    M, N, K, R = 3, 700, 1280, 16
    c, ids = _case(5, M, N, K, R, 128, 0, 0, pads=True, ties=True)
    ids[:, 9] = ids[:, 6]
    ids[1, 0] = ids[1, 12]
    if nan:
        c["codes"][ids[0, 7], 100] = 0x7F
        c["codes"][ids[2, 0], 3] = 0xFF
    want_i, want_v, want_p = orc.logit_rerank_e4m3(c["X"], c["codes"], c["scale"], 0, 128, ids, 0)
    got_i, got_v, got_p = _run(c, ids, N, K, 0)
    assert np.array_equal(got_i, want_i)
    same = lambda a, b: ((a.view(np.uint32) == b.view(np.uint32)) | (np.isnan(a) & np.isnan(b))).all()
    assert same(got_v, want_v)                                  # a NaN's sign and payload are not part of the contract
    assert np.array_equal(np.ascontiguousarray(got_p[..., 0]).view(np.uint32), np.ascontiguousarray(want_p[..., 0]).view(np.uint32))
    assert same(np.ascontiguousarray(got_p[..., 1]), np.ascontiguousarray(want_p[..., 1]))
    assert np.isnan(want_v).any() == nan
