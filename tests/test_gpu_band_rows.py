"""The activation-producer rows on the GPU, called through the row table the way the engine would:
quant_act_fp8, gated_quant_fp8 and rmsnorm_quant_fp8 bit for bit against the CPU oracle, and
rmsnorm_quant_fp8 bit for bit against the reference's own kernel (src/r3d_more.hip of libr3d, compiled
where it lay for sm_100a into oracle/_ref/libref_more.so)."""
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


def _bits(t):
    return t.view(torch.int16).cpu().numpy().view(np.uint16)


def _codes_equal(q, want):
    """e4m3 codes equal; a NaN code (0x7f / 0xff) may differ in sign only."""
    nan = (want & 0x7F) == 0x7F
    return np.array_equal(q & 0x7F, want & 0x7F) and np.array_equal(q[~nan], want[~nan])


@pytest.mark.parametrize("rows,n,group,f32", [(1, 5120, 128, False), (7, 1000, 128, False), (3, 200, 0, False),
                                              (4, 512, 512, True)])
def test_quant_act_row(rows, n, group, f32):
    rng = np.random.default_rng(rows * 31 + n)
    x = (rng.standard_normal((rows, n)) * 3).astype(np.float32)
    x[0, :3] = [0.0, 448.0 * 4, -1e-9]
    xb = gen.f32_to_bf16_bits(x)
    xd = gu.dev(x) if f32 else gu.dev(xb).view(torch.bfloat16)
    g = n if group <= 0 else group
    q = torch.zeros((rows, n), dtype=torch.uint8, device="cuda")
    s = torch.zeros((rows, (n + g - 1) // g), dtype=torch.float32, device="cuda")
    r = ops.quant_act_fp8_row(xd, q, s, group=group)
    torch.cuda.synchronize()
    assert r.name == "quant_act_fp8_act"
    want_q, want_s = orc.quant_act_fp8(x if f32 else orc.bf16_bits_to_f32(xb), g)
    assert np.array_equal(s.cpu().numpy().view(np.uint32), want_s.view(np.uint32))
    assert _codes_equal(q.cpu().numpy(), want_q)


@pytest.mark.parametrize("act", [None, "silu", "sigmoid"])
@pytest.mark.parametrize("M,n,group,f32", [(1, 128, 128, False), (5, 300, 128, False), (16, 13824, 128, False),
                                           (3, 256, 128, True)])
def test_gated_quant_row(M, n, group, f32, act):
    rng = np.random.default_rng(M * 1000 + n)
    bits = gen.f32_to_bf16_bits((rng.standard_normal((M, 2 * n)) * 4).astype(np.float32))
    # an f32 plane that holds bf16-exact values must give what the bf16 plane gives
    gd = gu.dev(orc.bf16_bits_to_f32(bits)) if f32 else gu.dev(bits).view(torch.bfloat16)
    q = torch.zeros((M, n), dtype=torch.uint8, device="cuda")
    s = torch.zeros((M, (n + group - 1) // group), dtype=torch.float32, device="cuda")
    ob = torch.zeros((M, n), dtype=torch.bfloat16, device="cuda")
    r = ops.gated_quant_fp8_row(gd, q, s, ob, group=group, act=act)
    torch.cuda.synchronize()
    assert r.name == "gated_quant_fp8_act"
    want_q, want_s, want_ob = orc.gated_quant_fp8(bits, group, act != "sigmoid", want_ob=True)
    assert np.array_equal(s.cpu().numpy().view(np.uint32), want_s.view(np.uint32))
    assert gu.same_bits_or_both_nan(_bits(ob), want_ob).all()
    assert _codes_equal(q.cpu().numpy(), want_q)


def _rms_case(M, n, seed, w_f32):
    rng = np.random.default_rng(seed)
    x = gen.f32_to_bf16_bits((rng.standard_normal((M, n)) * 2).astype(np.float32))
    res = gen.f32_to_bf16_bits((rng.standard_normal((M, n)) * 5).astype(np.float32))
    wv = (1 + 0.2 * rng.standard_normal(n)).astype(np.float32)
    w = wv if w_f32 else gen.f32_to_bf16_bits(wv)
    return x, res, w


def _rms_device(x, res, w, n, group, eps, wadd, out_f32):
    M = x.shape[0]
    xd = gu.dev(x).view(torch.bfloat16)
    rd = gu.dev(res).view(torch.bfloat16) if res is not None else None
    wd = gu.dev(w) if w.dtype == np.float32 else gu.dev(w).view(torch.bfloat16)
    q = torch.zeros((M, n), dtype=torch.uint8, device="cuda")
    s = torch.zeros((M, (n + group - 1) // group), dtype=torch.float32, device="cuda")
    ob = torch.zeros((M, n), dtype=torch.float32 if out_f32 else torch.bfloat16, device="cuda")
    return xd, rd, wd, q, s, ob


@pytest.mark.parametrize("M,n,with_res,w_f32,wadd,out_f32", [
    (1, 5120, False, False, None, False), (4, 5120, True, False, None, False), (3, 300, True, True, 1.0, True),
    (2, 30720, False, False, None, False), (5, 4096, True, False, 1.0, False), (1, 4, False, True, None, True)])
def test_rmsnorm_quant_row_bit_identical_to_oracle(M, n, with_res, w_f32, wadd, out_f32):
    x, res, w = _rms_case(M, n, 9000 + M + n, w_f32)
    if not with_res:
        res = None
    eps = 1e-6
    xd, rd, wd, q, s, ob = _rms_device(x, res, w, n, 128, eps, wadd, out_f32)
    r = ops.rmsnorm_quant_fp8(xd, wd, q, s, eps=eps, residual=rd, out=ob, group=128, wadd=wadd)
    torch.cuda.synchronize()
    assert r.name == "rmsnorm_quant_fp8"
    want = orc.rmsnorm_quant_fp8(x, w, eps, 128, wadd or 0.0, res)
    got_ob = gen.f32_to_bf16_bits(ob.cpu().numpy()) if out_f32 else _bits(ob)
    assert np.array_equal(got_ob, want["ob"])
    assert np.array_equal(s.cpu().numpy().view(np.uint32), want["scale"].view(np.uint32))
    assert np.array_equal(q.cpu().numpy(), want["q"])
    if with_res:
        assert np.array_equal(_bits(rd), want["res"])


def _desc(t, dt):
    return tensor_desc(t.data_ptr() if t is not None else None, dt, list(t.shape) if t is not None else [])


@pytest.mark.parametrize("M,n,with_res", [(1, 5120, False), (4, 5120, True), (3, 300, True), (2, 13824, False)])
def test_rmsnorm_quant_row_against_the_reference_kernel(M, n, with_res):
    R = orc.ref_more()
    if R is None:
        pytest.skip("oracle/_ref/libref_more.so not present")
    x, res, w = _rms_case(M, n, 9100 + M + n, False)
    eps = 1e-6
    xd, rd, wd, q, s, ob = _rms_device(x, res if with_res else None, w, n, 128, eps, None, False)
    ops.rmsnorm_quant_fp8(xd, wd, q, s, eps=eps, residual=rd, out=ob, group=128)
    # the reference's own entry and kernel on fresh copies of the same operands
    xr, rr, wr, qr, sr, obr = _rms_device(x, res if with_res else None, w, n, 128, eps, None, False)
    pack = ArgPack([_desc(xr, abi.RAD_BF16), _desc(rr, abi.RAD_BF16), _desc(wr, abi.RAD_BF16),
                    _desc(qr, abi.RAD_F8E4M3), _desc(sr, abi.RAD_F32), _desc(obr, abi.RAD_BF16)],
                   dict(M=M, n=n, eps=eps, group=128, dtype="bf16"))
    assert R.ref_more_rmsnorm_quant_fp8(C.byref(pack.args), None) == 0
    torch.cuda.synchronize()
    assert np.array_equal(_bits(ob), _bits(obr))
    assert np.array_equal(s.cpu().numpy().view(np.uint32), sr.cpu().numpy().view(np.uint32))
    assert np.array_equal(q.cpu().numpy(), qr.cpu().numpy())
    if with_res:
        assert np.array_equal(_bits(rd), _bits(rr))


@pytest.mark.parametrize("M,N,R,off,with_pairs", [(1, 151936, 32, 0, True), (4, 19072, 8, 132864, True),
                                                   (16, 19072, 1, 19072, False), (3, 8, 32, 5, True),
                                                   (2, 512, 32, 0, False), (5, 1000, 7, 0, True),
                                                   # a second block of eight items; a block whose last warp is partly
                                                   # filled; two full blocks; three passes (more than 4096 survivors)
                                                   (2, 4104, 32, 0, True), (1, 4616, 5, 3, False),
                                                   (2, 8192, 32, 0, False), (1, 600000, 32, 0, True)])
def test_row_topk_row_against_oracle(M, N, R, off, with_pairs):
    """Exact top-R with ties: the values are drawn from few distinct bf16 numbers so every row holds
    many equal candidates, plus +-inf and signed zeros; slots past the row's width are (-1, -inf)."""
    rng = np.random.default_rng(M * 7 + N + R)
    x = gen.f32_to_bf16_bits(np.round(rng.standard_normal((M, N)) * 8).astype(np.float32) / 4)
    x[0, :4] = [0x7F80, 0xFF80, 0x0000, 0x8000]
    x[-1, N - 1] = x[-1].view(np.int16).max()                 # a tie with an earlier column at the row's end
    xd = gu.dev(x).view(torch.bfloat16)
    idx = torch.full((M, R), -7, dtype=torch.int32, device="cuda")
    val = torch.zeros((M, R), dtype=torch.float32, device="cuda")
    pairs = torch.zeros((M, R, 2), dtype=torch.float32, device="cuda") if with_pairs else None
    r = ops.row_topk(xd, idx, val, pairs, R=R, vocab_off=off)
    torch.cuda.synchronize()
    assert r.name == "rowtopk_bf16"
    want_i, want_v = orc.row_topk(x, R, off)
    assert np.array_equal(idx.cpu().numpy(), want_i)
    assert np.array_equal(val.cpu().numpy().view(np.uint32), want_v.view(np.uint32))
    if with_pairs:
        p = pairs.cpu().numpy()
        assert np.array_equal(p[..., 0].copy().view(np.int32), want_i)
        assert np.array_equal(p[..., 1].view(np.uint32), want_v.view(np.uint32))


def test_sharded_row_topk_pairs_merge_to_the_unsharded_answer():
    """What the column-sharded head does with it: each slab reports its top-R with global ids
    (vocab_off = the slab's first column); the top-R of the concatenated pairs is the top-R of the row."""
    M, N, R, G = 4, 4096, 16, 4
    rng = np.random.default_rng(5)
    x = gen.f32_to_bf16_bits(np.round(rng.standard_normal((M, N)) * 16).astype(np.float32) / 8)
    want_i, want_v = orc.row_topk(x, R, 0)
    got_i, got_v = [], []
    for g in range(G):
        sl = np.ascontiguousarray(x[:, g * N // G:(g + 1) * N // G])
        idx = torch.zeros((M, R), dtype=torch.int32, device="cuda")
        val = torch.zeros((M, R), dtype=torch.float32, device="cuda")
        ops.row_topk(gu.dev(sl).view(torch.bfloat16), idx, val, None, R=R, vocab_off=g * N // G)
        torch.cuda.synchronize()
        got_i.append(idx.cpu().numpy()); got_v.append(val.cpu().numpy())
    ci, cv = np.concatenate(got_i, 1), np.concatenate(got_v, 1)
    for m in range(M):
        order = np.lexsort((ci[m], -cv[m]))[:R]                # value descending, then id ascending
        assert np.array_equal(ci[m][order], want_i[m]) and np.array_equal(cv[m][order], want_v[m])


@pytest.mark.parametrize("M,N,R,off", [(1, 151936, 32, 0), (4, 19072, 8, 132864), (3, 8, 32, 5), (5, 1000, 7, 0)])
def test_row_topk_row_against_the_reference_kernel(M, N, R, off):
    """The reference's own row_topk entry and kernel (src/r3d_more.hip, compiled for sm_100a) on the same
    rows, ties included: columns, values and the pairs plane must be identical. The rows are positive:
    in the reference's block reduction a thread that has no candidate left carries (0.0, -1), and its
    comparison lets that pair win against a real candidate whose value is negative, so on rows whose
    picks reach below zero it reports holes where its stated contract (exact top-R) has values. This
    library follows the contract (the oracle test above covers negative rows)."""
    Rf = orc.ref_more()
    if Rf is None:
        pytest.skip("oracle/_ref/libref_more.so not present")
    rng = np.random.default_rng(M * 11 + N + R)
    x = gen.f32_to_bf16_bits(np.round(rng.standard_normal((M, N)) * 8).astype(np.float32) / 4 + 16)
    xd = gu.dev(x).view(torch.bfloat16)
    out = []
    for _ in range(2):
        out.append((torch.full((M, R), -7, dtype=torch.int32, device="cuda"),
                    torch.zeros((M, R), dtype=torch.float32, device="cuda"),
                    torch.zeros((M, R, 2), dtype=torch.float32, device="cuda")))
    ops.row_topk(xd, *out[0], R=R, vocab_off=off)
    pack = ArgPack([_desc(xd, abi.RAD_BF16), _desc(out[1][0], abi.RAD_I32), _desc(out[1][1], abi.RAD_F32),
                    _desc(out[1][2], abi.RAD_F32)], dict(M=M, N=N, R=R, vocab_off=off, dtype="bf16"))
    assert Rf.ref_more_row_topk(C.byref(pack.args), None) == 0
    torch.cuda.synchronize()
    for a, b in zip(out[0], out[1]):
        assert np.array_equal(a.cpu().numpy().view(np.uint32), b.cpu().numpy().view(np.uint32))


@pytest.mark.parametrize("M,nv", [(1, 151936), (16, 151936), (4, 19072), (3, 7), (2, 513)])
def test_sample_argmax_row_against_oracle(M, nv):
    """Greedy over f32 logits with many ties (few distinct values), a row of all -inf and signed zeros;
    it must also be row_topk's first pick on the same values."""
    rng = np.random.default_rng(M + nv)
    lg = (np.round(rng.standard_normal((M, nv)) * 3) / 2).astype(np.float32)
    lg[0, :] = np.minimum(lg[0, :], 2.0)                       # the row's maximum occurs many times
    if M > 1:
        lg[1, :] = -np.inf
    if M > 2:
        lg[2, :] = np.where(rng.random(nv) < 0.5, np.float32(-0.0), np.float32(0.0))
    ld = gu.dev(lg)
    tok = torch.full((M,), -9, dtype=torch.int32, device="cuda")
    r = ops.sample_argmax(ld, tok)
    torch.cuda.synchronize()
    assert r.name == "sample_argmax_f32"
    want = orc.sample_argmax(lg)
    assert np.array_equal(tok.cpu().numpy(), want)
    assert np.array_equal(want, np.argmax(lg, axis=1).astype(np.int32))


def test_greedy_decode_tail_logits_then_argmax():
    """The end of a decode step as the engine issues it: logits_gemm (f32) then sample_argmax, against
    the oracle's logits and the oracle's argmax over them."""
    c = gen.case_logits(77, 4, 1024, 512, 128, 0)
    got = gu.logits_launch(c, abi.R3D_ARM_AUTO)
    ld = gu.dev(got)
    tok = torch.zeros((4,), dtype=torch.int32, device="cuda")
    ops.sample_argmax(ld, tok)
    torch.cuda.synchronize()
    assert np.array_equal(tok.cpu().numpy(), orc.sample_argmax(got))


def test_row_topk_with_the_launch_arena_allocates_nothing_and_agrees():
    """With the arena its scratch hook asks for, the row's first call at a new size leaves the device's free
    memory where it was (the survivor planes live in the arena); without the arena it falls back to planes of
    its own. Both give the same picks."""
    M, N, R = 3, 40000, 32
    rng = np.random.default_rng(12)
    x = gen.f32_to_bf16_bits(rng.standard_normal((M, N)).astype(np.float32))
    xd = gu.dev(x).view(torch.bfloat16)
    outs = []
    for arena in (True, False):
        idx = torch.zeros((M, R), dtype=torch.int32, device="cuda")
        val = torch.zeros((M, R), dtype=torch.float32, device="cuda")
        if arena:
            ops.row_topk(xd, idx, val, None, R=R)                     # the arena itself is created here
            torch.cuda.synchronize()
            free0 = torch.cuda.mem_get_info()[0]
            xs = gu.dev(gen.f32_to_bf16_bits(rng.standard_normal((5, N)).astype(np.float32))).view(torch.bfloat16)
            i5 = torch.zeros((5, R), dtype=torch.int32, device="cuda")
            v5 = torch.zeros((5, R), dtype=torch.float32, device="cuda")
            torch.cuda.synchronize()
            free1 = torch.cuda.mem_get_info()[0]
            ops.row_topk(xs, i5, v5, None, R=R)                        # more survivors than any call before
            torch.cuda.synchronize()
            assert torch.cuda.mem_get_info()[0] == free1 <= free0
        ops.row_topk(xd, idx, val, None, R=R, arena=arena)
        torch.cuda.synchronize()
        outs.append((idx.cpu().numpy(), val.cpu().numpy()))
    want_i, want_v = orc.row_topk(x, R, 0)
    for gi, gv in outs:
        assert np.array_equal(gi, want_i) and np.array_equal(gv.view(np.uint32), want_v.view(np.uint32))
