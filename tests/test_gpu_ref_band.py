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
