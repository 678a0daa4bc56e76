"""The all-gather fused into the GEMV epilogue (peer stores over NVLink + flags), on two GPUs:
each rank serves its slab of weight rows and every rank must end up with the unsharded result,
bit for bit, for the packed mxfp4 decode kernel, the LM-head kernel and the copy fallback.
Needs two GPUs; skipped otherwise. Ranks are child processes, one per GPU; a rank leaves only
after its stream is idle."""
import ctypes as C
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _gemm_q(abi, A, AS, B, BS, Y, M, N, K, arm):
    q = abi.R3dGemmQ()
    q.a, q.a_scale, q.b, q.b_scale = A.data_ptr(), AS.data_ptr(), B.data_ptr(), BS.data_ptr()
    q.y = Y.data_ptr() if Y is not None else None
    q.m, q.n, q.k, q.as_cols, q.bs_cols = M, N, K, K // 128, K // 32
    q.a_pitch, q.b_pitch, q.y_pitch, q.as_pitch, q.bs_pitch = K, K // 2, N, K // 128, K // 32
    q.rblk, q.bs_dtype, q.arm = 1, abi.RAD_E8M0, arm
    return q


def _rank(rank, world, port, out):
    import sys
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    import gen
    from libr3d_b200 import abi, ops
    from libr3d_b200.shard import PushGather, slab_of
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    ok = {}
    try:
        P = ops.plugin()
        dev = torch.device("cuda", rank)
        N, K = 1024, 2048
        slab = slab_of(N, world, rank)
        pg = PushGather(P, slot_bytes=16 * world * slab.padded * 4, slots=2)
        st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
        call = 0
        for M, arm in [(1, abi.R3D_ARM_AUTO), (2, abi.R3D_ARM_AUTO), (4, abi.R3D_ARM_AUTO), (3, abi.R3D_ARM_EXACT),
                       (9, abi.R3D_ARM_AUTO), (4, abi.R3D_ARM_AUTO)]:
            case = gen.case_mxfp4(900 + M + 10 * call, M, N, K)
            t = {k: torch.from_numpy(v).to(dev) for k, v in case.items()}
            full = torch.zeros((M, N), dtype=torch.bfloat16, device=dev)
            q = _gemm_q(abi, t["A"], t["AS"], t["B"], t["BS"], full, M, N, K, arm)
            assert P.lib.r3d_b200_gemm_mxfp4a8(C.byref(q), st) == 0           # the unsharded result
            Bl = t["B"][slab.start:slab.start + slab.rows].contiguous()
            BSl = t["BS"][slab.start:slab.start + slab.rows].contiguous()
            scratch = torch.zeros((M, slab.rows), dtype=torch.bfloat16, device=dev)
            ql = _gemm_q(abi, t["A"], t["AS"], Bl, BSl, scratch, M, slab.rows, K, arm)
            slot = call % 2
            assert P.lib.r3d_b200_gemm_mxfp4a8_push(C.byref(ql), pg.ptr, slot, slab.padded, st) == 0
            pg.wait()
            got = pg.buffer(slot, M, slab.padded, torch.bfloat16)[:, :N]
            torch.cuda.synchronize()
            ok[f"gemm M={M} arm={arm}"] = bool(torch.equal(got.view(torch.int16), full.view(torch.int16))) and pg.status() == 0
            call += 1
        # LM head: f32 logits
        for M in (1, 5, 16):
            c = gen.case_logits(70 + M, M, N, K, 128, 0)
            X, codes, scale = (torch.from_numpy(c[k]).to(dev) for k in ("X", "codes", "scale"))

            def lg(codes_, scale_, n_, y_):
                l = abi.R3dLogits()
                l.x, l.codes, l.scale = X.data_ptr(), codes_.data_ptr(), scale_.data_ptr()
                l.y = y_.data_ptr() if y_ is not None else None
                l.m, l.n, l.k, l.br = M, n_, K, 128
                l.scale_dtype, l.y_dtype, l.head_fmt, l.arm = abi.RAD_BF16, abi.RAD_F32, 0, abi.R3D_ARM_AUTO
                l.x_pitch, l.code_pitch, l.y_pitch, l.scale_pitch = K, K, n_, scale_.shape[1]
                return l
            full = torch.zeros((M, N), dtype=torch.float32, device=dev)
            assert P.lib.r3d_b200_logits(C.byref(lg(codes, scale, N, full)), st) == 0
            cl = codes[slab.start:slab.start + slab.rows].contiguous()
            sl = scale[slab.start // 128:(slab.start + slab.rows + 127) // 128].contiguous()
            slot = call % 2
            assert P.lib.r3d_b200_logits_push(C.byref(lg(cl, sl, slab.rows, None)), pg.ptr, slot, slab.padded, st) == 0
            pg.wait()
            got = pg.buffer(slot, M, slab.padded, torch.float32)[:, :N]
            torch.cuda.synchronize()
            ok[f"logits M={M}"] = bool(torch.equal(got.view(torch.int32), full.view(torch.int32))) and pg.status() == 0
            call += 1
        torch.cuda.synchronize()
        dist.barrier()
        pg.close()
    finally:
        out[rank] = ok
        dist.destroy_process_group()


def test_fused_gather_two_gpus_bit_identical_to_unsharded():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_rank, args=(2, _free_port(), out), nprocs=2, join=True)
    res = dict(out)
    assert set(res) == {0, 1}
    for r in (0, 1):
        assert res[r] and all(res[r].values()), res
