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


def test_push_epilogues_on_one_gpu_bit_identical_to_unsharded():
    """The pushing epilogues without a second GPU: two rank handles of one process on one device,
    connected by pointer; each "rank" serves its slab on the same stream and stores into both
    gathered buffers. No wait kernel runs (nothing here waits on another kernel): the stream is
    synchronised by the host and both buffers must hold the unsharded result bit for bit, for the
    packed mxfp4 kernel, the copy fallback, the M = 9 tcgen05 kernel, the fp8a8 band and the LM head."""
    import gen
    from libr3d_b200 import abi, ops
    from libr3d_b200.shard import slab_of
    P = ops.plugin()
    dev = torch.device("cuda", 0)
    world, N, K = 2, 1024, 2048
    slabs = [slab_of(N, world, r) for r in range(world)]
    n_pad = slabs[0].padded
    g = [C.c_void_p() for _ in range(world)]
    h = C.create_string_buffer(64)
    slot_bytes = 16 * world * n_pad * 4
    for r in range(world):
        assert P.lib.r3d_b200_gather_create(world, r, slot_bytes, 2, C.byref(g[r]), h) == 0
    for r in range(world):
        for p in range(world):
            if p != r:
                assert P.lib.r3d_b200_gather_connect_ptr(g[r], p, P.lib.r3d_b200_gather_base(g[p])) == 0
    P.lib.r3d_b200_gather_buffer.restype = C.c_void_p

    def gathered(r, slot, M, dtype):
        esz = torch.empty((), dtype=dtype).element_size()
        base = P.lib.r3d_b200_gather_buffer(g[r], slot)
        iface = {"shape": (M * world * n_pad * esz,), "typestr": "|u1", "data": (int(base), False), "version": 3}
        holder = type("_Dev", (), {"__cuda_array_interface__": iface})()
        return torch.as_tensor(holder, device=dev).view(dtype).view(M, world * n_pad)[:, :N]

    call = 0
    try:
        for M, arm in [(1, abi.R3D_ARM_AUTO), (4, abi.R3D_ARM_AUTO), (3, abi.R3D_ARM_EXACT), (9, abi.R3D_ARM_AUTO)]:
            case = gen.case_mxfp4(950 + M + 10 * call, M, N, K)
            t = {k: torch.from_numpy(v).to(dev) for k, v in case.items()}
            full = torch.zeros((M, N), dtype=torch.bfloat16, device=dev)
            q = _gemm_q(abi, t["A"], t["AS"], t["B"], t["BS"], full, M, N, K, arm)
            assert P.lib.r3d_b200_gemm_mxfp4a8(C.byref(q), None) == 0
            slot = call % 2
            keep = []
            for r, sl in enumerate(slabs):
                Bl = t["B"][sl.start:sl.start + sl.rows].contiguous()
                BSl = t["BS"][sl.start:sl.start + sl.rows].contiguous()
                scratch = torch.zeros((M, sl.rows), dtype=torch.bfloat16, device=dev)
                ql = _gemm_q(abi, t["A"], t["AS"], Bl, BSl, scratch, M, sl.rows, K, arm)
                keep.append((Bl, BSl, scratch, ql))
                assert P.lib.r3d_b200_gemm_mxfp4a8_push(C.byref(ql), g[r], slot, n_pad, None) == 0
            torch.cuda.synchronize()
            for r in range(world):
                assert torch.equal(gathered(r, slot, M, torch.bfloat16).view(torch.int16), full.view(torch.int16)), (M, arm, r)
            call += 1
        for M in (2, 16):                                                  # fp8a8 band
            case = gen.case_fp8(960 + M, M, N, K, "ref128")
            t = {k: torch.from_numpy(v).to(dev) for k, v in case.items() if k != "rblk"}

            def fq(B, BS, Y, n):
                q = abi.R3dGemmQ()
                q.a, q.a_scale, q.b, q.b_scale = t["A"].data_ptr(), t["AS"].data_ptr(), B.data_ptr(), BS.data_ptr()
                q.y = Y.data_ptr()
                q.m, q.n, q.k, q.as_cols, q.bs_cols = M, n, K, K // 128, K // 128
                q.a_pitch, q.b_pitch, q.y_pitch, q.as_pitch, q.bs_pitch = K, K, n, K // 128, K // 128
                q.rblk, q.bs_dtype, q.arm = 128, abi.RAD_BF16, abi.R3D_ARM_AUTO
                return q
            full = torch.zeros((M, N), dtype=torch.bfloat16, device=dev)
            assert P.lib.r3d_b200_gemm_fp8a8(C.byref(fq(t["B"], t["BS"], full, N)), None) == 0
            slot = call % 2
            keep = []
            for r, sl in enumerate(slabs):
                Bl = t["B"][sl.start:sl.start + sl.rows].contiguous()
                BSl = t["BS"][sl.start // 128:(sl.start + sl.rows + 127) // 128].contiguous()
                scratch = torch.zeros((M, sl.rows), dtype=torch.bfloat16, device=dev)
                ql = fq(Bl, BSl, scratch, sl.rows)
                keep.append((Bl, BSl, scratch, ql))
                assert P.lib.r3d_b200_gemm_fp8a8_push(C.byref(ql), g[r], slot, n_pad, None) == 0
            torch.cuda.synchronize()
            for r in range(world):
                assert torch.equal(gathered(r, slot, M, torch.bfloat16).view(torch.int16), full.view(torch.int16)), ("fp8a8", M, r)
            call += 1
        for M, ydt, tdt in ((1, abi.RAD_F32, torch.float32), (5, abi.RAD_BF16, torch.bfloat16), (16, abi.RAD_F32, torch.float32)):
            c = gen.case_logits(170 + M, M, N, K, 128, 0)
            X, codes, scale = (torch.from_numpy(c[k]).to(dev) for k in ("X", "codes", "scale"))

            def lg(codes_, scale_, n_, y_):
                l = abi.R3dLogits()
                l.x, l.codes, l.scale = X.data_ptr(), codes_.data_ptr(), scale_.data_ptr()
                l.y = y_.data_ptr() if y_ is not None else None
                l.m, l.n, l.k, l.br = M, n_, K, 128
                l.scale_dtype, l.y_dtype, l.head_fmt, l.arm = abi.RAD_BF16, ydt, 0, abi.R3D_ARM_AUTO
                l.x_pitch, l.code_pitch, l.y_pitch, l.scale_pitch = K, K, n_, scale_.shape[1]
                return l
            full = torch.zeros((M, N), dtype=tdt, device=dev)
            assert P.lib.r3d_b200_logits(C.byref(lg(codes, scale, N, full)), None) == 0
            slot = call % 2
            keep = []
            for r, sl in enumerate(slabs):
                cl = codes[sl.start:sl.start + sl.rows].contiguous()
                scl = scale[sl.start // 128:(sl.start + sl.rows + 127) // 128].contiguous()
                keep.append((cl, scl))
                assert P.lib.r3d_b200_logits_push(C.byref(lg(cl, scl, sl.rows, None)), g[r], slot, n_pad, None) == 0
            torch.cuda.synchronize()
            it = torch.int32 if tdt == torch.float32 else torch.int16
            for r in range(world):
                assert torch.equal(gathered(r, slot, M, tdt).view(it), full.view(it)), ("logits", M, r)
            call += 1
        assert P.lib.r3d_b200_stream_status() == 0
    finally:
        torch.cuda.synchronize()
        for r in range(world):
            P.lib.r3d_b200_gather_destroy(g[r])


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
