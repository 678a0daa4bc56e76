#!/usr/bin/env python
"""bench.py -- decode GEMV throughput of the mxfp4a8 band on B200.

Workload (N = 1 GPU): the 27B-class gate+up projection of the benchmark configuration
"mxfp4 decode GEMV band": K = 5120, N = 27648, M in {1, 2, 4}; e2m1 codes uniform over the 16
codes, one E8M0 scale per 32 of K uniform in [119, 123], activations bf16 N(0,1) quantised by
quant_act_fp8 (e4m3 + f32 scale per 128 of K). One step = the three calls (M = 1, 2, 4), each
over the next of `rot` distinct weight planes so that the stream never comes from L2.

  value      algorithmic GB/s of the whole job, inputs resident in HBM, device-timed
             (a recorded pass = CUDA graph of `rot` steps, replayed; CUDA events)
  e2e        the same metric through the declared-op API with HOST activations: per step the
             pinned-host -> device copy of the activations, three issues, device -> host read
             of the outputs
  roofline   the streaming kernel's algorithmic bytes per launch / its mean launch time
  cpu_baseline  the CPU restatement (oracle/) of the same step on the host cores, bounded sample

N > 1: every rank holds its own 27648-row slab (weak scaling: the sharded layer is G x wider) and
runs the same step; the all-gather of each bf16 output is fused into the GEMV epilogue (peer
stores over NVLink + a bounded device-side wait, --gather push, the default) or done by NCCL after
the kernel (--gather nccl); time = max over ranks.

--workload c5: the column-sharded LM head (strong scaling). --workload all [--cfg C1,..,C5]: every
configuration of the hot path on one GPU, one line each.

The line also carries `per_M` (each M timed alone), `spread` (the K-step region is timed five
times, the median is the value), `rows` (the band's other decode row on the same planes: the
int8-per-32 row the resolver picks by default), `rot_sweep` (2 / 4 / 8 rotating planes) and `c5`
(the sharded LM head, strong scaling, bf16 logits) and, on one GPU, `c4` (the prefill band at
M = 8192 in TFLOP/s against the measured MMA-issue rate).

--impl reference: the reference's arithmetic for this path on the host cores (the CPU
restatement, all cores; the reference has no CPU implementation of this path), same metric and
config; `reference_gpu` adds the reference's own kernels, compiled for sm_100a from where they lie
(oracle/_ref/libref_mxfp4.so), timed on the same GPU.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

K_DIM, N_DIM, MS = 5120, 27648, (1, 2, 4)
METRIC = "decode GEMV GB/s (mxfp4a8 band, M in {1,2,4}, K=5120, N=27648)"


def algo_bytes(M: int, n_rows: int = N_DIM) -> int:
    """codes + E8M0 scales + activation codes and scales + bf16 output"""
    return n_rows * K_DIM // 2 + n_rows * K_DIM // 32 + M * (K_DIM + K_DIM // 128 * 4) + M * n_rows * 2


STEP_BYTES = sum(algo_bytes(m) for m in MS)


class ClockSampler:
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc = index, None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *a):
        self.rows = []
        if self.proc:
            self.proc.terminate()
            try:
                out, _ = self.proc.communicate(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
                out = ""
            self.rows = [l.split(", ") for l in out.strip().splitlines() if l.count(",") >= 8]

    def summary(self) -> dict:
        if not getattr(self, "rows", None):
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        sm = [float(r[1]) for r in self.rows if r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in self.rows for n, v in zip(names, r[5:9]) if v.strip().lower() == "active"})
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": float(self.rows[0][2]) if self.rows else None,
                "power_w_max": max(float(r[3]) for r in self.rows), "samples": len(self.rows),
                "reasons": reasons}


def cpu_step_sample(rows: int, reps: int):
    """The CPU restatement over `rows` weight rows of one plane for M = 1, 2, 4."""
    import gen
    from oracle import oracle as orc
    cases = [gen.case_mxfp4(100 + m, m, rows, K_DIM) for m in MS]
    orc.lib().orc_set_threads(os.cpu_count() or 1)      # a launcher may have exported OMP_NUM_THREADS=1
    orc.gemm_mxfp4a8(**cases[0])
    t0 = time.perf_counter()
    for _ in range(reps):
        for c in cases:
            orc.gemm_mxfp4a8(**c)
    dt = (time.perf_counter() - t0) / reps
    nbytes = sum(algo_bytes(m, rows) for m in MS)
    return nbytes / dt / 1e9, dt, orc.lib().orc_num_threads()


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    rows = 1728            # 1/16 of the plane per step: the whole run stays within minutes
    import gen
    from oracle import oracle as orc
    cases = [gen.case_mxfp4(100 + m, m, rows, K_DIM) for m in MS]
    # rank 0 alone runs this arm, on all host cores (torch.distributed.run exports OMP_NUM_THREADS=1)
    orc.lib().orc_set_threads(os.cpu_count() or 1)
    for _ in range(max(args.warmup, 1)):
        for c in cases:
            orc.gemm_mxfp4a8(**c)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        for c in cases:
            orc.gemm_mxfp4a8(**c)
    dt = time.perf_counter() - t0
    nbytes = sum(algo_bytes(m, rows) for m in MS)
    val = nbytes * args.steps / dt / 1e9
    threads = orc.lib().orc_num_threads()
    sample = f"{rows} of {N_DIM} weight rows per step, M=1,2,4, full K"
    ref_gpu = reference_kernels_on_gpu(args)
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": val, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": "C2 mxfp4a8 decode GEMV, M in {1,2,4}, K=5120, N=27648 per GPU"},
        "cpu_baseline": {"value": val, "unit": "GB/s", "cores": threads, "kind": "port", "sample": sample,
                         "host_threads": threads},
        "e2e": {"value": val, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "reference_gpu": ref_gpu,
    }))


def reference_kernels_on_gpu(args):
    """The reference has no CPU implementation of this path: its implementation is GPU kernels
    (HIP). Where its band file has been compiled for sm_100a from where it lay (oracle/_ref/
    libref_mxfp4.so, through the HIP / rocWMMA stand-ins) and a GPU is present, the same C2 step is
    also timed through the reference's own entries and kernels on this GPU: the row its resolver
    would pick (the int8-per-32 decode row, priority 1200) and its fp32-walk decode row."""
    try:
        import ctypes as C
        import torch
        from oracle import oracle as orc
        if not torch.cuda.is_available():
            return {"unavailable": "no GPU"}
        R = orc.ref_gemm("mxfp4")
        if R is None:
            return {"unavailable": "oracle/_ref/libref_mxfp4.so not built"}
        from libr3d_b200 import abi
        from libr3d_b200.plugin import ArgPack, tensor_desc
        dev = torch.device("cuda", 0)
        torch.cuda.set_device(0)
        g = torch.Generator(device=dev).manual_seed(1234)
        rot = 4
        planes = [(torch.randint(0, 256, (N_DIM, K_DIM // 2), dtype=torch.uint8, device=dev, generator=g),
                   torch.randint(119, 124, (N_DIM, K_DIM // 32), dtype=torch.uint8, device=dev, generator=g))
                  for _ in range(rot)]
        import gen
        out = {}
        for name, entry in (("gemm_nt_q_mxfp4_decode_q8x", R.ref_mxfp4_gemm_nt_q_decode_q8x),
                            ("gemm_nt_q_mxfp4_decode", R.ref_mxfp4_gemm_nt_q_decode)):
            packs, keep = {}, []
            for m in MS:
                c = gen.case_mxfp4(100 + m, m, 128, K_DIM)
                A = torch.from_numpy(c["A"]).to(dev); AS = torch.from_numpy(c["AS"]).to(dev)
                y = torch.zeros((m, N_DIM), dtype=torch.bfloat16, device=dev)
                keep.append((A, AS, y))
                d = lambda t, dt: tensor_desc(t.data_ptr(), dt, list(t.shape))
                for p, (B, BS) in enumerate(planes):
                    packs[m, p] = ArgPack([d(A, abi.RAD_F8E4M3), d(AS, abi.RAD_F32),
                                           tensor_desc(B.data_ptr(), abi.RAD_FP4E2M1, [N_DIM, K_DIM], [K_DIM, 1]),
                                           d(BS, abi.RAD_E8M0), d(y, abi.RAD_BF16), tensor_desc(None, abi.RAD_F32, []),
                                           tensor_desc(None, abi.RAD_BF16, [])],
                                          dict(M=m, N=N_DIM, K=K_DIM, group=32, dtype="mxfp4a8"))

            def step(i):
                for m in MS:
                    rc = entry(C.byref(packs[m, i % rot].args), None)
                    if rc != 0:
                        raise RuntimeError(f"reference row {name} returned {rc}")
            for i in range(rot + 2):                      # first sight of every plane builds its caches
                step(i)
            torch.cuda.synchronize()
            steps = min(max(args.steps, 8), 100)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for i in range(steps):
                step(i)
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1)
            out[name] = {"value": STEP_BYTES * steps / (ms * 1e-3) / 1e9, "unit": "GB/s", "us_per_call": ms * 1e3 / (3 * steps),
                         "steps": steps, "nonzero": float(torch.count_nonzero(keep[-1][2].view(torch.int16))) / keep[-1][2].numel()}
        out["what"] = ("the reference's own entries and kernels (src/r3d_gemm_mxfp4.hip), compiled unmodified for sm_100a "
                       "through oracle/hipstub, timed on this GPU: direct issue, 4 rotating weight planes, CUDA events")
        return out
    except Exception as e:                                 # noqa: BLE001 - the CPU numbers above stand on their own
        return {"unavailable": f"{type(e).__name__}: {e}"}


def run_c5(args):
    """LM-head logits (configuration C5): N = 151936, K = 5120, M in {1, 4, 16}, e4m3 head with a
    bf16 scale per 128x128 block, column-sharded over the ranks (strong scaling: the head is
    split, every rank keeps 1/G of it), f32 logits all-gathered over NCCL. One JSON line with
    per-M times, the per-GPU HBM fraction of the GEMV alone and of GEMV + gather."""
    import numpy as np
    import torch
    import torch.distributed as dist
    import ctypes
    from libr3d_b200 import abi, ops, shard
    from libr3d_b200.plugin import planes_blob
    P = ops.plugin()

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    dev = torch.device("cuda", local)
    NV, K = 151936, 5120
    slab = shard.slab_of(NV, world, rank)
    rows = max(slab.rows, 128)
    g = torch.Generator(device=dev).manual_seed(99 + rank)
    rot = 2 if rows * K > 200e6 else 4
    blobs = []
    for _ in range(rot):
        codes = torch.randint(0, 127, (rows, K), dtype=torch.uint8, device=dev, generator=g)
        scale = (torch.rand(((rows + 127) // 128, K // 128), device=dev, generator=g) * 0.01 + 0.001).to(torch.bfloat16)
        hb = np.frombuffer(planes_blob([("codes", abi.RAD_F8E4M3, (1, 1), np.zeros((rows, K), np.uint8)),
                                        ("scale", abi.RAD_BF16, (128, 128), np.zeros(tuple(scale.shape), np.uint16))]),
                           np.uint8)
        blob = torch.from_numpy(hb.copy()).to(dev)
        hdr = abi.planes_round(blob.numel() - abi.planes_round(rows * K) - abi.planes_round(scale.numel() * 2))
        blob[hdr:hdr + rows * K] = codes.flatten()
        so = hdr + abi.planes_round(rows * K)
        blob[so:so + scale.numel() * 2] = scale.flatten().view(torch.uint8)
        blobs.append(blob)
        del codes
    res = {}
    peak = json.loads((ROOT / "MEASURED_PEAKS.json").read_text())["hbm_gbs"] if (ROOT / "MEASURED_PEAKS.json").exists() else 6650.0
    for M in (1, 4, 16):
        x = torch.randn((M, K), device=dev, generator=g).to(torch.bfloat16)
        y = torch.zeros((M, slab.padded), dtype=torch.float32, device=dev)
        yv = y[:, :rows]
        out_all = torch.empty((world * M, slab.padded), dtype=torch.float32, device=dev)

        if world > 1 and M == 1:
            pg = shard.PushGather(P, slot_bytes=16 * world * slab.padded * 4, slots=2)

        def head(i):
            blob = blobs[i % rot]
            l = abi.R3dLogits()
            l.x, l.y = x.data_ptr(), y.data_ptr()
            l.codes = blob.data_ptr() + hdr
            l.scale = blob.data_ptr() + hdr + abi.planes_round(rows * K)
            l.m, l.n, l.k, l.br = M, rows, K, 128
            l.scale_dtype, l.y_dtype, l.head_fmt, l.arm = abi.RAD_BF16, abi.RAD_F32, 0, abi.R3D_ARM_AUTO
            l.x_pitch, l.code_pitch, l.y_pitch, l.scale_pitch = K, K, slab.padded, K // 128
            return l
        heads = [head(i) for i in range(rot)]

        def step(i, gather=True):
            st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
            if world > 1 and gather:
                # the all-gather fused into the head's epilogue (peer stores + flags)
                assert P.lib.r3d_b200_logits_push(ctypes.byref(heads[i % rot]), pg.ptr, i % 2, slab.padded, st) == 0
                pg.wait(st.value)
            else:
                assert P.lib.r3d_b200_logits(ctypes.byref(heads[i % rot]), st) == 0

        times = {}
        for gather in (False, True):
            for i in range(args.warmup):
                step(i, gather)
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier(); torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for i in range(args.steps):
                step(i, gather)
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1)
            if world > 1:
                t = torch.tensor([ms], device=dev); dist.all_reduce(t, op=dist.ReduceOp.MAX); ms = float(t.item())
            times[gather] = ms / args.steps * 1e3
        wbytes = rows * K + ((rows + 127) // 128) * (K // 128) * 2 + M * K * 2 + M * rows * 4
        res[f"M{M}"] = {"us_gemv": times[False], "us_gemv_gather": times[True],
                        "per_gpu_GBs_gemv": wbytes / times[False] / 1e3,
                        "per_gpu_hbm_frac_gemv": wbytes / times[False] / 1e3 / peak,
                        "job_GBs_with_gather": wbytes * world / times[True] / 1e3}
    if rank == 0:
        print(json.dumps({"metric": "LM-head logits GEMV (e4m3 head, N=151936, K=5120), column-sharded",
                          "n_gpus": world, "scaling": "strong", "steps": args.steps, "warmup": args.warmup,
                          "rows_per_gpu": rows, "peak_GBs": peak, "issue": "r3d_b200_logits / r3d_b200_logits_push per call (host-issued, not a graph)", "gather": "fused into the epilogue: peer stores + flags" if world > 1 else "none",
                          "results": res}))
    if world > 1:
        dist.destroy_process_group()


def run_all(args):
    """Every configuration of the hot path on one GPU, through the C-ABI launch layer with the
    arm left to AUTO: C1 (fp8a8 M=1, 4096x4096), C2 (mxfp4a8 M=1,2,4), C3 (M=16 projections, both
    formats), C4 (prefill M=8192, both formats), C5 (LM head M=1,4,16). Decode shapes rotate
    enough distinct weight planes to exceed L2 and are timed as a replayed CUDA graph; prefill
    calls are timed directly. One JSON line: per configuration us per call, GB/s and fraction of the
    measured HBM peak (decode) or TFLOP/s (prefill)."""
    import ctypes as C
    import numpy as np
    import torch
    from libr3d_b200 import abi, ops
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    P = ops.plugin()
    g = torch.Generator(device=dev).manual_seed(7)
    peak = json.loads((ROOT / "MEASURED_PEAKS.json").read_text())["hbm_gbs"] if (ROOT / "MEASURED_PEAKS.json").exists() else 6650.0

    def timed(calls, reps):
        st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
        for fn in calls:
            fn(st)
        torch.cuda.synchronize()
        graph = None
        if len(calls) > 1:
            s = torch.cuda.Stream()
            s.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(s):
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=s):
                    for fn in calls:
                        fn(C.c_void_p(torch.cuda.current_stream().cuda_stream))
            torch.cuda.current_stream().wait_stream(s)
            for _ in range(3):
                graph.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            if graph is not None:
                graph.replay()
            else:
                calls[0](st)
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1e3 / (reps * len(calls))

    def gemm(kind, M, N, K, rot):
        """kind: mxfp4a8, fp8a8 (the reference's grids: bf16 scale per 128x128, f32 per token and 128 of K)
        or fp8a8/channel (one f32 scale per token, one per output channel: the benchmark's prefill contract)"""
        channel, mx8 = kind == "fp8a8/channel", kind == "mxfp4mx8"
        x = torch.randn((M, K), device=dev, generator=g).to(torch.bfloat16)
        A, AS = ops.quant_act_fp8(x, K if channel else 128)
        acols = 1 if channel else K // 128
        if mx8:
            # timing operands: e4m3 codes as above with an E8M0 byte per 32 columns (the values the
            # OCP-MX quantiser would store for N(0,1) activations lie around 127 - 8 + 1)
            AS = torch.randint(118, 122, (M, K // 32), dtype=torch.uint8, device=dev, generator=g)
            acols = K // 32
        keep, calls = [], []
        for _ in range(rot):
            if kind in ("mxfp4a8", "mxfp4mx8"):
                B = torch.randint(0, 256, (N, K // 2), dtype=torch.uint8, device=dev, generator=g)
                BS = torch.randint(119, 124, (N, K // 32), dtype=torch.uint8, device=dev, generator=g)
            elif channel:
                B = torch.randint(0, 127, (N, K), dtype=torch.uint8, device=dev, generator=g)
                BS = torch.rand((N, 1), device=dev, generator=g) * 0.01 + 0.001
            else:
                B = torch.randint(0, 127, (N, K), dtype=torch.uint8, device=dev, generator=g)
                BS = (torch.rand(((N + 127) // 128, K // 128), device=dev, generator=g) * 0.01 + 0.001).to(torch.bfloat16)
            Y = torch.zeros((M, N), dtype=torch.bfloat16, device=dev)
            q = abi.R3dGemmQ()
            q.a, q.a_scale, q.b, q.b_scale, q.y = A.data_ptr(), AS.data_ptr(), B.data_ptr(), BS.data_ptr(), Y.data_ptr()
            q.m, q.n, q.k, q.as_cols = M, N, K, acols
            q.a_pitch, q.y_pitch, q.as_pitch, q.arm = K, N, acols, abi.R3D_ARM_AUTO
            if kind in ("mxfp4a8", "mxfp4mx8"):
                q.bs_cols, q.rblk, q.bs_dtype, q.b_pitch, q.bs_pitch = K // 32, 1, abi.RAD_E8M0, K // 2, K // 32
                fn = P.lib.r3d_b200_gemm_mxfp4mx8 if mx8 else P.lib.r3d_b200_gemm_mxfp4a8
            elif channel:
                q.bs_cols, q.rblk, q.bs_dtype, q.b_pitch, q.bs_pitch = 1, 1, abi.RAD_F32, K, 1
                fn = P.lib.r3d_b200_gemm_fp8a8
            else:
                q.bs_cols, q.rblk, q.bs_dtype, q.b_pitch, q.bs_pitch = K // 128, 128, abi.RAD_BF16, K, K // 128
                fn = P.lib.r3d_b200_gemm_fp8a8
            keep.append((B, BS, Y, q))
            calls.append(lambda st, q=q, fn=fn: fn(C.byref(q), st))
        wbytes = N * K // 2 + N * K // 32 if kind in ("mxfp4a8", "mxfp4mx8") else N * K + ((N + 127) // 128) * (K // 128) * 2
        return calls, keep, wbytes + M * (K + K // 128 * 4) + M * N * 2

    out = []

    def decode_case(cfg, kind, M, N, K):
        wb = N * K // 2 if kind == "mxfp4a8" else N * K
        rot = max(2, int(400e6 // wb) + 1)
        calls, keep, nbytes = gemm(kind, M, N, K, rot)
        us = timed(calls, max(2, 400 // rot))
        ok = int(torch.count_nonzero(keep[0][2].view(torch.int16))) > 0.9 * M * N
        out.append({"cfg": cfg, "band": kind, "M": M, "N": N, "K": K, "us_per_call": round(us, 2),
                    "GBs": round(nbytes / us / 1e3, 1), "hbm_frac_of_measured": round(nbytes / us / 1e3 / peak, 3),
                    "planes": rot, "nonzero_ok": ok})
        del calls, keep
        torch.cuda.empty_cache()

    want = set(c.strip().upper() for c in args.cfg.split(",")) if args.cfg else {"C1", "C2", "C3", "C4", "C5", "ROWS", "W2A8"}
    if "C1" in want:
        decode_case("C1", "fp8a8", 1, 4096, 4096)
    if "C2" in want:
        for M in (1, 2, 4):
            decode_case("C2", "mxfp4a8", M, 27648, 5120)
    if "C3" in want:
        for kind in ("fp8a8", "mxfp4a8"):
            for (K, N) in ((5120, 6144), (5120, 5120), (5120, 27648), (13824, 5120)):
                decode_case("C3", kind, 16, N, K)
    if "C4" in want:
        MT = args.tokens
        for kind in ("fp8a8/channel", "mxfp4mx8", "fp8a8", "mxfp4a8"):
            for (K, N) in ((5120, 27648), (13824, 5120)):
                calls, keep, _ = gemm(kind, MT, N, K, 1)
                us = timed(calls, 10)
                out.append({"cfg": "C4", "band": kind, "M": MT, "N": N, "K": K, "us_per_call": round(us, 1),
                            "TFLOPs": round(2 * MT * N * K / us / 1e6, 1),
                            "nonzero_ok": int(torch.count_nonzero(keep[0][2].view(torch.int16))) > 0.9 * MT * N})
                del calls, keep
                torch.cuda.empty_cache()
    # C5: e4m3 head with a bf16 scale per 128x128 block, f32 logits
    NV, K = 151936, 5120
    heads = []
    for _ in range(2 if "C5" in want else 0):
        codes = torch.randint(0, 127, (NV, K), dtype=torch.uint8, device=dev, generator=g)
        scale = (torch.rand(((NV + 127) // 128, K // 128), device=dev, generator=g) * 0.01 + 0.001).to(torch.bfloat16)
        heads.append((codes, scale))
    for M in ((1, 4, 16) if "C5" in want else ()):
        x = torch.randn((M, K), device=dev, generator=g).to(torch.bfloat16)
        y = torch.zeros((M, NV), dtype=torch.float32, device=dev)
        ls = []
        for codes, scale in heads:
            l = abi.R3dLogits()
            l.x, l.codes, l.scale, l.y = x.data_ptr(), codes.data_ptr(), scale.data_ptr(), y.data_ptr()
            l.m, l.n, l.k, l.br = M, NV, K, 128
            l.scale_dtype, l.y_dtype, l.head_fmt, l.arm = abi.RAD_BF16, abi.RAD_F32, 0, abi.R3D_ARM_AUTO
            l.x_pitch, l.code_pitch, l.y_pitch, l.scale_pitch = K, K, NV, K // 128
            ls.append(l)
        calls = [lambda st, l=l: P.lib.r3d_b200_logits(C.byref(l), st) for l in ls]
        us = timed(calls, 20)
        nbytes = NV * K + ((NV + 127) // 128) * (K // 128) * 2 + M * K * 2 + M * NV * 4
        out.append({"cfg": "C5", "band": "logits e4m3", "M": M, "N": NV, "K": K, "us_per_call": round(us, 1),
                    "GBs": round(nbytes / us / 1e3, 1), "hbm_frac_of_measured": round(nbytes / us / 1e3 / peak, 3),
                    "planes": 2, "nonzero_ok": int(torch.count_nonzero(y)) > 0.9 * M * NV})
    # C5, mxfp4 head (e2m1 nibbles + one E8M0 byte per 32 columns; not a reference format), f32 logits
    heads4 = []
    for _ in range(2 if "C5" in want else 0):
        heads4.append((torch.randint(0, 256, (NV, K // 2), dtype=torch.uint8, device=dev, generator=g),
                       torch.randint(119, 124, (NV, K // 32), dtype=torch.uint8, device=dev, generator=g)))
    for M in ((1, 4, 16) if "C5" in want else ()):
        x = torch.randn((M, K), device=dev, generator=g).to(torch.bfloat16)
        y = torch.zeros((M, NV), dtype=torch.float32, device=dev)
        ls = []
        for codes, scale in heads4:
            l = abi.R3dLogits()
            l.x, l.codes, l.scale, l.y = x.data_ptr(), codes.data_ptr(), scale.data_ptr(), y.data_ptr()
            l.m, l.n, l.k, l.br = M, NV, K, 1
            l.scale_dtype, l.y_dtype, l.head_fmt, l.arm = abi.RAD_E8M0, abi.RAD_F32, 1, abi.R3D_ARM_AUTO
            l.x_pitch, l.code_pitch, l.y_pitch, l.scale_pitch = K, K // 2, NV, K // 32
            ls.append(l)
        calls = [lambda st, l=l: P.lib.r3d_b200_logits(C.byref(l), st) for l in ls]
        us = timed(calls, 20)
        nbytes = NV * K // 2 + NV * K // 32 + M * K * 2 + M * NV * 4
        out.append({"cfg": "C5", "band": "logits mxfp4", "M": M, "N": NV, "K": K, "us_per_call": round(us, 1),
                    "GBs": round(nbytes / us / 1e3, 1), "hbm_frac_of_measured": round(nbytes / us / 1e3 / peak, 3),
                    "planes": 2, "nonzero_ok": int(torch.count_nonzero(y)) > 0.9 * M * NV})
    del heads4
    if "ROWS" in want:
        # the rows either side of the bands, through their row entries: activation producers at the
        # model's widths and the per-shard top-R over bf16 logits
        def row_case(name, shape, nbytes, issue):
            calls = [lambda st, i=i: issue(i) for i in range(4)]
            us = timed(calls, 50)
            out.append({"cfg": "ROWS", "row": name, "shape": shape, "us_per_call": round(us, 2),
                        "GBs": round(nbytes / us / 1e3, 1)})
        for M in (1, 16):
            n = 5120
            xs = [torch.randn((M, n), device=dev, generator=g).to(torch.bfloat16) for _ in range(4)]
            rs = [torch.randn((M, n), device=dev, generator=g).to(torch.bfloat16) for _ in range(4)]
            w = torch.ones(n, device=dev, dtype=torch.bfloat16)
            q = torch.zeros((M, n), dtype=torch.uint8, device=dev)
            sc = torch.zeros((M, n // 128), dtype=torch.float32, device=dev)
            ob = torch.zeros((M, n), dtype=torch.bfloat16, device=dev)
            row_case("quant_act_fp8_act", f"M={M} n={n}", M * n * 3, lambda i: ops.quant_act_fp8_row(xs[i], q, sc))
            row_case("rmsnorm_quant_fp8 (+residual)", f"M={M} n={n}", M * n * 9,
                     lambda i: ops.rmsnorm_quant_fp8(xs[i], w, q, sc, eps=1e-6, residual=rs[i], out=ob))
            n2 = 13824
            gus = [torch.randn((M, 2 * n2), device=dev, generator=g).to(torch.bfloat16) for _ in range(4)]
            q2 = torch.zeros((M, n2), dtype=torch.uint8, device=dev)
            sc2 = torch.zeros((M, n2 // 128), dtype=torch.float32, device=dev)
            row_case("gated_quant_fp8_act", f"M={M} n={n2}", M * n2 * 5, lambda i: ops.gated_quant_fp8_row(gus[i], q2, sc2))
        for (M, N, R) in ((1, 151936, 32), (16, 151936, 8), (16, 19072, 32)):
            ls = [torch.randn((M, N), device=dev, generator=g).to(torch.bfloat16) for _ in range(4)]
            idx = torch.zeros((M, R), dtype=torch.int32, device=dev)
            val = torch.zeros((M, R), dtype=torch.float32, device=dev)
            pairs = torch.zeros((M, R, 2), dtype=torch.float32, device=dev)
            row_case("rowtopk_bf16", f"M={M} N={N} R={R}", M * N * 2, lambda i: ops.row_topk(ls[i], idx, val, pairs, R=R))
        # gemm_nt_q_gated @ fp8a8: the gate_up projection (2n = 27648 rows, K = 5120) with the gated quantiser
        # closing the call; bytes = the weight stream + operands + codes and scales out
        Kg, Ng = 5120, 27648
        wg = [(torch.randint(0, 127, (Ng, Kg), dtype=torch.uint8, device=dev, generator=g),
               (torch.rand((Ng // 128, Kg // 128), device=dev, generator=g) * 0.01 + 0.001).to(torch.bfloat16)) for _ in range(3)]
        for M in (1, 4, 8, 16):
            xg = torch.randn((M, Kg), device=dev, generator=g).to(torch.bfloat16)
            Ag, ASg = ops.quant_act_fp8(xg, 128)
            qg = torch.zeros((M, Ng // 2), dtype=torch.uint8, device=dev)
            sg = torch.zeros((M, Ng // 2 // 128), dtype=torch.float32, device=dev)
            scr = torch.empty(64 * Ng * 2, dtype=torch.uint8, device=dev)
            calls = [lambda st, i=i: ops.gemm_nt_q_gated(Ag, ASg, wg[i][0], wg[i][1], qg, sg, N=Ng, K=Kg, scratch=scr)
                     for i in range(3)]
            us = timed(calls, 30)
            nbytes = Ng * Kg + (Ng // 128) * (Kg // 128) * 2 + M * (Kg + Kg // 128 * 4) + M * (Ng // 2) + M * (Ng // 2 // 128) * 4
            out.append({"cfg": "ROWS", "row": "gemm_nt_q_gated_fp8a8", "shape": f"M={M} 2n={Ng} K={Kg}",
                        "us_per_call": round(us, 2), "GBs": round(nbytes / us / 1e3, 1),
                        "hbm_frac_of_measured": round(nbytes / us / 1e3 / peak, 3)})
        del wg
        torch.cuda.empty_cache()
        # the candidate rescoring row over the e4m3 head (each candidate reads its own row: 32 x 5120 bytes)
        from libr3d_b200.plugin import planes_blob
        NVr, Kr, R = 151936, 5120, 32
        hc = torch.randint(0, 127, (NVr, Kr), dtype=torch.uint8, generator=torch.Generator().manual_seed(5)).numpy()
        hs = np.full(((NVr + 127) // 128, Kr // 128), 0x3C00, np.uint16)       # f16 1.0
        blob = torch.from_numpy(np.frombuffer(planes_blob([("codes", abi.RAD_F8E4M3, (1, 1), hc),
                                                           ("scale", abi.RAD_F16, (128, 128), hs)]), np.uint8).copy()).to(dev)
        del hc
        for M in (1, 16):
            xs = [torch.randn((M, Kr), device=dev, generator=g).to(torch.bfloat16) for _ in range(4)]
            ids = [torch.randint(0, NVr, (M, R), dtype=torch.int32, device=dev, generator=g) for _ in range(4)]
            idx = torch.zeros((M, R), dtype=torch.int32, device=dev)
            val = torch.zeros((M, R), dtype=torch.float32, device=dev)
            row_case("logit_rerank_e4m3", f"M={M} N={NVr} K={Kr} R={R}", M * R * Kr,
                     lambda i: ops.logit_rerank(xs[i], blob, ids[i], idx, val, n_vocab=NVr, n_embd=Kr))
        del blob
        torch.cuda.empty_cache()
    if "W2A8" in want:
        # the draft head's 2-bit decode band (N = 248320 rows x K = 5120: 318 MB of codes a plane, two planes;
        # --w2-rows shrinks N for a profiler capture)
        from libr3d_b200.plugin import planes_blob
        Nw, Kw = args.w2_rows, 5120
        G = Kw // 128
        sc16 = np.full((Nw, G), 0x1E00, np.uint16)
        zp8 = np.ones((Nw, G), np.uint8)
        wblob = torch.from_numpy(np.frombuffer(planes_blob([("scale", abi.RAD_F16, (1, 128), sc16),
                                                            ("zero", abi.RAD_U8, (1, 128), zp8, G)]), np.uint8).copy()).to(dev)
        wb = [torch.randint(0, 256, (Nw, Kw // 4), dtype=torch.uint8, device=dev, generator=g) for _ in range(2)]
        for M in (1, 2, 4, 8, 16):
            a8 = torch.randint(-127, 128, (M, Kw), dtype=torch.int8, device=dev, generator=g)
            asc = torch.full((M,), 0.01, dtype=torch.float32, device=dev)
            asum = torch.zeros((G, 16), dtype=torch.float32, device=dev)
            asum[:, :M] = a8.view(M, G, 128).to(torch.float32).sum(-1).T
            yw = torch.zeros((M, Nw), dtype=torch.bfloat16, device=dev)
            calls = [lambda st, i=i: ops.gemm_w2a8(a8, asc, wb[i], wblob, yw, asum, N=Nw, K=Kw) for i in range(2)]
            us = timed(calls, 10)
            nbytes = Nw * Kw // 4 + Nw * G * 3 + M * Kw + M * Nw * 2
            out.append({"cfg": "W2A8", "row": "gemm_nt_q_w2a8_decode", "shape": f"M={M} N={Nw} K={Kw}",
                        "us_per_call": round(us, 2), "GBs": round(nbytes / us / 1e3, 1),
                        "hbm_frac_of_measured": round(nbytes / us / 1e3 / peak, 3)})
        del wb, wblob
        torch.cuda.empty_cache()
    for r in out:
        sys.stderr.write(json.dumps(r) + "\n")
    print(json.dumps({"workload": "all", "n_gpus": 1, "peak_GBs": peak, "peak_source": "measured", "timed_as":
                      "CUDA graph replay over rotating weight planes (decode), direct calls (prefill)",
                      "status": int(P.lib.r3d_b200_stream_status()), "results": out}))


def _peak():
    pk = ROOT / "MEASURED_PEAKS.json"
    if pk.exists():
        peaks = json.loads(pk.read_text())
        if "hbm_gbs" in peaks:
            return float(peaks["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def _record(fn, n: int):
    """Record n calls of fn(i) once (a CUDA graph: the engine's recorded pass) and return the graph."""
    import torch
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=s):
            for i in range(n):
                fn(i)
    torch.cuda.current_stream().wait_stream(s)
    return graph


def _timed(run, regions: int, fence):
    """`regions` device-timed repetitions of run(); returns the list of milliseconds."""
    import torch
    out = []
    for _ in range(regions):
        fence()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        run()
        e1.record()
        fence()
        out.append(e0.elapsed_time(e1))
    return out


def mma_peak(P, kind: int) -> float:
    """TFLOP/s of the MMA-issue kernel (operands resident in shared memory, nothing loaded or stored):
    the measured tensor-pipe rate the prefill fractions divide by. kind 0 e4m3 x e4m3, 1 block-scaled
    e2m1 x e4m3."""
    import torch
    iters = 4000
    vals = []
    for rep in range(4):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        flops = P.lib.r3d_b200_mma_peak(kind, iters, None)
        e1.record()
        torch.cuda.synchronize()
        if flops <= 0:
            return float("nan")
        if rep:
            vals.append(flops / (e0.elapsed_time(e1) * 1e-3) / 1e12)
    return statistics.median(vals)


def c4_record(P, dev):
    """The prefill band (configuration C4) as a sub-record: M = 8192 tokens over (K=5120, N=27648) and
    (K=13824, N=5120), fp8 W8A8 with per-channel / per-token f32 scales and mxfp4 weights x mxfp8
    activations; TFLOP/s and the fraction of the measured MMA-issue rate of the same tensor-core kind."""
    import ctypes as C
    import torch
    from libr3d_b200 import abi, ops
    g = torch.Generator(device=dev).manual_seed(4)
    peaks = {"fp8a8/channel": mma_peak(P, 0), "mxfp4mx8": mma_peak(P, 1)}
    M, res = 8192, []
    for kind in ("fp8a8/channel", "mxfp4mx8"):
        for (K, N) in ((5120, 27648), (13824, 5120)):
            x = torch.randn((M, K), device=dev, generator=g).to(torch.bfloat16)
            q = abi.R3dGemmQ()
            if kind == "mxfp4mx8":
                A, _ = ops.quant_act_fp8(x, 128)
                AS = torch.randint(118, 122, (M, K // 32), dtype=torch.uint8, device=dev, generator=g)
                B = torch.randint(0, 256, (N, K // 2), dtype=torch.uint8, device=dev, generator=g)
                BS = torch.randint(119, 124, (N, K // 32), dtype=torch.uint8, device=dev, generator=g)
                q.as_cols, q.as_pitch, q.bs_cols, q.bs_pitch, q.b_pitch = K // 32, K // 32, K // 32, K // 32, K // 2
                q.rblk, q.bs_dtype, fn = 1, abi.RAD_E8M0, P.lib.r3d_b200_gemm_mxfp4mx8
            else:
                A, AS = ops.quant_act_fp8(x, K)
                B = torch.randint(0, 127, (N, K), dtype=torch.uint8, device=dev, generator=g)
                BS = torch.rand((N, 1), device=dev, generator=g) * 0.01 + 0.001
                q.as_cols, q.as_pitch, q.bs_cols, q.bs_pitch, q.b_pitch = 1, 1, 1, 1, K
                q.rblk, q.bs_dtype, fn = 1, abi.RAD_F32, P.lib.r3d_b200_gemm_fp8a8
            Y = torch.zeros((M, N), dtype=torch.bfloat16, device=dev)
            q.a, q.a_scale, q.b, q.b_scale, q.y = A.data_ptr(), AS.data_ptr(), B.data_ptr(), BS.data_ptr(), Y.data_ptr()
            q.m, q.n, q.k, q.a_pitch, q.y_pitch, q.arm = M, N, K, K, N, abi.R3D_ARM_AUTO
            for _ in range(2):
                assert fn(C.byref(q), None) == 0
            torch.cuda.synchronize()
            ts = []
            for _ in range(3):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for _ in range(5):
                    fn(C.byref(q), None)
                e1.record()
                torch.cuda.synchronize()
                ts.append(e0.elapsed_time(e1) / 5)
            ms = statistics.median(ts)
            tf = 2.0 * M * N * K / (ms * 1e-3) / 1e12
            ok = int(torch.count_nonzero(Y.view(torch.int16))) > 0.9 * M * N
            res.append({"contract": kind, "M": M, "N": N, "K": K, "ms_per_call": round(ms, 4), "TFLOPs": round(tf, 1),
                        "frac_of_measured_mma_rate": round(tf / peaks[kind], 3), "frac_of_nominal_dense_fp8": round(tf / 4500.0, 3),
                        "nonzero_ok": ok})
            del x, A, AS, B, BS, Y
            torch.cuda.empty_cache()
    return {"workload": "C4 prefill, M=8192 (weights and activations larger than L2 together; 5 calls per region, median of 3)",
            "mma_issue_rate_TFLOPs": {k: round(v, 1) for k, v in peaks.items()},
            "mma_issue_rate_how": "r3d_b200_mma_peak: every CTA pair issues 16000 cta_group::2 MMAs from resident shared-memory tiles, CUDA events",
            "results": res, "status": int(P.lib.r3d_b200_stream_status())}


def c5_record(args, P, dev, world: int, rank: int, peak: float):
    """The sharded LM head (configuration C5) as a sub-record: N = 151936, K = 5120, M in {1, 4, 16},
    e4m3 head with a bf16 scale per 128x128 block, column slabs over the ranks (strong scaling),
    bf16 logits; per M the time of the head alone and with the all-gather of the logits fused into
    its epilogue, and the per-GPU HBM fraction."""
    import ctypes
    import torch
    import torch.distributed as dist
    from libr3d_b200 import abi, shard
    NV, K = 151936, 5120
    slab = shard.slab_of(NV, world, rank)
    rows = max(slab.rows, 128)
    g = torch.Generator(device=dev).manual_seed(99 + rank)
    rot = 2 if rows * K > 200e6 else 4
    heads = []
    for _ in range(rot):
        codes = torch.randint(0, 127, (rows, K), dtype=torch.uint8, device=dev, generator=g)
        scale = (torch.rand(((rows + 127) // 128, K // 128), device=dev, generator=g) * 0.01 + 0.001).to(torch.bfloat16)
        heads.append((codes, scale))
    pg = shard.PushGather(P, slot_bytes=16 * world * slab.padded * 2, slots=2) if world > 1 else None
    res = {}
    steps = 40
    for M in (1, 4, 16):
        x = torch.randn((M, K), device=dev, generator=g).to(torch.bfloat16)
        y = torch.zeros((M, slab.padded), dtype=torch.bfloat16, device=dev)
        ls = []
        for codes, scale in heads:
            l = abi.R3dLogits()
            l.x, l.y, l.codes, l.scale = x.data_ptr(), y.data_ptr(), codes.data_ptr(), scale.data_ptr()
            l.m, l.n, l.k, l.br = M, rows, K, 128
            l.scale_dtype, l.y_dtype, l.head_fmt, l.arm = abi.RAD_BF16, abi.RAD_BF16, 0, abi.R3D_ARM_AUTO
            l.x_pitch, l.code_pitch, l.y_pitch, l.scale_pitch = K, K, slab.padded, K // 128
            ls.append(l)

        def step(i, gather):
            st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
            if pg is not None and gather:
                assert P.lib.r3d_b200_logits_push(ctypes.byref(ls[i % rot]), pg.ptr, i % 2, slab.padded, st) == 0
                pg.wait(st.value)
            else:
                assert P.lib.r3d_b200_logits(ctypes.byref(ls[i % rot]), st) == 0

        times = {}
        for gather in ((False, True) if pg is not None else (False,)):
            for i in range(4):
                step(i, gather)
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier(); torch.cuda.synchronize()
            # a recorded pass of `rot` steps (rot is even: heads and gather slots repeat with it), replayed
            graph = _record(lambda i, gather=gather: step(i, gather), rot)
            graph.replay()
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier(); torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(steps // rot):
                graph.replay()
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1)
            if world > 1:
                t = torch.tensor([ms], device=dev); dist.all_reduce(t, op=dist.ReduceOp.MAX); ms = float(t.item())
            times[gather] = ms / (steps // rot * rot) * 1e3
            del graph
        wbytes = rows * K + ((rows + 127) // 128) * (K // 128) * 2 + M * K * 2 + M * rows * 2
        r = {"us_head": round(times[False], 2), "per_gpu_GBs": round(wbytes / times[False] / 1e3, 1),
             "per_gpu_hbm_frac": round(wbytes / times[False] / 1e3 / peak, 3)}
        if True in times:
            r["us_head_and_gather"] = round(times[True], 2)
        res[f"M{M}"] = r
    if pg is not None:
        pg.close()
    del heads
    torch.cuda.empty_cache()
    return {"workload": "C5 LM head, e4m3 codes + bf16 scale per 128x128, N=151936, K=5120, bf16 logits",
            "scaling": "strong", "rows_per_gpu": rows, "planes": rot, "steps": steps,
            "issue": "r3d_b200_logits / r3d_b200_logits_push (+ gather wait) recorded once per pass of `planes` steps and "
                     "replayed (CUDA graph), CUDA events, max over ranks",
            "gather": "fused into the head's epilogue: peer stores over NVLink + flags" if world > 1 else "none (one GPU)",
            "results": res}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=400)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--rot", type=int, default=8, help="distinct weight planes cycled (footprint > L2)")
    ap.add_argument("--row", default="gemm_nt_q_mxfp4_decode")
    ap.add_argument("--regions", type=int, default=5, help="how many times the K-step region is timed (median reported)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU-baseline leg")
    ap.add_argument("--no-sub", action="store_true", help="skip the sub-records (other row, plane sweep, C5)")
    ap.add_argument("--cfg", default="", help="--workload all: comma list of configurations to run (C1..C5, ROWS, W2A8), default all")
    ap.add_argument("--tokens", type=int, default=8192, help="--workload all: M of the prefill configuration C4")
    ap.add_argument("--w2-rows", type=int, default=248320, help="--workload all --cfg W2A8: rows of the 2-bit draft head")
    ap.add_argument("--gather", default="push", choices=["push", "nccl"],
                    help="N > 1: all-gather fused into the GEMV epilogue (push) or NCCL after it")
    ap.add_argument("--workload", default="c2", help="c2 (default, the headline), c5 (sharded LM head) or all (every configuration, one GPU)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        return run_reference(args)
    if args.workload == "c5":
        return run_c5(args)
    if args.workload == "all":
        return run_all(args)

    import torch
    import torch.distributed as dist
    from libr3d_b200 import ops, shard

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    dev = torch.device("cuda", local)
    P = ops.plugin()
    rot = max(args.rot, 1)
    peak, which = _peak()
    OTHER = "gemm_nt_q_mxfp4_decode_q8x" if args.row == "gemm_nt_q_mxfp4_decode" else "gemm_nt_q_mxfp4_decode"

    g = torch.Generator(device=dev).manual_seed(1234 + rank)
    planes = [(torch.randint(0, 256, (N_DIM, K_DIM // 2), dtype=torch.uint8, device=dev, generator=g),
               torch.randint(119, 124, (N_DIM, K_DIM // 32), dtype=torch.uint8, device=dev, generator=g))
              for _ in range(rot)]
    acts, outs, ops_ = {}, {}, {}
    for m in MS:
        x = torch.randn((m, K_DIM), device=dev, generator=g).to(torch.bfloat16)
        acts[m] = ops.quant_act_fp8(x, 128)
        outs[m] = torch.zeros((m, N_DIM), dtype=torch.bfloat16, device=dev)
        for row in (args.row, OTHER):
            for p in range(rot):
                ops_[row, m, p] = ops.BoundGemm(acts[m][0], acts[m][1], planes[p][0], planes[p][1], outs[m],
                                                dtype="mxfp4a8", N=N_DIM, K=K_DIM, row=row)
    gathered = {m: torch.empty((world * m, N_DIM), dtype=torch.bfloat16, device=dev) for m in MS} if world > 1 else None
    push = world > 1 and args.gather == "push"
    gather_note = ""
    pg = None
    if push:
        # the all-gather fused into the GEMV epilogue: peer stores over NVLink + flags, two slots.
        # Every rank must get its peer mappings; if one cannot, all ranks take the NCCL form.
        err = ""
        try:
            pg = shard.PushGather(P, slot_bytes=max(MS) * world * N_DIM * 2, slots=2)
        except Exception as e:                                  # noqa: BLE001 - reported in the JSON line
            err = f"{type(e).__name__}: {e}"
        okt = torch.tensor([1 if pg is not None else 0], device=dev)
        dist.all_reduce(okt, op=dist.ReduceOp.MIN)
        if int(okt.item()) == 0:
            push, gather_note = False, f"fused gather unavailable ({err or 'a peer failed'}): NCCL all_gather used"
            if pg is not None:
                pg.close()
    if push:
        pushed = {(m, p): shard.PushedGemm(pg, acts[m][0], acts[m][1], planes[p][0], planes[p][1], dtype="mxfp4a8",
                                           M=m, n_local=N_DIM, n_pad=N_DIM, K=K_DIM, scratch=outs[m])
                  for m in MS for p in range(rot)}

    def call(row: str, m: int, i: int, nrot: int = rot):
        if push:
            pushed[m, i % nrot].issue(i % 2)
            return
        ops_[row, m, i % nrot].issue()
        if world > 1:
            dist.all_gather_into_tensor(gathered[m], outs[m])

    def step(i: int, row: str = args.row, nrot: int = rot):
        for m in MS:
            call(row, m, i, nrot)

    def fence():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    for i in range(args.warmup):
        step(i)
    fence()
    probe = pushed[4, (args.warmup - 1) % rot].result((args.warmup - 1) % 2) if push else outs[4]
    assert int(torch.count_nonzero(probe.view(torch.int16))) > 0.9 * probe.numel()
    recordable = world == 1 or push

    def region_runner(row: str, nrot: int, steps: int):
        """run() issues exactly `steps` steps: replays of a recorded pass of nrot steps + the remainder"""
        if not recordable:
            return (lambda: [step(i, row, nrot) for i in range(steps)]), 0
        for i in range(nrot):                            # a row's first calls may build its scratch: not inside a recording
            step(i, row, nrot)
        torch.cuda.synchronize()
        lc = P.lib.r3d_b200_launch_count()
        graph = _record(lambda i: step(i, row, nrot), nrot)
        per_replay = P.lib.r3d_b200_launch_count() - lc
        replays, rem = divmod(steps, nrot)
        lc = P.lib.r3d_b200_launch_count()
        graph_rem = _record(lambda i: step(i, row, nrot), rem) if rem else None      # the last, shorter pass
        per_rem = P.lib.r3d_b200_launch_count() - lc
        for _ in range(3):
            graph.replay()
        if graph_rem is not None:
            graph_rem.replay()

        def run():
            for _ in range(replays):
                graph.replay()
            if graph_rem is not None:
                graph_rem.replay()
        run.keep = (graph, graph_rem)
        return run, per_replay * replays + per_rem

    # ---- device-timed region: exactly `steps` steps, timed `regions` times; the median is the value
    run_main, graph_launches = region_runner(args.row, rot, args.steps)
    fence()
    l0 = P.lib.r3d_b200_launch_count()
    with ClockSampler(local) as clk:
        time.sleep(0.25)
        ms_list = _timed(run_main, max(args.regions, 1), fence)
        time.sleep(0.25)
    direct_launches = (P.lib.r3d_b200_launch_count() - l0) // max(args.regions, 1)
    launches = graph_launches + direct_launches
    if world > 1:
        t = torch.tensor(ms_list, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_list = [float(v) for v in t.tolist()]
    ms = statistics.median(ms_list)
    value = STEP_BYTES * args.steps * world / (ms * 1e-3) / 1e9

    def per_m(row: str, nrot: int):
        """each M alone: a recorded pass of nrot calls over the rotating planes, median of 3 regions"""
        out = {}
        for m in MS:
            if recordable:
                call(row, m, 0, nrot)
                torch.cuda.synchronize()
                gph = _record(lambda i, m=m: call(row, m, i, nrot), nrot)
                for _ in range(3):
                    gph.replay()
                reps = max(2, 120 // nrot)
                msl = _timed(lambda: [gph.replay() for _ in range(reps)], 3, fence)
                n_calls = reps * nrot
            else:
                n_calls = 60
                msl = _timed(lambda: [call(row, m, i, nrot) for i in range(n_calls)], 3, fence)
            if world > 1:
                t = torch.tensor(msl, device=dev); dist.all_reduce(t, op=dist.ReduceOp.MAX); msl = [float(v) for v in t.tolist()]
            us = statistics.median(msl) * 1e3 / n_calls
            out[f"M{m}"] = {"us_per_call": round(us, 2), "GBs": round(algo_bytes(m) / us / 1e3, 1),
                            "hbm_frac": round(algo_bytes(m) / us / 1e3 / peak, 3)}
        return out

    def row_value(row: str, nrot: int, steps: int, regions: int):
        run, _ = region_runner(row, nrot, steps)
        msl = _timed(run, regions, fence)
        if world > 1:
            t = torch.tensor(msl, device=dev); dist.all_reduce(t, op=dist.ReduceOp.MAX); msl = [float(v) for v in t.tolist()]
        m_ = statistics.median(msl)
        return STEP_BYTES * steps * world / (m_ * 1e-3) / 1e9, m_ / steps

    per_m_main = per_m(args.row, rot)
    rows_rec, rot_sweep, c5, c4 = None, None, None, None
    if not args.no_sub:
        sub_steps = min(args.steps, 200)
        if not push:
            v_o, ms_o = row_value(OTHER, rot, sub_steps, 3)
            rows_rec = {OTHER: {"value": v_o, "unit": "GB/s", "ms_per_step": ms_o, "steps": sub_steps, "regions": 3,
                                "hbm_frac_per_gpu": v_o / world / peak, "per_M": per_m(OTHER, rot),
                                "what": ("the row the band resolver picks when no lever is set (priority 1200): int8-per-32 "
                                         "activation arm, exact integer dots on tcgen05 kind::mxf4, bit-identical to the reference row"
                                         if OTHER.endswith("_q8x") else "the fp32-walk decode row (priority 1100)")}}
        if world == 1:
            rot_sweep = {}
            for nrot in sorted({2, 4, rot}):
                if nrot <= rot:
                    v_r, _ = row_value(args.row, nrot, sub_steps, 3)
                    rot_sweep[str(nrot)] = {"planes_MB": round(nrot * (N_DIM * K_DIM // 2 + N_DIM * K_DIM // 32) / 1e6),
                                            "value": round(v_r, 1), "hbm_frac": round(v_r / peak, 3)}

    # ---- end to end: host activations in, host outputs back, through the declared ops
    # every step: ONE copy of the packed activations (codes + scales of the three calls) from
    # pinned host memory, three issues, ONE copy of the packed outputs back to pinned host memory.
    # Device and host buffers are doubled (step i uses set i % 2) so that a recorded pass can run
    # the copies of one step beside the kernels of its neighbours; the kernels themselves stay on
    # one stream in step order (the library's activation scratch and the ranks' call counts need it).
    in_bytes = sum(acts[m][0].numel() + acts[m][1].numel() * 4 for m in MS)
    h_in = torch.empty(in_bytes, dtype=torch.uint8).pin_memory()
    d_ins = [torch.empty(in_bytes, dtype=torch.uint8, device=dev) for _ in range(2)]
    d_outs = [torch.empty((sum(MS), N_DIM), dtype=torch.bfloat16, device=dev) for _ in range(2)]
    h_outs = [torch.empty((sum(MS), N_DIM), dtype=torch.bfloat16).pin_memory() for _ in range(2)]
    e2e_ops, e2e_out, off, row_at = {}, {}, 0, 0
    for m in MS:
        na, ns = acts[m][0].numel(), acts[m][1].numel() * 4
        h_in[off:off + na].copy_(acts[m][0].flatten().cpu())
        h_in[off + na:off + na + ns].copy_(acts[m][1].flatten().view(torch.uint8).cpu())
        for bset in range(2):
            a_v = d_ins[bset][off:off + na].view(m, K_DIM)
            s_v = d_ins[bset][off + na:off + na + ns].view(torch.float32).view(m, K_DIM // 128)
            e2e_out[m, bset] = d_outs[bset][row_at:row_at + m]
            for p in range(rot):
                e2e_ops[m, p, bset] = (shard.PushedGemm(pg, a_v, s_v, planes[p][0], planes[p][1], dtype="mxfp4a8", M=m,
                                                        n_local=N_DIM, n_pad=N_DIM, K=K_DIM, scratch=e2e_out[m, bset]) if push else
                                       ops.BoundGemm(a_v, s_v, planes[p][0], planes[p][1], e2e_out[m, bset],
                                                     dtype="mxfp4a8", N=N_DIM, K=K_DIM, row=args.row))
        off += na + ns
        row_at += m
    h2d, d2h = in_bytes, h_outs[0].numel() * 2

    def rows_e2e(i: int):
        """the row issues of step i on the current stream (buffer set i % 2, plane i % rot)"""
        bset = i % 2
        if push:
            # every rank ends up with the full [m, world * N] result in its slot; the host reads
            # back this rank's own columns of it (the same bytes per rank as at N = 1)
            for m in MS:
                e2e_ops[m, i % rot, bset].issue(i % 2)
                e2e_out[m, bset].copy_(e2e_ops[m, i % rot, bset].result(i % 2)[:, rank * N_DIM:(rank + 1) * N_DIM])
        else:
            for m in MS:
                e2e_ops[m, i % rot, bset].issue()
            if world > 1:
                for m in MS:
                    dist.all_gather_into_tensor(gathered[m], e2e_out[m, bset])

    def step_e2e_body(i: int):
        """copy in, the row issues, copy out of step i, all on the current stream"""
        d_ins[i % 2].copy_(h_in, non_blocking=True)
        rows_e2e(i)
        h_outs[i % 2].copy_(d_outs[i % 2], non_blocking=True)

    e2e_period = rot if rot % 2 == 0 else 2 * rot          # (plane, buffer set) pairs repeat with this period
    s_k, s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()

    def pass_e2e_body():
        """one pass of e2e_period steps on the current stream (s_k) with the copies forked to s_in and
        s_out: step i's copy-in waits only for step i - 2's rows (its buffer set is free), its rows for
        that copy and for step i - 2's copy-out, its copy-out for its rows"""
        ev_k, ev_out = {}, {}
        s_in.wait_stream(s_k)
        s_out.wait_stream(s_k)
        for i in range(e2e_period):
            bset = i % 2
            with torch.cuda.stream(s_in):
                if i >= 2:
                    s_in.wait_event(ev_k[i - 2])
                d_ins[bset].copy_(h_in, non_blocking=True)
                ev_in = torch.cuda.Event()
                ev_in.record()
            s_k.wait_event(ev_in)
            if i >= 2:
                s_k.wait_event(ev_out[i - 2])
            rows_e2e(i)
            ev_k[i] = torch.cuda.Event()
            ev_k[i].record()
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_k[i])
                h_outs[bset].copy_(d_outs[bset], non_blocking=True)
                ev_out[i] = torch.cuda.Event()
                ev_out[i].record()
        s_k.wait_stream(s_in)
        s_k.wait_stream(s_out)

    # The engine records a pass once and replays it. Two forms are timed. "serial": the copy in, the
    # row issues and the copy out of one step are one recording per (weight plane, buffer set); the
    # host waits for step i before it issues step i + 1. "pipelined": one recording holds a pass of
    # e2e_period steps with the copies forked as above; the host waits once per pass. If recording
    # is not possible (the NCCL-gather form), both are issued directly.
    e2e_graphs, e2e_pass, e2e_how = None, None, "direct issue"
    s_k.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s_k):
        for i in range(2):
            step_e2e_body(i)
        pass_e2e_body()
    torch.cuda.synchronize()
    if recordable:
        try:
            e2e_graphs = []
            with torch.cuda.stream(s_k):
                for i in range(e2e_period):
                    gph = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(gph, stream=s_k):
                        step_e2e_body(i)
                    e2e_graphs.append(gph)
                e2e_pass = torch.cuda.CUDAGraph()
                with torch.cuda.graph(e2e_pass, stream=s_k):
                    pass_e2e_body()
            torch.cuda.synchronize()
            e2e_how = "replay of recordings"
        except Exception as ex:                          # noqa: BLE001 - fall back to direct issue, and say so
            sys.stderr.write(f"bench: end-to-end step not recordable ({type(ex).__name__}: {ex}); issuing directly\n")
            e2e_graphs, e2e_pass = None, None
            torch.cuda.synchronize()

    def run_serial(n: int):
        with torch.cuda.stream(s_k):
            for i in range(n):
                if e2e_graphs is not None:
                    e2e_graphs[i % e2e_period].replay()
                else:
                    step_e2e_body(i)
                s_k.synchronize()                          # the caller reads the step's result

    def run_pipelined(n: int):
        with torch.cuda.stream(s_k):
            for _ in range(n // e2e_period):
                if e2e_pass is not None:
                    e2e_pass.replay()
                else:
                    pass_e2e_body()
                s_k.synchronize()                          # the caller reads the pass's results

    e2e_steps = max(e2e_period, min(args.steps, 200) // e2e_period * e2e_period)
    run_serial(4)
    run_pipelined(e2e_period)

    def e2e_of(run):
        lst = _timed(lambda: run(e2e_steps), 3, fence)
        if world > 1:
            t = torch.tensor(lst, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            lst = [float(v) for v in t.tolist()]
        return STEP_BYTES * e2e_steps * world / (statistics.median(lst) * 1e-3) / 1e9, lst

    e2e_serial, _ = e2e_of(run_serial)
    e2e, ms_e_list = e2e_of(run_pipelined)
    # what the last two steps of the last pass left in host memory == the same calls issued alone
    torch.cuda.synchronize()
    for i in (e2e_period - 2, e2e_period - 1):
        row_at = 0
        for m in MS:
            if push:
                pushed[m, i % rot].issue(i % 2)
                ref = pushed[m, i % rot].result(i % 2)[:, rank * N_DIM:(rank + 1) * N_DIM]
            else:
                ops_[args.row, m, i % rot].issue()
                ref = outs[m]
            torch.cuda.synchronize()
            got = h_outs[i % 2][row_at:row_at + m]
            assert torch.equal(ref.cpu().view(torch.int16), got.view(torch.int16)), f"end-to-end result differs (step {i}, M={m})"
            row_at += m

    if not args.no_sub:
        if pg is not None and push:
            # the C5 record makes its own exchange buffers; release this one's slots first
            pass
        try:
            c5 = c5_record(args, P, dev, world, rank, peak)
        except Exception as ex:                          # noqa: BLE001 - the headline stands without the sub-record
            c5 = {"unavailable": f"{type(ex).__name__}: {ex}"}
        if world == 1:
            try:
                c4 = c4_record(P, dev)
            except Exception as ex:                      # noqa: BLE001
                c4 = {"unavailable": f"{type(ex).__name__}: {ex}"}

    if rank == 0:
        per_launch_s = ms * 1e-3 / (3 * args.steps)
        achieved = (STEP_BYTES / 3) / per_launch_s / 1e9
        traffic = None
        tf = ROOT / "profiles" / "traffic.json"
        if tf.exists():
            tj = json.loads(tf.read_text())
            traffic = tj.get("k_tc_q8x_c2_bytes_per_call" if args.row.endswith("_q8x") else "k_tc_mxf4_c2_bytes_per_call")
        vals = [STEP_BYTES * args.steps * world / (m_ * 1e-3) / 1e9 for m_ in ms_list]
        line = {
            "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "e2m1 x e4m3 -> f32", "data": "synthetic",
            "config": {"workload": "C2 mxfp4a8 decode GEMV, M in {1,2,4}, K=5120, N=27648 per GPU",
                       "row": args.row, "rot_planes": rot,
                       "l2": f"inputs larger than L2: {rot} rotating weight planes, "
                             f"{rot * (N_DIM * K_DIM // 2 + N_DIM * K_DIM // 32) / 1e6:.0f} MB",
                       "timed_as": ("CUDA graph replay of recorded steps" if recordable else "direct issue")
                                   + f"; the {args.steps}-step region timed {len(ms_list)} times, median reported",
                       "parallelism": "1 GPU" if world == 1 else
                                      (f"column slabs x{world}, all-gather fused into the GEMV epilogue (peer stores + flags)"
                                       if push else f"column slabs x{world} + NCCL all_gather per call"
                                       + (f" [{gather_note}]" if gather_note else ""))},
            "spread": {"regions": len(ms_list), "value_min": min(vals), "value_max": max(vals),
                       "rel": (max(vals) - min(vals)) / value},
            "per_M": per_m_main,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "peak_source": which, "traffic": traffic,
                         "kernel": ("k_tc_q8x<MT,WALK,HW,EW> (one per call, after its k_q8x_split)" if args.row.endswith("_q8x")
                                    else "k_tc_mxf4<NP,MT> (one per call, after its k_mxf4_split)"),
                         "bytes_per_launch": STEP_BYTES / 3,
                         "us_per_launch": per_launch_s * 1e6},
            "e2e": {"value": e2e, "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "timed_as": e2e_how + f": a pass of {e2e_period} steps, each step's copy-in and copy-out on side "
                                          "streams beside its neighbours' kernels (two buffer sets), the host waits once per pass",
                    "serial": {"value": e2e_serial, "unit": "GB/s",
                               "timed_as": "copy in, rows, copy out on one stream; the host waits for step i before issuing step i + 1"},
                    "steps": e2e_steps, "regions": len(ms_e_list),
                    "checked": "host results of the last pass bit-equal to the same calls issued alone"},
            "gpu_launches": int(launches),
            "clocks": clk.summary(),
        }
        if rows_rec is not None:
            line["rows"] = rows_rec
        if rot_sweep is not None:
            line["rot_sweep"] = rot_sweep
        if c5 is not None:
            line["c5"] = c5
        if c4 is not None:
            line["c4"] = c4
        if world == 1 and not args.no_cpu:
            v, dt, threads = cpu_step_sample(N_DIM, 3)
            line["cpu_baseline"] = {"value": v, "unit": "GB/s", "cores": threads, "kind": "port",
                                    "sample": f"3 full steps (M=1,2,4 over one 27648x5120 plane), {dt:.2f} s each"}
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
