"""Writes the golden input/output vectors under tests/golden/ (small .npz files).

The reference's arbiter (radiance libref) is not shipped with it, and its kernels run only on a
GPU (they are HIP sources, compiled for the B200 through stand-in headers by oracle/Makefile and
run beside the oracle in the -m gpu tests), so nothing of the reference itself can be executed in
the GPU-less container these vectors are made in. They are therefore outputs of the CPU
restatement (oracle/) on (a) the reference tools' own seeded fixtures and (b) small draws of the
benchmark distributions. They freeze the oracle: a later
edit that changes any output byte fails tests/test_oracle_gemm.py::test_golden_vectors, and
the GPU tests use the same files where the reference tree is absent.

    python tests/golden/make_golden.py
"""
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent))
sys.path.insert(0, str(HERE.parent.parent))
import gen  # noqa: E402
from oracle import oracle as orc  # noqa: E402


def main():
    # fp8a8: the analytic unit fixture and one draw per scale grid
    c, _ = gen.fixture_fp8_unit(3, 256, 20)
    np.savez_compressed(HERE / "fp8a8_unit.npz", kind="fp8a8", **c,
                        Y=orc.gemm_fp8a8(c["A"], c["AS"], c["B"], c["BS"], 1))
    for grid, (M, N, K) in {"ref128": (5, 200, 384), "row": (8, 72, 256), "channel": (1, 96, 512)}.items():
        c = gen.case_fp8(101, M, N, K, grid)
        np.savez_compressed(HERE / f"fp8a8_{grid}.npz", kind="fp8a8", **c,
                            Y=orc.gemm_fp8a8(c["A"], c["AS"], c["B"], c["BS"], c["rblk"]))
    # mxfp4a8: the probe tool's srand(777) fixture, a benchmark-distribution draw, torture bytes
    c = gen.fixture_probe_m4(3, 512, 40)
    np.savez_compressed(HERE / "mxfp4a8_probe777.npz", kind="mxfp4a8", **c, Y=orc.gemm_mxfp4a8(**c))
    c = gen.case_mxfp4(102, 4, 96, 1024)
    np.savez_compressed(HERE / "mxfp4a8_c2dist.npz", kind="mxfp4a8", **c, Y=orc.gemm_mxfp4a8(**c))
    c = gen.case_mxfp4(103, 2, 64, 512)
    rng = np.random.default_rng(7)
    c["BS"][:] = rng.choice(np.array([0, 1, 127, 254, 255], np.uint8), size=c["BS"].shape,
                            p=[.1, .1, .7, .05, .05])
    c["B"][::3] = 0x7F                                            # codes 7 and 15: +-6
    np.savez_compressed(HERE / "mxfp4a8_torture.npz", kind="mxfp4a8", **c, Y=orc.gemm_mxfp4a8(**c))
    for walk in (0, 1):
        c = gen.case_mxfp4(104 + walk, 4 if walk else 2, 80, 1280)
        np.savez_compressed(HERE / f"mxfp4a8_q8x_walk{walk}.npz", kind="mxfp4a8_q8x", walk=walk, **c,
                            Y=orc.gemm_mxfp4_q8x(c["A"], c["AS"], c["B"], c["BS"], walk))
    # logits: two of the reference unit test's geometries
    for (N, K, M, br, sdt) in [(130, 300, 5, 128, 0), (200, 512, 2, 1, 2)]:
        c = gen.case_logits(105, M, N, K, br, sdt)
        np.savez_compressed(HERE / f"logits_e4m3_N{N}_K{K}_M{M}.npz", kind="logits_e4m3", **c,
                            Y=orc.logits_e4m3(c["X"], c["codes"], c["scale"], sdt, br))


if __name__ == "__main__":
    main()
