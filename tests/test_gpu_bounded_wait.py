"""A device-side wait that nothing satisfies must run out, report through its status word and
leave the context usable: the gather wait of a rank whose peer never pushes."""
import ctypes as C
import time

import numpy as np
import pytest
import torch

import gen
import gpu_util as gu
from libr3d_b200 import abi, ops
from oracle import oracle as orc

pytestmark = pytest.mark.gpu


def test_gather_wait_expires_with_status_and_context_survives():
    P = ops.plugin()
    g = [C.c_void_p(), C.c_void_p()]
    h = C.create_string_buffer(64)
    for r in (0, 1):                                     # two "ranks" of one process, same GPU
        assert P.lib.r3d_b200_gather_create(2, r, 4096, 2, C.byref(g[r]), h) == 0
    assert P.lib.r3d_b200_gather_connect_ptr(g[0], 1, P.lib.r3d_b200_gather_base(g[1])) == 0
    assert P.lib.r3d_b200_gather_connect_ptr(g[1], 0, P.lib.r3d_b200_gather_base(g[0])) == 0
    assert P.lib.r3d_b200_gather_status(g[0]) == 0
    t0 = time.time()
    assert P.lib.r3d_b200_gather_wait(g[0], None) == 0   # rank 1 never waits, so never publishes
    torch.cuda.synchronize()
    dt = time.time() - t0
    assert P.lib.r3d_b200_gather_status(g[0]) == 2       # 1 + the rank that did not arrive
    assert 0.2 < dt < 10.0, dt                           # ~2e9 clocks, not forever
    # the context is intact: a normal call still computes correctly
    case = gen.case_mxfp4(1, 2, 256, 512)
    assert np.array_equal(gu.gemm_launch("mxfp4a8", case, abi.R3D_ARM_EXACT), orc.gemm_mxfp4a8(**case))
    for r in (0, 1):
        P.lib.r3d_b200_gather_destroy(g[r])
