"""Host-side harness for libr3d_b200.so: loads the plugin the way the radiance loader does
(ABI version check, schema and row enumeration), resolves a band to a row by constraints
and priority, and issues ops through the row's `launch` pointer with hand-built RadArgs.

This is the Python twin of the reference's dlopen tools (tools/rows_dump.cpp,
tools/probe_m4_entry.cpp, tools/bench_gemv_prof.cpp:88-117 of libr3d). It holds no
arithmetic: if the shared object is missing or has no usable device, calls fail loudly.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Iterable

from . import abi

SO_PATH = Path(__file__).resolve().parent / "libr3d_b200.so"

# every symbol include/rad_abi.h and include/r3d_b200.h declare
EXPORTS = [
    "rad_plugin_abi_version", "rad_plugin_info", "rad_kernel_schema_count",
    "rad_kernel_schema_at", "rad_kernel_count", "rad_kernel_at",
    "r3d_rad_gemm_nt_q_fp8", "r3d_rad_gemm_nt_q_fp8_decode", "r3d_rad_gemm_nt_q",
    "r3d_rad_gemm_nt_q_mxfp4_decode", "r3d_rad_gemm_nt_q_mxfp4_decode_q8x",
    "r3d_rad_gemm_nt_q_gated_fp8", "r3d_rad_gemm_nt_q_gated_fp8_scratch", "r3d_b200_gated_quant_fp8",
    "r3d_rad_row_topk_scratch", "r3d_rad_sample_argmax_scratch",
    "r3d_rad_quant_act_fp8", "r3d_rad_gated_quant_fp8", "r3d_rad_rmsnorm_quant_fp8", "r3d_rad_row_topk", "r3d_rad_sample_argmax",
    "r3d_mxfp4_q8x_off", "r3d_rad_logits_gemm_e4m3", "r3d_layout_head", "r3d_relayout_head",
    "r3d_unrelayout_head",
    "r3d_b200_gemm_fp8a8", "r3d_b200_gemm_mxfp4a8", "r3d_b200_gemm_mxfp4a8_q8x",
    "r3d_b200_gemm_mxfp4a8_q8x_static", "r3d_b200_q8x_on_tensor_core", "r3d_b200_gemm_mxfp4mx8",
    "r3d_rad_gemm_nt_q_mx8", "r3d_b200_mma_peak", "r3d_rad_logit_rerank_e4m3", "r3d_b200_forget_head",
    "r3d_rad_gemm_nt_q_w2a8_decode", "r3d_layout_gemm_w2a8", "r3d_relayout_gemm_w2a8", "r3d_unrelayout_gemm_w2a8",
    "r3d_b200_gemm_w2a8",
    "r3d_b200_gemm_fp8a8_gated",
    "r3d_b200_logits", "r3d_b200_quant_act_fp8", "r3d_b200_pick_arm_fp8a8",
    "r3d_b200_pick_arm_mxfp4a8", "r3d_b200_launch_count", "r3d_b200_stream_status",
    "r3d_b200_gather_create", "r3d_b200_gather_connect", "r3d_b200_gather_buffer", "r3d_b200_gather_wait",
    "r3d_b200_gather_status", "r3d_b200_gather_destroy", "r3d_b200_gather_connect_ptr", "r3d_b200_gather_base", "r3d_b200_gemm_mxfp4a8_push",
    "r3d_b200_gemm_fp8a8_push", "r3d_b200_logits_push",
]


@dataclass
class Row:
    name: str
    op: str
    priority: int
    domain: int
    constraints: list[tuple[str, int, int, str | None]]
    launch: int
    has_layout: bool
    has_scratch: bool = False


def _holds(c: tuple[str, int, int, str | None], query: dict[str, Any]) -> bool:
    """One constraint against a band query. A constraint on a key the query does not carry
    does not hold (src/r3d_rows.cpp:1105-1110 of libr3d)."""
    key, op, ival, sval = c
    if key not in query:
        return False
    v = query[key]
    if op == abi.RAD_C_IN:
        return isinstance(v, str) and v in (sval or "").split()
    if not isinstance(v, int):
        return False
    if op == abi.RAD_C_EQ:
        return v == ival
    if op == abi.RAD_C_LE:
        return v <= ival
    if op == abi.RAD_C_GE:
        return v >= ival
    if op == abi.RAD_C_DIV:
        return ival != 0 and v % ival == 0
    return False


class Plugin:
    def __init__(self, path: Path | str = SO_PATH):
        path = Path(path)
        if not path.exists():
            raise FileNotFoundError(
                f"{path} is not built: run `python -m libr3d_b200.build` (nvcc, sm_100a). "
                "There is no fallback implementation.")
        self.lib = C.CDLL(str(path))
        L = self.lib
        L.rad_plugin_abi_version.restype = C.c_uint32
        L.rad_plugin_info.restype = C.POINTER(abi.RadPluginInfo)
        L.rad_kernel_schema_at.restype = C.POINTER(abi.RadOpSchema)
        L.rad_kernel_schema_at.argtypes = [C.c_int]
        L.rad_kernel_at.restype = C.POINTER(abi.RadKernelInfo)
        L.rad_kernel_at.argtypes = [C.c_int]
        L.r3d_mxfp4_q8x_off.restype = C.c_bool
        L.r3d_b200_launch_count.restype = C.c_longlong
        for f in ("r3d_b200_gemm_fp8a8", "r3d_b200_gemm_mxfp4a8", "r3d_b200_gemm_mxfp4mx8"):
            getattr(L, f).argtypes = [C.POINTER(abi.R3dGemmQ), C.c_void_p]
        L.r3d_b200_gemm_mxfp4a8_q8x.argtypes = [C.POINTER(abi.R3dGemmQ), C.c_void_p, C.c_void_p,
                                                C.c_int, C.c_void_p]
        L.r3d_b200_gemm_mxfp4a8_q8x_static.argtypes = [C.POINTER(abi.R3dGemmQ), C.c_int, C.c_void_p]
        L.r3d_b200_q8x_on_tensor_core.argtypes = [C.POINTER(abi.R3dGemmQ)]
        L.r3d_b200_mma_peak.argtypes = [C.c_int, C.c_int, C.c_void_p]
        L.r3d_b200_mma_peak.restype = C.c_double
        L.r3d_b200_logits.argtypes = [C.POINTER(abi.R3dLogits), C.c_void_p]
        L.r3d_rad_gemm_nt_q_gated_fp8_scratch.restype = C.c_int64
        L.r3d_rad_gemm_nt_q_gated_fp8_scratch.argtypes = [C.POINTER(abi.RadArgs)]
        for hook in (L.r3d_rad_row_topk_scratch, L.r3d_rad_sample_argmax_scratch):
            hook.restype = C.c_int64
            hook.argtypes = [C.POINTER(abi.RadArgs)]
        L.r3d_b200_gated_quant_fp8.argtypes = [C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.c_void_p, C.c_int64,
                                               C.c_void_p, C.c_int32, C.c_int64, C.c_int32, C.c_int32, C.c_int32,
                                               C.c_int32, C.c_void_p]
        L.r3d_b200_gather_create.argtypes = [C.c_int, C.c_int, C.c_int64, C.c_int, C.POINTER(C.c_void_p), C.c_char_p]
        L.r3d_b200_gather_connect.argtypes = [C.c_void_p, C.c_char_p]
        L.r3d_b200_gather_buffer.argtypes = [C.c_void_p, C.c_int]
        L.r3d_b200_gather_buffer.restype = C.c_void_p
        L.r3d_b200_gather_wait.argtypes = [C.c_void_p, C.c_void_p]
        L.r3d_b200_gather_status.argtypes = [C.c_void_p]
        L.r3d_b200_gather_destroy.argtypes = [C.c_void_p]
        L.r3d_b200_gather_destroy.restype = None
        L.r3d_b200_gather_connect_ptr.argtypes = [C.c_void_p, C.c_int, C.c_void_p]
        L.r3d_b200_gather_base.argtypes = [C.c_void_p]
        L.r3d_b200_gather_base.restype = C.c_void_p
        for f in ("r3d_b200_gemm_mxfp4a8_push", "r3d_b200_gemm_fp8a8_push"):
            getattr(L, f).argtypes = [C.POINTER(abi.R3dGemmQ), C.c_void_p, C.c_int, C.c_int64, C.c_void_p]
        L.r3d_b200_logits_push.argtypes = [C.POINTER(abi.R3dLogits), C.c_void_p, C.c_int, C.c_int64, C.c_void_p]
        L.r3d_b200_quant_act_fp8.argtypes = [C.c_void_p, C.c_int32, C.c_int64, C.c_void_p,
                                             C.c_int64, C.c_void_p, C.c_int64, C.c_int32,
                                             C.c_int32, C.c_int32, C.c_void_p]
        if L.rad_plugin_abi_version() != abi.RAD_ABI_VERSION:
            raise RuntimeError("plugin ABI version differs from the engine's: refused")
        self._launch_t = C.CFUNCTYPE(C.c_int, C.POINTER(abi.RadArgs), C.c_void_p)

    # ------------------------------------------------------------------ enumeration
    def info(self) -> dict[str, Any]:
        i = self.lib.rad_plugin_info().contents
        return dict(kind=i.kind, name=i.name.decode(), version=i.version.decode(),
                    description=i.description.decode(), targets=i.targets.decode())

    def schemas(self) -> dict[str, dict[str, list]]:
        out = {}
        for k in range(self.lib.rad_kernel_schema_count()):
            s = self.lib.rad_kernel_schema_at(k).contents
            out[s.op.decode()] = dict(
                params=[(s.params[j].name.decode(), s.params[j].type, s.params[j].need)
                        for j in range(s.n_params)],
                operands=[(s.operands[j].name.decode(), s.operands[j].dir, s.operands[j].optional)
                          for j in range(s.n_operands)])
        return out

    def rows(self) -> list[Row]:
        out = []
        for k in range(self.lib.rad_kernel_count()):
            r = self.lib.rad_kernel_at(k).contents
            cons = [(r.constraints[j].key.decode(), r.constraints[j].op, r.constraints[j].ival,
                     r.constraints[j].sval.decode() if r.constraints[j].sval else None)
                    for j in range(r.n_constraints)]
            out.append(Row(r.name.decode(), r.op.decode(), r.priority, r.domain, cons,
                           r.launch or 0, bool(r.layout), bool(r.scratch)))
        return out

    def resolve(self, op: str, query: dict[str, Any]) -> Row | None:
        """The row a band with these parameters lands on: all constraints hold, highest
        priority wins, first declared breaks ties."""
        best = None
        for r in self.rows():
            if r.op != op or not all(_holds(c, query) for c in r.constraints):
                continue
            if best is None or r.priority > best.priority:
                best = r
        return best

    # ------------------------------------------------------------------ issue
    def entry(self, symbol: str):
        f = getattr(self.lib, symbol)
        f.restype = C.c_int
        f.argtypes = [C.POINTER(abi.RadArgs), C.c_void_p]
        return f

    def launch_row(self, row: Row, args: "ArgPack", stream: int = 0) -> int:
        return self._launch_t(row.launch)(C.byref(args.args), C.c_void_p(stream))


def tensor_desc(data_ptr: int | None, dtype: int, shape: Iterable[int],
                stride: Iterable[int] | None = None) -> abi.RadTensor:
    """A RadTensor; strides in elements, row-major when omitted. data_ptr None = absent."""
    shape = list(shape)
    t = abi.RadTensor()
    t.data = data_ptr
    t.dtype = dtype
    t.rank = len(shape)
    if stride is None:
        stride, acc = [0] * len(shape), 1
        for i in range(len(shape) - 1, -1, -1):
            stride[i] = acc
            acc *= shape[i]
    for i, (s, st) in enumerate(zip(shape, stride)):
        t.shape[i] = s
        t.stride[i] = st
    return t


class ArgPack:
    """Owns the ctypes arrays behind one RadArgs so they outlive the call."""

    def __init__(self, tensors: list[abi.RadTensor], params: dict[str, Any],
                 scratch: int | None = None, scratch_bytes: int = 0):
        self.t = (abi.RadTensor * len(tensors))(*tensors)
        plist = []
        self._keep = []
        for k, v in params.items():
            p = abi.RadParam()
            kb = k.encode()
            self._keep.append(kb)
            p.key = kb
            if isinstance(v, str):
                vb = v.encode()
                self._keep.append(vb)
                p.kind, p.sval = abi.RAD_PK_STR, vb
            elif isinstance(v, float):
                p.kind, p.dval = abi.RAD_PK_F64, v
            else:
                p.kind, p.ival = abi.RAD_PK_INT, int(v)
            plist.append(p)
        self.p = (abi.RadParam * max(1, len(plist)))(*plist)
        self.args = abi.RadArgs()
        self.args.t = self.t
        self.args.n_t = len(tensors)
        self.args.p = self.p
        self.args.n_p = len(plist)
        self.args.scratch = scratch
        self.args.scratch_bytes = scratch_bytes


def planes_blob(planes: list[tuple[str, int, tuple[int, int], "Any"]]) -> bytes:
    """Join weight planes into one rad.planes blob (the recipe of tools/bench_w2a8.cpp:84-105
    of libr3d). `planes` = [(role, rad_dtype, (block_rows, block_cols), 2-D numpy array[, logical columns])]."""
    import numpy as np

    n = len(planes)
    head = C.sizeof(abi.RadPlanesHeader) + n * C.sizeof(abi.RadPlanesEntry)
    off = abi.planes_round(head)
    entries, payloads = [], []
    for role, dt, block, arr, *rest in planes:
        arr = np.ascontiguousarray(arr)
        e = abi.RadPlanesEntry()
        e.role = role.encode()
        e.dtype, e.kind = dt, abi.RAD_PLANE_TILED
        e.block[0], e.block[1] = block
        e.rows, e.cols = arr.shape
        if rest:                              # logical columns of a sub-byte plane (u4: two a byte)
            e.cols = rest[0]
        e.row_bytes = arr.strides[0]
        e.offset = off
        entries.append(e)
        payloads.append((off, arr.tobytes()))
        off = abi.planes_round(off + arr.nbytes)
    buf = bytearray(off)
    h = abi.RadPlanesHeader()
    h.magic, h.n_planes, h.bytes = abi.RAD_PLANES_MAGIC, n, off
    buf[:C.sizeof(h)] = bytes(h)
    p = C.sizeof(h)
    for e in entries:
        buf[p:p + C.sizeof(e)] = bytes(e)
        p += C.sizeof(e)
    for o, b in payloads:
        buf[o:o + len(b)] = b
    return bytes(buf)
