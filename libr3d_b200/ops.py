"""The ops of the quantised-matmul path as a caller issues them: `gemm_nt_q` and
`logits_gemm`, with device tensors (torch is used for device memory and streams only).

Each call does what the radiance engine does for the op: resolve the band to a row by the
rows' constraints and priorities, then call that row's `launch` with a RadArgs on the
current CUDA stream. Nothing is computed here.
"""
from __future__ import annotations

from typing import Any

import torch

from . import abi
from .plugin import ArgPack, Plugin, Row, tensor_desc

_plugin: Plugin | None = None


def plugin() -> Plugin:
    global _plugin
    if _plugin is None:
        _plugin = Plugin()
    return _plugin


class RowRefused(RuntimeError):
    def __init__(self, row: str, rc: int):
        super().__init__(f"row {row} returned {abi.STATUS_NAMES[rc] if 0 <= rc < 7 else rc}")
        self.rc = rc


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _desc(t: torch.Tensor | None, dtype: int, shape=None, stride=None) -> abi.RadTensor:
    if t is None:
        return tensor_desc(None, dtype, [])
    return tensor_desc(t.data_ptr(), dtype, shape if shape is not None else t.shape,
                       stride if stride is not None else t.stride())


def gemm_nt_q(a: torch.Tensor, a_scale: torch.Tensor, b: torch.Tensor, b_scale: torch.Tensor,
              y: torch.Tensor, *, dtype: str, N: int, K: int, group: int | None = None,
              M_param: int | None = None, row: str | None = None) -> Row:
    """y[M,N] (bf16, given as a uint16/bfloat16 tensor) = a[M,K] @ dequant(b)[N,K]^T.

    a: uint8 e4m3 codes [M,K]; a_scale: float32 [M, K/128]
    dtype "fp8a8":   b uint8 e4m3 codes [N,K]; b_scale bf16 (or f32) [N/128 | N, K/128]
    dtype "mxfp4a8": b uint8 packed e2m1 [N,K/2] (low nibble = even k); b_scale uint8 E8M0 [N,K/32]
    `row` forces a row by name; otherwise the band is resolved like the engine would.
    Returns the row that served the call; raises RowRefused on a nonzero status.
    """
    P = plugin()
    M = y.numel() // N
    if group is None:
        group = 128 if dtype == "fp8a8" else 32
    query: dict[str, Any] = dict(M=M_param if M_param is not None else M, N=N, K=K,
                                 group=group, dtype=dtype)
    if row is None:
        r = P.resolve("gemm_nt_q", query)
        if r is None:
            raise RuntimeError(f"no row serves gemm_nt_q {query}")
    else:
        r = next(x for x in P.rows() if x.name == row)
    if dtype == "fp8a8":
        bdesc = _desc(b, abi.RAD_F8E4M3)
        sdt = abi.RAD_F32 if b_scale.dtype == torch.float32 else abi.RAD_BF16
    else:
        bdesc = _desc(b, abi.RAD_FP4E2M1, shape=[b.shape[0], K], stride=[K, 1])
        sdt = abi.RAD_E8M0
    tensors = [_desc(a, abi.RAD_F8E4M3), _desc(a_scale, abi.RAD_F32), bdesc,
               _desc(b_scale, sdt), _desc(y, abi.RAD_BF16), _desc(None, abi.RAD_F32),
               _desc(None, abi.RAD_BF16)]
    pack = ArgPack(tensors, query)
    rc = P.launch_row(r, pack, _stream())
    if rc != abi.RAD_OK:
        raise RowRefused(r.name, rc)
    return r


def gemm_nt_q_gated(a: torch.Tensor, a_scale: torch.Tensor, b: torch.Tensor, b_scale: torch.Tensor,
                    q: torch.Tensor, scale: torch.Tensor, *, N: int, K: int, act: str = "silu",
                    group: int = 128, out: torch.Tensor | None = None,
                    scratch: torch.Tensor | None = None) -> Row:
    """q[M, N/2] (e4m3 codes), scale[M, N/2/group] (f32) = gated_quant_fp8(a @ dequant(b)^T) for a
    [N = 2n, K] fp8a8 gate_up weight, gate half first; `out` optionally receives the gated product
    (bf16 or f32). `scratch` is the launch arena (default: what the row's scratch hook asks for)."""
    P = plugin()
    n = N // 2
    M = q.numel() // n
    query: dict[str, Any] = dict(M=M, N=N, K=K, group=group, dtype="fp8a8", act=act)
    r = P.resolve("gemm_nt_q_gated", query)
    if r is None:
        raise RuntimeError(f"no row serves gemm_nt_q_gated {query}")
    sdt = abi.RAD_F32 if b_scale.dtype == torch.float32 else abi.RAD_BF16
    odt = abi.RAD_F32 if (out is not None and out.dtype == torch.float32) else abi.RAD_BF16
    tensors = [_desc(a, abi.RAD_F8E4M3), _desc(a_scale, abi.RAD_F32), _desc(b, abi.RAD_F8E4M3),
               _desc(b_scale, sdt), _desc(q, abi.RAD_F8E4M3), _desc(scale, abi.RAD_F32),
               _desc(out, odt), _desc(None, abi.RAD_F32)]
    if scratch is None:
        probe = ArgPack(tensors, query)
        need = int(P.lib.r3d_rad_gemm_nt_q_gated_fp8_scratch(probe.args))
        scratch = torch.empty(need, dtype=torch.uint8, device=a.device)
    pack = ArgPack(tensors, query, scratch=scratch.data_ptr(), scratch_bytes=scratch.numel() * scratch.element_size())
    rc = P.launch_row(r, pack, _stream())
    if rc != abi.RAD_OK:
        raise RowRefused(r.name, rc)
    return r


def logits_gemm(x: torch.Tensor, head_blob: torch.Tensor, logits: torch.Tensor, *, n_vocab: int,
                n_embd: int) -> Row:
    """logits[M, n_vocab] f32 = x[M, n_embd] bf16 @ head^T, head a joined rad.planes blob
    (uint8 device tensor) of e4m3 codes + block scales."""
    P = plugin()
    M = logits.numel() // n_vocab
    query = dict(M=M, n_vocab=n_vocab, n_embd=n_embd, dtype="bf16")
    r = P.resolve("logits_gemm", query)
    if r is None:
        raise RuntimeError(f"no row serves logits_gemm {query}")
    tensors = [_desc(x, abi.RAD_BF16), _desc(head_blob, abi.RAD_U8), _desc(logits, abi.RAD_F32)]
    rc = P.launch_row(r, ArgPack(tensors, query), _stream())
    if rc != abi.RAD_OK:
        raise RowRefused(r.name, rc)
    return r


def gemm_w2a8(a: torch.Tensor, a_scale: torch.Tensor, b: torch.Tensor, bs_blob: torch.Tensor, y: torch.Tensor,
              a_sum: torch.Tensor, *, N: int, K: int, M_param: int | None = None) -> Row:
    """y[M,N] bf16 = a[M,K] (int8, quant_act_i8's step order, f32 scale a row) @ dequant(b)[N,K]^T for the
    draft head's 2-bit weight: b uint8 [N, K/4] (four codes a byte), bs_blob the joined rad.planes blob of
    its f16 scale and u8/u4 zero per (row, 128 of K), a_sum f32 [K/128, mpad] the activation's group sums."""
    P = plugin()
    M = y.numel() // N
    query: dict[str, Any] = dict(M=M_param if M_param is not None else M, N=N, K=K, group=128, dtype="w2a8")
    r = P.resolve("gemm_nt_q", query)
    if r is None:
        raise RuntimeError(f"no row serves gemm_nt_q {query}")
    tensors = [_desc(a, abi.RAD_I8), _desc(a_scale, abi.RAD_F32), _desc(b, abi.RAD_U2, shape=[N, K], stride=[K, 1]),
               _desc(bs_blob, abi.RAD_U8), _desc(y, abi.RAD_BF16), _desc(a_sum, abi.RAD_F32), _desc(None, abi.RAD_BF16)]
    rc = P.launch_row(r, ArgPack(tensors, query), _stream())
    if rc != abi.RAD_OK:
        raise RowRefused(r.name, rc)
    return r


def logit_rerank(x: torch.Tensor, head_blob: torch.Tensor, idx_in: torch.Tensor, idx: torch.Tensor,
                 val: torch.Tensor, pairs: torch.Tensor | None = None, *, n_vocab: int, n_embd: int,
                 vocab_off: int = 0) -> Row:
    """R candidate ids a row (idx_in int32 [M, R], global ids) rescored exactly against the joined e4m3
    head and re-sorted: idx int32 [M, R], val f32 [M, R], optional pairs f32 [M, R, 2] (id bits, value).
    x is bf16 or f32 [M, n_embd]."""
    P = plugin()
    M, R = idx_in.shape
    query = dict(M=M, R=R, n_vocab=n_vocab, n_embd=n_embd, vocab_off=vocab_off, dtype="bf16")
    r = P.resolve("logit_rerank", query)
    if r is None:
        raise RuntimeError(f"no row serves logit_rerank {query}")
    xdt = abi.RAD_F32 if x.dtype == torch.float32 else abi.RAD_BF16
    tensors = [_desc(x, xdt), _desc(head_blob, abi.RAD_U8), _desc(idx_in, abi.RAD_I32), _desc(idx, abi.RAD_I32),
               _desc(val, abi.RAD_F32), _desc(pairs, abi.RAD_F32)]
    rc = P.launch_row(r, ArgPack(tensors, query), _stream())
    if rc != abi.RAD_OK:
        raise RowRefused(r.name, rc)
    return r


def quant_act_fp8(x: torch.Tensor, group: int = 128) -> tuple[torch.Tensor, torch.Tensor]:
    """bf16/f32 activations [rows, n] -> (e4m3 codes uint8 [rows, n], f32 scale [rows, n/group])."""
    P = plugin()
    rows, n = x.shape
    ngrp = (n + group - 1) // group
    q = torch.empty((rows, n), dtype=torch.uint8, device=x.device)
    s = torch.empty((rows, ngrp), dtype=torch.float32, device=x.device)
    xdt = abi.RAD_F32 if x.dtype == torch.float32 else abi.RAD_BF16
    rc = P.lib.r3d_b200_quant_act_fp8(x.data_ptr(), xdt, x.stride(0), q.data_ptr(), q.stride(0),
                                      s.data_ptr(), s.stride(0), rows, n, group, _stream())
    if rc != abi.RAD_OK:
        raise RowRefused("quant_act_fp8", rc)
    return q, s


def _act_dt(t: torch.Tensor) -> tuple[int, str]:
    return (abi.RAD_F32, "f32") if t.dtype == torch.float32 else (abi.RAD_BF16, "bf16")


_ARENA: dict[tuple[int, int], torch.Tensor] = {}


def _arena(nbytes: int, device: torch.device) -> torch.Tensor:
    """the launch arena an engine hands a row whose scratch hook asks for one: kept per device, grown only"""
    key = (device.index or 0, 0)
    t = _ARENA.get(key)
    if t is None or t.numel() < nbytes:
        t = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _ARENA[key] = t
    return t


def _issue(op: str, query: dict, tensors: list, scratch_hook=None, device: torch.device | None = None) -> Row:
    P = plugin()
    r = P.resolve(op, query)
    if r is None:
        raise RuntimeError(f"no row serves {op} {query}")
    pack = ArgPack(tensors, query)
    if scratch_hook is not None and device is not None:
        need = int(scratch_hook(pack.args))
        if need > 0:
            arena = _arena(need, device)
            pack = ArgPack(tensors, query, scratch=arena.data_ptr(), scratch_bytes=arena.numel())
    rc = P.launch_row(r, pack, _stream())
    if rc != abi.RAD_OK:
        raise RowRefused(r.name, rc)
    return r


def quant_act_fp8_row(x: torch.Tensor, q: torch.Tensor, scale: torch.Tensor, *, group: int = 128) -> Row:
    """The quant_act_fp8 op through its row: x [M, n] bf16/f32 -> q e4m3 (uint8) [M, n], scale f32."""
    dt, name = _act_dt(x)
    query = dict(M=x.shape[0], n=x.shape[-1], group=group, dtype=name)
    return _issue("quant_act_fp8", query, [_desc(x, dt), _desc(q, abi.RAD_F8E4M3), _desc(scale, abi.RAD_F32)])


def gated_quant_fp8_row(gate_up: torch.Tensor, q: torch.Tensor, scale: torch.Tensor,
                        out: torch.Tensor | None = None, *, group: int = 128, act: str | None = None) -> Row:
    """The gated_quant_fp8 op through its row: gate_up [M, 2n] (gate half first) -> q [M, n], scale and,
    when `out` is given, the bf16/f32 gated product."""
    dt, name = _act_dt(gate_up)
    query = dict(M=gate_up.shape[0], n=gate_up.shape[-1] // 2, group=group, dtype=name)
    if act is not None:
        query["act"] = act
    odt = _act_dt(out)[0] if out is not None else abi.RAD_BF16
    return _issue("gated_quant_fp8", query, [_desc(gate_up, dt), _desc(q, abi.RAD_F8E4M3),
                                             _desc(scale, abi.RAD_F32), _desc(out, odt)])


def rmsnorm_quant_fp8(x: torch.Tensor, w: torch.Tensor, q: torch.Tensor, scale: torch.Tensor, *, eps: float,
                      residual: torch.Tensor | None = None, out: torch.Tensor | None = None,
                      group: int = 128, wadd: float | None = None) -> Row:
    """The rmsnorm_quant_fp8 op through its row: x [M, n] bf16, w [n]; `residual` (bf16, updated in place
    with the narrowed sum) selects the fused-add form; `out` receives the bf16/f32 norm output."""
    query = dict(M=x.shape[0], n=x.shape[-1], eps=float(eps), group=group, dtype="bf16")
    if wadd is not None:
        query["wadd"] = float(wadd)
    odt = _act_dt(out)[0] if out is not None else abi.RAD_BF16
    return _issue("rmsnorm_quant_fp8", query, [_desc(x, abi.RAD_BF16), _desc(residual, abi.RAD_BF16),
                                               _desc(w, _act_dt(w)[0]), _desc(q, abi.RAD_F8E4M3),
                                               _desc(scale, abi.RAD_F32), _desc(out, odt)])


def row_topk(x: torch.Tensor, idx: torch.Tensor, val: torch.Tensor, pairs: torch.Tensor | None = None, *,
             R: int, vocab_off: int | None = None, arena: bool = True) -> Row:
    """The row_topk op through its row: x [M, N] bf16 -> idx i32 [M, R], val f32 [M, R] and, when given,
    pairs f32 [M, R, 2] holding (bits of the int32 id, value). `arena`: hand the row the launch arena its
    scratch hook asks for (as an engine does); without it the row uses planes of its own."""
    query = dict(M=x.shape[0], N=x.shape[-1], R=R, dtype="bf16")
    if vocab_off is not None:
        query["vocab_off"] = int(vocab_off)
    return _issue("row_topk", query, [_desc(x, abi.RAD_BF16), _desc(idx, abi.RAD_I32), _desc(val, abi.RAD_F32),
                                      _desc(pairs, abi.RAD_F32)],
                  plugin().lib.r3d_rad_row_topk_scratch if arena else None, x.device)


def sample_argmax(logits: torch.Tensor, token: torch.Tensor, params: torch.Tensor | None = None) -> Row:
    """The sample_argmax op through its row: logits f32 [M, n_vocab] -> token i32 [M] (greedy, ties to the
    lower id). `params` is the engine's per-row parameter blob; the row does not read it."""
    query = dict(M=logits.shape[0], n_vocab=logits.shape[1])
    return _issue("sample_argmax", query, [_desc(logits, abi.RAD_F32), _desc(params, abi.RAD_U8),
                                           _desc(token, abi.RAD_I32)],
                  plugin().lib.r3d_rad_sample_argmax_scratch, logits.device)


class BoundGemm:
    """A gemm_nt_q band declared once and issued many times, the way the engine uses a row:
    the row is resolved and the RadArgs built at declare time over fixed device buffers; each
    `issue()` is one call of the row's launch pointer on the current stream. Buffers must
    outlive the object."""

    def __init__(self, a: torch.Tensor, a_scale: torch.Tensor, b: torch.Tensor,
                 b_scale: torch.Tensor, y: torch.Tensor, *, dtype: str, N: int, K: int,
                 row: str | None = None):
        P = plugin()
        M = y.numel() // N
        group = 128 if dtype == "fp8a8" else 32
        query: dict[str, Any] = dict(M=M, N=N, K=K, group=group, dtype=dtype)
        self.row = (P.resolve("gemm_nt_q", query) if row is None
                    else next(x for x in P.rows() if x.name == row))
        if self.row is None:
            raise RuntimeError(f"no row serves gemm_nt_q {query}")
        if dtype == "fp8a8":
            bdesc = _desc(b, abi.RAD_F8E4M3)
            sdt = abi.RAD_F32 if b_scale.dtype == torch.float32 else abi.RAD_BF16
        else:
            bdesc = _desc(b, abi.RAD_FP4E2M1, shape=[b.shape[0], K], stride=[K, 1])
            sdt = abi.RAD_E8M0
        self._keep = (a, a_scale, b, b_scale, y)
        self.pack = ArgPack([_desc(a, abi.RAD_F8E4M3), _desc(a_scale, abi.RAD_F32), bdesc,
                             _desc(b_scale, sdt), _desc(y, abi.RAD_BF16),
                             _desc(None, abi.RAD_F32), _desc(None, abi.RAD_BF16)], query)
        self._fn = P._launch_t(self.row.launch)
        import ctypes as _C
        self._argp = _C.byref(self.pack.args)
        self._C = _C

    def issue(self) -> None:
        rc = self._fn(self._argp, self._C.c_void_p(_stream()))
        if rc != abi.RAD_OK:
            raise RowRefused(self.row.name, rc)
