"""Column sharding of the LM head and the large-N projections across the GPUs of one node.

Every output column y[:, n] depends on one weight row, so the weight rows are split into
contiguous slabs, one per rank; activations are replicated; each rank runs the unchanged
single-GPU row on its slab and the bf16/f32 outputs are all-gathered over NCCL (NVLink).
No reduction crosses ranks, so the gathered result is bit-identical to the unsharded one.
The reference is single-rank ("vocab_off is the shard origin and stays 0",
src/r3d_rows.cpp:281-284 of libr3d); this module has no counterpart there.

Host-side logic only (torch.distributed for the exchange): it runs unchanged on the gloo
backend for CPU tests.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import torch
import torch.distributed as dist


@dataclass(frozen=True)
class Slab:
    start: int        # first weight row of this rank
    rows: int         # live rows of this rank (0 for a rank past the end)
    padded: int       # slab height every rank uses in the gather (equal counts)


def slab_of(n_rows: int, world: int, rank: int, granule: int = 128) -> Slab:
    """Contiguous slabs of `granule`-row tiles, equal except that trailing ranks may be
    short or empty: ceil(tiles / world) tiles each. 151936 rows = 1187 tiles of 128."""
    tiles = (n_rows + granule - 1) // granule
    per = (tiles + world - 1) // world
    padded = per * granule
    start = min(rank * padded, n_rows)
    rows = max(0, min(n_rows - start, padded))
    return Slab(start, rows, padded)


def gather_columns(y_local: torch.Tensor, n_rows: int, granule: int = 128,
                   group: dist.ProcessGroup | None = None) -> torch.Tensor:
    """y_local [M, slab.padded] (columns past slab.rows are don't-care) from every rank ->
    y [M, n_rows] on every rank, columns in weight-row order."""
    world = dist.get_world_size(group)
    M, padded = y_local.shape
    if world == 1:
        return y_local[:, :n_rows]
    buf = torch.empty((world, M, padded), dtype=y_local.dtype, device=y_local.device)
    # concatenation form: [world * M, P] <- [M, P] from every rank, rank-major
    dist.all_gather_into_tensor(buf.view(world * M, padded), y_local.contiguous(), group=group)
    # [G, M, P] -> [M, G*P]: rank-major columns are already in weight-row order
    return buf.permute(1, 0, 2).reshape(M, world * padded)[:, :n_rows]


def gather_topk(pairs_local: torch.Tensor, group: dist.ProcessGroup | None = None) -> tuple[torch.Tensor, torch.Tensor]:
    """The exchange behind a column-sharded head that samples: every rank ran row_topk over its own
    slab with `vocab_off` = the slab's first column and hands in its pairs plane [M, R, 2] (f32 words:
    the bits of the int32 global id, the value; a hole is id -1 / -inf). The planes are all-gathered
    (M * R * 8 bytes per rank instead of the logits) and merged under the same order the rows use --
    value descending, ties to the lower id, holes last -- into idx int32 [M, R], val f32 [M, R] on
    every rank: the unsharded row_topk's answer. The merge is tiny (world * R candidates per row) and
    runs as tensor ops on whatever device holds the planes."""
    world = dist.get_world_size(group)
    M, R, _ = pairs_local.shape
    flat = pairs_local.contiguous().view(M, 2 * R)
    if world > 1:
        buf = torch.empty((world * M, 2 * R), dtype=flat.dtype, device=flat.device)
        dist.all_gather_into_tensor(buf, flat, group=group)
        cand = buf.view(world, M, R, 2).permute(1, 0, 2, 3).reshape(M, world * R, 2)
    else:
        cand = flat.view(M, R, 2)
    ids = cand[..., 0].contiguous().view(torch.int32)
    vals = cand[..., 1].contiguous()
    big = torch.iinfo(torch.int32).max
    key_id = torch.where(ids < 0, torch.full_like(ids, big), ids)
    order = torch.sort(key_id, dim=1, stable=True).indices                    # ids ascending, holes last
    v1 = torch.gather(vals, 1, order)
    order2 = torch.sort(v1, dim=1, descending=True, stable=True).indices      # then values descending, stably
    pick = torch.gather(order, 1, order2)[:, :R]
    return torch.gather(ids, 1, pick), torch.gather(vals, 1, pick)


class PushGather:
    """The fused form of the gather: the serving kernel's epilogue stores this rank's columns
    into every rank's [M, world * n_pad] buffer over NVLink (CUDA IPC peer mappings) and raises
    a flag; wait() enqueues the bounded device-side wait for all ranks. Two slots are used
    alternately by the caller so that a peer's next push never lands on a result still in use.

    Construction is collective: every rank of `group` creates its buffer and the 64-byte IPC
    handles are exchanged with all_gather_object. Needs the CUDA plugin (no CPU path)."""

    def __init__(self, plugin, slot_bytes: int, slots: int = 2, group: dist.ProcessGroup | None = None):
        self.lib = plugin.lib
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.slots, self.slot_bytes = slots, slot_bytes
        handle = C.create_string_buffer(64)
        ptr = C.c_void_p()
        rc = self.lib.r3d_b200_gather_create(self.world, self.rank, slot_bytes, slots, C.byref(ptr), handle)
        self.ptr = ptr if rc == 0 else None
        # every rank takes part in both exchanges whatever happened locally, so that a failure on
        # one rank becomes the same exception on all of them instead of a stuck collective
        handles: list = [None] * self.world
        dist.all_gather_object(handles, handle.raw if rc == 0 else None, group=group)
        if rc == 0 and all(h is not None for h in handles):
            rc = self.lib.r3d_b200_gather_connect(self.ptr, b"".join(handles))
        elif rc == 0:
            rc = -1
        codes: list = [None] * self.world
        dist.all_gather_object(codes, int(rc), group=group)
        if any(c != 0 for c in codes):
            self.close()
            raise RuntimeError(f"fused gather set-up failed, per-rank status {codes}")
        dist.barrier(group=group)

    def buffer(self, slot: int, M: int, n_pad: int, dtype: torch.dtype) -> torch.Tensor:
        """This rank's gathered [M, world * n_pad] view of a slot (valid after wait())."""
        esz = torch.empty((), dtype=dtype).element_size()
        n = M * self.world * n_pad
        if n * esz > self.slot_bytes:
            raise ValueError("slot too small for this shape")
        base = self.lib.r3d_b200_gather_buffer(self.ptr, slot)
        iface = {"shape": (n * esz,), "typestr": "|u1", "data": (int(base), False), "version": 3}
        holder = type("_Dev", (), {"__cuda_array_interface__": iface})()
        return torch.as_tensor(holder, device="cuda").view(dtype).view(M, self.world * n_pad)

    def wait(self, stream: int | None = None) -> None:
        st = stream if stream is not None else torch.cuda.current_stream().cuda_stream
        rc = self.lib.r3d_b200_gather_wait(self.ptr, C.c_void_p(st))
        if rc != 0:
            raise RuntimeError(f"r3d_b200_gather_wait failed with status {rc}")

    def status(self) -> int:
        return int(self.lib.r3d_b200_gather_status(self.ptr))

    def close(self) -> None:
        if getattr(self, "ptr", None):
            self.lib.r3d_b200_gather_destroy(self.ptr)
        self.ptr = None


class PushedGemm:
    """One column slab of an mxfp4a8 / fp8a8 gemm_nt_q band, declared once over fixed device buffers
    and issued many times: issue(slot) launches the slab's GEMV with the all-gather fused into
    its epilogue, then the wait; result(slot) is this rank's [M, world * n_pad] view."""

    def __init__(self, pg: PushGather, a: torch.Tensor, a_scale: torch.Tensor, b: torch.Tensor,
                 b_scale: torch.Tensor, *, dtype: str, M: int, n_local: int, n_pad: int, K: int,
                 scratch: torch.Tensor | None = None):
        from . import abi
        self.pg, self.M, self.n_pad = pg, M, n_pad
        q = abi.R3dGemmQ()
        q.a, q.a_scale, q.b, q.b_scale = a.data_ptr(), a_scale.data_ptr(), b.data_ptr(), b_scale.data_ptr()
        q.y = scratch.data_ptr() if scratch is not None else None
        q.m, q.n, q.k = M, n_local, K
        q.as_cols, q.a_pitch, q.as_pitch, q.y_pitch = a_scale.shape[1], a.stride(0), a_scale.stride(0), n_local
        if dtype == "mxfp4a8":
            q.bs_cols, q.rblk, q.bs_dtype = K // 32, 1, abi.RAD_E8M0
            q.b_pitch, q.bs_pitch = b.stride(0), b_scale.stride(0)
            self._fn = pg.lib.r3d_b200_gemm_mxfp4a8_push
        else:
            q.bs_cols, q.bs_dtype = b_scale.shape[1], (abi.RAD_F32 if b_scale.dtype == torch.float32 else abi.RAD_BF16)
            q.rblk = 128 if b_scale.shape[0] < n_local else 1
            q.b_pitch, q.bs_pitch = b.stride(0), b_scale.stride(0)
            self._fn = pg.lib.r3d_b200_gemm_fp8a8_push
        q.arm = abi.R3D_ARM_AUTO
        self._q, self._keep = q, (a, a_scale, b, b_scale, scratch)

    def issue(self, slot: int) -> None:
        st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
        rc = self._fn(C.byref(self._q), self.pg.ptr, slot, self.n_pad, st)
        if rc != 0:
            raise RuntimeError(f"sharded gemm refused with status {rc}")
        self.pg.wait(st.value)

    def result(self, slot: int) -> torch.Tensor:
        return self.pg.buffer(slot, self.M, self.n_pad, torch.bfloat16)
