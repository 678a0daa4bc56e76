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
