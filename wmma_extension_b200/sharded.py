"""Multi-GPU execution of the TCEC SGEMM: one process per GPU over ``torch.distributed``.

Two shardings, neither of which splits K, so no reduction is ever needed:

* batch sharding  - rank r owns a contiguous slice of the independent matrices of a
  batched GEMM; there is no collective on the data path.
* column sharding - rank r owns a block of columns of B and of C; A lives on one
  rank and is broadcast (NCCL over NVLink on GPUs) in row panels into every rank's
  own memory, each panel's GEMM overlapping the next panel's broadcast.  B is split
  into operand panels once per call, not once per row panel.

The reference is single-GPU (no collective call site exists in it); this module is
the host logic the multi-GPU configurations of the benchmark add around the C ABI.
The local compute functions are injectable so the same plumbing runs under the
``gloo`` backend on CPU tensors in tests.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, List, Optional, Tuple

import torch
import torch.distributed as dist


def batch_shard(batch: int, rank: int, world: int) -> Tuple[int, int]:
    """(first, count) of the matrices rank ``rank`` owns; earlier ranks take the remainder."""
    if world <= 0 or not (0 <= rank < world) or batch < 0:
        raise ValueError("bad shard request")
    base, rem = divmod(batch, world)
    first = rank * base + min(rank, rem)
    return first, base + (1 if rank < rem else 0)


def column_shard(n: int, rank: int, world: int, align: int = 256) -> Tuple[int, int]:
    """(first column, count) of the column block rank ``rank`` owns.

    Blocks are multiples of ``align`` columns (one output tile) except the last
    non-empty one, so no tile straddles two ranks.
    """
    if world <= 0 or not (0 <= rank < world) or n < 0 or align <= 0:
        raise ValueError("bad shard request")
    units = (n + align - 1) // align
    first_u, cnt_u = batch_shard(units, rank, world)
    first = min(first_u * align, n)
    last = min((first_u + cnt_u) * align, n)
    return first, last - first


def row_panels(m: int, panel_rows: int) -> List[Tuple[int, int]]:
    """[(first row, rows)] covering m rows; panel_rows is rounded up to a multiple of 128."""
    if m < 0 or panel_rows <= 0:
        raise ValueError("bad panel request")
    panel_rows = ((panel_rows + 127) // 128) * 128
    return [(r, min(panel_rows, m - r)) for r in range(0, m, panel_rows)]


@dataclass
class LocalOps:
    """Local compute used by the sharded drivers (CUDA library by default)."""

    prepare_b: Callable[[torch.Tensor], object]
    gemm_panel: Callable[[torch.Tensor, object, torch.Tensor], None]  # (A panel, prepared B, C rows)


def cuda_ops(policy: str = "fp16_ec", reserve_sms: int = 0) -> LocalOps:
    """Local compute through the CUDA library.  The GEMM's persistent CTAs take every register
    of their SM, so a broadcast kernel launched beside it only runs where the GEMM has no CTA,
    and a GEMM CTA that has to wait for such an SM delays the whole launch.  ``reserve_sms`` keeps
    that many SMs out of the GEMM's grid (as many as the broadcast uses channels)."""
    from . import tcec

    def prepare_b(b_local: torch.Tensor):
        k, n = b_local.shape
        return (tcec.pack_b(b_local, policy), k, n)

    def gemm_panel(a_panel: torch.Tensor, prepared, c_rows: torch.Tensor) -> None:
        b_packed, k, n = prepared
        a_packed = tcec.pack_a(a_panel, policy)
        if reserve_sms:
            tcec.set_option("reserve_sms", reserve_sms)
        try:
            tcec.sgemm_packed(a_packed, b_packed, a_panel.shape[0], n, k, c_rows, policy=policy)
        finally:
            if reserve_sms:
                tcec.set_option("reserve_sms", 0)

    return LocalOps(prepare_b, gemm_panel)


def sgemm_column_sharded(a_root: Optional[torch.Tensor], b_local: torch.Tensor, c_local: torch.Tensor,
                         m: int, k: int, *, root: int = 0, panel_rows: int = 2048,
                         ops: Optional[LocalOps] = None, group=None,
                         a_buffers: Optional[List[torch.Tensor]] = None) -> torch.Tensor:
    """C[:, cols] = A @ B[:, cols] on every rank, with A (m x k, row-major) held by ``root``.

    ``b_local`` is this rank's (k x n_local) column block, ``c_local`` its (m x n_local)
    output block.  A reaches the other ranks by broadcast, one row panel at a time,
    double-buffered: panel p+1 is in flight while panel p is multiplied.  Every rank
    ends up having read A only from its own memory.
    """
    rank = dist.get_rank(group)
    world = dist.get_world_size(group)
    ops = ops or cuda_ops()
    if rank == root:
        if a_root is None or tuple(a_root.shape) != (m, k) or not a_root.is_contiguous():
            raise ValueError("root must pass a contiguous (m, k) matrix")
    panels = row_panels(m, panel_rows)
    prepared = ops.prepare_b(b_local) if b_local.shape[1] > 0 else None
    if world == 1:
        for r0, rows in panels:
            if prepared is not None:
                ops.gemm_panel(a_root[r0:r0 + rows], prepared, c_local[r0:r0 + rows])
        return c_local

    max_rows = max(rows for _, rows in panels) if panels else 0
    if a_buffers is None and rank != root:
        a_buffers = [torch.empty((max_rows, k), dtype=b_local.dtype, device=b_local.device) for _ in range(2)]

    def panel_tensor(i: int) -> torch.Tensor:
        r0, rows = panels[i]
        if rank == root:
            return a_root[r0:r0 + rows]
        return a_buffers[i % 2][:rows]

    works = [None] * len(panels)
    if panels:
        works[0] = dist.broadcast(panel_tensor(0), src=root, group=group, async_op=True)
    for i, (r0, rows) in enumerate(panels):
        works[i].wait()
        if i + 1 < len(panels):
            # Buffer (i+1) % 2 was last read by panel i-1's GEMM, queued on this stream before
            # the wait above; the collective's stream is ordered after it by the work handle.
            works[i + 1] = dist.broadcast(panel_tensor(i + 1), src=root, group=group, async_op=True)
        if prepared is not None:
            ops.gemm_panel(panel_tensor(i), prepared, c_local[r0:r0 + rows])
    return c_local


def sgemm_batch_sharded(a_local: torch.Tensor, b_local: torch.Tensor, c_local: Optional[torch.Tensor] = None,
                        *, policy: str = "fp16_ec") -> torch.Tensor:
    """This rank's slice of a batched GEMM ([count, m, k] x [count, k, n]); no communication."""
    from . import tcec

    if a_local.shape[0] == 0:
        return c_local if c_local is not None else a_local.new_empty((0, a_local.shape[1], b_local.shape[2]))
    return tcec.sgemm_strided_batched(a_local, b_local, c_local, policy=policy)
