"""Multi-GPU execution of the TCEC SGEMM with one process per GPU over ``torch.distributed``.

Two shardings, neither of which splits K, so no reduction is ever needed:

* batch sharding  - rank r owns a contiguous slice of the independent matrices of a
  batched GEMM; there is no collective on the data path.
* column sharding - rank r owns a block of columns of B and of C; A lives on one
  rank and is broadcast (NCCL over NVLink on GPUs) in row panels into every rank's
  own memory.

On GPUs both are thin callers of the C ABI (``tcec_sgemm_column_shard``,
``tcec_sgemm_strided_batched``): the library owns its NCCL communicator, created here from an
id that ``torch.distributed`` carries to the ranks.  The same plumbing also runs with injected
local compute under the ``gloo`` backend on CPU tensors, which is how its host logic - shard
arithmetic, panel order, what happens when a rank fails - is tested without a GPU.

The reference is single-GPU (no collective call site exists in it); this module is the host
logic the multi-GPU configurations of the benchmark add around the C ABI.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, List, Optional, Tuple

import torch
import torch.distributed as dist

OK, ERR_LOCAL, ERR_COMM, ERR_PEER = 0, 1, 2, 3


class ShardError(RuntimeError):
    """A rank's local compute failed, a collective failed, or another rank reported a failure."""

    def __init__(self, status: int, what: str):
        self.status = status
        super().__init__(what)


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
    """Local compute injected into the column-sharded driver (tests; a caller's own kernels)."""

    prepare_b: Callable[[torch.Tensor], object]
    gemm_panel: Callable[[torch.Tensor, object, torch.Tensor], None]  # (A panel, prepared B, C rows)


_comm_ready = {}


def init_library_comm(group=None) -> None:
    """Gives the CUDA library its own communicator for ``group`` (once): rank 0 obtains the id,
    ``torch.distributed`` carries it, every rank joins with its current device."""
    from . import tcec

    key = id(group) if group is not None else 0
    if _comm_ready.get(key):
        return
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    box = [tcec.comm_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(box, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
    tcec.comm_init_rank(world, rank, box[0])
    _comm_ready[key] = True


def sgemm_column_sharded(a_root: Optional[torch.Tensor], b_local: torch.Tensor, c_local: torch.Tensor,
                         m: int, k: int, *, root: int = 0, panel_rows: int = 2048,
                         ops: Optional[LocalOps] = None, group=None, policy: str = "fp16_ec") -> torch.Tensor:
    """C[:, cols] = A @ B[:, cols] on every rank, with A (m x k) held by ``root``.

    ``b_local`` is this rank's (k x n_local) column block, ``c_local`` its (m x n_local) output
    block.  Without ``ops`` the operands are CUDA tensors and the call is ``tcec_sgemm_column_shard``
    (the library broadcasts split row panels of A with NCCL and multiplies them as they arrive).
    With ``ops`` the broadcast runs here, panel by panel through ``torch.distributed``, and the
    local compute is the caller's; a failure of any rank's compute is reported on every rank.
    """
    rank = dist.get_rank(group)
    world = dist.get_world_size(group)
    if rank == root:
        if a_root is None or tuple(a_root.shape) != (m, k):
            raise ValueError("root must pass an (m, k) matrix")
    if ops is None:
        from . import tcec

        if world > 1:
            init_library_comm(group)
        return tcec.sgemm_column_shard(a_root if rank == root else None, b_local, c_local, m, k, root=root,
                                       policy=policy)

    panels = row_panels(m, panel_rows)
    status, what = OK, ""
    prepared = None
    try:
        prepared = ops.prepare_b(b_local) if b_local.shape[1] > 0 else None
    except Exception as e:  # keep taking part in the broadcasts: the other ranks must not block on this one
        status, what = ERR_LOCAL, f"prepare_b failed on rank {rank}: {e}"
    src = dist.get_global_rank(group, root) if group is not None else root
    buf = None
    for r0, rows in panels:
        if rank == root:
            panel = a_root[r0:r0 + rows].contiguous()
        else:
            if buf is None or buf.shape[0] < rows:
                buf = torch.empty((rows, k), dtype=b_local.dtype, device=b_local.device)
            panel = buf[:rows]
        if world > 1:
            try:
                dist.broadcast(panel, src=src, group=group)
            except Exception as e:
                raise ShardError(ERR_COMM, f"broadcast of rows {r0}..{r0 + rows} failed on rank {rank}: {e}") from e
        if status == OK and prepared is not None:
            try:
                ops.gemm_panel(panel, prepared, c_local[r0:r0 + rows])
            except Exception as e:
                status, what = ERR_LOCAL, f"gemm_panel failed on rank {rank} at row {r0}: {e}"
    if world > 1:
        # every rank learns whether any rank failed (the only extra collective: one word per call)
        word = torch.tensor([status], dtype=torch.int32, device=b_local.device)
        try:
            dist.all_reduce(word, op=dist.ReduceOp.MAX, group=group)
        except Exception as e:
            raise ShardError(ERR_COMM, f"status exchange failed on rank {rank}: {e}") from e
        if status == OK and int(word.item()) != OK:
            status, what = ERR_PEER, "another rank reported a failure"
    if status != OK:
        raise ShardError(status, what)
    return c_local


def sgemm_batch_sharded(a_local: torch.Tensor, b_local: torch.Tensor, c_local: Optional[torch.Tensor] = None,
                        *, policy: str = "fp16_ec") -> torch.Tensor:
    """This rank's slice of a batched GEMM ([count, m, k] x [count, k, n]); no communication."""
    from . import tcec

    if a_local.shape[0] == 0:
        return c_local if c_local is not None else a_local.new_empty((0, a_local.shape[1], b_local.shape[2]))
    return tcec.sgemm_strided_batched(a_local, b_local, c_local, policy=policy)
