"""Scan-level data parallelism: scans are independent (the batch index is part of every
coordinate key and normalisation runs on stored statistics), so a batch is split by scan across
the GPUs of one box, every rank holds a full copy of the weights and runs its shard on its own
stream, and the only communication is one gather of the outputs per batch.  The reference has no
multi-GPU code at all; this module is what a caller of it would have to add."""
from typing import List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

__all__ = ["shard_range", "balanced_assignment", "gather_rows", "gather_rows_padded", "PaddedGather"]


def shard_range(n_items: int, world_size: int, rank: int) -> Tuple[int, int]:
    """Contiguous [lo, hi) slice of n_items for `rank`; the first n_items % world_size ranks get
    one extra item."""
    if world_size < 1 or not (0 <= rank < world_size):
        raise ValueError(f"bad rank {rank} for world size {world_size}")
    base, extra = divmod(n_items, world_size)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def balanced_assignment(sizes: Sequence[int], world_size: int) -> List[List[int]]:
    """Greedy longest-first assignment of items (e.g. scans by voxel count) to ranks; returns the
    item indices of every rank.  Deterministic for equal inputs on every rank."""
    order = sorted(range(len(sizes)), key=lambda i: (-sizes[i], i))
    loads = [0] * world_size
    out: List[List[int]] = [[] for _ in range(world_size)]
    for i in order:
        r = min(range(world_size), key=lambda k: (loads[k], k))
        out[r].append(i)
        loads[r] += sizes[i]
    return [sorted(v) for v in out]


def gather_rows(local: torch.Tensor, group: Optional[dist.ProcessGroup] = None) -> Tuple[torch.Tensor, List[int]]:
    """All-gather of row-major [n_r, C] tensors with a different row count per rank.
    Returns (rows of all ranks concatenated in rank order, list of per-rank row counts).
    Two collectives: the counts (world_size int64) and the rows padded to the largest count."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return local, [local.shape[0]]
    world = dist.get_world_size(group)
    n = torch.tensor([local.shape[0]], dtype=torch.int64, device=local.device)
    counts = torch.empty(world, dtype=torch.int64, device=local.device)
    dist.all_gather_into_tensor(counts, n, group=group)
    counts_host = counts.cpu().tolist()
    mx = max(counts_host)
    padded = local
    if local.shape[0] != mx:
        padded = torch.zeros((mx,) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
        padded[: local.shape[0]] = local
    buf = torch.empty((world * mx,) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(buf, padded.contiguous(), group=group)
    parts = [buf[r * mx: r * mx + counts_host[r]] for r in range(world)]
    return torch.cat(parts, 0), counts_host


def gather_rows_padded(local: torch.Tensor, max_rows: int, group: Optional[dist.ProcessGroup] = None
                       ) -> Tuple[torch.Tensor, torch.Tensor]:
    """All-gather for a caller that knows an upper bound of the per-rank row count: no host read.
    Returns (buffer [world, max_rows, C] whose slice [r, :counts[r]] holds rank r's rows, counts as
    an int64 device tensor [world]).  Rows beyond a rank's count are unspecified.  Two collectives
    queued on the current stream; nothing waits for the device."""
    if local.shape[0] > max_rows:
        raise ValueError(f"{local.shape[0]} rows exceed max_rows={max_rows}")
    n = torch.tensor([local.shape[0]], dtype=torch.int64).to(local.device, non_blocking=True)
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        buf = torch.empty((1, max_rows) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
        buf[0, : local.shape[0]] = local
        return buf, n
    world = dist.get_world_size(group)
    counts = torch.empty(world, dtype=torch.int64, device=local.device)
    dist.all_gather_into_tensor(counts, n, group=group)
    padded = torch.empty((max_rows,) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
    padded[: local.shape[0]] = local
    buf = torch.empty((world, max_rows) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(buf.view((world * max_rows,) + tuple(local.shape[1:])), padded, group=group)
    return buf, counts


class PaddedGather:
    """gather_rows_padded with its buffers allocated once: for a loop that gathers the output of every
    step, where the per-call allocations and small host calls would otherwise be paid each time.
    All calls must be made on the same stream (the buffers are reused in stream order).  Returns views
    of the internal buffers, valid until the next call.

    The row count never passes through reused host memory (a queued host-to-device copy reads its source
    when it runs, not when it is queued, so a later call could overwrite it first): a count the host knows
    travels as a kernel argument (`fill_`), a count the host does not know is given as a device tensor."""

    def __init__(self, max_rows: int, cols: int, dtype: torch.dtype, device,
                 group: Optional[dist.ProcessGroup] = None) -> None:
        self.group = group
        self.world = dist.get_world_size(group) if (dist.is_available() and dist.is_initialized()) else 1
        self.max_rows = max_rows
        self.padded = torch.zeros((max_rows, cols), dtype=dtype, device=device)
        self.buf = torch.empty((self.world, max_rows, cols), dtype=dtype, device=device)
        self.n_dev = torch.zeros(1, dtype=torch.int64, device=device)
        self.counts = torch.zeros(self.world, dtype=torch.int64, device=device)

    def __call__(self, local: torch.Tensor, n_dev: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
        """`local`: this rank's rows.  Without `n_dev` all of them count; with `n_dev` (an integer tensor of one
        element on the device) `local` holds `max_rows` rows of which the first `n_dev[0]` count."""
        rows = local.shape[0]
        if rows > self.max_rows:
            raise ValueError(f"{rows} rows exceed max_rows={self.max_rows}")
        if n_dev is None:
            self.n_dev.fill_(rows)
        else:
            self.n_dev.copy_(n_dev.reshape(1))
        if rows == self.max_rows and local.is_contiguous():
            src = local                       # already padded: gathered in place
        else:
            self.padded[:rows].copy_(local)
            src = self.padded
        if self.world == 1:
            self.counts.copy_(self.n_dev)
            self.buf[0].copy_(src)
        else:
            dist.all_gather_into_tensor(self.counts, self.n_dev, group=self.group)
            dist.all_gather_into_tensor(self.buf.view(self.world * self.max_rows, -1), src, group=self.group)
        return self.buf, self.counts
