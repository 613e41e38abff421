"""Batch sharding of a KSMM workload across the GPUs of one node.

Every batch column (batch-last) or row (batch-first) of a Kronecker-sparse
product is independent and the factors are tiny, so the batch dimension is
split into contiguous ranges, the weights are replicated, and the hot path
needs no collective.  The only communication is the optional gather of the
outputs (NCCL all-gather over NVLink on GPUs, gloo in CPU tests).

The reference has no multi-device code at all (its only affordance is a
``--device-id`` flag, src/ksmm_py/benchmark/ksmm_time.py:24); this module is
new functionality.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def shard_range(batch, rank, world_size):
    """Contiguous [start, stop) of the batch owned by ``rank``; the first
    ``batch % world_size`` ranks get one extra element."""
    if world_size <= 0 or not (0 <= rank < world_size):
        raise ValueError(f"bad rank {rank} / world size {world_size}")
    base, extra = divmod(int(batch), world_size)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def shard_batch(x, bs_last, rank, world_size):
    """The rank's contiguous local copy of a global 2-D activation.  A column
    slice of a batch-last tensor is not contiguous, so it is materialised."""
    n = x.shape[1] if bs_last else x.shape[0]
    lo, hi = shard_range(n, rank, world_size)
    return (x[:, lo:hi] if bs_last else x[lo:hi]).contiguous()


def gather_output(y_local, bs_last, batch, group=None):
    """All-gather the per-rank outputs back into the global (out, batch) /
    (batch, out) tensor.  Uneven shards are padded to the largest shard for
    the collective and trimmed afterwards."""
    world = dist.get_world_size(group)
    sizes = [shard_range(batch, r, world)[1] - shard_range(batch, r, world)[0] for r in range(world)]
    mx = max(sizes)
    feat = y_local.shape[0] if bs_last else y_local.shape[1]
    rows = y_local.t().contiguous() if bs_last else y_local      # (local batch, feat)
    if rows.shape[0] < mx:
        pad = torch.zeros(mx - rows.shape[0], feat, dtype=rows.dtype, device=rows.device)
        rows = torch.cat([rows, pad], dim=0)
    parts = [torch.empty_like(rows) for _ in range(world)]
    dist.all_gather(parts, rows.contiguous(), group=group)
    full = torch.cat([p[:s] for p, s in zip(parts, sizes)], dim=0)  # (batch, feat)
    return full.t().contiguous() if bs_last else full
