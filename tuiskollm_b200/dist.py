"""Multi-GPU plumbing for the two places the path shards (one process per GPU,
``torch.distributed`` over NCCL; gloo works for the host logic on CPU).

* LM head: vocabulary rows are split contiguously; every rank streams its shard and
  produces per-token ``(max, global index)`` pairs; one all-gather of ``8 * rows`` bytes per
  rank and a first-maximum merge give the greedy token.  Logits stay sharded.
* Layer slice: QKV / GDN-input / gate-up are column-parallel (weight rows split), down is
  row-parallel (reduction split) followed by one all-reduce of the ``[rows, hidden]`` partial
  sums.  Norm and activation quantisation are replicated.

The reference is single-GPU (no NCCL/MPI anywhere in it); this layer is new design.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist


@dataclass(frozen=True)
class Shard:
    rows: int     # rows (or reduction columns) owned by this rank
    offset: int   # first global row / column


def vocab_shard(vocab: int, world: int, rank: int) -> Shard:
    """Contiguous vocabulary shard; every shard must keep the projection's row granularity."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world of {world}")
    if vocab % (world * 16) != 0:
        raise ValueError(f"vocabulary {vocab} does not split into {world} shards of a multiple of 16 rows")
    rows = vocab // world
    return Shard(rows, rank * rows)


def column_shard(out_rows: int, world: int, rank: int, granule: int = 128) -> Shard:
    """Column-parallel split of a projection's output rows (QKV, GDN-input, gate/up)."""
    if out_rows % (world * granule) != 0:
        raise ValueError(f"{out_rows} rows do not split into {world} shards of a multiple of {granule}")
    rows = out_rows // world
    return Shard(rows, rank * rows)


def reduction_shard(columns: int, world: int, rank: int, granule: int = 64) -> Shard:
    """Row-parallel split of the down projection's reduction length (NVFP4: whole groups of
    four 16-column scale blocks per shard)."""
    if columns % (world * granule) != 0:
        raise ValueError(f"{columns} columns do not split into {world} shards of a multiple of {granule}")
    cols = columns // world
    return Shard(cols, rank * cols)


def gather_pairs(pairs: torch.Tensor, gathered: torch.Tensor, group=None) -> None:
    """All-gather of the per-rank ``[rows, 2]`` int32 pair planes into ``[world, rows, 2]``."""
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        gathered.view(-1)[: pairs.numel()].copy_(pairs.view(-1))
        return
    dist.all_gather_into_tensor(gathered.view(-1), pairs.view(-1), group=group)


def alloc_exchange(rows: int, world: int, device, group=None):
    """Symmetric peer-mapped exchange buffer for the fused argmax exchange: returns
    ``(buffer, handle, addresses)`` where ``addresses[i]`` is rank i's buffer as mapped in this
    process (torch symmetric memory over NVLink peer access).  Collective: every rank calls it."""
    import torch.distributed._symmetric_memory as symm

    from .ops import exchange_bytes

    words = (exchange_bytes(rows, world) + 7) // 8
    buf = symm.empty(words, dtype=torch.int64, device=device)
    buf.zero_()
    torch.cuda.synchronize()
    grp = group if group is not None else dist.group.WORLD
    try:
        handle = symm.rendezvous(buf, grp)
    except TypeError:
        handle = symm.rendezvous(buf, grp.group_name)
    addresses = [int(a) for a in handle.buffer_ptrs]
    if len(addresses) != world:
        raise RuntimeError("symmetric memory returned %d peer addresses for %d ranks" % (len(addresses), world))
    dist.barrier(group=group)
    return buf, handle, addresses


def alloc_peer_sum(capacity_values: int, world: int, device, group=None):
    """Symmetric peer-mapped exchange buffer for :func:`tuiskollm_b200.ops.peer_sum_bf16`:
    returns ``(buffer, handle, addresses)`` as :func:`alloc_exchange` does.  Collective."""
    import torch.distributed._symmetric_memory as symm

    from .ops import peer_sum_bytes

    words = (peer_sum_bytes(capacity_values, world) + 7) // 8
    buf = symm.empty(words, dtype=torch.int64, device=device)
    buf.zero_()
    torch.cuda.synchronize()
    grp = group if group is not None else dist.group.WORLD
    try:
        handle = symm.rendezvous(buf, grp)
    except TypeError:
        handle = symm.rendezvous(buf, grp.group_name)
    addresses = [int(a) for a in handle.buffer_ptrs]
    if len(addresses) != world:
        raise RuntimeError("symmetric memory returned %d peer addresses for %d ranks" % (len(addresses), world))
    dist.barrier(group=group)
    return buf, handle, addresses


class ShardedLmHead:
    """One rank's part of the vocabulary-sharded LM head with fused greedy selection."""

    def __init__(self, context, vocab: int, rank: int = 0, world: int = 1, group=None,
                 peer_addresses=None):
        """``peer_addresses`` (from :func:`alloc_exchange`) selects the fused peer-store
        exchange; without it the pairs travel through one NCCL all-gather."""
        from .ops import LmHeadOp

        self.shard = vocab_shard(vocab, world, rank)
        self.world = world
        self.rank = rank
        self.group = group
        self.peer_addresses = peer_addresses
        self.op = LmHeadOp(context, self.shard.rows, self.shard.offset)

    def launch(self, stream, rows, input, activation_codes, activation_scales, weight_codes,
               weight_scales, output, logits_f32, argmax_scratch, pairs, gathered, merged):
        """Projection + per-shard argmax, then (world > 1) all-gather + merge into ``merged``."""
        if self.world > 1 and self.peer_addresses is not None:
            self.op.launch_sharded(stream, rows, input, activation_codes, activation_scales,
                                   weight_codes, weight_scales, output, logits_f32, argmax_scratch,
                                   self.world, self.rank, self.peer_addresses, merged)
            return merged
        self.op.launch(stream, rows, input, activation_codes, activation_scales, weight_codes,
                       weight_scales, output, logits_f32, argmax_scratch, pairs)
        if self.world > 1:
            gather_pairs(pairs, gathered, self.group)
            self.op.merge(stream, rows, self.world, gathered, merged)
        return merged if self.world > 1 else pairs
