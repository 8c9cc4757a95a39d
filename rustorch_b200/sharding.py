"""Host-side partitioning of the attention path across the GPUs of one box.

The reference has no multi-device attention (its NCCL layer is a single-rank stub,
crates/rustorch-cuda/src/nccl.rs:116-143).  The path shards in two ways:

* prefill and batched decode: (batch, head) units / sequences are independent — the unit the
  reference's rayon loop parallelises over (crates/rustorch-attention/src/cpu_forward.rs:219-226).
  Each rank takes a contiguous slab (`shard_units`) or a length-balanced set of sequences
  (`balance_sequences`); no collective is needed.
* long-context decode: the KV range is split contiguously (`kv_shard`); every rank produces a
  normalised partial (O f32 [rows, D], LSE [rows]), the ranks exchange one packed record each
  (`pack_partial` + `all_gather_partials`) and merge locally with the combine_tiles algebra
  (crates/rustorch-attention/src/online_softmax.rs:105-131).

Everything here is plain torch / torch.distributed plumbing and runs on CPU (gloo) as well as on
GPUs (nccl); the arithmetic lives in the CUDA library.
"""
from __future__ import annotations

from typing import List, Sequence, Tuple


def shard_units(n_units: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous, balanced [begin, end) slice of `n_units` independent units for `rank`."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError(f"bad rank {rank} for world size {world}")
    base, extra = divmod(max(n_units, 0), world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def kv_shard(kv_len: int, world: int, rank: int, align: int = 1) -> Tuple[int, int]:
    """Contiguous KV range [begin, end) of `rank`; shard boundaries are multiples of `align`."""
    blocks = (max(kv_len, 0) + align - 1) // align
    b0, b1 = shard_units(blocks, world, rank)
    return min(b0 * align, kv_len), min(b1 * align, kv_len)


def balance_sequences(costs: Sequence[float], world: int) -> List[List[int]]:
    """Longest-processing-time assignment of sequences to ranks; returns the indices of each rank.

    `costs[i]` is the work of sequence i (sum of lengths for decode, length squared for causal
    prefill).  Greedy LPT keeps the heaviest rank within 4/3 of the optimum.
    """
    loads = [0.0] * world
    out: List[List[int]] = [[] for _ in range(world)]
    for i in sorted(range(len(costs)), key=lambda j: (-costs[j], j)):
        r = min(range(world), key=lambda x: (loads[x], x))
        out[r].append(i)
        loads[r] += float(costs[i])
    return [sorted(ix) for ix in out]


def pack_partial(o, lse):
    """(O [rows, D] f32, LSE [rows] f32) -> one contiguous record [rows, D + 1]."""
    import torch
    return torch.cat([o, lse.unsqueeze(-1)], dim=-1).contiguous()


def unpack_partials(records):
    """[R, rows, D + 1] -> (O [R, rows, D], LSE [R, rows]), both contiguous."""
    return records[..., :-1].contiguous(), records[..., -1].contiguous()


def all_gather_partials(record, group=None):
    """All-gather one packed record per rank -> [world, rows, D + 1] (rank order = KV order)."""
    import torch
    import torch.distributed as dist
    world = dist.get_world_size(group)
    out = torch.empty((world,) + tuple(record.shape), dtype=record.dtype, device=record.device)
    if dist.get_backend(group) == "nccl":
        dist.all_gather_into_tensor(out, record.contiguous(), group=group)
    else:  # gloo has no flat-tensor all-gather
        dist.all_gather(list(out.unbind(0)), record.contiguous(), group=group)
    return out
