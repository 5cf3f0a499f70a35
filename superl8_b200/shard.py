"""Sharding of the path's independent units across the GPUs of one box.

A unit is one (batch element, KV head) with its Hq/Hkv query heads: its K mean, K/V tiles,
scales and outputs are private to it (the reference reduces K over keys only,
superl8/quant/core.py:81-85, and maps query heads to KV heads by integer division,
csrc/include/attn_int8_fwd.cuh:72), so ranks never exchange data on the hot path.  The only
collectives are the ones a harness wants: a barrier, the max-over-ranks of a time, and a
gather of outputs for a correctness check.
"""

from __future__ import annotations

import torch
import torch.distributed as dist


def unit_range(n_units: int, world: int, rank: int) -> range:
    """Contiguous, balanced slice of ``n_units`` for ``rank`` (sizes differ by at most one)."""
    if not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world of {world}")
    base, extra = divmod(n_units, world)
    start = rank * base + min(rank, extra)
    return range(start, start + base + (1 if rank < extra else 0))


def batch_range(B: int, Hkv: int, world: int, rank: int):
    """Shard (batch, kv-head) units but keep whole batch elements together when possible:
    returns (batch_range, kv_head_range).  world <= B splits batches; otherwise world must be a
    multiple of B and every batch element's KV heads are split across world // B ranks."""
    if world <= B:
        return unit_range(B, world, rank), range(Hkv)
    if world % B or Hkv % (world // B):
        raise ValueError(f"cannot split B={B}, Hkv={Hkv} over {world} ranks")
    per = world // B
    b = rank // per
    return range(b, b + 1), unit_range(Hkv, per, rank % per)


def balance_by_length(lengths, world: int) -> list[list[int]]:
    """Longest-first greedy assignment of sequences to ranks (decode: work is proportional to
    the context length).  Returns, per rank, the list of sequence indices it owns."""
    order = sorted(range(len(lengths)), key=lambda i: (-int(lengths[i]), i))
    loads = [0] * world
    owned: list[list[int]] = [[] for _ in range(world)]
    for i in order:
        r = min(range(world), key=lambda k: (loads[k], k))
        owned[r].append(i)
        loads[r] += int(lengths[i])
    for o in owned:
        o.sort()
    return owned


def max_over_ranks(value: float, device=None) -> float:
    """A job is as slow as its slowest rank."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return float(value)
    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def gather_batch(local: torch.Tensor) -> torch.Tensor:
    """All-gathers equally shaped per-rank outputs along dim 0 (correctness checks only)."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return local
    parts = [torch.empty_like(local) for _ in range(dist.get_world_size())]
    dist.all_gather(parts, local.contiguous())
    return torch.cat(parts, dim=0)
