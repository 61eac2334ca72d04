"""Host-side helpers for the two multi-GPU modes of the KV-cache path.  One process per GPU;
`torch.distributed` is plumbing only (NCCL on GPUs, gloo in the CPU tests).

* request-parallel (default): sequences are independent, so requests are dealt to ranks and
  every rank runs the single-GPU path on its own pool, block tables and radix tree.  No
  collective on the data path; requests that share a prefix are routed to the same rank so
  that prefix blocks are shared where they live.
* KV-head-sharded (one very long sequence): rank r holds KV heads [r*Hkv/G, (r+1)*Hkv/G) of
  every block and the query heads that read them; attention is exact per head, the only
  exchange is an all-gather of the per-head outputs.
"""
from __future__ import annotations

import hashlib
from typing import List, Sequence, Tuple


def deal_requests(num_requests: int, world: int, rank: int) -> List[int]:
    """Request ids served by `rank`: contiguous, sizes differ by at most one."""
    base, extra = divmod(num_requests, world)
    start = rank * base + min(rank, extra)
    return list(range(start, start + base + (1 if rank < extra else 0)))


def route_by_prefix(tokens: Sequence[int], world: int, prefix_len: int = 16) -> int:
    """Rank that owns a request: a hash of its first `prefix_len` token ids, so requests with a
    common prefix land on the rank whose radix tree already holds that prefix."""
    head = ",".join(str(int(t)) for t in tokens[:prefix_len]).encode()
    return int.from_bytes(hashlib.blake2b(head, digest_size=8).digest(), "little") % world


def kv_head_shard(rank: int, world: int, q_heads: int, kv_heads: int) -> Tuple[range, range]:
    """(kv head range, q head range) of `rank`; kv_heads must be divisible by world."""
    if kv_heads % world:
        raise ValueError(f"{kv_heads} KV heads cannot be split over {world} ranks")
    per = kv_heads // world
    mul = q_heads // kv_heads
    return range(rank * per, (rank + 1) * per), range(rank * per * mul, (rank + 1) * per * mul)


def gather_head_outputs(out_shard, world: int):
    """All-gather of per-rank attention outputs [batch, q_heads/world * head_size] into
    [batch, q_heads * head_size] (head-major, rank order = head order)."""
    import torch
    import torch.distributed as dist
    if world == 1:
        return out_shard
    parts = [torch.empty_like(out_shard) for _ in range(world)]
    dist.all_gather(parts, out_shard.contiguous())
    return torch.cat(parts, dim=-1)


def max_over_ranks(value: float, world: int, device=None) -> float:
    import torch
    import torch.distributed as dist
    if world == 1:
        return value
    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def sum_over_ranks(values: Sequence[float], world: int, device=None) -> List[float]:
    import torch
    import torch.distributed as dist
    t = torch.tensor(list(values), dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(t)
    return t.tolist()
