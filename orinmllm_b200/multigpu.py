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
    """Request ids served by `rank` when nothing is known about their sizes: contiguous, counts
    differ by at most one."""
    base, extra = divmod(num_requests, world)
    start = rank * base + min(rank, extra)
    return list(range(start, start + base + (1 if rank < extra else 0)))


def deal_requests_by_load(loads: Sequence[float], world: int, equal_counts: bool = False) -> List[List[int]]:
    """Request ids per rank, balanced by load (KV bytes = cached tokens): longest first, each to
    the rank that holds the least so far (ties to the lower rank).  With equal_counts every rank
    gets the same number of requests, give or take one (a fixed batch per GPU); a full rank is
    passed over.  Deterministic: every rank computes the same deal from the same loads."""
    n = len(loads)
    order = sorted(range(n), key=lambda i: (-float(loads[i]), i))
    cap = [(n // world) + (1 if r < n % world else 0) for r in range(world)] if equal_counts else [n] * world
    held = [0.0] * world
    out: List[List[int]] = [[] for _ in range(world)]
    for i in order:
        r = min((r for r in range(world) if len(out[r]) < cap[r]), key=lambda r: (held[r], r))
        out[r].append(i)
        held[r] += float(loads[i])
    return [sorted(ids) for ids in out]


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
    [batch, q_heads * head_size] (head-major, rank order = head order) through
    torch.distributed: the form the CPU (gloo) tests of the sharding arithmetic use.  On GPUs
    the exchange is HeadExchange (C++ / NCCL on the kernel's stream, no allocation)."""
    import torch
    import torch.distributed as dist
    if world == 1:
        return out_shard
    parts = [torch.empty_like(out_shard) for _ in range(world)]
    dist.all_gather(parts, out_shard.contiguous())
    return torch.cat(parts, dim=-1)


class HeadExchange:
    """The all-gather of per-head attention outputs of the KV-head-sharded mode through the C ABI
    of include/kpx_comm.h (lib/libkpx_comm.so: NCCL issued from C++ on the caller's stream, into a
    buffer the caller owns; capturable with the attention launch it follows).  torch.distributed
    only carries the 128-byte communicator id to the ranks."""

    def __init__(self, world: int, rank: int):
        import ctypes as C
        import torch.distributed as dist
        from . import capi
        path = capi.LIB_DIR / "libkpx_comm.so"
        if not path.exists():
            raise RuntimeError(f"{path} is missing: build it (python -m orinmllm_b200.build; needs NCCL)")
        self.lib = C.CDLL(str(path))
        self.lib.kpx_comm_make_id.argtypes = [C.c_void_p]
        self.lib.kpx_comm_create.argtypes = [C.POINTER(C.c_void_p), C.c_void_p, C.c_int32, C.c_int32]
        self.lib.kpx_comm_destroy.argtypes = [C.c_void_p]
        self.lib.kpx_allgather_heads.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p]
        self.lib.kpx_allgather_head_rows.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int64,
                                                     C.c_void_p]
        self.world, self.rank = world, rank
        ident = C.create_string_buffer(128)
        if rank == 0:
            capi.check(self.lib.kpx_comm_make_id(ident), "kpx_comm_make_id")
        if world > 1:
            box = [bytes(ident.raw)]
            dist.broadcast_object_list(box, src=0)
            ident = C.create_string_buffer(box[0], 128)
        handle = C.c_void_p()
        capi.check(self.lib.kpx_comm_create(C.byref(handle), ident, world, rank), "kpx_comm_create")
        self._h = handle

    def gather(self, shard, full, batch: int = 1, stream=None) -> None:
        """shard [batch, heads_per_rank*head_size] of this rank -> full [batch, q_heads*head_size]."""
        from . import capi
        row_bytes = shard.numel() * shard.element_size() // batch
        if batch == 1:
            rc = self.lib.kpx_allgather_heads(self._h, capi.ptr(shard), capi.ptr(full), row_bytes, capi._stream(stream))
        else:
            rc = self.lib.kpx_allgather_head_rows(self._h, capi.ptr(shard), capi.ptr(full), batch, row_bytes,
                                                  capi._stream(stream))
        capi.check(rc, "kpx_allgather_heads")

    def close(self):
        if getattr(self, "_h", None):
            self.lib.kpx_comm_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


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
