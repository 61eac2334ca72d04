"""The N > 1 host logic on CPU: world_size-2 gloo ranks (rendezvous on 127.0.0.1)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from orinmllm_b200 import multigpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q, kc, vc, result):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from tests import kvtest
    oracle = kvtest.load_oracle()
    H, HKV, D = 8, 4, 128
    n = kc.shape[0]
    # KV-head-sharded: this rank's KV heads and the query heads that read them
    kv_r, q_r = multigpu.kv_head_shard(rank, world, H, HKV)
    kcs = np.ascontiguousarray(kc.reshape(n, HKV, D)[:, kv_r.start:kv_r.stop].reshape(n, -1))
    vcs = np.ascontiguousarray(vc.reshape(n, HKV, D)[:, kv_r.start:kv_r.stop].reshape(n, -1))
    qs = np.ascontiguousarray(q.reshape(H, D)[q_r.start:q_r.stop].reshape(-1))
    out = oracle.mha(n - 1, len(q_r), 0, n, len(kv_r) * D, H // HKV, D, qs, kcs.reshape(-1), vcs.reshape(-1))
    full = multigpu.gather_head_outputs(torch.from_numpy(out)[None, :], world)
    # request-parallel bookkeeping: whole-job totals and max-over-ranks time
    mine = multigpu.deal_requests(11, world, rank)
    tot = multigpu.sum_over_ranks([float(len(mine)), 100.0 * (rank + 1)], world)
    worst = multigpu.max_over_ranks(5.0 + rank, world)
    if rank == 0:
        result.put((full.numpy(), tot, worst))
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_gloo_head_sharding_and_aggregation(oracle):
    rng = np.random.default_rng(0)
    H, HKV, D, n = 8, 4, 128, 70
    q = rng.standard_normal(H * D).astype(np.float32)
    kc = rng.standard_normal((n, HKV * D)).astype(np.float32)
    vc = rng.standard_normal((n, HKV * D)).astype(np.float32)
    ctx = mp.get_context("spawn")
    result = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q, kc, vc, result)) for r in range(2)]
    for p in procs:
        p.start()
    full, tot, worst = result.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    ref = oracle.mha(n - 1, H, 0, n, HKV * D, H // HKV, D, q, kc.reshape(-1), vc.reshape(-1))
    assert np.array_equal(full[0], ref)          # sharding by KV head is exact
    assert tot == [11.0, 300.0] and worst == 6.0


def test_request_dealing_and_prefix_routing():
    for world in (1, 2, 4, 8):
        seen = sorted(i for r in range(world) for i in multigpu.deal_requests(513, world, r))
        assert seen == list(range(513))
        sizes = [len(multigpu.deal_requests(513, world, r)) for r in range(world)]
        assert max(sizes) - min(sizes) <= 1
    prefix = list(range(100, 132))
    a = multigpu.route_by_prefix(prefix + [1, 2, 3], 8)
    b = multigpu.route_by_prefix(prefix + [9, 9], 8)
    assert a == b and 0 <= a < 8
    with pytest.raises(ValueError):
        multigpu.kv_head_shard(0, 3, 32, 8)
    kv, qh = multigpu.kv_head_shard(3, 4, 32, 8)
    assert (kv.start, kv.stop, qh.start, qh.stop) == (6, 8, 24, 32)


def test_dealing_by_load_balances_skewed_lengths():
    rng = np.random.default_rng(3)
    # a skewed set: a few very long requests among many short ones
    lens = np.concatenate([rng.integers(128, 600, 480), rng.integers(20000, 32768, 32)])
    rng.shuffle(lens)
    for world in (2, 4, 8):
        for equal in (False, True):
            deal = multigpu.deal_requests_by_load(lens, world, equal_counts=equal)
            assert sorted(i for ids in deal for i in ids) == list(range(len(lens)))
            loads = [int(lens[ids].sum()) for ids in deal]
            assert (max(loads) - min(loads)) / np.mean(loads) < 0.02, (world, equal, loads)
            if equal:
                assert {len(ids) for ids in deal} == {len(lens) // world}
        # contiguous dealing of the same set is far off balance
        naive = [int(lens[multigpu.deal_requests(len(lens), world, r)].sum()) for r in range(world)]
        assert (max(naive) - min(naive)) / np.mean(naive) > 0.05
    assert multigpu.deal_requests_by_load([5.0, 1.0, 1.0], 2) == [[0], [1, 2]]


def _deal_worker(rank, world, port, result):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    # every rank draws the same global set and computes the same deal; the totals add up
    lens = np.random.default_rng(2024).integers(128, 4097, size=64 * world)
    mine = multigpu.deal_requests_by_load(lens, world, equal_counts=True)[rank]
    tot = multigpu.sum_over_ranks([float(len(mine)), float(lens[mine].sum())], world)
    if rank == 0:
        result.put((tot, float(lens.sum()), float(lens[mine].sum())))
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_gloo_dealing_by_load_is_consistent():
    ctx = mp.get_context("spawn")
    result = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_deal_worker, args=(r, 2, port, result)) for r in range(2)]
    for p in procs:
        p.start()
    tot, all_tokens, rank0_tokens = result.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert tot == [128.0, all_tokens]
    assert abs(rank0_tokens - all_tokens / 2) / all_tokens < 0.005
