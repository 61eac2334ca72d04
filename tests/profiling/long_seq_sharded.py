"""One 131072-token sequence at the Qwen3-8B attention shape sharded by KV head over the ranks
(8 KV heads -> 8/G per GPU), with the all-gather of the per-head outputs issued from C++ (NCCL on
the attention's stream, include/kpx_comm.h).  Checks the gathered row on rank 0 against the CPU
oracle, then reports, per layer-step: the decode kernel time (max over ranks) and its KV GB/s per
GPU; the exchange behind the attention of the same step (includes the ranks' launch skew); the
exchange alone, back to back; and attention + exchange replayed as one CUDA graph.  Run with 1
process or under torchrun:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node G --master-addr 127.0.0.1 \
        tests/profiling/long_seq_sharded.py
"""
import json
import os
import sys
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))
from orinmllm_b200 import capi, multigpu  # noqa: E402

H, HKV, D, BS, CTX, ITERS = 32, 8, 128, 16, 131072, 20
rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
local = int(os.environ.get("LOCAL_RANK", 0))
torch.cuda.set_device(local)
dev = torch.device("cuda", local)
if world > 1:
    dist.init_process_group("nccl", device_id=dev)
kv_r, q_r = multigpu.kv_head_shard(rank, world, H, HKV)
hkv, hq = len(kv_r), len(q_r)
nb = CTX // BS
rng = np.random.default_rng(5)                      # same table on every rank (replicated)
perm = rng.permutation(nb).astype(np.int32)
table = torch.from_numpy(perm[None, :].copy()).to(dev)
# the whole sequence's K/V and the query from one seed on every rank; a rank keeps its heads
g = torch.Generator(device=dev).manual_seed(11)
kp_all = torch.randn(nb, HKV, BS, D, generator=g, device=dev, dtype=torch.float32).to(torch.float16)
vp_all = torch.randn(nb, HKV, BS, D, generator=g, device=dev, dtype=torch.float32).to(torch.float16)
q_all = torch.randn(1, H * D, generator=g, device=dev, dtype=torch.float32).to(torch.float16)
kp = kp_all[:, kv_r.start:kv_r.stop].contiguous()
vp = vp_all[:, kv_r.start:kv_r.stop].contiguous()
q = q_all[:, q_r.start * D:q_r.stop * D].contiguous()
if rank != 0:
    del kp_all, vp_all
out = torch.empty_like(q)
full = torch.zeros(1, H * D, device=dev, dtype=torch.float16)
lens = torch.tensor([CTX], dtype=torch.int32, device=dev)
lay = capi.layout_paged(capi.KPX_F16, hkv, D, BS, nb)
nbytes = capi.decode_workspace_bytes(1, hq, hkv)
ws = torch.empty(nbytes, dtype=torch.uint8, device=dev)
capi.workspace_init(ws, nbytes)
exchange = multigpu.HeadExchange(world, rank)


def attend(stream=None):
    capi.paged_decode(out, q, kp, vp, lay, table, nb, lens, 0, 1, hq, 1 / np.sqrt(D), ws, nbytes, stream=stream)


def gather(stream=None):
    exchange.gather(out, full, 1, stream=stream)


for _ in range(3):
    attend()
    gather()
torch.cuda.synchronize()
# ---- correctness of the gathered row (rank 0 holds the whole sequence for this)
if rank == 0:
    from tests import kvtest
    oracle = kvtest.load_oracle()
    ref = oracle.paged_decode(q_all.float().cpu().numpy(), kp_all.float().cpu().numpy(), vp_all.float().cpu().numpy(),
                              perm[None, :], np.array([CTX], np.int32), H, HKV, D, BS, threads=oracle.max_threads())
    max_abs, max_rel = kvtest.assert_attention_close(full.float().cpu().numpy(), ref, "gathered row")
    del kp_all, vp_all
else:
    max_abs = max_rel = 0.0
# ---- the many-row form of the exchange (rows in head order on every rank)
rows = 3
mine = torch.full((rows, hq * D), float(rank + 1), device=dev, dtype=torch.float16) + \
    torch.arange(rows, device=dev, dtype=torch.float16)[:, None]
wide = torch.zeros(rows, H * D, device=dev, dtype=torch.float16)
exchange.gather(mine, wide, rows)
torch.cuda.synchronize()
for r in range(world):
    want = float(r + 1) + torch.arange(rows, device=dev, dtype=torch.float16)[:, None]
    assert torch.equal(wide[:, r * hq * D:(r + 1) * hq * D], want.expand(rows, hq * D)), "row exchange"
ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
t_attn, t_gather = [], []
for _ in range(ITERS):
    if world > 1:
        dist.barrier()
    ev[0].record()
    attend()
    ev[1].record()
    gather()
    ev[2].record()
    torch.cuda.synchronize()
    t_attn.append(ev[0].elapsed_time(ev[1]))
    t_gather.append(ev[1].elapsed_time(ev[2]))
# the exchange alone: back to back, so that the ranks' launch skew after the barrier (which the
# bracket above includes) drops out
n_alone = 50
torch.cuda.synchronize()
if world > 1:
    dist.barrier()
ev[0].record()
for _ in range(n_alone):
    gather()
ev[1].record()
torch.cuda.synchronize()
alone = multigpu.max_over_ranks(ev[0].elapsed_time(ev[1]) / n_alone, world, dev)
# attention + exchange of `layers` layer-steps as one CUDA graph (what a decode step replays)
layers = 36
side = torch.cuda.Stream(dev)
graph = torch.cuda.CUDAGraph()
with torch.cuda.graph(graph, stream=side):
    for _ in range(layers):
        attend(side.cuda_stream)
        gather(side.cuda_stream)
for _ in range(2):
    graph.replay()
torch.cuda.synchronize()
if world > 1:
    dist.barrier()
ev[0].record()
for _ in range(5):
    graph.replay()
ev[1].record()
torch.cuda.synchronize()
step = multigpu.max_over_ranks(ev[0].elapsed_time(ev[1]) / 5 / layers, world, dev)
attn = multigpu.max_over_ranks(float(np.median(t_attn)), world, dev)
gath = multigpu.max_over_ranks(float(np.median(t_gather)), world, dev)
assert capi.workspace_status(ws) == 0
if rank == 0:
    kv_bytes = CTX * hkv * D * 2 * 2
    print(json.dumps({"n_gpus": world, "kv_heads_per_gpu": hkv, "ctx": CTX, "attention_us": round(attn * 1e3, 1),
                      "kv_gbs_per_gpu": round(kv_bytes / attn / 1e6, 1), "exchange_behind_attention_us": round(gath * 1e3, 1),
                      "exchange_alone_us": round(alone * 1e3, 1),
                      "graph_layer_step_us": round(step * 1e3, 1),
                      "graph_kv_gbs_per_gpu": round(kv_bytes / step / 1e6, 1),
                      "kv_mb_per_gpu": round(kv_bytes / 1e6, 1), "gathered_row_max_abs_err": max_abs}))
# a captured graph keeps the communicator's work alive: it goes first, or destroying the
# communicator waits for ever
del graph
torch.cuda.synchronize()
exchange.close()
if world > 1:
    dist.destroy_process_group()
