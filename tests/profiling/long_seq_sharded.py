"""BASELINE.json configs[4](b): one 131072-token sequence at the Qwen3-8B attention shape sharded by
KV head over the ranks (8 KV heads -> 8/G per GPU), NCCL all-gather of the per-head outputs.
Reports, per layer-step, the decode kernel time (max over ranks), its KV GB/s per GPU, and the
all-gather latency separately: behind the attention of the same step (includes the ranks'
launch skew) and alone, back to back.  Run with 1 process or under torchrun:

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
table = torch.from_numpy(rng.permutation(nb).astype(np.int32)[None, :]).to(dev)
kp = torch.randn(nb, hkv, BS, D, device=dev, dtype=torch.float16)
vp = torch.randn(nb, hkv, BS, D, device=dev, dtype=torch.float16)
q = torch.randn(1, hq * D, device=dev, dtype=torch.float16)
out = torch.empty_like(q)
lens = torch.tensor([CTX], dtype=torch.int32, device=dev)
lay = capi.layout_paged(capi.KPX_F16, hkv, D, BS, nb)
nbytes = capi.decode_workspace_bytes(1, hq, hkv)
ws = torch.empty(nbytes, dtype=torch.uint8, device=dev)
capi.workspace_init(ws, nbytes)


def attend():
    capi.paged_decode(out, q, kp, vp, lay, table, nb, lens, 0, 1, hq, 1 / np.sqrt(D), ws, nbytes)


for _ in range(3):
    attend()
    full = multigpu.gather_head_outputs(out, world)
torch.cuda.synchronize()
ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
t_attn, t_gather = [], []
for _ in range(ITERS):
    if world > 1:
        dist.barrier()
    ev[0].record()
    attend()
    ev[1].record()
    full = multigpu.gather_head_outputs(out, world)
    ev[2].record()
    torch.cuda.synchronize()
    t_attn.append(ev[0].elapsed_time(ev[1]))
    t_gather.append(ev[1].elapsed_time(ev[2]))
# the all-gather alone: back to back, so that the ranks' launch skew after the barrier (which the
# bracket above includes) drops out
n_alone = 50
torch.cuda.synchronize()
if world > 1:
    dist.barrier()
ev[0].record()
for _ in range(n_alone):
    full = multigpu.gather_head_outputs(out, world)
ev[1].record()
torch.cuda.synchronize()
alone = multigpu.max_over_ranks(ev[0].elapsed_time(ev[1]) / n_alone, world, dev)
attn = multigpu.max_over_ranks(float(np.median(t_attn)), world, dev)
gath = multigpu.max_over_ranks(float(np.median(t_gather)), world, dev)
assert capi.workspace_status(ws) == 0 and full.shape[-1] == H * D
if rank == 0:
    kv_bytes = CTX * hkv * D * 2 * 2
    print(json.dumps({"n_gpus": world, "kv_heads_per_gpu": hkv, "ctx": CTX, "attention_us": round(attn * 1e3, 1),
                      "kv_gbs_per_gpu": round(kv_bytes / attn / 1e6, 1), "allgather_us": round(gath * 1e3, 1),
                      "allgather_alone_us": round(alone * 1e3, 1),
                      "kv_mb_per_gpu": round(kv_bytes / 1e6, 1)}))
if world > 1:
    dist.destroy_process_group()
