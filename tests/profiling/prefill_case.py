"""Chunked prefill at the Qwen2.5-7B attention shape (28 Q / 4 KV heads,
d=128, bf16, 4 sequences of 2048 tokens in 512-token chunks, block 16, seeded random block
placement) on random data: times every chunk call with CUDA events (alone and synchronised, then
queued back to back for the device time) and prints TFLOP/s on the causal-exact FLOP count.  Also the small case the ncu capture under profiles/ was taken on.

    python tests/profiling/prefill_case.py [reps] [path]      path: 0 tensor-core tiles, 1 streaming
"""
import sys
from pathlib import Path

import numpy as np
import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))
from orinmllm_b200 import capi  # noqa: E402

reps = int(sys.argv[1]) if len(sys.argv) > 1 else 3
path = int(sys.argv[2]) if len(sys.argv) > 2 else 0
capi.lib().kpx_internal_set_prefill_path(path)
H, HKV, D, BS, B, PROMPT, CHUNK = 28, 4, 128, 16, 4, 2048, 512
rng = np.random.default_rng(3)
nb = int(B * PROMPT / BS * 1.25)
perm = rng.permutation(nb).astype(np.int32)
table = perm[:B * PROMPT // BS].reshape(B, PROMPT // BS).copy()
dt = torch.bfloat16
kp = torch.randn(nb, HKV, BS, D, device="cuda", dtype=dt)
vp = torch.randn(nb, HKV, BS, D, device="cuda", dtype=dt)
q = torch.randn(B * CHUNK, H * D, device="cuda", dtype=dt)
out = torch.empty_like(q)
lay = capi.layout_paged(capi.KPX_BF16, HKV, D, BS, nb)
bt = torch.from_numpy(table).cuda()
cu = (np.arange(B + 1) * CHUNK).astype(np.int32)
nbytes = capi.prefill_workspace_bytes(B * CHUNK, H, HKV, D)
ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
capi.workspace_init(ws, nbytes)
NCH = PROMPT // CHUNK
flops = [B * 4.0 * H * D * sum(c * CHUNK + i + 1 for i in range(CHUNK)) for c in range(NCH)]
starts = [np.full(B, c * CHUNK, np.int32) for c in range(NCH)]


def call(c):
    capi.paged_prefill(out, q, kp, vp, lay, bt, table.shape[1], cu, starts[c], B, H, 1 / np.sqrt(D), ws, nbytes)


# (1) one call at a time, synchronised: what a caller that waits for each chunk sees (host
#     work of the call included)
for rep in range(reps):
    for c in range(NCH):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        call(c)
        e1.record()
        torch.cuda.synchronize()
        if rep == reps - 1:
            ms = e0.elapsed_time(e1)
            print(f"chunk {c} alone : {ms * 1e3:8.1f} us  {flops[c] / ms / 1e9:8.1f} TFLOP/s (causal-exact)")
# (2) device time: each chunk's call queued `queued` times back to back behind a long-running
#     filler so that the host is ahead of the device; events bracket the queued calls
queued = 20
filler = torch.empty(1 << 28, dtype=torch.float32, device="cuda")
total_ms = 0.0
for c in range(NCH):
    for _ in range(3):
        filler.add_(1.0)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(queued):
        call(c)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / queued
    total_ms += ms
    print(f"chunk {c} queued: {ms * 1e3:8.1f} us  {flops[c] / ms / 1e9:8.1f} TFLOP/s (causal-exact)")
print("status", capi.workspace_status(ws))
print(f"all chunks (device time): {sum(flops) / total_ms / 1e9:.1f} TFLOP/s, {total_ms * 1e3:.1f} us per 4x2048-token prefill layer")

# (3) the chunk step as the path runs it: RoPE + append of the chunk's 4 x 512 new rows into the
#     pool, then the attention call; queued as in (2)
k_new = torch.randn(B * CHUNK, HKV * D, device="cuda", dtype=dt)
v_new = torch.randn(B * CHUNK, HKV * D, device="cuda", dtype=dt)
sin = torch.empty(PROMPT * D, device="cuda", dtype=torch.float32)
cos = torch.empty_like(sin)
capi.sin_cos_cache(sin, cos, D, PROMPT, 1e6)
step_ms = 0.0
for c in range(NCH):
    pos = np.tile(np.arange(c * CHUNK, (c + 1) * CHUNK), B).astype(np.int32)
    seq = np.repeat(np.arange(B), CHUNK)
    slots = table[seq, pos // BS].astype(np.int64) * BS + pos % BS
    d_pos, d_slots = torch.from_numpy(pos).cuda(), torch.from_numpy(slots).cuda()
    for _ in range(3):
        filler.add_(1.0)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(queued):
        capi.rope_append(q, k_new, v_new, H, d_pos, sin, cos, kp, vp, lay, d_slots, B * CHUNK)
        call(c)
    e1.record()
    torch.cuda.synchronize()
    step_ms += e0.elapsed_time(e1) / queued
print(f"all chunks with RoPE+append (device time): {step_ms * 1e3:.1f} us per layer = "
      f"{B * PROMPT / step_ms / 1e3:.1f} M tokens/s per layer, {sum(flops) / step_ms / 1e9:.1f} TFLOP/s of attention")
