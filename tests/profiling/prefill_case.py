"""BASELINE configs[2] (chunked prefill at the Qwen2.5-7B attention shape: 28 Q / 4 KV heads,
d=128, bf16, 4 sequences of 2048 tokens in 512-token chunks, block 16, seeded random block
placement) on random data: times every chunk call with CUDA events and prints TFLOP/s on the
causal-exact FLOP count.  Also the small case the ncu capture under profiles/ was taken on.

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
total_ms, total_flop = 0.0, 0.0
for rep in range(reps):
    for c in range(PROMPT // CHUNK):
        sp = np.full(B, c * CHUNK, np.int32)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        capi.paged_prefill(out, q, kp, vp, lay, bt, table.shape[1], cu, sp, B, H, 1 / np.sqrt(D), ws, nbytes)
        e1.record()
        torch.cuda.synchronize()
        flop = B * 4.0 * H * D * sum(c * CHUNK + i + 1 for i in range(CHUNK))
        ms = e0.elapsed_time(e1)
        if rep == reps - 1:
            print(f"chunk {c}: {ms * 1e3:8.1f} us  {flop / ms / 1e9:8.1f} TFLOP/s (causal-exact)")
        if rep > 0 or reps == 1:
            total_ms += ms
            total_flop += flop
print("status", capi.workspace_status(ws))
print(f"all chunks: {total_flop / total_ms / 1e9:.1f} TFLOP/s, {total_ms / max(1, reps - 1) * 1e3:.1f} us per 4x2048-token prefill layer")
