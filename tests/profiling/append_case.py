"""The append kernels alone at Qwen3-8B attention shape (8 KV heads x 128, fp16, block 16), the
new rows of consecutive positions filling blocks that sit at seeded random places in the pool
(64 tokens: one slot each in 64 different blocks, as in a decode step):

  plain    kpx_append: K and V rows copied into the pools (read 4 KB + write 4 KB per token)
  rope     kpx_rope_append: q (8 KB) and k rotated in place, k and v stored into the pools
           (read 16 KB, write 10 KB in place + 4 KB to the pools per token: 26 KB counted as
           q+k+v read, q+k written back, k+v stored = 8+2+2 + 8+2 + 2+2 KB)

at three sizes: 64 tokens (one decode step of the headline batch), 2048 (one prefill step of
4 x 512) and 131072 (bulk, larger than L2: the one the HBM figure is read from).

    python tests/profiling/append_case.py [bulk_tokens] [launches]

Prints device time (CUDA events, median of the launches) and algorithmic GB/s per case.
"""
import sys
from pathlib import Path

import numpy as np
import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))
from orinmllm_b200 import capi  # noqa: E402

H, HKV, D, BS = 32, 8, 128, 16
bulk = int(sys.argv[1]) if len(sys.argv) > 1 else 131072
launches = int(sys.argv[2]) if len(sys.argv) > 2 else 5
rng = np.random.default_rng(77)
nb = int(np.ceil(bulk / BS * 1.25))
kp = torch.zeros(nb, HKV, BS, D, device="cuda", dtype=torch.float16)
vp = torch.zeros_like(kp)
lay = capi.layout_paged(capi.KPX_F16, HKV, D, BS, nb)
max_pos = 4096
sin = torch.empty(max_pos * D, device="cuda", dtype=torch.float32)
cos = torch.empty_like(sin)
capi.sin_cos_cache(sin, cos, D, max_pos, 1e6)
flush = torch.zeros(64 << 20, dtype=torch.int32, device="cuda")  # 256 MB, larger than L2; read, so it leaves no dirty lines


def timed(fn):
    ms = []
    for _ in range(launches):
        flush.sum()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ms.append(e0.elapsed_time(e1))
    return float(np.median(ms))


for n in (64, 2048, bulk):
    if n <= 64:
        sl = rng.permutation(nb)[:n].astype(np.int64) * BS + rng.integers(0, BS, n)
        ps = rng.integers(0, max_pos, n)
    else:
        blocks = rng.permutation(nb)[:(n + BS - 1) // BS].astype(np.int64)
        sl = (blocks[:, None] * BS + np.arange(BS)[None, :]).reshape(-1)[:n]
        ps = np.arange(n) % max_pos
    slots = torch.from_numpy(sl.astype(np.int64)).cuda()
    pos = torch.from_numpy(ps.astype(np.int32)).cuda()
    q = torch.randn(n, H * D, device="cuda", dtype=torch.float16)
    k = torch.randn(n, HKV * D, device="cuda", dtype=torch.float16)
    v = torch.randn(n, HKV * D, device="cuda", dtype=torch.float16)
    t = timed(lambda: capi.append(kp, vp, lay, k, v, slot_mapping=slots, num_tokens=n))
    b = n * HKV * D * 2 * 2 * 2
    print(f"plain  {n:7d} tokens: {t * 1e3:8.1f} us, {b / 1e6:8.2f} MB read+written = {b / t / 1e6:7.1f} GB/s")
    t = timed(lambda: capi.rope_append(q, k, v, H, pos, sin, cos, kp, vp, lay, slots, n))
    b = n * D * 2 * ((H + 2 * HKV) + (H + HKV) + 2 * HKV)
    print(f"rope   {n:7d} tokens: {t * 1e3:8.1f} us, {b / 1e6:8.2f} MB read+written = {b / t / 1e6:7.1f} GB/s")
    del q, k, v

# the same bytes as the bulk plain case moved by the framework's contiguous copy, for scale
src = torch.randn(2, bulk, HKV * D, device="cuda", dtype=torch.float16)
dst = torch.empty_like(src)
t = timed(lambda: dst.copy_(src))
b = src.numel() * 2 * 2
print(f"contiguous device copy of the same size: {t * 1e3:8.1f} us, {b / 1e6:8.2f} MB read+written = {b / t / 1e6:7.1f} GB/s")
