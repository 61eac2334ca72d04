"""One layer of the headline decode workload (Qwen3-8B attention shape, bs=64, ctx U[128,4096],
fp16, block 16; ~0.7 GB of pools) launched a few times: the small case the ncu captures
summarised under profiles/ were taken on.

    python tests/profiling/decode_case.py [launches] [large|overlapped]

`overlapped` launches the three-small-CTAs-per-SM form (kpx_paged_decode_overlapped), `large`
(default) the one-CTA-per-SM form (kpx_paged_decode).
"""
import sys
from pathlib import Path

import numpy as np
import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))
from orinmllm_b200 import capi  # noqa: E402

B, H, HKV = 64, 32, 8
launches = int(sys.argv[1]) if len(sys.argv) > 1 else 3
decode = capi.paged_decode_overlapped if len(sys.argv) > 2 and sys.argv[2] == "overlapped" else capi.paged_decode
rng = np.random.default_rng(2024)
lens = rng.integers(128, 4097, size=B).astype(np.int32)
nblk = (lens + 15) // 16
nb = int(np.ceil(nblk.sum() * 1.25))
perm = rng.permutation(nb).astype(np.int32)
table = np.full((B, int(nblk.max())), -1, np.int32)
c = 0
for i, n in enumerate(nblk):
    table[i, :n] = perm[c:c + n]
    c += n
kp = torch.randn(nb, HKV, 16, 128, device="cuda", dtype=torch.float16)
vp = torch.randn(nb, HKV, 16, 128, device="cuda", dtype=torch.float16)
q = torch.randn(B, H * 128, device="cuda", dtype=torch.float16)
out = torch.empty_like(q)
lay = capi.layout_paged(capi.KPX_F16, HKV, 128, 16, nb)
nbytes = capi.decode_workspace_bytes(B, H, HKV)
ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
capi.workspace_init(ws, nbytes)
bt, sl = torch.from_numpy(table).cuda(), torch.from_numpy(lens).cuda()
for _ in range(launches):
    decode(out, q, kp, vp, lay, bt, table.shape[1], sl, 0, B, H, 1 / np.sqrt(128), ws, nbytes)
torch.cuda.synchronize()
print("status", capi.workspace_status(ws), "tokens", int(lens.sum()), "kv_bytes", int(lens.sum()) * HKV * 128 * 4)
