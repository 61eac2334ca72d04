"""The NCCL head exchange of the KV-head-sharded mode through its C ABI (include/kpx_comm.h) on one
GPU: a communicator of one rank (the all-gather is then a copy), the single-row and the
many-row form, eagerly and captured in a CUDA graph with the attention launch it follows.  More
than one rank is exercised by tests/profiling/long_seq_sharded.py under torchrun."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_exchange_one_rank_eager_and_captured(native_libs):
    import torch
    from orinmllm_b200 import capi, multigpu
    if not (capi.LIB_DIR / "libkpx_comm.so").exists():
        pytest.skip("libkpx_comm.so not built (no NCCL at build time)")
    ex = multigpu.HeadExchange(1, 0)
    shard = torch.randn(1, 32 * 128, device="cuda").to(torch.float16)
    full = torch.zeros_like(shard)
    ex.gather(shard, full, 1)
    torch.cuda.synchronize()
    assert torch.equal(shard, full)
    rows = torch.randn(5, 4 * 128, device="cuda").to(torch.float16)
    full_rows = torch.zeros_like(rows)
    ex.gather(rows, full_rows, 5)
    torch.cuda.synchronize()
    assert torch.equal(rows, full_rows)
    # captured behind a decode launch: replay with new data gives the new rows
    nb, hkv, h = 40, 2, 8
    kp = torch.randn(nb, hkv, 16, 128, device="cuda").to(torch.float16)
    vp = torch.randn(nb, hkv, 16, 128, device="cuda").to(torch.float16)
    q = torch.randn(1, h * 128, device="cuda").to(torch.float16)
    out, gathered = torch.zeros_like(q), torch.zeros_like(q)
    table = torch.arange(nb, dtype=torch.int32, device="cuda")[None, :].contiguous()
    lens = torch.tensor([500], dtype=torch.int32, device="cuda")
    lay = capi.layout_paged(capi.KPX_F16, hkv, 128, 16, nb)
    nbytes = capi.decode_workspace_bytes(1, h, hkv)
    ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    capi.workspace_init(ws, nbytes)
    run = lambda s=None: (capi.paged_decode(out, q, kp, vp, lay, table, nb, lens, 0, 1, h, 0.088, ws, nbytes, stream=s),
                          ex.gather(out, gathered, 1, stream=s))
    run()
    torch.cuda.synchronize()
    eager = gathered.clone()
    side = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        run(side.cuda_stream)
    gathered.zero_()
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(gathered, eager)
    q.copy_(torch.randn_like(q))
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(gathered, out) and not torch.equal(gathered, eager)
    assert capi.workspace_status(ws) == 0
    del graph  # before the communicator: captured work keeps it alive
    torch.cuda.synchronize()
    ex.close()
