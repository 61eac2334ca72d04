"""A decode step (RoPE + append + paged decode, several layers) captured once in a CUDA graph and
replayed with new tokens: the entry points take every per-step quantity (positions, slots, block
table, lengths) from device memory and make no allocation or host synchronisation, as the
reference requires of its graph path (kuiper/include/base/cuda_graph.h:59-290,
qwen_base.cpp:683-756).  Replays must give bit-identical results to the same calls made eagerly."""
import numpy as np
import pytest

from tests import kvtest

pytestmark = pytest.mark.gpu


def test_decode_step_replays_from_a_cuda_graph(native_libs):
    import torch
    from orinmllm_b200 import capi, kvm

    L, H, HKV, D, BS, B = 3, 32, 8, 128, 16, 12
    nb = 600
    rng = np.random.default_rng(8)
    g = torch.Generator(device="cuda").manual_seed(1)
    mgr = kvm.KvManager(nb, BS, seed=2)
    lay = capi.layout_paged(capi.KPX_F16, HKV, D, BS, nb)
    kp = torch.randn(L, nb, HKV, BS, D, generator=g, device="cuda", dtype=torch.float16)
    vp = torch.randn(L, nb, HKV, BS, D, generator=g, device="cuda", dtype=torch.float16)
    sin = torch.empty(4096 * D, device="cuda", dtype=torch.float32)
    cos = torch.empty_like(sin)
    capi.sin_cos_cache(sin, cos, D, 4096, 1e6)
    seqs = [mgr.add_sequence() for _ in range(B)]
    lens = rng.integers(5, 600, B)
    for s, n in zip(seqs, lens):
        mgr.append(s, int(n))
    width = 48  # fixed table width of the captured launch (blocks for up to 768 tokens)
    # device-resident step inputs, updated in place between replays
    d_pos = torch.zeros(B, dtype=torch.int32, device="cuda")
    d_slots = torch.zeros(B, dtype=torch.int64, device="cuda")
    d_lens = torch.zeros(B, dtype=torch.int32, device="cuda")
    d_table = torch.full((B, width), -1, dtype=torch.int32, device="cuda")
    d_q = torch.zeros(L, B, H * D, device="cuda", dtype=torch.float16)
    d_k = torch.zeros(L, B, HKV * D, device="cuda", dtype=torch.float16)
    d_v = torch.zeros(L, B, HKV * D, device="cuda", dtype=torch.float16)
    d_out = torch.zeros(L, B, H * D, device="cuda", dtype=torch.float16)
    nbytes = capi.decode_workspace_bytes(B, H, HKV)
    ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    capi.workspace_init(ws, nbytes)

    def next_inputs():
        slots = np.array([mgr.append(s, 1)[0] for s in seqs], np.int64)
        pos = np.array([mgr.length(s) - 1 for s in seqs], np.int32)
        d_pos.copy_(torch.from_numpy(pos))
        d_slots.copy_(torch.from_numpy(slots))
        d_lens.copy_(torch.from_numpy(pos + 1))
        d_table.copy_(torch.from_numpy(mgr.block_table(seqs, width)))
        d_q.copy_(torch.randn(d_q.shape, generator=g, device="cuda", dtype=torch.float32))
        d_k.copy_(torch.randn(d_k.shape, generator=g, device="cuda", dtype=torch.float32))
        d_v.copy_(torch.randn(d_v.shape, generator=g, device="cuda", dtype=torch.float32))

    def step(q, k, out, kpool, vpool):
        for l in range(L):
            capi.rope_append(q[l], k[l], d_v[l], H, d_pos, sin, cos, kpool[l], vpool[l], lay, d_slots, B)
            capi.paged_decode(out[l], q[l], kpool[l], vpool[l], lay, d_table, width, d_lens, 0, B, H,
                              1.0 / np.sqrt(D), ws, nbytes)

    # warm-up outside capture (first-use attribute calls, lazy module load)
    next_inputs()
    step(d_q.clone(), d_k.clone(), torch.empty_like(d_out), kp.clone(), vp.clone())
    torch.cuda.synchronize()

    graph = torch.cuda.CUDAGraph()
    # q and k are rotated in place by rope_append: the graph works on copies made inside it
    g_q, g_k = torch.empty_like(d_q), torch.empty_like(d_k)
    with torch.cuda.graph(graph):
        g_q.copy_(d_q)
        g_k.copy_(d_k)
        step(g_q, g_k, d_out, kp, vp)
    for _ in range(3):
        next_inputs()
        # eager reference on clones of the pools as they are before the step
        kp_ref, vp_ref = kp.clone(), vp.clone()
        out_ref = torch.empty_like(d_out)
        step(d_q.clone(), d_k.clone(), out_ref, kp_ref, vp_ref)
        graph.replay()
        torch.cuda.synchronize()
        assert capi.workspace_status(ws) == 0
        assert torch.equal(d_out, out_ref), "graph replay differs from the eager launches"
        assert torch.equal(kp, kp_ref) and torch.equal(vp, vp_ref), "appended rows differ"
