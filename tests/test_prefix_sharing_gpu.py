"""Prefix-cache block sharing end to end on the GPU (the shared-prefix request pattern, reduced):
requests sharing a common prefix map its blocks by reference through the radix tree, the
partly filled last shared block is copied on first write (all layers, device kernel), block
reference counts are mirrored on the device, and every request's attention output equals the
oracle run on that request's own unshared K/V history."""
import numpy as np
import pytest

from tests import kvtest

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("plen,slen", [(64, 24), (100, 28)])  # aligned (no COW) / unaligned (COW)
def test_shared_prefix_requests(native_libs, oracle, plen, slen):
    import torch
    from orinmllm_b200 import capi, kvm

    L, H, HKV, D, BS = 2, 32, 8, 128, 16
    R, STEPS = 10, 5
    rng = np.random.default_rng(11)
    nb = 200
    dtype = "f16"
    mgr = kvm.KvManager(nb, BS, seed=5, min_prefix_length=4)
    lay = capi.layout_paged(capi.KPX_F16, HKV, D, BS, nb)
    layer_stride = nb * HKV * BS * D
    kp = kvtest.to_device(kvtest.poison((L, nb, HKV, BS, D), dtype), dtype)
    vp = kvtest.to_device(kvtest.poison((L, nb, HKV, BS, D), dtype), dtype)
    refc = torch.zeros(nb, dtype=torch.int32, device="cuda")
    errc = torch.zeros(1, dtype=torch.int32, device="cuda")
    staging = torch.empty(1 << 16, dtype=torch.uint8, device="cuda")
    kv_dim = HKV * D

    def rows(n):
        return (kvtest.to_storage(rng.standard_normal((L, n, kv_dim)).astype(np.float32), dtype),
                kvtest.to_storage(rng.standard_normal((L, n, kv_dim)).astype(np.float32), dtype))

    prefix_tokens = rng.integers(0, 151936, plen).tolist()
    pk, pv = rows(plen)
    hist_k, hist_v, seqs, toks_of = [], [], [], []

    def write(seq, k_rows, v_rows, n):
        slots = torch.from_numpy(mgr.append(seq, n)).cuda()
        # copy-on-write and reference counts reach the device before the new rows land
        mgr.flush_device(refc, errc, kp, vp, lay, L, layer_stride, staging, staging.numel())
        for l in range(L):
            capi.append(kp[l], vp[l], lay, kvtest.to_device(k_rows[l], dtype), kvtest.to_device(v_rows[l], dtype),
                        slots, num_tokens=n)

    for r in range(R):
        suffix = rng.integers(0, 151936, slen).tolist()
        toks = prefix_tokens + suffix
        s = mgr.add_sequence()
        m = mgr.match_prefix(s, toks)
        assert m == (0 if r == 0 else plen)
        sk, sv = rows(slen)
        if m == 0:
            write(s, np.concatenate([pk, sk], 1), np.concatenate([pv, sv], 1), plen + slen)
            mgr.insert_prefix(s, prefix_tokens)
        else:
            write(s, sk, sv, slen)
        mgr.insert_prefix(s, toks)
        hist_k.append(np.concatenate([pk, sk], 1))
        hist_v.append(np.concatenate([pv, sv], 1))
        seqs.append(s)
        toks_of.append(toks)
    assert mgr.cow_events == (0 if plen % BS == 0 else R - 1)
    assert mgr.num_shared >= plen // BS

    ws_bytes = capi.decode_workspace_bytes(R, H, HKV)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device="cuda")
    capi.workspace_init(ws, ws_bytes)
    for step in range(STEPS):
        dk, dv = rows(R)  # one new token per request, per layer
        slots = np.empty(R, np.int64)
        for i, s in enumerate(seqs):
            slots[i] = mgr.append(s, 1)[0]
        mgr.flush_device(refc, errc, kp, vp, lay, L, layer_stride, staging, staging.numel())
        for i in range(R):
            hist_k[i] = np.concatenate([hist_k[i], dk[:, i:i + 1]], 1)
            hist_v[i] = np.concatenate([hist_v[i], dv[:, i:i + 1]], 1)
        d_slots = torch.from_numpy(slots).cuda()
        lens = np.array([mgr.length(s) for s in seqs], np.int32)
        table = mgr.block_table(seqs)
        q = kvtest.to_storage(rng.standard_normal((R, H * D)).astype(np.float32), dtype)
        for l in range(L):
            capi.append(kp[l], vp[l], lay, kvtest.to_device(dk[l], dtype), kvtest.to_device(dv[l], dtype),
                        d_slots, num_tokens=R)
            out = torch.empty(R, H * D, dtype=torch.float16, device="cuda")
            capi.paged_decode(out, kvtest.to_device(q, dtype), kp[l], vp[l], lay, torch.from_numpy(table).cuda(),
                              table.shape[1], torch.from_numpy(lens).cuda(), 0, R, H, 1.0 / np.sqrt(D), ws, ws_bytes)
            got = out.cpu().numpy().astype(np.float32)
            for i in range(R):
                n = int(lens[i])
                ref = oracle.mha(n - 1, H, 0, n, kv_dim, H // HKV, D, q[i].astype(np.float32),
                                 hist_k[i][l].astype(np.float32).reshape(-1), hist_v[i][l].astype(np.float32).reshape(-1))
                kvtest.assert_attention_close(got[i], ref, f"request {i} layer {l} step {step}", dtype)
    assert capi.workspace_status(ws) == 0
    # cache contents seen through every request's block table = its own unshared history
    kp_h, vp_h = kp.cpu().numpy(), vp.cpu().numpy()
    table = mgr.block_table(seqs)
    for i, s in enumerate(seqs):
        n = mgr.length(s)
        for l in range(L):
            gk = oracle.gather_paged(kp_h[l], table[i], n, HKV, D, BS)
            gv = oracle.gather_paged(vp_h[l], table[i], n, HKV, D, BS)
            assert np.array_equal(gk.view(np.uint8), hist_k[i][l].view(np.uint8))
            assert np.array_equal(gv.view(np.uint8), hist_v[i][l].view(np.uint8))
    # device mirror of the reference counts = host counts; nothing was refused
    assert refc.cpu().numpy().tolist() == mgr.ref_counts().tolist()
    assert int(errc.item()) == 0
    # Releasing the sequences and evicting returns every block except the shared prefix span:
    # like the reference, eviction only drops terminal LEAVES, and the prefix node has children,
    # so its blocks stay cached (one reference each, held by the tree).
    for s in seqs:
        mgr.free_sequence(s)
    mgr.evict(0)
    mgr.flush_device(refc, errc, kp, vp, lay, L, layer_stride, staging, staging.numel())
    kept = -(-plen // BS)
    assert mgr.num_free == nb - kept
    rc = refc.cpu().numpy()
    assert rc.tolist() == mgr.ref_counts().tolist() and int(rc.sum()) == kept and int(rc.max()) == 1
    assert int(errc.item()) == 0
