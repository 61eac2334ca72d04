"""Parity at the full sizes of the named workloads (the other test files run them reduced):

* chunked prefill, Qwen2.5-7B attention shape (28 Q / 4 KV heads, d 128), bf16, 4 sequences of
  2048-token prompts in 512-token chunks, RoPE theta 1e6 on Q/K before the append, seeded random
  block placement; every 5th query row of every head against the oracle;
* prefix-cache reuse, Qwen3-8B shape (32/8, fp16, block 16): 256 requests sharing a 1024-token
  prefix + 256 own tokens (and the unaligned 1000 + 280 that makes copy-on-write fire), 128 decode
  steps each, through the request scheduler; pool state against the host manager bit for bit,
  outputs of sampled requests / positions against the oracle;
* one 131 072-token sequence as its 8 / 4 / 2 / 1 KV-head shards (what each GPU of 1 / 2 / 4 / 8
  holds), run one after another on one GPU, every shard against the oracle's heads.
"""
from concurrent.futures import ThreadPoolExecutor

import numpy as np
import pytest

from tests import kvtest

pytestmark = pytest.mark.gpu


def test_chunked_prefill_4x2048_chunk512_bf16_full_size(native_libs, oracle):
    import torch
    from orinmllm_b200 import capi
    H, HKV, D, BS = 28, 4, 128, 16
    B, T, CH, dtype = 4, 2048, 512, "bf16"
    dim, kv_dim = H * D, HKV * D
    rng = np.random.default_rng(303)
    nblk_seq = T // BS
    nb = int(B * nblk_seq * 1.25)
    perm = rng.permutation(nb).astype(np.int32)
    table = perm[:B * nblk_seq].reshape(B, nblk_seq).copy()
    sin, cos = oracle.sin_cos_cache(D, T, 1e6)
    q_st = kvtest.to_storage(rng.standard_normal((B, T, dim), np.float32), dtype)
    k_st = kvtest.to_storage(rng.standard_normal((B, T, kv_dim), np.float32), dtype)
    v_st = kvtest.to_storage(rng.standard_normal((B, T, kv_dim), np.float32), dtype)
    # ---- oracle side: rotate in fp32 from the stored values, one rounding, contiguous caches
    q_rot = kvtest.storage_to_f32(q_st, dtype).copy()
    k_rot = kvtest.storage_to_f32(k_st, dtype).copy()
    for b in range(B):
        oracle.rope_batched(0, q_rot[b], k_rot[b], D, sin, cos)
    q_rot_st, k_rot_st = kvtest.to_storage(q_rot, dtype), kvtest.to_storage(k_rot, dtype)
    q_ref = kvtest.storage_to_f32(q_rot_st, dtype)
    k_ref = kvtest.storage_to_f32(k_rot_st, dtype)
    v_ref = kvtest.storage_to_f32(v_st, dtype)
    # ---- device: per chunk, RoPE + append of the chunk's rows, then the chunk's attention
    code = capi.dtype_code(kvtest.torch_dtype(dtype))
    lay = capi.layout_paged(code, HKV, D, BS, nb)
    shape = (nb, HKV, BS, D)
    kp = kvtest.to_device(kvtest.poison(shape, dtype), dtype)
    vp = kvtest.to_device(kvtest.poison(shape, dtype), dtype)
    d_table = torch.from_numpy(table).cuda()
    d_sin, d_cos = torch.from_numpy(sin).cuda(), torch.from_numpy(cos).cuda()
    nbytes = capi.prefill_workspace_bytes(B * CH, H, HKV, D)
    ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    capi.workspace_init(ws, nbytes)
    got = np.empty((B, T, dim), np.float32)
    cu = (np.arange(B + 1) * CH).astype(np.int32)
    for c0 in range(0, T, CH):
        pos = np.tile(np.arange(c0, c0 + CH, dtype=np.int32), B)
        slots = np.concatenate([table[b, np.arange(c0, c0 + CH) // BS].astype(np.int64) * BS + np.arange(c0, c0 + CH) % BS
                                for b in range(B)])
        dq = kvtest.to_device(np.ascontiguousarray(q_st[:, c0:c0 + CH]).reshape(B * CH, dim), dtype)
        dk = kvtest.to_device(np.ascontiguousarray(k_st[:, c0:c0 + CH]).reshape(B * CH, kv_dim), dtype)
        dv = kvtest.to_device(np.ascontiguousarray(v_st[:, c0:c0 + CH]).reshape(B * CH, kv_dim), dtype)
        capi.rope_append(dq, dk, dv, H, torch.from_numpy(pos).cuda(), d_sin, d_cos, kp, vp, lay,
                         torch.from_numpy(slots).cuda(), B * CH)
        out = torch.full_like(dq, float("nan"))
        capi.paged_prefill(out, dq, kp, vp, lay, d_table, nblk_seq, cu, np.full(B, c0, np.int32), B, H,
                           1.0 / np.sqrt(D), ws, nbytes)
        assert capi.workspace_status(ws) == 0
        got[:, c0:c0 + CH] = kvtest.storage_to_f32(kvtest.from_device(out, dtype), dtype).reshape(B, CH, dim)
    # appended cache contents: bit-exact against the rotated rows scattered on the host
    kp_ref, vp_ref = kvtest.poison(shape, dtype), kvtest.poison(shape, dtype)
    all_slots = np.concatenate([table[b, np.arange(T) // BS].astype(np.int64) * BS + np.arange(T) % BS for b in range(B)])
    oracle.append_paged(kp_ref, k_rot_st.reshape(B * T, kv_dim), all_slots, HKV, D, BS)
    oracle.append_paged(vp_ref, v_st.reshape(B * T, kv_dim), all_slots, HKV, D, BS)
    assert np.array_equal(kvtest.from_device(kp, dtype).view(np.uint8), kp_ref.view(np.uint8))
    assert np.array_equal(kvtest.from_device(vp, dtype).view(np.uint8), vp_ref.view(np.uint8))
    # ---- every 5th query row (all heads) against the oracle, rows spread over host threads
    kvtest.BF16_BEYOND_ATOL.update(elements=0, beyond=0)
    rows = [(b, t) for b in range(B) for t in range(b % 5, T, 5)]

    def one(bt):
        b, t = bt
        ref = oracle.mha_prefill(t, q_ref[b, t:t + 1], H, t + 1, kv_dim, H // HKV, D, k_ref[b, :t + 1].reshape(-1),
                                 v_ref[b, :t + 1].reshape(-1), threads=1)
        return kvtest.attention_errors(got[b, t:t + 1], ref), ref

    worst = (0.0, 0.0)
    with ThreadPoolExecutor(max_workers=oracle.max_threads()) as pool:
        for (b, t), (err, ref) in zip(rows, pool.map(one, rows)):
            kvtest.assert_attention_close(got[b, t:t + 1], ref, f"prefill 4x2048 seq {b} row {t}", dtype)
            worst = (max(worst[0], err[0]), max(worst[1], err[1]))
    n = kvtest.BF16_BEYOND_ATOL
    print(f"full-size chunked prefill: {len(rows)} rows checked, max_abs={worst[0]:.3e} max_rel={worst[1]:.3e}; "
          f"bf16 outputs beyond the plain 2e-3: {n['beyond']} of {n['elements']}")


def _oracle_rows(oracle, sim, tokens, positions):
    """Reference outputs [L, dim] of one request at the given cache positions, from its token list."""
    import torch
    H, HKV, D = sim.H, sim.HKV, sim.D
    n = max(positions) + 1
    ids = torch.from_numpy(np.asarray(tokens[:n], np.int64) % sim.vocab).cuda()
    sin = sim.sin[:(n + 1) * D].cpu().numpy()
    cos = sim.cos[:(n + 1) * D].cpu().numpy()
    per_layer = []
    for l in range(sim.L):
        q = sim.Eq[l, ids].float().cpu().numpy()
        k = sim.Ek[l, ids].float().cpu().numpy()
        v = np.ascontiguousarray(sim.Ev[l, ids].float().cpu().numpy())
        oracle.rope_batched(0, q, k, D, sin, cos)
        q = kvtest.storage_to_f32(kvtest.to_storage(q, "f16"), "f16")
        k = np.ascontiguousarray(kvtest.storage_to_f32(kvtest.to_storage(k, "f16"), "f16"))
        per_layer.append({p: oracle.mha_prefill(p, q[p:p + 1], H, p + 1, HKV * D, H // HKV, D, k[:p + 1].reshape(-1),
                                                v[:p + 1].reshape(-1), threads=1)[0] for p in positions})
    return {p: np.stack([per_layer[l][p] for l in range(sim.L)]) for p in positions}


@pytest.mark.parametrize("prefix,suffix", [(1024, 256), (1000, 280)])
def test_prefix_reuse_256_requests_full_size(native_libs, oracle, prefix, suffix):
    from tests.serving_sim import ServingSim
    n_req, gen = 256, 129  # 129 sampled tokens = 128 decode steps with a cached position each
    sim = ServingSim(num_layers=1, q_heads=32, kv_heads=8, num_blocks=8192, seed=3, prefill_chunk=512,
                     max_prefill_tokens=4096, max_decode_batch=256, record=True, poison=True,
                     record_ids=[0, 1, 97, 255])
    rng = np.random.default_rng(1)
    common = rng.integers(0, 151936, prefix)
    first = sim.sched.submit(np.concatenate([common, rng.integers(0, 151936, suffix)]), 1, also_register=prefix)
    sim.run()
    followers = [sim.sched.submit(np.concatenate([common, rng.integers(0, 151936, suffix)]), gen) for _ in range(n_req - 1)]
    mid = {}

    def hook(d):
        if sim.sched.stats()["decode_steps"] == 64 and not mid:
            sim._flush()
            mid["dev"], mid["host"] = sim.refc.cpu().numpy().copy(), sim.manager.ref_counts().copy()
            mid["shared"] = sim.manager.num_shared

    sim.run(decode_hook=hook)
    st = sim.sched.stats()
    assert st["finished"] == n_req and st["reused_tokens"] == (n_req - 1) * prefix
    assert st["decode_steps"] == 128 and sim.decode_launches == 128
    # block accounting: shared prefix blocks once, the followers' own blocks each
    own = -(-(prefix + suffix + gen - 1) // 16) - prefix // 16       # blocks a follower takes from the free list
    first_kept = -(-(prefix + suffix) // 16)
    assert st["peak_blocks_in_use"] == first_kept + (n_req - 1) * own
    assert sim.manager.cow_events == (0 if prefix % 16 == 0 else n_req - 1)
    # device reference counts equal the host's, mid-run (255 sequences sharing) and at the end
    assert np.array_equal(mid["dev"], mid["host"]) and mid["shared"] >= prefix // 16
    assert int(mid["host"].max()) >= n_req - 1
    assert np.array_equal(sim.refc.cpu().numpy(), sim.manager.ref_counts())
    # outputs of sampled requests at sampled positions: prefill rows, first and last decode steps
    worst = 0.0
    for rid in (first, followers[0], followers[96], followers[-1]):
        toks = sim.sched.tokens(rid)
        got = sim.outputs[rid]
        reused = sim.sched.reused_tokens(rid)
        assert sorted(got) == list(range(reused, len(toks) - 1))
        have = sorted(got)
        picks = sorted(set([have[0], have[len(have) // 3], have[-1]] + have[suffix - 2:suffix + 2] + have[::97]))
        ref = _oracle_rows(oracle, sim, toks, picks)
        for p in picks:
            a, _ = kvtest.assert_attention_close(got[p], ref[p], f"request {rid} position {p}")
            worst = max(worst, a)
    print(f"prefix {prefix}+{suffix}: peak blocks {st['peak_blocks_in_use']}, cow {sim.manager.cow_events}, "
          f"worst max-abs over sampled outputs {worst:.2e}")


def test_long_sequence_kv_head_shards_on_one_gpu(native_libs, oracle):
    """131 072 tokens, Qwen3-8B heads: the 8 / 4 / 2 / 1 KV-head shards that 1 / 2 / 4 / 8 GPUs hold,
    launched one after another here; the small-launch form and the two-level assembly run at
    their real sizes."""
    import torch
    from orinmllm_b200 import capi
    H, HKV, D, BS, T = 32, 8, 128, 16, 131072
    kv_mul = H // HKV
    rng = np.random.default_rng(77)
    nblk = T // BS
    nb = nblk + 64
    perm = rng.permutation(nb).astype(np.int32)[:nblk]
    g = torch.Generator(device="cuda").manual_seed(5)
    kp = torch.randn(nb, HKV, BS, D, generator=g, device="cuda", dtype=torch.float32).to(torch.float16)
    vp = torch.randn(nb, HKV, BS, D, generator=g, device="cuda", dtype=torch.float32).to(torch.float16)
    q = torch.randn(1, H * D, generator=g, device="cuda", dtype=torch.float32).to(torch.float16)
    table = torch.from_numpy(perm[None, :].copy()).cuda()
    lens = torch.tensor([T], dtype=torch.int32, device="cuda")
    ref = oracle.paged_decode(q.float().cpu().numpy(), kp.float().cpu().numpy(), vp.float().cpu().numpy(), perm[None, :],
                              np.array([T], np.int32), H, HKV, D, BS, threads=oracle.max_threads())
    for shard_heads in (8, 4, 2, 1):
        worst = 0.0
        for first_head in range(0, HKV, shard_heads):
            ks = kp[:, first_head:first_head + shard_heads].contiguous()
            vs = vp[:, first_head:first_head + shard_heads].contiguous()
            qs = q[:, first_head * kv_mul * D:(first_head + shard_heads) * kv_mul * D].contiguous()
            lay = capi.layout_paged(capi.KPX_F16, shard_heads, D, BS, nb)
            nbytes = capi.decode_workspace_bytes(1, shard_heads * kv_mul, shard_heads)
            ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
            capi.workspace_init(ws, nbytes)
            out = torch.full_like(qs, float("nan"))
            capi.paged_decode(out, qs, ks, vs, lay, table, nblk, lens, 0, 1, shard_heads * kv_mul, 1 / np.sqrt(D), ws, nbytes)
            assert capi.workspace_status(ws) == 0
            want = ref[:, first_head * kv_mul * D:(first_head + shard_heads) * kv_mul * D]
            a, _ = kvtest.assert_attention_close(out.float().cpu().numpy(), want, f"{shard_heads}-head shard at head {first_head}")
            worst = max(worst, a)
            if shard_heads <= 2 and first_head >= 2 * shard_heads:
                break  # two shards of the narrow shapes are enough
        print(f"131072 tokens, {shard_heads} KV heads per shard: max abs err {worst:.2e}")
