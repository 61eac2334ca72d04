"""Chunked prefill over the paged cache against the CPU oracle (causal attention of a chunk of
queries at positions start_pos.. against cache rows 0..start_pos+i)."""
import numpy as np
import pytest

from tests import kvtest

pytestmark = pytest.mark.gpu


def _run_chunked(oracle, dtype, q_heads, kv_heads, prompt_lens, chunk, seed=0, atol_note=""):
    import torch
    from orinmllm_b200 import capi, kvm

    D, BS = 128, 16
    rng = np.random.default_rng(seed)
    B = len(prompt_lens)
    nb = sum(-(-l // BS) for l in prompt_lens) + 5
    mgr = kvm.KvManager(nb, BS, seed=seed + 1)
    seqs = [mgr.add_sequence() for _ in range(B)]
    lay = capi.layout_paged(capi.dtype_code(kvtest.torch_dtype(dtype)), kv_heads, D, BS, nb)
    shape = (nb, kv_heads, BS, D)
    kp = kvtest.to_device(kvtest.poison(shape, dtype), dtype)
    vp = kvtest.to_device(kvtest.poison(shape, dtype), dtype)
    kp_ref, vp_ref = kvtest.poison(shape, dtype), kvtest.poison(shape, dtype)
    kv_dim, dim = kv_heads * D, q_heads * D
    k_all = [kvtest.to_storage(rng.standard_normal((l, kv_dim)).astype(np.float32), dtype) for l in prompt_lens]
    v_all = [kvtest.to_storage(rng.standard_normal((l, kv_dim)).astype(np.float32), dtype) for l in prompt_lens]
    q_all = [kvtest.to_storage(rng.standard_normal((l, dim)).astype(np.float32), dtype) for l in prompt_lens]
    worst = (0.0, 0.0)
    start = [0] * B
    max_blocks = max(-(-l // BS) for l in prompt_lens)
    while any(start[b] < prompt_lens[b] for b in range(B)):
        active = [b for b in range(B) if start[b] < prompt_lens[b]]
        n = [min(chunk, prompt_lens[b] - start[b]) for b in active]
        # 1. append the chunk's K/V rows (slots from the manager)
        slots = np.concatenate([mgr.append(seqs[b], n_b) for b, n_b in zip(active, n)])
        k_rows = np.concatenate([k_all[b][start[b]:start[b] + n_b] for b, n_b in zip(active, n)])
        v_rows = np.concatenate([v_all[b][start[b]:start[b] + n_b] for b, n_b in zip(active, n)])
        capi.append(kp, vp, lay, kvtest.to_device(k_rows, dtype), kvtest.to_device(v_rows, dtype),
                    torch.from_numpy(slots).cuda(), num_tokens=len(slots))
        oracle.append_paged(kp_ref, k_rows, slots, kv_heads, D, BS)
        oracle.append_paged(vp_ref, v_rows, slots, kv_heads, D, BS)
        # 2. attention of the chunk's queries
        q_rows = np.concatenate([q_all[b][start[b]:start[b] + n_b] for b, n_b in zip(active, n)])
        dq = kvtest.to_device(q_rows, dtype)
        out = torch.full_like(dq, float("nan"))
        table = mgr.block_table([seqs[b] for b in active], max_blocks)
        cu = np.concatenate([[0], np.cumsum(n)]).astype(np.int32)
        sp = np.array([start[b] for b in active], np.int32)
        nbytes = capi.prefill_workspace_bytes(int(cu[-1]), q_heads, kv_heads, D)
        ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
        capi.workspace_init(ws, nbytes)
        # oracle: gather each sequence to the reference's contiguous layout, causal MHA
        refs = []
        for i, (b, n_b) in enumerate(zip(active, n)):
            length = start[b] + n_b
            kc = kvtest.storage_to_f32(oracle.gather_paged(kp_ref, table[i], length, kv_heads, D, BS), dtype)
            vc = kvtest.storage_to_f32(oracle.gather_paged(vp_ref, table[i], length, kv_heads, D, BS), dtype)
            refs.append(oracle.mha_prefill(start[b], kvtest.storage_to_f32(q_rows[cu[i]:cu[i + 1]], dtype), q_heads,
                                           length, kv_dim, q_heads // kv_heads, D, kc.reshape(-1), vc.reshape(-1),
                                           threads=oracle.max_threads()))
        # tensor-core tiles with the key range whole / cut in 2 / cut in 4 parts and merged / cut by
        # the library's own rule, and the per-query streaming path: each against the oracle
        d_table = torch.from_numpy(table).cuda()
        for path, split in ((0, 0), (0, 2), (0, 4), (0, -1), (1, -1)):
            if dtype == "f32" and (path, split) != (0, -1):
                continue  # fp32 pools always take the streaming path
            capi.lib().kpx_internal_set_prefill_path(path)
            capi.lib().kpx_internal_set_prefill_split(split)
            out.fill_(float("nan"))
            capi.paged_prefill(out, dq, kp, vp, lay, d_table, max_blocks, cu, sp, len(active), q_heads,
                               1.0 / np.sqrt(D), ws, nbytes)
            assert capi.workspace_status(ws) == 0
            got = kvtest.storage_to_f32(kvtest.from_device(out, dtype), dtype)
            for i, b in enumerate(active):
                e = kvtest.assert_attention_close(
                    got[cu[i]:cu[i + 1]], refs[i],
                    f"prefill {dtype} path {path} split {split} seq {b} start {start[b]} {atol_note}", dtype)
                worst = (max(worst[0], e[0]), max(worst[1], e[1]))
        capi.lib().kpx_internal_set_prefill_path(0)
        capi.lib().kpx_internal_set_prefill_split(-1)
        for b, n_b in zip(active, n):
            start[b] += n_b
    # cache contents after all chunks: bit-exact
    assert np.array_equal(kvtest.from_device(kp, dtype).view(np.uint8), kp_ref.view(np.uint8))
    assert np.array_equal(kvtest.from_device(vp, dtype).view(np.uint8), vp_ref.view(np.uint8))
    return worst


@pytest.mark.parametrize("dtype", ["bf16", "f16", "f32"])
def test_prefill_small_ragged(native_libs, oracle, dtype):
    _run_chunked(oracle, dtype, 28, 4, [1, 37, 130, 200], chunk=64, seed=3)


def test_prefill_qwen3_shape(native_libs, oracle):
    _run_chunked(oracle, "f16", 32, 8, [300, 129], chunk=128, seed=4)


def test_prefill_config3_shape_reduced(native_libs, oracle):
    # Qwen2.5-7B attention shape (28 Q / 4 KV heads, d=128, bf16, chunks of 512, block 16) with
    # 2 sequences of 1024 tokens so the CPU oracle finishes in seconds
    worst = _run_chunked(oracle, "bf16", 28, 4, [1024, 1024], chunk=512, seed=5)
    print("config-3 (reduced) prefill parity: max_abs=%.3e max_rel=%.3e" % worst)


@pytest.mark.parametrize("dtype", ["f16", "bf16"])
def test_prefill_reference_cache_layout(native_libs, oracle, dtype):
    """The reference's token-major cache [seq_len][kv_dim] (16-bit) through the tensor-core path:
    the TMA tensor maps take the layout's strides, the block table is the identity, and a chunk
    that starts inside a block and ends inside another is handled (start 40, 300 queries)."""
    import torch
    from orinmllm_b200 import capi
    H, HKV, D, S = 12, 2, 128, 512
    start, n = 40, 300
    rng = np.random.default_rng(17)
    kv_dim = HKV * D
    kc = kvtest.to_storage(rng.standard_normal((S, kv_dim)).astype(np.float32), dtype)
    vc = kvtest.to_storage(rng.standard_normal((S, kv_dim)).astype(np.float32), dtype)
    q = kvtest.to_storage(rng.standard_normal((n, H * D)).astype(np.float32), dtype)
    lay = capi.layout_contiguous(capi.dtype_code(kvtest.torch_dtype(dtype)), HKV, D, 16, S // 16)
    table = torch.arange(S // 16, dtype=torch.int32, device="cuda")[None, :].contiguous()
    dq, dk, dv = kvtest.to_device(q, dtype), kvtest.to_device(kc, dtype), kvtest.to_device(vc, dtype)
    out = torch.full_like(dq, float("nan"))
    nbytes = capi.prefill_workspace_bytes(n, H, HKV, D)
    ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    capi.workspace_init(ws, nbytes)
    ref = oracle.mha_prefill(start, kvtest.storage_to_f32(q, dtype), H, S, kv_dim, H // HKV, D,
                             kvtest.storage_to_f32(kc, dtype).reshape(-1), kvtest.storage_to_f32(vc, dtype).reshape(-1),
                             threads=oracle.max_threads())
    for path in (0, 1):
        capi.lib().kpx_internal_set_prefill_path(path)
        out.fill_(float("nan"))
        capi.paged_prefill(out, dq, dk, dv, lay, table, S // 16, np.array([0, n], np.int32),
                           np.array([start], np.int32), 1, H, 1.0 / np.sqrt(D), ws, nbytes)
        assert capi.workspace_status(ws) == 0
        got = kvtest.storage_to_f32(kvtest.from_device(out, dtype), dtype)
        kvtest.assert_attention_close(got, ref, f"prefill reference layout {dtype} path {path}", dtype)
    capi.lib().kpx_internal_set_prefill_path(0)
