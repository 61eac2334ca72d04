"""Bit-exact parity of append, RoPE(+append), COW copy and refcount kernels with the oracle."""
import numpy as np
import pytest

from tests import kvtest

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", ["f16", "bf16", "f32"])
def test_append_scatter_bit_exact(native_libs, oracle, dtype):
    import torch
    from orinmllm_b200 import capi
    case = kvtest.make_paged_case(3, dtype, 28, 4, [0, 1, 16, 33, 512, 5])
    lay = capi.layout_paged(capi.dtype_code(kvtest.torch_dtype(dtype)), 4, 128, 16, case.num_blocks)
    shape = (case.num_blocks, 4, 16, 128)
    kp = kvtest.to_device(kvtest.poison(shape, dtype), dtype)
    vp = kvtest.to_device(kvtest.poison(shape, dtype), dtype)
    slots = case.slot_mapping.copy()
    slots[7] = -1  # padding token: skipped
    case.slot_mapping = slots
    capi.append(kp, vp, lay, kvtest.to_device(case.k_rows, dtype), kvtest.to_device(case.v_rows, dtype),
                torch.from_numpy(slots).cuda(), num_tokens=case.total_tokens)
    kr, vr = kvtest.oracle_pools(oracle, case)
    assert np.array_equal(kvtest.from_device(kp, dtype).view(np.uint8), kr.view(np.uint8))
    assert np.array_equal(kvtest.from_device(vp, dtype).view(np.uint8), vr.view(np.uint8))


@pytest.mark.parametrize("kv_heads,lens,k_only", [
    (4, [6000, 5000, 1203], False),   # far more tokens than resident CTAs: every unrolled step of the token loop
    (4, [6000, 5000, 1203], True),    # K pool alone (KVCacheLayer appends K and V in separate calls)
    (40, [3000, 1500], False),        # a token wider than one CTA: the flat-index kernel, several passes
])
def test_append_large_and_wide_bit_exact(native_libs, oracle, kv_heads, lens, k_only):
    import torch
    from orinmllm_b200 import capi
    dtype = "f16"
    case = kvtest.make_paged_case(5, dtype, kv_heads, kv_heads, lens)
    lay = capi.layout_paged(capi.dtype_code(kvtest.torch_dtype(dtype)), kv_heads, 128, 16, case.num_blocks)
    shape = (case.num_blocks, kv_heads, 16, 128)
    kp = kvtest.to_device(kvtest.poison(shape, dtype), dtype)
    vp = kvtest.to_device(kvtest.poison(shape, dtype), dtype)
    slots = case.slot_mapping.copy()
    slots[::97] = -1  # padding tokens: skipped
    case.slot_mapping = slots
    d_slots = torch.from_numpy(slots).cuda()
    if k_only:
        capi.append(kp, None, lay, kvtest.to_device(case.k_rows, dtype), None, d_slots, num_tokens=case.total_tokens)
    else:
        capi.append(kp, vp, lay, kvtest.to_device(case.k_rows, dtype), kvtest.to_device(case.v_rows, dtype),
                    d_slots, num_tokens=case.total_tokens)
    kr, vr = kvtest.oracle_pools(oracle, case)
    assert np.array_equal(kvtest.from_device(kp, dtype).view(np.uint8), kr.view(np.uint8))
    if k_only:
        assert np.array_equal(kvtest.from_device(vp, dtype).view(np.uint8), kvtest.poison(shape, dtype).view(np.uint8))
    else:
        assert np.array_equal(kvtest.from_device(vp, dtype).view(np.uint8), vr.view(np.uint8))


def test_append_at_device_position_reference_layout(native_libs, oracle):
    """KVCacheLayer semantics: cache [S, kv_dim], row *pos (device int32) <- src."""
    import torch
    from orinmllm_b200 import capi
    S, kv_dim = 50, 256
    lay = capi.layout_contiguous(capi.KPX_F32, 2, 128, 16)
    rng = np.random.default_rng(0)
    cache = rng.standard_normal((S, kv_dim)).astype(np.float32)
    src = rng.standard_normal((1, kv_dim)).astype(np.float32)
    d_cache = torch.from_numpy(cache).cuda()
    pos = torch.tensor([37], dtype=torch.int32, device="cuda")
    capi.append(d_cache, None, lay, torch.from_numpy(src).cuda(), None, None, pos, 0, 1)
    ref = cache.copy()
    oracle.lib.orc_append_contiguous(ref.reshape(-1), src.reshape(-1), 37, kv_dim, 0, S)
    assert np.array_equal(d_cache.cpu().numpy(), ref)


@pytest.mark.parametrize("dtype", ["f16", "bf16", "f32"])
def test_rope_append_bit_exact(native_libs, oracle, dtype):
    """RoPE'd Q/K rows and the appended pools equal the CPU statement bit for bit when both
    sides read the same sin/cos tables (products are not fused on either side)."""
    import torch
    from orinmllm_b200 import capi
    H, HKV, D = 28, 4, 128
    n, start = 40, 100
    rng = np.random.default_rng(8)
    sin, cos = oracle.sin_cos_cache(D, 256, 1e6)
    q32 = rng.standard_normal((n, H * D)).astype(np.float32)
    k32 = rng.standard_normal((n, HKV * D)).astype(np.float32)
    v32 = rng.standard_normal((n, HKV * D)).astype(np.float32)
    q_st, k_st, v_st = (kvtest.to_storage(x, dtype) for x in (q32, k32, v32))
    # oracle: fp32 math on the stored values, one rounding at the end
    q_ref = kvtest.storage_to_f32(q_st, dtype).copy()
    k_ref = kvtest.storage_to_f32(k_st, dtype).copy()
    oracle.rope_batched(start, q_ref, k_ref, D, sin, cos)
    q_ref_st, k_ref_st = kvtest.to_storage(q_ref, dtype), kvtest.to_storage(k_ref, dtype)
    nblk = 12
    perm = rng.permutation(nblk).astype(np.int64)
    pos = np.arange(start, start + n)
    slots = perm[(pos - 96) // 16] * 16 + pos % 16
    shape = (nblk, HKV, 16, D)
    kp_ref, vp_ref = kvtest.poison(shape, dtype), kvtest.poison(shape, dtype)
    oracle.append_paged(kp_ref, k_ref_st, slots, HKV, D, 16)
    oracle.append_paged(vp_ref, v_st, slots, HKV, D, 16)
    # device
    lay = capi.layout_paged(capi.dtype_code(kvtest.torch_dtype(dtype)), HKV, D, 16, nblk)
    dq, dk, dv = (kvtest.to_device(x, dtype) for x in (q_st, k_st, v_st))
    kp = kvtest.to_device(kvtest.poison(shape, dtype), dtype)
    vp = kvtest.to_device(kvtest.poison(shape, dtype), dtype)
    capi.rope_append(dq, dk, dv, H, torch.from_numpy(pos.astype(np.int32)).cuda(),
                     torch.from_numpy(sin).cuda(), torch.from_numpy(cos).cuda(), kp, vp, lay,
                     torch.from_numpy(slots).cuda(), n)
    assert np.array_equal(kvtest.from_device(dq, dtype).view(np.uint8), q_ref_st.view(np.uint8))
    assert np.array_equal(kvtest.from_device(dk, dtype).view(np.uint8), k_ref_st.view(np.uint8))
    assert np.array_equal(kvtest.from_device(kp, dtype).view(np.uint8), kp_ref.view(np.uint8))
    assert np.array_equal(kvtest.from_device(vp, dtype).view(np.uint8), vp_ref.view(np.uint8))


@pytest.mark.parametrize("dtype", ["f16", "bf16", "f32"])
@pytest.mark.parametrize("which", ["both", "k_only"])
def test_norm_rope_append_matches_oracle(native_libs, oracle, dtype, which):
    """Per-head RMSNorm (Qwen3 q/k norm) fused in front of RoPE + append.  The sum of squares is
    a tree over lanes on the device and sequential in the oracle, so rows agree to a few fp32
    ulps before the one rounding to the cache dtype: at most one ulp of that dtype apart.  The
    pool rows are bit-identical to the K rows the call returns, V rows are copied untouched."""
    import torch
    from orinmllm_b200 import capi
    H, HKV, D = 16, 4, 128
    n, start = 37, 5
    rng = np.random.default_rng(12)
    sin, cos = oracle.sin_cos_cache(D, 64, 1e6)
    q32 = rng.standard_normal((n, H * D)).astype(np.float32) * 3.0
    k32 = rng.standard_normal((n, HKV * D)).astype(np.float32) * 0.2
    v32 = rng.standard_normal((n, HKV * D)).astype(np.float32)
    wq = (1.0 + 0.1 * rng.standard_normal(D)).astype(np.float32)
    wk = (1.0 + 0.1 * rng.standard_normal(D)).astype(np.float32)
    q_st, k_st, v_st = (kvtest.to_storage(x, dtype) for x in (q32, k32, v32))
    q_ref = kvtest.storage_to_f32(q_st, dtype).copy()
    k_ref = kvtest.storage_to_f32(k_st, dtype).copy()
    if which == "both":
        oracle.rmsnorm_heads(q_ref, H, D, wq, 1e-6)
    oracle.rmsnorm_heads(k_ref, HKV, D, wk, 1e-6)
    oracle.rope_batched(start, q_ref, k_ref, D, sin, cos)
    nblk = 6
    perm = rng.permutation(nblk).astype(np.int64)
    pos = np.arange(start, start + n)
    slots = perm[pos // 16] * 16 + pos % 16
    shape = (nblk, HKV, 16, D)
    lay = capi.layout_paged(capi.dtype_code(kvtest.torch_dtype(dtype)), HKV, D, 16, nblk)
    dq, dk, dv = (kvtest.to_device(x, dtype) for x in (q_st, k_st, v_st))
    kp = kvtest.to_device(kvtest.poison(shape, dtype), dtype)
    vp = kvtest.to_device(kvtest.poison(shape, dtype), dtype)
    capi.norm_rope_append(dq, dk, dv, H, torch.from_numpy(wq).cuda() if which == "both" else None,
                          torch.from_numpy(wk).cuda(), 1e-6, torch.from_numpy(pos.astype(np.int32)).cuda(),
                          torch.from_numpy(sin).cuda(), torch.from_numpy(cos).cuda(), kp, vp, lay,
                          torch.from_numpy(slots).cuda(), n)
    got_q = kvtest.storage_to_f32(kvtest.from_device(dq, dtype), dtype)
    got_k = kvtest.storage_to_f32(kvtest.from_device(dk, dtype), dtype)
    ulp = {"f16": 2.0 ** -10, "bf16": 2.0 ** -7, "f32": 2.0 ** -21}[dtype]  # one ulp, relative, with slack for fp32
    for got, ref, name in ((got_q, q_ref, "q"), (got_k, k_ref, "k")):
        err = np.abs(got - ref)
        bound = ulp * np.maximum(np.abs(ref), 1e-3) + 1e-6
        assert np.all(err <= bound), f"{name}: worst {float((err / bound).max()):.2f} x bound"
    # the pool holds exactly the K rows the call returned, and the V rows as given
    kp_ref, vp_ref = kvtest.poison(shape, dtype), kvtest.poison(shape, dtype)
    oracle.append_paged(kp_ref, kvtest.from_device(dk, dtype), slots, HKV, D, 16)
    oracle.append_paged(vp_ref, v_st, slots, HKV, D, 16)
    assert np.array_equal(kvtest.from_device(kp, dtype).view(np.uint8), kp_ref.view(np.uint8))
    assert np.array_equal(kvtest.from_device(vp, dtype).view(np.uint8), vp_ref.view(np.uint8))
    # a normalised head has mean square ~ mean(w^2) before the rotation, which preserves it
    ms = (got_k.reshape(n, HKV, D) ** 2).mean(-1)
    assert np.allclose(ms, (wk ** 2).mean(), rtol=0.2)


def test_sin_cos_cache_close_to_cpu_table(native_libs, oracle):
    import torch
    from orinmllm_b200 import capi
    s = torch.empty(300, 128, device="cuda")
    c = torch.empty(300, 128, device="cuda")
    capi.sin_cos_cache(s, c, 128, 300, 1e6)
    sr, cr = oracle.sin_cos_cache(128, 300, 1e6)
    # device powf/sinf differ from libm in the last bits; the angle reaches 299 rad
    assert np.abs(s.cpu().numpy() - sr).max() < 1e-4
    assert np.abs(c.cpu().numpy() - cr).max() < 1e-4


def test_config1_reference_layout_decode_fp32(native_libs, oracle):
    """The CPU-runnable anchor case (Qwen2.5-1.5B attention shape, 512 cached + 1 new token) on the GPU through the reference's own cache layout: 12 Q / 2 KV
    heads, d=128, 512 cached + 1 new token, fp32, contiguous cache, device-resident pos."""
    import torch
    from orinmllm_b200 import capi
    H, HKV, D, S = 12, 2, 128, 520
    rng = np.random.default_rng(1)
    kc = np.zeros((S, HKV * D), np.float32)
    vc = np.zeros((S, HKV * D), np.float32)
    kc[:512] = rng.standard_normal((512, HKV * D), np.float32)
    vc[:512] = rng.standard_normal((512, HKV * D), np.float32)
    kc[513:], vc[513:] = np.nan, np.nan  # rows beyond pos must never be read
    q = rng.standard_normal((1, H * D)).astype(np.float32)
    k = rng.standard_normal((1, HKV * D)).astype(np.float32)
    v = rng.standard_normal((1, HKV * D)).astype(np.float32)
    sin, cos = oracle.sin_cos_cache(D, S, 1e6)
    # oracle
    q_ref, k_ref = q.copy(), k.copy()
    oracle.rope(512, q_ref[0], k_ref[0], D, sin, cos)
    kc_ref, vc_ref = kc.copy(), vc.copy()
    kc_ref[512], vc_ref[512] = k_ref[0], v[0]
    ref = oracle.mha(512, H, 0, S, HKV * D, H // HKV, D, q_ref[0],
                     np.nan_to_num(kc_ref).reshape(-1), np.nan_to_num(vc_ref).reshape(-1))
    # device: rope, append at *pos, attend pos+1 rows
    lay = capi.layout_contiguous(capi.KPX_F32, HKV, D, 16)
    dq, dk, dv = (torch.from_numpy(x).cuda() for x in (q, k, v))
    dkc, dvc = torch.from_numpy(kc).cuda(), torch.from_numpy(vc).cuda()
    pos = torch.tensor([512], dtype=torch.int32, device="cuda")
    capi.rope_append(dq, dk, None, H, pos, torch.from_numpy(sin).cuda(), torch.from_numpy(cos).cuda(),
                     None, None, lay, None, 1)
    capi.append(dkc, dvc, lay, dk, dv, None, pos, 0, 1)
    assert np.array_equal(dkc.cpu().numpy()[512], kc_ref[512])
    out = torch.empty_like(dq)
    nbytes = capi.decode_workspace_bytes(1, H, HKV)
    ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    capi.workspace_init(ws, nbytes)
    capi.paged_decode(out, dq, dkc, dvc, lay, None, 0, pos, 1, 1, H, 1.0 / np.sqrt(D), ws, nbytes)
    assert capi.workspace_status(ws) == 0
    max_abs, max_rel = kvtest.assert_attention_close(out.cpu().numpy()[0], ref, "config 1", "f32")
    assert max_abs < 1e-5  # fp32 end to end


def test_cow_copy_and_refcounts(native_libs):
    import torch
    from orinmllm_b200 import capi
    L, nb, HKV = 3, 10, 4
    lay = capi.layout_paged(capi.KPX_F16, HKV, 128, 16, nb)
    kp = torch.randn(L, nb, HKV, 16, 128, device="cuda", dtype=torch.float16)
    vp = torch.randn(L, nb, HKV, 16, 128, device="cuda", dtype=torch.float16)
    k0, v0 = kp.clone(), vp.clone()
    src = torch.tensor([2, 7], dtype=torch.int32, device="cuda")
    dst = torch.tensor([5, 0], dtype=torch.int32, device="cuda")
    capi.cow_copy_blocks(kp, vp, lay, L, nb * HKV * 16 * 128, src, dst, 2)
    k0[:, 5], k0[:, 0] = k0[:, 2].clone(), k0[:, 7].clone()
    v0[:, 5], v0[:, 0] = v0[:, 2].clone(), v0[:, 7].clone()
    assert torch.equal(kp, k0) and torch.equal(vp, v0)
    rc = torch.zeros(nb, dtype=torch.int32, device="cuda")
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    ids = torch.tensor([1, 1, 3, 9, 12], dtype=torch.int32, device="cuda")
    dl = torch.tensor([1, 1, 2, 1, 1], dtype=torch.int32, device="cuda")
    capi.refcount_update(rc, nb, ids, dl, 5, err)
    # a second launch releases: increments and decrements of one block are ordered by launch
    ids2 = torch.tensor([3, 4], dtype=torch.int32, device="cuda")
    dl2 = torch.tensor([-1, -1], dtype=torch.int32, device="cuda")
    capi.refcount_update(rc, nb, ids2, dl2, 2, err)
    # id 12 is out of range, block 4 would go negative: both refused and counted
    assert rc.cpu().tolist() == [0, 2, 0, 1, 0, 0, 0, 0, 0, 1]
    assert int(err.item()) == 2
