"""The one-launch decode step (RoPE + append + attention, kpx_rope_append_decode) against the
oracle and against the three-step path it replaces (kpx_rope_append then kpx_paged_decode)."""
import numpy as np
import pytest

from tests import kvtest

pytestmark = pytest.mark.gpu


def _step_case(seed, dtype, heads, cached_lens):
    """A paged case whose tables cover cached_lens + 1 tokens; the last token of every sequence
    is the step's new token (rows not yet rotated, not yet in the pool)."""
    H, HKV = heads
    cached = np.asarray(cached_lens, np.int32)
    case = kvtest.make_paged_case(seed, dtype, H, HKV, cached + 1)
    ends = np.cumsum(case.seq_lens)            # row index one past each sequence's tokens
    new_rows = ends - 1
    keep = np.ones(case.total_tokens, bool)
    keep[new_rows] = False
    return case, cached, new_rows, keep


def _run(oracle, dtype, heads, cached_lens, seed=21, flags=0, table_identity=False):
    import torch
    from orinmllm_b200 import capi
    H, HKV = heads
    D, BS = 128, 16
    case, cached, new_rows, keep = _step_case(seed, dtype, heads, cached_lens)
    b = len(cached)
    rng = np.random.default_rng(seed + 1)
    max_pos = int(cached.max()) + 2
    sin, cos = oracle.sin_cos_cache(D, max_pos, 1e6)
    # the step's inputs: unrotated q, k and v rows of the new tokens, in the storage dtype
    q_st = case.q
    k_new_st = case.k_rows[new_rows]
    v_new_st = case.v_rows[new_rows]
    # ---- expectation on the CPU: rotate (fp32 math on stored values, one rounding), append, attend
    q_rot = kvtest.storage_to_f32(q_st, dtype).copy()
    k_rot = kvtest.storage_to_f32(k_new_st, dtype).copy()
    for i in range(b):
        oracle.rope(int(cached[i]), q_rot[i], k_rot[i], D, sin, cos)
    q_rot_st, k_rot_st = kvtest.to_storage(q_rot, dtype), kvtest.to_storage(k_rot, dtype)
    exp = kvtest.PagedCase(dtype, H, HKV, D, BS, case.seq_lens, case.num_blocks, case.block_table,
                           case.k_rows.copy(), case.v_rows, case.slot_mapping, q_rot_st)
    exp.k_rows[new_rows] = k_rot_st
    kp_ref, vp_ref = kvtest.oracle_pools(oracle, exp)
    ref = kvtest.oracle_decode(oracle, exp, kp_ref, vp_ref, threads=oracle.max_threads())
    # ---- device: pools hold the cached tokens only
    code = capi.dtype_code(kvtest.torch_dtype(dtype))
    lay = capi.layout_paged(code, HKV, D, BS, case.num_blocks)
    shape = (case.num_blocks, HKV, BS, D)
    kp = kvtest.to_device(kvtest.poison(shape, dtype), dtype)
    vp = kvtest.to_device(kvtest.poison(shape, dtype), dtype)
    d_slots = torch.from_numpy(case.slot_mapping[keep]).cuda()
    if keep.any():
        capi.append(kp, vp, lay, kvtest.to_device(case.k_rows[keep], dtype), kvtest.to_device(case.v_rows[keep], dtype),
                    d_slots, num_tokens=int(keep.sum()))
    kp2, vp2 = kp.clone(), vp.clone()
    dq, dk, dv = (kvtest.to_device(x, dtype) for x in (q_st, k_new_st, v_new_st))
    d_pos = torch.from_numpy(cached).cuda()
    d_table = torch.from_numpy(case.block_table).cuda()
    d_sin, d_cos = torch.from_numpy(sin).cuda(), torch.from_numpy(cos).cuda()
    nbytes = capi.decode_workspace_bytes(b, H, HKV, D)
    ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    capi.workspace_init(ws, nbytes)
    out = torch.full_like(dq, float("nan"))
    scale = 1.0 / np.sqrt(D)
    capi.rope_append_decode(out, dq, dk, dv, d_sin, d_cos, kp, vp, lay, d_table, case.block_table.shape[1],
                            d_pos, b, H, scale, ws, nbytes, flags)
    assert capi.workspace_status(ws) == 0
    # inputs are not rotated in place
    assert np.array_equal(kvtest.from_device(dq, dtype).view(np.uint8), q_st.view(np.uint8))
    assert np.array_equal(kvtest.from_device(dk, dtype).view(np.uint8), k_new_st.view(np.uint8))
    # pools: bit-exact with the CPU statement (cached rows untouched, new rows rotated + stored)
    assert np.array_equal(kvtest.from_device(kp, dtype).view(np.uint8), kp_ref.view(np.uint8)), "K pool"
    assert np.array_equal(kvtest.from_device(vp, dtype).view(np.uint8), vp_ref.view(np.uint8)), "V pool"
    got = kvtest.storage_to_f32(kvtest.from_device(out, dtype), dtype)
    kvtest.assert_attention_close(got, ref, f"fused step {dtype} H={H}/{HKV}", dtype)
    # ---- the three-step path on copies of the pools: same pools bit for bit, same outputs
    # within the attention tolerance (the new token is added in a different order)
    dq2, dk2 = dq.clone(), dk.clone()
    new_slots = torch.from_numpy(case.slot_mapping[new_rows]).cuda()
    capi.rope_append(dq2, dk2, dv, H, d_pos, d_sin, d_cos, kp2, vp2, lay, new_slots, b)
    out2 = torch.full_like(dq, float("nan"))
    capi.paged_decode(out2, dq2, kp2, vp2, lay, d_table, case.block_table.shape[1], d_pos, 1, b, H, scale, ws, nbytes)
    assert capi.workspace_status(ws) == 0
    assert torch.equal(kp.view(torch.uint8), kp2.view(torch.uint8)) and torch.equal(vp.view(torch.uint8), vp2.view(torch.uint8))
    got2 = kvtest.storage_to_f32(kvtest.from_device(out2, dtype), dtype)
    kvtest.assert_attention_close(got, got2, "fused vs three-step", dtype)


@pytest.mark.parametrize("dtype", ["f16", "bf16", "f32"])
@pytest.mark.parametrize("heads", [(32, 8), (12, 2), (28, 4), (8, 8), (16, 2)])
def test_fused_step_small(native_libs, oracle, dtype, heads):
    # cached lengths around the block boundaries; 0 = the new token is the sequence's first
    _run(oracle, dtype, heads, [0, 1, 15, 16, 17, 31, 32, 100, 513, 0, 64])


@pytest.mark.parametrize("flags", [0, 1])
def test_fused_step_headline_shape(native_libs, oracle, flags):
    """bs 64, ctx U[128,4096], 32/8 heads, fp16: both CTA forms."""
    rng = np.random.default_rng(2024)
    lens = rng.integers(128, 4097, size=64)
    _run(oracle, "f16", (32, 8), lens, seed=5, flags=flags)


def test_fused_step_long_cut_items(native_libs, oracle):
    """Sequences long enough to be cut into many pieces: only the piece that ends the item may
    add the new token."""
    _run(oracle, "bf16", (32, 8), [20000, 3, 9000, 16 * 700], seed=9)
    _run(oracle, "f16", (4, 1), [50000], seed=10, flags=1)


def test_fused_step_rejects_bad_arguments(native_libs):
    import torch
    from orinmllm_b200 import capi
    lay = capi.layout_paged(capi.KPX_F16, 8, 128, 16, 4)
    t = torch.zeros(4096, dtype=torch.float16, device="cuda")
    f = torch.zeros(4096, dtype=torch.float32, device="cuda")
    i = torch.zeros(16, dtype=torch.int32, device="cuda")
    ws = torch.zeros(capi.decode_workspace_bytes(1, 32, 8), dtype=torch.uint8, device="cuda")
    lib = capi.lib()
    import ctypes as C
    args = lambda k_new, flags: (capi.ptr(t), capi.ptr(t), k_new, capi.ptr(t), capi.ptr(f), capi.ptr(f), capi.ptr(t),
                                 capi.ptr(t), C.byref(lay), capi.ptr(i), 4, capi.ptr(i), 1, 32, 0.1, capi.ptr(ws),
                                 ws.numel(), flags, None)
    assert lib.kpx_rope_append_decode(*args(None, 0)) == capi.KPX_ERR_INVALID_ARGUMENT
    assert lib.kpx_rope_append_decode(*args(capi.ptr(t), 6)) == capi.KPX_ERR_INVALID_ARGUMENT
    assert lib.kpx_rope_append_decode(*args(capi.ptr(t) + 2, 0)) == capi.KPX_ERR_INVALID_ARGUMENT


def test_fused_step_many_sequences_in_slices(native_libs, oracle):
    """More sequences than one launch's prefix table holds: the entry point slices the batch, and
    every slice must pick up its own rows of q / k_new / v_new / positions."""
    rng = np.random.default_rng(3)
    _run(oracle, "f16", (8, 2), rng.integers(0, 70, size=700), seed=33)


@pytest.mark.parametrize("dtype", ["f32", "f16"])
def test_fused_step_reference_cache_layout(native_libs, oracle, dtype):
    """The reference's own cache [seq_len][kv_dim] (token-major, no block table, batch 1): the step
    rotates q and k, stores row `pos` of the K and V caches and attends rows 0..pos, which is
    RoPEGpuPosLayer -> KVCacheLayer x2 -> MHAGpuPosLayer in one launch."""
    import torch
    from orinmllm_b200 import capi
    H, HKV, D, S, pos = 12, 2, 128, 544, 512
    kv_dim = HKV * D
    rng = np.random.default_rng(12)
    kc = kvtest.to_storage(rng.standard_normal((S, kv_dim)).astype(np.float32), dtype)
    vc = kvtest.to_storage(rng.standard_normal((S, kv_dim)).astype(np.float32), dtype)
    q = kvtest.to_storage(rng.standard_normal((1, H * D)).astype(np.float32), dtype)
    kn = kvtest.to_storage(rng.standard_normal((1, kv_dim)).astype(np.float32), dtype)
    vn = kvtest.to_storage(rng.standard_normal((1, kv_dim)).astype(np.float32), dtype)
    sin, cos = oracle.sin_cos_cache(D, S, 1e6)
    # CPU statement: rotate, store row pos, attend 0..pos over the contiguous cache
    q_rot, k_rot = kvtest.storage_to_f32(q, dtype).copy(), kvtest.storage_to_f32(kn, dtype).copy()
    oracle.rope(pos, q_rot[0], k_rot[0], D, sin, cos)
    q_rot = kvtest.storage_to_f32(kvtest.to_storage(q_rot, dtype), dtype)
    kc_ref, vc_ref = kc.copy(), vc.copy()
    kc_ref[pos] = kvtest.to_storage(k_rot, dtype)[0]
    vc_ref[pos] = vn[0]
    ref = oracle.mha(pos, H, 0, S, kv_dim, H // HKV, D, q_rot[0], kvtest.storage_to_f32(kc_ref, dtype).reshape(-1),
                     kvtest.storage_to_f32(vc_ref, dtype).reshape(-1))
    lay = capi.layout_contiguous(capi.dtype_code(kvtest.torch_dtype(dtype)), HKV, D, 16, S // 16)
    dk, dv = kvtest.to_device(kc, dtype), kvtest.to_device(vc, dtype)
    dq, dkn, dvn = kvtest.to_device(q, dtype), kvtest.to_device(kn, dtype), kvtest.to_device(vn, dtype)
    out = torch.full_like(dq, float("nan"))
    nbytes = capi.decode_workspace_bytes(1, H, HKV)
    ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    capi.workspace_init(ws, nbytes)
    d_pos = torch.tensor([pos], dtype=torch.int32, device="cuda")
    capi.rope_append_decode(out, dq, dkn, dvn, torch.from_numpy(sin).cuda(), torch.from_numpy(cos).cuda(), dk, dv, lay,
                            None, 0, d_pos, 1, H, 1 / np.sqrt(D), ws, nbytes, 0)
    assert capi.workspace_status(ws) == 0
    assert np.array_equal(kvtest.from_device(dk, dtype).view(np.uint8), kc_ref.view(np.uint8))
    assert np.array_equal(kvtest.from_device(dv, dtype).view(np.uint8), vc_ref.view(np.uint8))
    got = kvtest.storage_to_f32(kvtest.from_device(out, dtype), dtype)
    kvtest.assert_attention_close(got[0], ref, f"fused step, reference layout {dtype}", dtype)
