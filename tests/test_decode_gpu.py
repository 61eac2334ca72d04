"""Parity of the CUDA append + paged decode path with the CPU oracle, through the C ABI."""
import numpy as np
import pytest

from tests import kvtest

pytestmark = pytest.mark.gpu


def _run_case(oracle, case, check_append=True, launches=1):
    import torch
    from orinmllm_b200 import capi

    dt = case.dtype
    code = capi.dtype_code(kvtest.torch_dtype(dt))
    lay = capi.layout_paged(code, case.kv_heads, case.head_size, case.block_size, case.num_blocks)
    shape = (case.num_blocks, case.kv_heads, case.block_size, case.head_size)
    kp = kvtest.to_device(kvtest.poison(shape, dt), dt)
    vp = kvtest.to_device(kvtest.poison(shape, dt), dt)
    if case.total_tokens:
        capi.append(kp, vp, lay, kvtest.to_device(case.k_rows, dt), kvtest.to_device(case.v_rows, dt),
                    torch.from_numpy(case.slot_mapping).cuda(), num_tokens=case.total_tokens)
    kp_ref, vp_ref = kvtest.oracle_pools(oracle, case)
    if check_append:
        # appended cache contents are bit-exact (compare raw bytes, NaN poison included)
        assert np.array_equal(kvtest.from_device(kp, dt).view(np.uint8), kp_ref.view(np.uint8))
        assert np.array_equal(kvtest.from_device(vp, dt).view(np.uint8), vp_ref.view(np.uint8))
    b = len(case.seq_lens)
    q = kvtest.to_device(case.q, dt)
    out = torch.full_like(q, float("nan"))
    nbytes = capi.decode_workspace_bytes(b, case.q_heads, case.kv_heads, case.head_size)
    ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    capi.workspace_init(ws, nbytes)
    first = None
    for _ in range(launches):  # later launches reuse the workspace as the earlier ones left it
        out.fill_(float("nan"))
        capi.paged_decode(out, q, kp, vp, lay, torch.from_numpy(case.block_table).cuda(),
                          case.block_table.shape[1], torch.from_numpy(case.seq_lens).cuda(), 0, b,
                          case.q_heads, 1.0 / np.sqrt(case.head_size), ws, nbytes)
        assert capi.workspace_status(ws) == 0
        if first is None:
            first = out.clone()
        else:
            assert torch.equal(first.view(torch.uint8), out.view(torch.uint8)), "a repeated launch differs"
    got = kvtest.storage_to_f32(kvtest.from_device(out, dt), dt)
    ref = kvtest.oracle_decode(oracle, case, kp_ref, vp_ref, threads=oracle.max_threads())
    return kvtest.assert_attention_close(got, ref, f"decode {dt} H={case.q_heads}/{case.kv_heads}", dt)


@pytest.mark.parametrize("dtype", ["f16", "bf16", "f32"])
@pytest.mark.parametrize("heads", [(32, 8), (12, 2), (28, 4), (8, 8), (4, 2), (16, 2)])
def test_decode_small(native_libs, oracle, dtype, heads):
    lens = [1, 15, 16, 17, 63, 64, 65, 128, 200, 513]
    case = kvtest.make_paged_case(11, dtype, heads[0], heads[1], lens)
    _run_case(oracle, case)


@pytest.mark.parametrize("dtype", ["f16", "bf16"])
def test_decode_ragged_and_empty(native_libs, oracle, dtype):
    lens = [0, 5, 0, 1000, 3, 0, 77, 2049]
    case = kvtest.make_paged_case(5, dtype, 32, 8, lens)
    _run_case(oracle, case)


def test_decode_single_long(native_libs, oracle):
    # one sequence spread over every persistent CTA: exercises the split-KV merge
    case = kvtest.make_paged_case(7, "f16", 32, 8, [20000])
    _run_case(oracle, case)


@pytest.mark.parametrize("dtype,heads", [("f16", (8, 2)), ("bf16", (14, 2)), ("f16", (2, 2))])
def test_decode_long_items_two_level_assembly(native_libs, oracle, dtype, heads):
    """Sequences long enough that one (sequence, KV head) item is cut into hundreds of pieces: the
    pieces are merged per group of warps and then per item.  Launched three times on the same
    workspace (the counters of both levels must have reset themselves)."""
    case = kvtest.make_paged_case(5, dtype, heads[0], heads[1], [60000, 17, 45000, 3000])
    _run_case(oracle, case, check_append=False, launches=3)


def test_decode_many_short(native_libs, oracle):
    # many items per CTA range
    rng = np.random.default_rng(3)
    lens = rng.integers(1, 40, size=300)
    case = kvtest.make_paged_case(9, "f16", 32, 8, lens)
    _run_case(oracle, case)


def test_decode_batch_slices(native_libs, oracle):
    # more sequences than one launch's prefix table holds (1024): sliced launches
    rng = np.random.default_rng(4)
    lens = rng.integers(0, 50, size=1500)
    case = kvtest.make_paged_case(10, "f16", 8, 2, lens)
    _run_case(oracle, case, check_append=False)


def test_decode_headline_shape(native_libs, oracle):
    # Qwen3-8B attention shape, batch 64, ctx uniform in [128, 4096], fp16, block 16
    rng = np.random.default_rng(2024)
    lens = rng.integers(128, 4097, size=64)
    case = kvtest.make_paged_case(2024, "f16", 32, 8, lens)
    max_abs, max_rel = _run_case(oracle, case)
    print(f"headline parity: max_abs={max_abs:.3e} max_rel={max_rel:.3e}")


@pytest.mark.parametrize("dtype,heads", [("f16", (28, 4)), ("bf16", (28, 4)), ("f16", (40, 8)), ("f16", (64, 8))])
def test_decode_headline_size_five_to_eight_heads_per_kv_head(native_libs, oracle, dtype, heads):
    # Qwen2.5-7B attention shape (28 Q / 4 KV heads: seven query heads per KV head) and its
    # neighbours at the headline batch: served in passes of four heads (padding heads of the last
    # pass carry a zero query and are never written)
    rng = np.random.default_rng(77)
    lens = rng.integers(128, 4097, size=64)
    case = kvtest.make_paged_case(77, dtype, heads[0], heads[1], lens)
    max_abs, max_rel = _run_case(oracle, case, launches=2)
    print(f"{heads[0]}/{heads[1]} heads {dtype}: max_abs={max_abs:.3e} max_rel={max_rel:.3e}")


def test_decode_placement_invariance(native_libs, oracle):
    # the same sequences through two different block placements give bit-identical outputs
    import torch
    from orinmllm_b200 import capi
    lens = [100, 999, 31]
    outs = []
    for seed in (1, 2):
        case = kvtest.make_paged_case(21, "f16", 32, 8, lens)
        rng = np.random.default_rng(seed)
        perm = rng.permutation(case.num_blocks).astype(np.int32)
        table = np.where(case.block_table >= 0, perm[np.maximum(case.block_table, 0)], -1).astype(np.int32)
        slots = []
        for i, l in enumerate(lens):
            pos = np.arange(l)
            slots.append(table[i, pos // 16].astype(np.int64) * 16 + pos % 16)
        case.block_table, case.slot_mapping = table, np.concatenate(slots)
        lay = capi.layout_paged(capi.KPX_F16, 8, 128, 16, case.num_blocks)
        shape = (case.num_blocks, 8, 16, 128)
        kp = kvtest.to_device(kvtest.poison(shape, "f16"), "f16")
        vp = kvtest.to_device(kvtest.poison(shape, "f16"), "f16")
        capi.append(kp, vp, lay, kvtest.to_device(case.k_rows, "f16"), kvtest.to_device(case.v_rows, "f16"),
                    torch.from_numpy(case.slot_mapping).cuda(), num_tokens=case.total_tokens)
        q = kvtest.to_device(case.q, "f16")
        out = torch.empty_like(q)
        nbytes = capi.decode_workspace_bytes(3, 32, 8)
        ws = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
        capi.paged_decode(out, q, kp, vp, lay, torch.from_numpy(table).cuda(), table.shape[1],
                          torch.from_numpy(case.seq_lens).cuda(), 0, 3, 32, 1.0 / np.sqrt(128), ws, nbytes)
        outs.append(out.cpu())
    assert torch.equal(outs[0], outs[1])


@pytest.mark.parametrize("knobs", [(0, 12, 4), (1 << 20, 20, 0), (1 << 20, 3, 1), (1 << 20, 12, 4)])
@pytest.mark.parametrize("dtype,heads,lens", [
    ("f16", (32, 8), [4096]),                 # one sequence: every item is cut into many pieces
    ("bf16", (12, 2), [300, 9000, 17, 0, 64]),
    ("f32", (8, 8), [2000, 1]),
    ("f16", (4, 1), [40000]),                 # one KV head of one long sequence (the sharded case)
])
def test_decode_small_launch_forms(native_libs, oracle, knobs, dtype, heads, lens):
    """Launches with few blocks per warp run a form of the kernel that cuts the work into fewer,
    longer ranges on CTA-minor warp numbers.  Whatever the cut (off; as coarse as 20 blocks per
    range with idle SMs allowed; as fine as 3), outputs meet the oracle, twice in a row on the
    same workspace."""
    from orinmllm_b200 import capi
    lib = capi.lib()
    try:
        lib.kpx_internal_set_decode_small(*knobs)
        case = kvtest.make_paged_case(29, dtype, heads[0], heads[1], lens)
        _run_case(oracle, case, check_append=False, launches=2)
    finally:
        lib.kpx_internal_set_decode_small(12, 12, 4)
