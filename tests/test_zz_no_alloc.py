"""kpx_paged_decode_static: decode for callers that can neither allocate device memory nor
pass a workspace (a plugin in a host that owns the heap, a kernel registry whose signature
has inputs and outputs only).  Its scratch is an array built into the library, shared by
every call on the device, so the test runs it twice in a row on different inputs and holds
each result to the workspace entry point's result on the same inputs.

This file sorts last on purpose: a run that stops at the first failure has then already
run every other test.
"""
import numpy as np
import pytest

from tests import kvtest

pytestmark = pytest.mark.gpu


def _decode_both_ways(case):
    import torch
    from orinmllm_b200 import capi

    dt = case.dtype
    lay = capi.layout_paged(capi.dtype_code(kvtest.torch_dtype(dt)), case.kv_heads, case.head_size,
                            case.block_size, case.num_blocks)
    shape = (case.num_blocks, case.kv_heads, case.block_size, case.head_size)
    kp = kvtest.to_device(kvtest.poison(shape, dt), dt)
    vp = kvtest.to_device(kvtest.poison(shape, dt), dt)
    capi.append(kp, vp, lay, kvtest.to_device(case.k_rows, dt), kvtest.to_device(case.v_rows, dt),
                torch.from_numpy(case.slot_mapping).cuda(), num_tokens=case.total_tokens)
    b = len(case.seq_lens)
    q = kvtest.to_device(case.q, dt)
    table = torch.from_numpy(case.block_table).cuda()
    lens = torch.from_numpy(case.seq_lens).cuda()
    scale = 1.0 / np.sqrt(case.head_size)
    # existing entry point, caller-owned workspace
    nbytes = capi.decode_workspace_bytes(b, case.q_heads, case.kv_heads, case.head_size)
    ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    capi.workspace_init(ws, nbytes)
    want = torch.full_like(q, float("nan"))
    capi.paged_decode(want, q, kp, vp, lay, table, case.block_table.shape[1], lens, 0, b,
                      case.q_heads, scale, ws, nbytes)
    assert capi.workspace_status(ws) == 0
    # new entry point: no workspace argument, nothing allocated inside
    got = torch.full_like(q, float("nan"))
    capi.paged_decode_static(got, q, kp, vp, lay, table, case.block_table.shape[1], lens, 0, b,
                             case.q_heads, scale)
    torch.cuda.synchronize()
    return (kvtest.storage_to_f32(kvtest.from_device(got, dt), dt),
            kvtest.storage_to_f32(kvtest.from_device(want, dt), dt))


def test_static_scratch_decode_matches_workspace_decode_twice(native_libs):
    # call 1: many items cut by range boundaries (partials + piece counters in use)
    case1 = kvtest.make_paged_case(41, "f16", 32, 8, [3000, 17, 1, 640, 0, 2222, 129, 4096])
    got1, want1 = _decode_both_ways(case1)
    kvtest.assert_attention_close(got1, want1, "static scratch, call 1", "f16")
    assert np.array_equal(got1, want1)
    # call 2, right after, different lengths and data: must not see call 1's leftovers
    case2 = kvtest.make_paged_case(42, "f16", 32, 8, [5, 5000, 900, 64, 1500])
    got2, want2 = _decode_both_ways(case2)
    kvtest.assert_attention_close(got2, want2, "static scratch, call 2", "f16")
    assert np.array_equal(got2, want2)


def test_static_scratch_rejects_sizes_beyond_its_limit(native_libs):
    import ctypes
    from orinmllm_b200 import capi
    # 32 KV heads x 1 head group = 32 items per sequence > 16: refused before any CUDA work
    lay = capi.layout_paged(capi.KPX_F16, 32, 128, 16)
    rc = capi.lib().kpx_paged_decode_static(1, 1, 1, 1, ctypes.byref(lay), None, 0, None, 1, 1, 32,
                                            1.0, None)
    assert rc == capi.KPX_ERR_STATIC_SCRATCH_LIMIT
    assert "built-in scratch" in capi.status_string(rc)
