"""A bounded device-side wait that runs out: the kernel must return, the workspace status must say
KPX_ERR_DEVICE_TIMEOUT, and after the workspace has started over the next launch must be right.

The failure is made without faulting or hanging anything: a test-only knob of the library makes
ONE warp announce its first tile request to its barrier without issuing the copy, and shortens
the poll limit of the bounded waits; that warp gives up after the limit, raises the status word
and retires, every other warp finishes as usual."""
import numpy as np
import pytest

from tests import kvtest

pytestmark = pytest.mark.gpu


def _setup(oracle):
    import torch
    from orinmllm_b200 import capi
    rng = np.random.default_rng(31)
    lens = rng.integers(600, 3000, size=24)
    case = kvtest.make_paged_case(31, "f16", 32, 8, lens)
    lay = capi.layout_paged(capi.KPX_F16, 8, 128, 16, case.num_blocks)
    kp_ref, vp_ref = kvtest.oracle_pools(oracle, case)
    kp, vp = kvtest.to_device(kp_ref, "f16"), kvtest.to_device(vp_ref, "f16")
    q = kvtest.to_device(case.q, "f16")
    nbytes = capi.decode_workspace_bytes(len(lens), 32, 8)
    ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    capi.workspace_init(ws, nbytes)
    ref = kvtest.oracle_decode(oracle, case, kp_ref, vp_ref, threads=oracle.max_threads())
    table, d_lens = torch.from_numpy(case.block_table).cuda(), torch.from_numpy(case.seq_lens).cuda()

    def launch(entry=capi.paged_decode):
        out = torch.full_like(q, float("nan"))
        entry(out, q, kp, vp, lay, table, case.block_table.shape[1], d_lens, 0, len(lens), 32, 1 / np.sqrt(128),
              ws, nbytes)
        return out

    return capi, ws, nbytes, ref, launch


@pytest.mark.parametrize("form", ["large", "overlapped"])
@pytest.mark.parametrize("recover", ["status_read", "explicit_init"])
def test_decode_wait_runs_out_and_the_workspace_recovers(native_libs, oracle, form, recover):
    import torch
    capi, ws, nbytes, ref, launch = _setup(oracle)
    entry = capi.paged_decode if form == "large" else capi.paged_decode_overlapped
    lib = capi.lib()
    good = launch(entry)
    assert capi.workspace_status(ws) == 0
    kvtest.assert_attention_close(good.float().cpu().numpy(), ref, "before the fault")
    lib.kpx_internal_set_decode_fault(3000, 7)  # warp 7 never gets its first tile; waits give up after 3000 polls
    try:
        broken = launch(entry)
        torch.cuda.synchronize()  # the kernel has returned
    finally:
        lib.kpx_internal_set_decode_fault(0, -1)
    bad_rows = torch.isnan(broken.float()).any(dim=1).sum().item()
    assert bad_rows >= 1, "the withheld warp's item cannot have been assembled"
    if recover == "status_read":
        assert capi.workspace_status(ws) == capi.KPX_ERR_DEVICE_TIMEOUT  # reading it wipes the workspace
        assert capi.workspace_status(ws) == 0
    else:
        capi.workspace_init(ws, nbytes)  # a caller that saw the failure some other way
    again = launch(entry)
    assert capi.workspace_status(ws) == 0
    assert torch.equal(again.view(torch.uint8), good.view(torch.uint8)), "the launch after recovery differs"


@pytest.mark.parametrize("tile", [0, 1, 2], ids=["first_k_tile", "first_v_tile", "second_k_tile"])
def test_prefill_wait_runs_out_and_the_next_call_is_right(native_libs, oracle, tile):
    """The tensor-core prefill kernel: one CTA never gets one of its tiles (the first K tile: the
    MMA warp gives up before its first scores; the first V tile or the second K tile: it gives
    up inside its loop, on the progress words, with scores and weights of the first tile
    already exchanged).  The roles give up in step (the loader on its barrier, the MMA warp on
    the give-up word, the softmax threads by vote), tensor memory is freed, the kernel returns,
    the status says so, and the same call made again is right."""
    import torch
    from orinmllm_b200 import capi
    H, HKV, D, n, start = 8, 2, 128, 300, 212
    length = start + n
    case = kvtest.make_paged_case(13, "bf16", H, HKV, [length])
    lay = capi.layout_paged(capi.KPX_BF16, HKV, D, 16, case.num_blocks)
    kp_ref, vp_ref = kvtest.oracle_pools(oracle, case)
    kp, vp = kvtest.to_device(kp_ref, "bf16"), kvtest.to_device(vp_ref, "bf16")
    rng = np.random.default_rng(5)
    q_st = kvtest.to_storage(rng.standard_normal((n, H * D)).astype(np.float32), "bf16")
    dq = kvtest.to_device(q_st, "bf16")
    table = torch.from_numpy(case.block_table).cuda()
    nbytes = capi.prefill_workspace_bytes(n, H, HKV, D)
    ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    capi.workspace_init(ws, nbytes)
    cu, sp = np.array([0, n], np.int32), np.array([start], np.int32)

    def call():
        out = torch.full_like(dq, float("nan"))
        capi.paged_prefill(out, dq, kp, vp, lay, table, case.block_table.shape[1], cu, sp, 1, H, 1 / np.sqrt(D), ws, nbytes)
        return out

    kc = kvtest.storage_to_f32(oracle.gather_paged(kp_ref, case.block_table[0], length, HKV, D, 16), "bf16")
    vc = kvtest.storage_to_f32(oracle.gather_paged(vp_ref, case.block_table[0], length, HKV, D, 16), "bf16")
    ref = oracle.mha_prefill(start, kvtest.storage_to_f32(q_st, "bf16"), H, length, HKV * D, H // HKV, D,
                             kc.reshape(-1), vc.reshape(-1), threads=oracle.max_threads())
    lib = capi.lib()
    lib.kpx_internal_set_prefill_fault(3000, tile << 16)  # CTA 0, the tile chosen above
    if tile:
        lib.kpx_internal_set_prefill_split(0)  # whole pairs, so that CTA 0 has a second key tile
    try:
        broken = call()
        torch.cuda.synchronize()  # the kernel has returned
    finally:
        lib.kpx_internal_set_prefill_fault(0, -1)
        lib.kpx_internal_set_prefill_split(-1)
    assert capi.workspace_status(ws) == capi.KPX_ERR_DEVICE_TIMEOUT
    # the withheld CTA's rows are missing: NaN where it owned them outright, wrong (its share of
    # the keys left out) where the call was cut along the keys and merged
    b = broken.float().cpu().numpy()
    assert np.isnan(b).any() or np.nanmax(np.abs(b - ref)) > 10 * kvtest.ATOL
    good = call()
    assert capi.workspace_status(ws) == 0
    got = kvtest.storage_to_f32(kvtest.from_device(good, "bf16"), "bf16")
    kvtest.assert_attention_close(got, ref, "prefill after a timed-out call", "bf16")
