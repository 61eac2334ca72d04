"""Error behaviour through the C ABI: bad arguments are refused before any launch with a status
code (nothing aborts), and data errors that only the device can see (a block id outside the
pool) are clamped, reported through the workspace status word and cleared by reading it."""
import ctypes

import numpy as np
import pytest

from tests import kvtest

pytestmark = pytest.mark.gpu


def _decode_setup(dtype="f16"):
    import torch
    from orinmllm_b200 import capi
    case = kvtest.make_paged_case(2, dtype, 8, 2, [40, 300, 17])
    lay = capi.layout_paged(capi.KPX_F16, 2, 128, 16, case.num_blocks)
    g = torch.Generator(device="cuda").manual_seed(0)
    shape = (case.num_blocks, 2, 16, 128)
    kp = torch.randn(shape, generator=g, device="cuda", dtype=torch.float16)
    vp = torch.randn(shape, generator=g, device="cuda", dtype=torch.float16)
    q = torch.randn(3, 8 * 128, generator=g, device="cuda", dtype=torch.float16)
    nbytes = capi.decode_workspace_bytes(3, 8, 2)
    ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    capi.workspace_init(ws, nbytes)
    return case, lay, kp, vp, q, ws, nbytes


def test_decode_reports_block_ids_outside_the_pool(native_libs):
    import torch
    from orinmllm_b200 import capi
    case, lay, kp, vp, q, ws, nbytes = _decode_setup()
    lens = torch.from_numpy(case.seq_lens).cuda()
    good = torch.from_numpy(case.block_table).cuda()
    out_good = torch.empty_like(q)
    capi.paged_decode(out_good, q, kp, vp, lay, good, good.shape[1], lens, 0, 3, 8, 0.1, ws, nbytes)
    assert capi.workspace_status(ws) == 0
    for bad_id in (case.num_blocks, case.num_blocks + 12345, -7):
        table = case.block_table.copy()
        table[1, 3] = bad_id  # inside sequence 1's 19 blocks
        out = torch.empty_like(q)
        capi.paged_decode(out, q, kp, vp, lay, torch.from_numpy(table).cuda(), table.shape[1], lens, 0, 3, 8, 0.1,
                          ws, nbytes)
        assert capi.workspace_status(ws) == capi.KPX_ERR_INVALID_ARGUMENT
        assert capi.workspace_status(ws) == 0, "reading the status clears it"
        assert torch.isfinite(out.float()).all()
        # the sequences whose tables are intact are unaffected
        assert torch.equal(out[0], out_good[0]) and torch.equal(out[2], out_good[2])
    # and the workspace is usable again without re-initialisation
    out = torch.empty_like(q)
    capi.paged_decode(out, q, kp, vp, lay, good, good.shape[1], lens, 0, 3, 8, 0.1, ws, nbytes)
    assert capi.workspace_status(ws) == 0 and torch.equal(out, out_good)


def test_prefill_reports_block_ids_outside_the_pool(native_libs):
    import torch
    from orinmllm_b200 import capi
    H, HKV, nb = 8, 2, 64
    lay = capi.layout_paged(capi.KPX_BF16, HKV, 128, 16, nb)
    g = torch.Generator(device="cuda").manual_seed(1)
    kp = torch.randn(nb, HKV, 16, 128, generator=g, device="cuda", dtype=torch.float32).bfloat16()
    vp = torch.randn(nb, HKV, 16, 128, generator=g, device="cuda", dtype=torch.float32).bfloat16()
    n = 200
    q = torch.randn(n, H * 128, generator=g, device="cuda", dtype=torch.float32).bfloat16()
    out = torch.empty_like(q)
    table = np.arange(13, dtype=np.int32)[None, :].copy()
    table[0, 5] = nb + 3
    nbytes = capi.prefill_workspace_bytes(n, H, HKV)
    ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    capi.workspace_init(ws, nbytes)
    capi.paged_prefill(out, q, kp, vp, lay, torch.from_numpy(table).cuda(), 13, np.array([0, n], np.int32),
                       np.array([0], np.int32), 1, H, 0.1, ws, nbytes)
    assert capi.workspace_status(ws) == capi.KPX_ERR_INVALID_ARGUMENT
    assert torch.isfinite(out.float()).all()


def test_arguments_are_refused_with_status_codes(native_libs):
    import torch
    from orinmllm_b200 import capi
    case, lay, kp, vp, q, ws, nbytes = _decode_setup()
    L = capi.lib()
    lens = torch.from_numpy(case.seq_lens).cuda()
    table = torch.from_numpy(case.block_table).cuda()
    out = torch.empty_like(q)

    def decode(**kw):
        a = dict(out=out.data_ptr(), q=q.data_ptr(), kp=kp.data_ptr(), vp=vp.data_ptr(), lay=lay,
                 table=table.data_ptr(), width=table.shape[1], lens=lens.data_ptr(), batch=3, heads=8,
                 ws=ws.data_ptr(), nbytes=nbytes)
        a.update(kw)
        return L.kpx_paged_decode(a["out"], a["q"], a["kp"], a["vp"], ctypes.byref(a["lay"]), a["table"], a["width"],
                                  a["lens"], 0, a["batch"], a["heads"], 0.1, a["ws"], a["nbytes"], None)

    assert decode() == 0
    assert decode(nbytes=nbytes - 1) == capi.KPX_ERR_WORKSPACE_TOO_SMALL
    assert decode(ws=None) == capi.KPX_ERR_INVALID_ARGUMENT
    assert decode(q=q.data_ptr() + 2) == capi.KPX_ERR_INVALID_ARGUMENT      # 16-byte alignment
    assert decode(heads=7) == capi.KPX_ERR_INVALID_ARGUMENT                 # not a multiple of the KV heads
    assert decode(width=0) == capi.KPX_ERR_INVALID_ARGUMENT
    assert decode(batch=-1) == capi.KPX_ERR_INVALID_ARGUMENT
    assert decode(batch=0) == 0
    odd = capi.layout_paged(capi.KPX_F16, 2, 96, 16, case.num_blocks)
    assert decode(lay=odd) == capi.KPX_ERR_UNIMPLEMENTED                    # head size other than 128
    torch.cuda.synchronize()
    assert capi.workspace_status(ws) == 0


def test_refcount_underflow_is_counted(native_libs):
    import torch
    from orinmllm_b200 import capi
    refc = torch.tensor([1, 0, 2, 0], dtype=torch.int32, device="cuda")
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    ids = torch.tensor([0, 1, 2], dtype=torch.int32, device="cuda")
    deltas = torch.tensor([-1, -1, -1], dtype=torch.int32, device="cuda")
    capi.refcount_update(refc, 4, ids, deltas, 3, err)
    torch.cuda.synchronize()
    assert refc.tolist()[0] == 0 and refc.tolist()[2] == 1
    assert int(err.item()) >= 1  # block 1 went below zero
