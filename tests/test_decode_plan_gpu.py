"""The plan of a decode step (kpx_decode_plan / kpx_paged_decode_planned): launches with a plan
give the same bits as launches without one, in both kernel forms, and a plan that does not fit a
launch is ignored."""
import numpy as np
import pytest

from tests import kvtest

pytestmark = pytest.mark.gpu


def _setup(oracle, case):
    import torch
    from orinmllm_b200 import capi

    dt = case.dtype
    lay = capi.layout_paged(capi.dtype_code(kvtest.torch_dtype(dt)), case.kv_heads, case.head_size,
                            case.block_size, case.num_blocks)
    kp_ref, vp_ref = kvtest.oracle_pools(oracle, case)
    kp, vp = kvtest.to_device(kp_ref, dt), kvtest.to_device(vp_ref, dt)
    b = len(case.seq_lens)
    q = kvtest.to_device(case.q, dt)
    nbytes = capi.decode_workspace_bytes(b, case.q_heads, case.kv_heads, case.head_size)
    ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    capi.workspace_init(ws, nbytes)
    table = torch.from_numpy(case.block_table).cuda()
    lens = torch.from_numpy(case.seq_lens).cuda()
    plan_bytes = capi.decode_plan_bytes()
    plan = torch.zeros(plan_bytes, dtype=torch.uint8, device="cuda")
    return dict(lay=lay, kp=kp, vp=vp, kp_ref=kp_ref, vp_ref=vp_ref, q=q, ws=ws, nbytes=nbytes, table=table,
                lens=lens, plan=plan, plan_bytes=plan_bytes, b=b)


def _decode(case, s, plan, flags, lens=None, b=None):
    import torch
    from orinmllm_b200 import capi

    b = s["b"] if b is None else b
    out = torch.full_like(s["q"][:b], float("nan"))
    capi.paged_decode_planned(out, s["q"], s["kp"], s["vp"], s["lay"], s["table"], case.block_table.shape[1],
                              s["lens"] if lens is None else lens, 0, b, case.q_heads,
                              1.0 / np.sqrt(case.head_size), s["ws"], s["nbytes"], plan, flags)
    assert capi.workspace_status(s["ws"]) == 0
    return out


def _make_plan(case, s, lens=None, b=None):
    from orinmllm_b200 import capi

    capi.decode_plan(s["plan"], s["plan_bytes"], s["lay"], s["table"], case.block_table.shape[1],
                     s["lens"] if lens is None else lens, 0, s["b"] if b is None else b, case.q_heads)


@pytest.mark.parametrize("dtype,heads", [("f16", (32, 8)), ("bf16", (28, 4)), ("f32", (12, 2)), ("f16", (8, 8))])
@pytest.mark.parametrize("flags", [0, 1], ids=["one_cta", "overlapped"])
def test_planned_launch_gives_the_same_bits(native_libs, oracle, dtype, heads, flags):
    """Enough blocks per warp for the long-range form (the one that takes a plan), ragged lengths
    with empty sequences among them; checked against the oracle once and bit for bit against the
    launch without a plan."""
    import torch

    rng = np.random.default_rng(31)
    lens = [int(x) for x in rng.integers(700, 2500, size=40)]
    lens[3] = 0
    lens[17] = 0
    lens[39] = 1
    case = kvtest.make_paged_case(17, dtype, heads[0], heads[1], lens)
    s = _setup(oracle, case)
    plain = _decode(case, s, None, flags)
    _make_plan(case, s)
    head = s["plan"][:32].view(torch.int32).cpu().numpy()
    assert head[0] == 0x4B50504C and head[1] == len(lens) and head[4] == 0
    planned = _decode(case, s, s["plan"], flags)
    assert torch.equal(plain.view(torch.uint8), planned.view(torch.uint8)), "a planned launch differs"
    got = kvtest.storage_to_f32(kvtest.from_device(planned, dtype), dtype)
    ref = kvtest.oracle_decode(oracle, case, s["kp_ref"], s["vp_ref"], threads=oracle.max_threads())
    kvtest.assert_attention_close(got, ref, f"planned decode {dtype} H={heads}", dtype)


def test_plan_follows_the_lengths_of_each_step(native_libs, oracle):
    """Two steps with different lengths on one plan buffer: the plan is made again for the second
    step and both steps equal their unplanned launches."""
    import torch

    rng = np.random.default_rng(7)
    lens = [int(x) for x in rng.integers(900, 2000, size=32)]
    case = kvtest.make_paged_case(23, "f16", 32, 8, lens)
    s = _setup(oracle, case)
    shorter = torch.from_numpy((case.seq_lens - 37).astype(np.int32)).cuda()
    for step_lens in (shorter, s["lens"]):
        _make_plan(case, s, lens=step_lens)
        planned = _decode(case, s, s["plan"], 1, lens=step_lens)
        plain = _decode(case, s, None, 1, lens=step_lens)
        assert torch.equal(plain.view(torch.uint8), planned.view(torch.uint8))


def test_plan_that_does_not_fit_is_ignored(native_libs, oracle):
    """A plan made for another batch size, a zeroed plan and a launch short enough for the
    short-range form: each launch works everything out itself and is right."""
    import torch

    rng = np.random.default_rng(11)
    lens = [int(x) for x in rng.integers(700, 1500, size=40)]
    case = kvtest.make_paged_case(29, "f16", 32, 8, lens)
    s = _setup(oracle, case)
    plain = _decode(case, s, None, 0)
    _make_plan(case, s, b=16)                       # plan of the first 16 sequences only
    assert torch.equal(plain.view(torch.uint8), _decode(case, s, s["plan"], 0).view(torch.uint8))
    s["plan"].zero_()
    assert torch.equal(plain.view(torch.uint8), _decode(case, s, s["plan"], 0).view(torch.uint8))
    # three short sequences: the short-range form, which does not read plans
    small = kvtest.make_paged_case(5, "f16", 32, 8, [40, 3, 130])
    t = _setup(oracle, small)
    base = _decode(small, t, None, 0)
    _make_plan(small, t)
    assert torch.equal(base.view(torch.uint8), _decode(small, t, t["plan"], 0).view(torch.uint8))
    got = kvtest.storage_to_f32(kvtest.from_device(base, "f16"), "f16")
    ref = kvtest.oracle_decode(oracle, small, t["kp_ref"], t["vp_ref"], threads=oracle.max_threads())
    kvtest.assert_attention_close(got, ref, "short launch with a plan it ignores", "f16")


def test_plan_argument_checks(native_libs):
    import torch
    from orinmllm_b200 import capi

    lay = capi.layout_paged(capi.KPX_F16, 8, 128, 16, 64)
    plan = torch.zeros(capi.decode_plan_bytes(), dtype=torch.uint8, device="cuda")
    table = torch.zeros(4, 4, dtype=torch.int32, device="cuda")
    lens = torch.zeros(4, dtype=torch.int32, device="cuda")
    with pytest.raises(capi.KpxError):
        capi.decode_plan(plan, 64, lay, table, 4, lens, 0, 4, 32)          # buffer too small
    with pytest.raises(capi.KpxError):
        capi.decode_plan(plan, plan.numel(), lay, table, 4, lens, 0, 4, 30)  # heads do not divide
    with pytest.raises(capi.KpxError):
        capi.decode_plan(None, plan.numel(), lay, table, 4, lens, 0, 4, 32)
