"""The hand-off to the step after the path: the output projection Wo
(kuiper/source/model/qwen_base.cpp:136-140 for decode, :464-474 for prefill) reads the attention
output as a row-major [rows, heads*head_size] matrix.  The kernels write exactly that layout, so
a GEMM consumes their output buffer as it is: no transpose, no copy.  Here a library GEMM stands
for Wo (the weight GEMMs are outside the path) and the product is checked against the oracle's
attention output times the same weights."""
import numpy as np
import pytest

from tests import kvtest

pytestmark = pytest.mark.gpu


def test_decode_and_prefill_outputs_feed_the_output_projection_as_they_are(native_libs, oracle):
    import torch
    from orinmllm_b200 import capi
    H, HKV, D, dim_out = 32, 8, 128, 512
    rng = np.random.default_rng(41)
    lens = rng.integers(100, 900, size=24)
    case = kvtest.make_paged_case(41, "f16", H, HKV, lens)
    lay = capi.layout_paged(capi.KPX_F16, HKV, D, 16, case.num_blocks)
    kp_ref, vp_ref = kvtest.oracle_pools(oracle, case)
    kp, vp = kvtest.to_device(kp_ref, "f16"), kvtest.to_device(vp_ref, "f16")
    q = kvtest.to_device(case.q, "f16")
    out = torch.full_like(q, float("nan"))
    nbytes = capi.decode_workspace_bytes(len(lens), H, HKV)
    ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    capi.workspace_init(ws, nbytes)
    table, d_lens = torch.from_numpy(case.block_table).cuda(), torch.from_numpy(case.seq_lens).cuda()
    capi.paged_decode(out, q, kp, vp, lay, table, case.block_table.shape[1], d_lens, 0, len(lens), H, 1 / np.sqrt(D),
                      ws, nbytes)
    assert capi.workspace_status(ws) == 0
    # the buffer the kernel wrote IS the GEMM's left operand: [batch, H*D], row stride H*D
    assert out.is_contiguous() and out.shape == (len(lens), H * D) and out.stride() == (H * D, 1)
    wo = torch.from_numpy((rng.standard_normal((dim_out, H * D)) / np.sqrt(H * D)).astype(np.float32)).cuda()
    projected = torch.matmul(out, wo.to(torch.float16).t()).float().cpu().numpy()     # rows @ Wo^T
    ref = kvtest.oracle_decode(oracle, case, kp_ref, vp_ref, threads=oracle.max_threads())
    want = ref.astype(np.float64) @ wo.to(torch.float16).float().cpu().numpy().astype(np.float64).T
    # each output of the projection sums 4096 products of values that are each right to 2e-3
    assert np.abs(projected - want).max() <= 5e-3
    # the same through the prefill entry point: 3 sequences' chunks, rows in cu_q_lens order
    n = [40, 128, 7]
    cu = np.concatenate([[0], np.cumsum(n)]).astype(np.int32)
    start = np.array([int(lens[i]) - n[i] for i in range(3)], np.int32)   # the chunk = each sequence's last n tokens
    qp = torch.randn(int(cu[-1]), H * D, device="cuda").to(torch.float16)
    outp = torch.full_like(qp, float("nan"))
    pbytes = capi.prefill_workspace_bytes(int(cu[-1]), H, HKV, D)
    pws = torch.empty(pbytes, dtype=torch.uint8, device="cuda")
    capi.workspace_init(pws, pbytes)
    capi.paged_prefill(outp, qp, kp, vp, lay, table[:3].contiguous(), case.block_table.shape[1], cu, start, 3, H,
                       1 / np.sqrt(D), pws, pbytes)
    assert capi.workspace_status(pws) == 0
    assert outp.is_contiguous() and outp.stride() == (H * D, 1)
    proj_p = torch.matmul(outp, wo.to(torch.float16).t()).float().cpu().numpy()
    refs = []
    for i in range(3):
        length = int(lens[i])
        kc = kvtest.storage_to_f32(oracle.gather_paged(kp_ref, case.block_table[i], length, HKV, D, 16), "f16")
        vc = kvtest.storage_to_f32(oracle.gather_paged(vp_ref, case.block_table[i], length, HKV, D, 16), "f16")
        refs.append(oracle.mha_prefill(int(start[i]), qp[cu[i]:cu[i + 1]].float().cpu().numpy(), H, length, HKV * D,
                                       H // HKV, D, kc.reshape(-1), vc.reshape(-1), threads=oracle.max_threads()))
    want_p = np.concatenate(refs).astype(np.float64) @ wo.to(torch.float16).float().cpu().numpy().astype(np.float64).T
    assert np.abs(proj_p - want_p).max() <= 5e-3
