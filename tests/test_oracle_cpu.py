"""CPU-only checks of the oracle itself (the checker must be trusted before it checks)."""
import numpy as np
import pytest

from tests import kvtest


def _config1(oracle, seed=1):
    """The CPU-runnable anchor case: Qwen2.5-1.5B attention shape, 512 cached tokens + 1 new, fp32."""
    H, HKV, D, S = 12, 2, 128, 520
    rng = np.random.default_rng(seed)
    kc = np.zeros((1, S, HKV * D), np.float32)
    vc = np.zeros((1, S, HKV * D), np.float32)
    kc[0, :512] = rng.standard_normal((512, HKV * D), np.float32)
    vc[0, :512] = rng.standard_normal((512, HKV * D), np.float32)
    q = rng.standard_normal(H * D, np.float32)
    k = rng.standard_normal(HKV * D, np.float32)
    v = rng.standard_normal(HKV * D, np.float32)
    sin, cos = oracle.sin_cos_cache(D, S, 1e6)
    oracle.rope(512, q, k, D, sin, cos)
    kc[0, 512], vc[0, 512] = k, v
    return H, HKV, D, S, q, kc, vc


def test_config1_cpu_anchor_matches_float64_shadow(oracle):
    H, HKV, D, S, q, kc, vc = _config1(oracle)
    out = oracle.mha(512, H, 0, S, HKV * D, H // HKV, D, q, kc.reshape(-1), vc.reshape(-1))
    ref = oracle.mha_f64(512, H, 0, S, HKV * D, H // HKV, D, q, kc.reshape(-1), vc.reshape(-1))
    assert out.shape == (H * D,)
    assert np.abs(out - ref).max() < 2e-6  # the oracle's own fp32 rounding, 3 orders below 2e-3


def test_softmax_matches_numpy(oracle):
    rng = np.random.default_rng(0)
    x = rng.standard_normal(513).astype(np.float32) * 4
    y = x.copy()
    oracle.lib.orc_softmax_inplace(y, len(y))
    e = np.exp(x.astype(np.float64) - x.max())
    assert np.allclose(y, e / e.sum(), rtol=1e-5, atol=1e-8)
    assert abs(float(y.sum()) - 1.0) < 1e-5


def test_sin_cos_table_definition(oracle):
    sin, cos = oracle.sin_cos_cache(128, 64, 1e6)
    pos, k = 37, 20
    freq = np.float32(1.0) / np.float32(np.power(np.float32(1e6), np.float32(k) / np.float32(128)))
    assert abs(sin[pos, k] - np.sin(np.float32(pos) * freq)) < 1e-6
    assert np.all(sin[0] == 0) and np.all(cos[0] == 1)


def test_rope_is_a_rotation_of_half_split_pairs(oracle):
    D = 128
    rng = np.random.default_rng(3)
    q = rng.standard_normal(4 * D).astype(np.float32)
    k = rng.standard_normal(2 * D).astype(np.float32)
    q0, k0 = q.copy(), k.copy()
    sin, cos = oracle.sin_cos_cache(D, 100, 1e6)
    oracle.rope(77, q, k, D, sin, cos)
    # norms of every (j, j+64) pair are preserved; position 0 is the identity
    for vec, ref in ((q, q0), (k, k0)):
        a = vec.reshape(-1, 2, D // 2)
        b = ref.reshape(-1, 2, D // 2)
        assert np.allclose((a ** 2).sum(1), (b ** 2).sum(1), rtol=1e-5)
    j = 5
    c, s = cos[77, 2 * j], sin[77, 2 * j]
    assert q[j] == np.float32(q0[j] * c) - np.float32(q0[j + 64] * s)
    q1 = q0.copy()
    oracle.rope(0, q1, None, D, sin, cos)
    assert np.array_equal(q1, q0)


@pytest.mark.parametrize("dtype", ["f16", "bf16", "f32"])
def test_paged_gather_equals_contiguous(oracle, dtype):
    """Paged state gathered through the block table equals the contiguous cache the
    reference would hold, so orc_mha on the gather IS the reference arithmetic."""
    case = kvtest.make_paged_case(5, dtype, 12, 2, [1, 16, 17, 300])
    kp, vp = kvtest.oracle_pools(oracle, case)
    start = 0
    for b, n in enumerate(case.seq_lens):
        got = oracle.gather_paged(kp, case.block_table[b], int(n), case.kv_heads, 128, 16)
        assert np.array_equal(got.view(np.uint8), case.k_rows[start:start + n].view(np.uint8))
        start += int(n)


def test_paged_decode_equals_per_sequence_mha(oracle):
    case = kvtest.make_paged_case(6, "f32", 8, 2, [40, 7, 129])
    kp, vp = kvtest.oracle_pools(oracle, case)
    out = kvtest.oracle_decode(oracle, case, kp, vp)
    start = 0
    for b, n in enumerate(case.seq_lens):
        n = int(n)
        kc = np.ascontiguousarray(case.k_rows[start:start + n]).reshape(-1)
        vc = np.ascontiguousarray(case.v_rows[start:start + n]).reshape(-1)
        ref = oracle.mha(n - 1, 8, 0, n, 256, 4, 128, case.q[b], kc, vc)
        assert np.array_equal(out[b], ref)
        start += n


def test_prefill_oracle_is_causal(oracle):
    rng = np.random.default_rng(9)
    H, HKV, D, S = 4, 2, 128, 48
    kc = rng.standard_normal((S, HKV * D), np.float32)
    vc = rng.standard_normal((S, HKV * D), np.float32)
    q = rng.standard_normal((8, H * D), np.float32)
    out = oracle.mha_prefill(16, q, H, S, HKV * D, 2, D, kc.reshape(-1), vc.reshape(-1))
    kc2 = kc.copy()
    kc2[30:] = 99.0  # rows beyond every query's horizon (16+7=23) must not matter
    out2 = oracle.mha_prefill(16, q, H, S, HKV * D, 2, D, kc2.reshape(-1), vc.reshape(-1))
    assert np.array_equal(out, out2)
    one = oracle.mha(16 + 3, H, 0, S, HKV * D, 2, D, q[3], kc.reshape(-1), vc.reshape(-1))
    assert np.array_equal(out[3], one)


def test_rmsnorm_heads_definition(oracle):
    """w * x / sqrt(mean(x^2) + eps) per head row (cpu/rmsnorm_kernel.cpp:26-34)."""
    rng = np.random.default_rng(4)
    x = rng.standard_normal((5, 3 * 128)).astype(np.float32)
    w = rng.standard_normal(128).astype(np.float32)
    ref = x.reshape(5, 3, 128).astype(np.float64)
    ref = w * ref / np.sqrt((ref ** 2).mean(-1, keepdims=True) + 1e-6)
    got = x.copy()
    oracle.rmsnorm_heads(got, 3, 128, w, 1e-6)
    assert np.allclose(got.reshape(5, 3, 128), ref, rtol=2e-6, atol=1e-6)
