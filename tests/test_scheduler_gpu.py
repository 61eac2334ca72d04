"""The request scheduler driving the kernels end to end on the GPU: concurrent requests that
share a token prefix (mapped by reference, copy-on-write on the first append into the shared
partial block), chunked prefill, batched decode, admission in waves.  Every attention output a
request produced equals the oracle run on that request's own contiguous K/V history."""
import numpy as np
import pytest

from tests import kvtest

pytestmark = pytest.mark.gpu


def oracle_outputs(oracle, sim, tokens, n_cached):
    """[L, n_cached, dim] reference outputs of one request from its token list alone.  The rotation
    uses the sin/cos table the device path used (an input of the RoPE op, as in the reference):
    the device's table and the host's differ in the last bit here and there, and one 16-bit
    rounding flip of a stored q or k element moves an output by up to ~2e-4."""
    import torch
    L, H, HKV, D = sim.L, sim.H, sim.HKV, sim.D
    ids = torch.from_numpy(np.asarray(tokens[:n_cached], np.int64) % sim.vocab).cuda()
    sin = sim.sin[:(n_cached + 1) * D].cpu().numpy()
    cos = sim.cos[:(n_cached + 1) * D].cpu().numpy()
    outs = []
    for l in range(L):
        q = sim.Eq[l, ids].float().cpu().numpy()
        k = sim.Ek[l, ids].float().cpu().numpy()
        v = sim.Ev[l, ids].float().cpu().numpy()
        oracle.rope_batched(0, q, k, D, sin, cos)
        # the kernel stores the rotated rows in the cache dtype
        q = kvtest.storage_to_f32(kvtest.to_storage(q, "f16"), "f16")
        k = kvtest.storage_to_f32(kvtest.to_storage(k, "f16"), "f16")
        outs.append(oracle.mha_prefill(0, q, H, n_cached, HKV * D, H // HKV, D, np.ascontiguousarray(k),
                                       np.ascontiguousarray(v), threads=oracle.max_threads()))
    return np.stack(outs)


@pytest.mark.parametrize("prefix,suffix", [(64, 40), (100, 52)])  # aligned / unaligned (copy-on-write)
def test_shared_prefix_serving_loop_matches_oracle(native_libs, oracle, prefix, suffix):
    from tests.serving_sim import ServingSim
    sim = ServingSim(num_layers=2, q_heads=16, kv_heads=4, num_blocks=400, seed=3, prefill_chunk=48,
                     max_prefill_tokens=160, max_decode_batch=64, record=True, poison=True)
    rng = np.random.default_rng(21)
    common = rng.integers(0, 151936, prefix)
    first = sim.sched.submit(np.concatenate([common, rng.integers(0, 151936, suffix)]), 1, also_register=prefix)
    sim.run()
    followers = [sim.sched.submit(np.concatenate([common, rng.integers(0, 151936, suffix + 3 * i)]), 6 + i)
                 for i in range(7)]
    sim.run()
    assert sim.manager.cow_events == (7 if prefix % 16 else 0)
    worst = 0.0
    for rid in [first] + followers:
        toks = sim.sched.tokens(rid)
        n_cached = len(toks) - 1
        reused = sim.sched.reused_tokens(rid)
        assert reused == (0 if rid == first else prefix)
        ref = oracle_outputs(oracle, sim, toks, n_cached)
        got = sim.outputs[rid]
        assert sorted(got) == list(range(reused, n_cached)), "every computed position was recorded exactly once"
        for pos, rows in got.items():
            a, r = kvtest.assert_attention_close(rows, ref[:, pos, :], f"request {rid} position {pos}")
            worst = max(worst, a)
    # device reference counts mirror the host's
    assert np.array_equal(sim.refc.cpu().numpy(), sim.manager.ref_counts())
    print(f"worst max-abs over all requests: {worst:.2e}")


def test_admission_waves_on_a_small_pool(native_libs, oracle):
    from tests.serving_sim import ServingSim
    sim = ServingSim(num_layers=1, q_heads=8, kv_heads=2, num_blocks=60, seed=5, prefill_chunk=64,
                     max_prefill_tokens=128, max_decode_batch=32, use_prefix_cache=False, record=True, poison=True)
    rng = np.random.default_rng(2)
    rids = [sim.sched.submit(rng.integers(0, 151936, int(rng.integers(30, 200))), int(rng.integers(2, 12)))
            for _ in range(24)]
    sim.run()
    st = sim.sched.stats()
    assert st["finished"] == 24 and st["admission_stalls"] > 0 and st["peak_blocks_in_use"] <= 60
    assert sim.manager.num_free == 60
    for rid in rids[::5]:
        toks = sim.sched.tokens(rid)
        ref = oracle_outputs(oracle, sim, toks, len(toks) - 1)
        for pos, rows in sim.outputs[rid].items():
            kvtest.assert_attention_close(rows, ref[:, pos, :], f"request {rid} position {pos}")


def test_two_turn_conversation_with_gap_fill(native_libs, oracle):
    """Turn 1 ends, the last sampled token and the template's suffix are prefilled (the
    reference's end-of-turn fix-up), the history is registered; turn 2 = history + a new message
    reuses all of it.  The pool starts as NaN, so a reused position that nobody wrote would show."""
    from tests.serving_sim import ServingSim
    sim = ServingSim(num_layers=2, q_heads=16, kv_heads=4, num_blocks=200, seed=11, prefill_chunk=32,
                     max_prefill_tokens=96, max_decode_batch=16, record=True, poison=True)
    rng = np.random.default_rng(8)
    suffix = np.array([198, 271], np.int32)
    t1 = sim.sched.submit_turn(rng.integers(0, 151936, 45), 9, suffix)
    other = sim.sched.submit(rng.integers(0, 151936, 70), 4)   # an unrelated request in the same batches
    sim.run()
    hist = sim.sched.tokens(t1)
    assert len(hist) == 45 + 9 + 2 and sim.sched.stats()["gap_tokens"] == 3
    t2 = sim.sched.submit_turn(np.concatenate([hist, rng.integers(0, 151936, 21)]), 5, suffix)
    sim.run()
    assert sim.sched.reused_tokens(t2) == len(hist) and sim.manager.cow_events == 1
    worst = 0.0
    for rid, reused in ((t1, 0), (t2, len(hist)), (other, 0)):
        toks = sim.sched.tokens(rid)
        n_cached = len(toks) if rid != other else len(toks) - 1
        ref = oracle_outputs(oracle, sim, toks, n_cached)
        got = sim.outputs[rid]
        assert sorted(got) == list(range(reused, n_cached))
        for pos, rows in got.items():
            a, r = kvtest.assert_attention_close(rows, ref[:, pos, :], f"request {rid} position {pos}")
            worst = max(worst, a)
    assert np.array_equal(sim.refc.cpu().numpy(), sim.manager.ref_counts())
    print(f"worst max-abs over the conversation: {worst:.2e}")
