"""Host-side request scheduler (base::KVScheduler through include/kpx_sched.h): admission by free
blocks, prefix reuse with copy-on-write, and the work lists handed to the kernels.  No GPU."""
import numpy as np
import pytest

from orinmllm_b200 import kvm, sched

BS = 16


def drive(s, sample=lambda rid, step: 7, prefill_hook=None, decode_hook=None, max_steps=100000):
    """Run the scheduler dry (no device): admit, prefill steps, decode steps, until idle."""
    steps = 0
    while s.num_waiting or s.num_running:
        s.admit()
        progressed = False
        while True:
            p = s.next_prefill()
            if p is None:
                break
            progressed = True
            if prefill_hook:
                prefill_hook(p)
            s.complete_prefill([sample(int(r), steps) for r in p.request_ids])
        d = s.next_decode()
        if d is not None:
            progressed = True
            if decode_hook:
                decode_hook(d)
            s.complete_decode([sample(int(r), steps) for r in d.request_ids])
        steps += 1
        assert progressed, "scheduler made no progress with requests outstanding"
        assert steps < max_steps
    return steps


def check_slots(step_positions, slot_mapping, table_row):
    for pos, slot in zip(step_positions, slot_mapping):
        assert slot == int(table_row[pos // BS]) * BS + pos % BS


def test_work_lists_are_consistent_and_chunked():
    m = kvm.KvManager(512, BS, seed=3)
    s = sched.Scheduler(m, prefill_chunk=48, max_prefill_tokens=100, max_prefill_rows=8, use_prefix_cache=False)
    rng = np.random.default_rng(0)
    prompts = {s.submit(rng.integers(0, 1000, n), 5): n for n in (130, 20, 75)}
    seen = {rid: 0 for rid in prompts}

    def on_prefill(p):
        assert p.positions.size <= 100 and len(p.request_ids) <= 8
        assert p.cu_q_lens[0] == 0 and p.cu_q_lens[-1] == p.positions.size
        for i, rid in enumerate(p.request_ids):
            a, b = p.cu_q_lens[i], p.cu_q_lens[i + 1]
            assert 0 < b - a <= 48
            assert p.start_pos[i] == seen[int(rid)]
            assert list(p.positions[a:b]) == list(range(seen[int(rid)], seen[int(rid)] + b - a))
            check_slots(p.positions[a:b], p.slot_mapping[a:b], p.block_table[i])
            seen[int(rid)] += b - a
            assert p.completes[i] == (seen[int(rid)] == prompts[int(rid)])

    def on_decode(d):
        for i, rid in enumerate(d.request_ids):
            assert d.positions[i] == seen[int(rid)]
            assert d.seq_lens[i] == seen[int(rid)] + 1
            check_slots(d.positions[i:i + 1], d.slot_mapping[i:i + 1], d.block_table[i])
            seen[int(rid)] += 1

    drive(s, prefill_hook=on_prefill, decode_hook=on_decode)
    st = s.stats()
    assert st["finished"] == 3 and st["prefilled_tokens"] == 225 and st["decoded_tokens"] == 3 * 4
    for rid, n in prompts.items():
        assert s.state(rid) == 3 and len(s.tokens(rid)) == n + 5
    assert m.num_free == 512  # no prefix cache: everything came back


@pytest.mark.parametrize("prefix,suffix", [(64, 24), (60, 28)])
def test_prefix_reuse_and_copy_on_write(prefix, suffix):
    m = kvm.KvManager(2048, BS, seed=1)
    s = sched.Scheduler(m, prefill_chunk=32)
    rng = np.random.default_rng(5)
    common = rng.integers(0, 151936, prefix)
    first = s.submit(np.concatenate([common, rng.integers(0, 151936, suffix)]), 1, also_register=prefix)
    drive(s)
    assert s.reused_tokens(first) == 0
    others = [s.submit(np.concatenate([common, rng.integers(0, 151936, suffix)]), 9) for _ in range(12)]
    drive(s)
    for rid in others:
        assert s.reused_tokens(rid) == prefix
        assert s.state(rid) == 3
    st = s.stats()
    assert st["reused_tokens"] == 12 * prefix
    assert st["prefilled_tokens"] == (prefix + suffix) + 12 * suffix
    # an unaligned prefix ends in a shared, partly filled block: every follower copies it once
    assert m.cow_events == (12 if prefix % BS else 0)
    ps = m.prefix_stats()
    assert ps["cache_hits"] == 12


def test_full_hit_recomputes_the_last_prompt_token():
    m = kvm.KvManager(256, BS, seed=2)
    s = sched.Scheduler(m)
    prompt = np.arange(100, 150, dtype=np.int32)
    a = s.submit(prompt, 1)
    drive(s)
    b = s.submit(prompt, 3)
    drive(s)
    assert s.reused_tokens(a) == 0 and s.reused_tokens(b) == len(prompt) - 1
    assert s.stats()["prefilled_tokens"] == len(prompt) + 1


def test_admission_waves_never_exhaust_the_pool():
    nblocks = 200
    m = kvm.KvManager(nblocks, BS, seed=9)
    s = sched.Scheduler(m, prefill_chunk=64, max_prefill_tokens=256, use_prefix_cache=False)
    rng = np.random.default_rng(11)
    want = {}
    for _ in range(60):
        n, g = int(rng.integers(20, 400)), int(rng.integers(1, 40))
        want[s.submit(rng.integers(0, 1000, n), g)] = n + g
    peak_running = 0

    def watch(_):
        nonlocal peak_running
        peak_running = max(peak_running, s.num_running)
        assert m.num_free >= 0

    drive(s, prefill_hook=watch, decode_hook=watch)
    st = s.stats()
    assert st["finished"] == 60 and st["admission_stalls"] > 0
    assert 0 < st["peak_blocks_in_use"] <= nblocks
    assert peak_running < 60  # it really ran in waves
    for rid, total in want.items():
        assert len(s.tokens(rid)) == total
    assert m.num_free == nblocks


def test_shared_prompt_workload_block_count():
    """256 requests = common 1024-id prefix + unique 256-id suffix, 128 decode steps each: the pool
    holds 64 shared blocks plus 24 private blocks per request."""
    n_req, prefix, suffix, gen = 256, 1024, 256, 129  # 129 sampled tokens = 128 cached decode positions
    m = kvm.KvManager(8192, BS, seed=4)
    s = sched.Scheduler(m, prefill_chunk=512, max_prefill_tokens=4096, max_decode_batch=256)
    rng = np.random.default_rng(1)
    common = rng.integers(0, 151936, prefix)
    first = s.submit(np.concatenate([common, rng.integers(0, 151936, suffix)]), 1, also_register=prefix)
    drive(s)
    s.forget(first)
    for _ in range(n_req - 1):
        s.submit(np.concatenate([common, rng.integers(0, 151936, suffix)]), gen)
    drive(s)
    st = s.stats()
    assert st["finished"] == n_req and st["reused_tokens"] == (n_req - 1) * prefix
    per_request = (suffix + gen - 1 + BS - 1) // BS  # 24
    # request 0 keeps its 16 suffix blocks in the tree; the 255 followers ran together
    assert st["peak_blocks_in_use"] == prefix // BS + suffix // BS + (n_req - 1) * per_request
    assert m.cow_events == 0


def test_turn_end_gap_fill_registers_the_whole_history():
    """The end-of-turn fix-up of the reference (demo/inference_common.h:1334-1358): the last
    sampled token and the template's separators are prefilled without sampling, the whole
    history is registered, and the next turn's prompt reuses all of it."""
    m = kvm.KvManager(256, BS, seed=4)
    s = sched.Scheduler(m, prefill_chunk=8)
    prompt = np.arange(1000, 1037, dtype=np.int32)
    suffix = np.array([198, 199], np.int32)
    gap_rows = []

    def prefill_hook(p):
        for i, rid in enumerate(p.request_ids):
            if s.state(int(rid)) == 4:
                a, b = p.cu_q_lens[i], p.cu_q_lens[i + 1]
                gap_rows.append((list(p.positions[a:b]), list(p.token_ids[a:b]), int(p.completes[i])))
                check_slots(p.positions[a:b], p.slot_mapping[a:b], p.block_table[i])

    t1 = s.submit_turn(prompt, 5, suffix)
    drive(s, sample=lambda rid, step: 500 + step, prefill_hook=prefill_hook)
    hist = s.tokens(t1)
    assert len(hist) == len(prompt) + 5 + len(suffix) and list(hist[-2:]) == [198, 199]
    # the gap: the last sampled token, then the suffix, at the positions after the cached ones; never sampled from
    n_cached = len(prompt) + 4
    assert [x for r in gap_rows for x in r[0]] == list(range(n_cached, n_cached + 3))
    assert [x for r in gap_rows for x in r[1]] == list(hist[n_cached:])
    assert all(r[2] == 0 for r in gap_rows)
    st = s.stats()
    assert st["gap_tokens"] == 3 and st["prefilled_tokens"] == len(prompt) + 3 and st["finished"] == 1
    assert m.num_free == 256 - (len(hist) + BS - 1) // BS  # only the registered span holds blocks
    # next turn: history + a new message; everything cached is reused (whole blocks by reference,
    # the partial last block copied on first write)
    t2 = s.submit_turn(np.concatenate([hist, np.arange(2000, 2010, dtype=np.int32)]), 3, suffix)
    drive(s, sample=lambda rid, step: 700 + step)
    assert s.reused_tokens(t2) == len(hist)
    assert m.cow_events == (1 if len(hist) % BS else 0)
    # without the gap fill the registered span stops before the last sampled token
    m2 = kvm.KvManager(256, BS, seed=4)
    s2 = sched.Scheduler(m2, prefill_chunk=8)
    u1 = s2.submit(prompt, 5)
    drive(s2, sample=lambda rid, step: 500 + step)
    h2 = s2.tokens(u1)
    u2 = s2.submit(np.concatenate([h2, suffix, np.arange(2000, 2010, dtype=np.int32)]), 3)
    drive(s2)
    assert s2.reused_tokens(u2) == len(h2) - 1


def test_gap_fill_blocks_are_reserved_at_admission():
    """A turn whose gap crosses into new blocks cannot run the pool dry: the blocks of the last
    sampled token and the suffix are part of the reservation."""
    m = kvm.KvManager(8, BS, seed=1)
    s = sched.Scheduler(m, use_prefix_cache=False)
    suffix = np.arange(40, dtype=np.int32)                  # 3 more blocks at the end
    a = s.submit_turn(np.arange(30, dtype=np.int32), 3, suffix)   # 30 + 3 + 40 = 73 tokens = 5 blocks
    b = s.submit_turn(np.arange(30, dtype=np.int32), 3, suffix)   # does not fit beside a
    s.admit()
    assert s.state(a) == 1 and s.state(b) == 0
    drive(s)
    st = s.stats()
    assert st["finished"] == 2 and st["admission_stalls"] > 0 and st["peak_blocks_in_use"] <= 8
    assert st["gap_tokens"] == 2 * 41 and m.num_free == 8


def test_end_tokens_finish_a_request_early():
    """kpx_sched_set_end_tokens: a sampled end token stops the request before max_new_tokens (the
    reference's is_sentence_ending check, demo/inference_common.h:1204); with a turn suffix the
    end token and the suffix are then prefilled and registered."""
    m = kvm.KvManager(128, BS, seed=3)
    s = sched.Scheduler(m)
    s.set_end_tokens([151645, 151643])
    prompt = np.arange(50, 90, dtype=np.int32)
    # sampled: 11, 12, 151645 (end) ...
    seq = iter([11, 12, 151645, 13, 14, 15, 16, 17])
    a = s.submit_turn(prompt, 8, [198])
    drive(s, sample=lambda rid, step: next(seq))
    toks = s.tokens(a)
    assert list(toks[len(prompt):]) == [11, 12, 151645, 198]
    st = s.stats()
    assert st["decoded_tokens"] == 2 and st["gap_tokens"] == 2 and st["finished"] == 1
    b = s.submit(np.concatenate([toks, [7, 8, 9]]).astype(np.int32), 2)
    drive(s, sample=lambda rid, step: 5)
    assert s.reused_tokens(b) == len(toks)
    s.set_end_tokens([])
    c = s.submit(prompt + 1000, 3)
    drive(s, sample=lambda rid, step: 151645)   # no longer an end token
    assert len(s.tokens(c)) == len(prompt) + 3


def test_admission_reclaims_cached_blocks_when_the_pool_is_short():
    """An idle pool whose free blocks plus the blocks held by unreferenced cached spans cover a
    request must admit it: 8 blocks, a finished 40-token request keeps 3 in the tree, the next
    request needs all 8."""
    m = kvm.KvManager(8, BS, seed=1)
    s = sched.Scheduler(m)
    a = s.submit(np.arange(40, dtype=np.int32), 1)
    drive(s)
    assert s.state(a) == 3 and m.num_free == 5 and m.cached_tokens == 40
    b = s.submit(np.arange(1000, 1100, dtype=np.int32), 8 * BS - 100 + 1)  # last cached token is number 128
    assert s.admit() == 1, "the request fits once the cached span is dropped"
    drive(s)
    assert s.state(b) == 3
    assert m.prefix_stats()["eviction_count"] >= 1


def test_small_shortfall_drops_only_the_oldest_span():
    import time
    m = kvm.KvManager(16, BS, seed=2)
    s = sched.Scheduler(m)
    prompts = [np.arange(100 * i, 100 * i + 48, dtype=np.int32) for i in range(1, 5)]  # 3 blocks each
    for p in prompts:
        s.submit(p, 1)
        drive(s)
        time.sleep(0.003)  # distinct last-access times (milliseconds)
    assert m.num_free == 4
    # needs 6 blocks: 2 short, so exactly one 3-block span (the oldest) has to go
    c = s.submit(np.arange(5000, 5090, dtype=np.int32), 7)
    assert s.admit() == 1
    assert m.cached_tokens == 3 * 48
    # the three younger prompts still hit, the oldest does not (looked up through the pool
    # manager, which maps blocks by reference and allocates nothing)
    hits = []
    for p in prompts:
        seq = m.add_sequence()
        n = m.match_prefix(seq, np.concatenate([p, [7, 8, 9]]).astype(np.int32))
        if n:
            m.release_prefix(p[:n])
        m.free_sequence(seq)
        hits.append(n)
    assert hits == [0, 48, 48, 48]
    drive(s)
    assert s.state(c) == 3


def test_request_larger_than_the_pool_is_refused_at_submit():
    m = kvm.KvManager(8, BS, seed=3)
    s = sched.Scheduler(m)
    with pytest.raises(ValueError):
        s.submit(np.arange(100, dtype=np.int32), 8 * BS - 100 + 2)   # last cached token would be number 129
    with pytest.raises(ValueError):
        s.submit_turn(np.arange(100, dtype=np.int32), 20, turn_suffix=[1] * 9)   # 100 + 20 + 9 > 128
    ok = s.submit(np.arange(100, dtype=np.int32), 8 * BS - 100 + 1)
    drive(s)
    assert s.state(ok) == 3


def test_multi_turn_histories_are_reclaimable_without_clear():
    """Every turn registers a longer history on top of the previous one, so the earlier spans
    become inner nodes of the tree.  They must still give their blocks back under pressure."""
    nblocks = 24
    m = kvm.KvManager(nblocks, BS, seed=5)
    s = sched.Scheduler(m, prefill_chunk=16)
    hist = np.arange(300, 330, dtype=np.int32)
    for turn in range(4):
        rid = s.submit_turn(hist, 6, turn_suffix=[198, 199], also_register=len(hist) if turn == 0 else 0)
        drive(s, sample=lambda r, step: 900 + step)
        hist = np.concatenate([s.tokens(rid), np.arange(4000 + 10 * turn, 4010 + 10 * turn, dtype=np.int32)])
    held = nblocks - m.num_free
    assert held > 0 and m.prefix_stats()["cache_hits"] == 3
    # a request that needs the whole pool: only possible if every span can be dropped
    big = s.submit(np.arange(9000, 9000 + 200, dtype=np.int32), nblocks * BS - 200 + 1)
    assert s.admit() == 1
    assert m.cached_tokens == 0
    drive(s)
    assert s.state(big) == 3


@pytest.mark.parametrize("seed", [1, 2, 3, 4, 5])
def test_random_serving_mix_always_progresses_and_conserves_blocks(seed):
    """A soak of the host logic: random prompts (many sharing prefixes of random lengths, so
    spans nest, split and get evicted), random generation lengths, some multi-turn requests,
    on a pool small enough that admission has to reclaim cached spans all the time.  The loop must
    never stall, blocks are conserved at every step, and once everything has finished the cache
    can give every block back."""
    rng = np.random.default_rng(seed)
    nblocks = 96
    m = kvm.KvManager(nblocks, BS, seed=seed)
    s = sched.Scheduler(m, prefill_chunk=40, max_prefill_tokens=160, max_prefill_rows=6, max_decode_batch=12)
    stems = [rng.integers(0, 151936, int(rng.integers(10, 200))) for _ in range(6)]
    submitted, refused = [], 0
    pending = 140

    def submit_some(k):
        nonlocal pending, refused
        for _ in range(k):
            if pending == 0:
                return
            pending -= 1
            stem = stems[int(rng.integers(0, len(stems)))]
            cut = int(rng.integers(1, len(stem) + 1))
            prompt = np.concatenate([stem[:cut], rng.integers(0, 151936, int(rng.integers(1, 120)))]).astype(np.int32)
            gen = int(rng.integers(1, 60))
            try:
                if rng.random() < 0.3:
                    rid = s.submit_turn(prompt, gen, turn_suffix=list(rng.integers(0, 1000, int(rng.integers(0, 4)))),
                                        also_register=cut if rng.random() < 0.5 else 0)
                else:
                    rid = s.submit(prompt, gen, also_register=cut if rng.random() < 0.5 else 0)
                submitted.append(rid)
            except ValueError:
                refused += 1  # larger than the whole pool

    def check_conservation(_=None):
        counts = m.ref_counts()
        assert m.num_free == int((counts == 0).sum()), "free list and reference counts disagree"
        assert counts.min() >= 0

    submit_some(20)
    steps = 0
    while s.num_waiting or s.num_running or pending:
        submit_some(int(rng.integers(0, 4)))
        s.admit()
        progressed = False
        while True:
            p = s.next_prefill()
            if p is None:
                break
            progressed = True
            check_conservation()
            s.complete_prefill([int(rng.integers(0, 151936)) for _ in p.request_ids])
        d = s.next_decode()
        if d is not None:
            progressed = True
            check_conservation()
            s.complete_decode([int(rng.integers(0, 151936)) for _ in d.request_ids])
        steps += 1
        assert progressed or not (s.num_waiting or s.num_running), "requests outstanding and nothing runnable"
        assert steps < 20000
    st = s.stats()
    assert st["finished"] == len(submitted) and st["finished"] + refused == 140
    assert st["reused_tokens"] > 0 and st["admission_stalls"] > 0
    check_conservation()
    # everything has finished: a request as large as the pool must be admissible (every span reclaimable)
    big = s.submit(np.arange(700000, 700000 + 100, dtype=np.int32), nblocks * BS - 100 + 1)
    assert s.admit() == 1
    drive(s)
    assert s.state(big) == 3
