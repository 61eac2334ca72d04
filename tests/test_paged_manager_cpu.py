"""The C++ KV-cache manager against the Python specification: block tables, slot mappings,
refcounts, free-list order and copy-on-write decisions, bit for bit, on seeded random call
sequences.  CPU only (the manager is host code)."""
import numpy as np
import pytest

from tests.paged_spec import SpecPool


@pytest.fixture(scope="module")
def kvm_mod(native_libs):
    from orinmllm_b200 import build, kvm
    build.build_host()
    return kvm


def _compare(mgr, spec, live):
    assert mgr.num_free == len(spec.free)
    assert mgr.ref_counts().tolist() == spec.ref
    assert mgr.cow_events == spec.cow_events
    for s in live:
        assert mgr.length(s) == spec.seqs[s][1]
        width = max(len(spec.seqs[s][0]), 1)
        assert mgr.block_table_row(s, width).tolist() == spec.table_row(s, width)


@pytest.mark.parametrize("seed", [1, 2, 3])
def test_random_sessions_match_spec(kvm_mod, seed):
    rng = np.random.default_rng(seed)
    nb = 96
    mgr = kvm_mod.KvManager(nb, 16, seed=seed, shuffle=True, min_prefix_length=4)
    spec = SpecPool(nb, 16, seed=seed, shuffle=True, min_prefix_length=4)
    live, tokens_of = [], {}
    library = []  # token sequences inserted so far
    for step in range(600):
        r = rng.random()
        if r < 0.25 or not live:
            s, s2 = mgr.add_sequence(), spec.add_sequence()
            assert s == s2
            if library and rng.random() < 0.7:
                base = library[rng.integers(len(library))]
                toks = base[:rng.integers(1, len(base) + 1)] + rng.integers(0, 50, rng.integers(0, 30)).tolist()
            else:
                toks = rng.integers(0, 50, rng.integers(1, 60)).tolist()
            m1 = mgr.match_prefix(s, toks)
            m2 = spec.match_prefix(s, toks)
            assert m1 == m2
            rest = len(toks) - m1
            rc, slots = mgr.try_append(s, rest)
            want = spec.append(s, rest)
            if want is None:
                assert rc == 8  # out of blocks, nothing changed
                mgr.free_sequence(s)
                spec.free_sequence(s)
            else:
                assert rc == 0 and slots.tolist() == want
                live.append(s)
                tokens_of[s] = toks
        elif r < 0.65:
            s = live[rng.integers(len(live))]
            n = int(rng.integers(1, 4))
            rc, slots = mgr.try_append(s, n)
            want = spec.append(s, n)
            if want is None:
                assert rc == 8
            else:
                assert rc == 0 and slots.tolist() == want
                tokens_of[s] = tokens_of[s] + rng.integers(0, 50, n).tolist()
        elif r < 0.85:
            s = live[rng.integers(len(live))]
            mgr.insert_prefix(s, tokens_of[s])
            spec.insert_prefix(s, tokens_of[s])
            library.append(list(tokens_of[s]))
        else:
            s = live.pop(rng.integers(len(live)))
            mgr.free_sequence(s)
            spec.free_sequence(s)
        _compare(mgr, spec, live)
    assert spec.cow_events > 0, "the scenario must exercise copy-on-write"
    # logs: replaying the deltas from zero reproduces the counts; copies are the COW pairs
    blocks, deltas, src, dst = mgr.take_pending()
    acc = np.zeros(nb, np.int64)
    np.add.at(acc, blocks, deltas)
    assert acc.tolist() == spec.ref
    assert list(zip(src.tolist(), dst.tolist())) == spec.copies
    mgr.close()


def test_free_list_is_the_seeded_permutation(kvm_mod):
    mgr = kvm_mod.KvManager(40, 16, seed=99)
    spec = SpecPool(40, 16, seed=99)
    s = mgr.add_sequence()
    spec.add_sequence()
    slots = mgr.append(s, 40 * 16)
    assert slots.tolist() == spec.append(0, 40 * 16)
    assert sorted(mgr.block_table_row(s, 40).tolist()) == list(range(40))
    assert mgr.block_table_row(s, 40).tolist() != list(range(40))
    rc, _ = mgr.try_append(s, 1)
    assert rc == 8 and mgr.length(s) == 640  # exhausted: error, no state change
    ident = kvm_mod.KvManager(8, 16, seed=1, shuffle=False)
    t = ident.add_sequence()
    ident.append(t, 8 * 16)
    assert ident.block_table_row(t, 8).tolist() == list(range(8))


def test_config4_block_accounting(kvm_mod):
    """The prefix-reuse workload at full size on the host: 256 requests share a 1024-id prefix and add
    256 unique ids, then 128 decode tokens each.  Aligned sizes: 64 shared blocks, no COW.
    Unaligned variant (prefix 1000 + suffix 280): the 63rd block is shared partially and every
    request copies it on its first append."""
    rng = np.random.default_rng(4)
    for plen, slen, expect_cow in ((1024, 256, 0), (1000, 280, 255)):
        prefix = rng.integers(0, 151936, plen).tolist()
        mgr = kvm_mod.KvManager(8192, 16, seed=7)
        spec = SpecPool(8192, 16, seed=7)
        seqs = []
        for i in range(256):
            toks = prefix + rng.integers(0, 151936, slen).tolist()
            s = mgr.add_sequence()
            spec.add_sequence()
            m = mgr.match_prefix(s, toks)
            assert m == (0 if i == 0 else plen) == spec.match_prefix(s, toks)
            assert mgr.append(s, len(toks) - m).tolist() == spec.append(s, len(toks) - m)
            if i == 0:
                mgr.insert_prefix(s, prefix)
                spec.insert_prefix(s, prefix)
            mgr.insert_prefix(s, toks)
            spec.insert_prefix(s, toks)
            for _ in range(128):
                assert mgr.append(s, 1).tolist() == spec.append(s, 1)
            if m:
                mgr.release_prefix(prefix)
            seqs.append(s)
        assert mgr.cow_events == expect_cow == spec.cow_events
        assert mgr.ref_counts().tolist() == spec.ref
        assert mgr.num_free == len(spec.free)
        shared_full = plen // 16
        rc = mgr.ref_counts()
        table0 = mgr.block_table_row(seqs[0], 128)
        # full prefix blocks: 256 sequences + the prefix span + 256 full-sequence spans
        assert all(rc[b] == 256 + 1 + 256 for b in table0[:shared_full])
        st = mgr.prefix_stats()
        assert st["cache_hits"] == 255 and st["cache_misses"] == 1 and st["tokens_reused"] == 255 * plen
        if not expect_cow:
            # 64 shared blocks + 24 private blocks per request (256 suffix + 128 decoded tokens)
            assert 8192 - mgr.num_free == 64 + 256 * 24
        mgr.close()
