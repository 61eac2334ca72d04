"""Pins the plain-C oracle (oracle/kv_oracle.c) to the reference project's own CPU kernels.

Two sources of truth, both produced by the reference's unmodified cpu/*.cpp files compiled
against the glog / Armadillo stand-ins (oracle/Makefile, target `ref`):
  * tests/golden/ref_cpu_golden.npz, committed (written by tests/golden/make_ref_cpu_golden.py);
  * oracle/_ref/libref_cpu*.so themselves, where they have been built (they travel with the
    working tree but are not in the history).
With every reduction in index order (`seq`) the oracle must equal the reference bit for bit;
with Armadillo's own two-running-sums loops (`arma`) it must agree within 1e-6 absolute, the
room Armadillo's unspecified summation order leaves.
"""
import numpy as np
import pytest

from tests import refcpu

TOL_ARMA = 1e-6


@pytest.fixture(scope="module")
def golden():
    assert refcpu.GOLDEN.exists(), "tests/golden/ref_cpu_golden.npz is missing"
    return dict(np.load(refcpu.GOLDEN))


@pytest.fixture(scope="module")
def oracle_outputs(oracle):
    return refcpu.run_all(refcpu.OracleAsImpl(oracle))


def _compare(name, got, want, exact):
    assert got.shape == want.shape, name
    if exact:
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), \
            f"{name}: {int((got.view(np.uint32) != want.view(np.uint32)).sum())} elements differ in bits"
    else:
        err = float(np.abs(got.astype(np.float64) - want.astype(np.float64)).max())
        assert err <= TOL_ARMA, f"{name}: max abs diff {err:.3e} > {TOL_ARMA}"


def test_oracle_equals_reference_golden_bit_for_bit_in_index_order(golden, oracle_outputs):
    keys = [k for k in golden if k.startswith("seq/")]
    assert len(keys) == len(oracle_outputs)
    for k in keys:
        _compare(k, oracle_outputs[k[4:]], golden[k], exact=True)


def test_oracle_within_1e6_of_reference_golden_with_armadillo_order(golden, oracle_outputs):
    for k in [k for k in golden if k.startswith("arma/")]:
        short = k[5:]
        _compare(k, oracle_outputs[short], golden[k], exact=short.split(".")[1] in refcpu.EXACT_KEYS)


@pytest.mark.parametrize("sequential", [True, False], ids=["seq", "arma"])
def test_reference_library_reproduces_its_golden_and_the_oracle(sequential, golden, oracle_outputs):
    """Where the reference-compiled library is present: it must reproduce the committed golden
    (so the file is not stale) and the oracle must match it live, on a second seed too."""
    impl = refcpu.load(sequential)
    if impl is None:
        pytest.skip("oracle/_ref/libref_cpu*.so not built here (needs the reference checkout)")
    assert impl.sequential == sequential
    prefix = "seq/" if sequential else "arma/"
    for key, val in refcpu.run_all(impl).items():
        _compare(prefix + key, val, golden[prefix + key], exact=True)
    # fresh seeds, not in the golden file
    from tests import kvtest
    orc = refcpu.OracleAsImpl(kvtest.load_oracle())
    for name, fn in refcpu.CASES.items():
        a, b = fn(impl, seed=101), fn(orc, seed=101)
        for key in a:
            _compare(f"{name}.{key}@101", b[key], a[key], exact=sequential or key in refcpu.EXACT_KEYS)


def test_sin_cos_table_equals_reference(golden, oracle):
    """sin_cos_cache_calc_cpu (Qwen branch, theta 1e6) against orc_sin_cos_cache: same libm
    calls in the same order, so the tables agree in every bit."""
    sin, cos = oracle.sin_cos_cache(128, 140, 1e6)
    assert np.array_equal(sin[100:108].view(np.uint32), golden["seq/rope_chunk.sin_tail"].view(np.uint32))
    assert np.array_equal(cos[100:108].view(np.uint32), golden["arma/rope_chunk.cos_tail"].view(np.uint32))
