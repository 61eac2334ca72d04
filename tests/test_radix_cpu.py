"""Radix tree / prefix cache: this repository's headers against the reference, bit for bit.

Golden fixtures under tests/golden/ were produced by the trace driver compiled against the
REFERENCE headers (tests/golden/make_radix_golden.py).  Here the same driver is compiled
against include/kuiper/base/*.h and must print identical text.  Where the reference checkout
is present (the build container), the reference's own two test programs are additionally
compiled against this repository's headers and must pass.
"""
import os
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
GOLDEN = ROOT / "tests" / "golden"
from tests import buildtools  # noqa: E402

REF = buildtools.reference_checkout() or Path("/nonexistent")
NAMES = ["tree_a", "tree_b", "cache_a", "cache_b", "config4"]


@pytest.fixture(scope="module")
def trace_bin(tmp_path_factory):
    out = tmp_path_factory.mktemp("radix") / "radix_trace"
    subprocess.run(["g++", "-std=c++17", "-O2", "-pthread", "-I", str(ROOT / "include" / "kuiper"),
                    "-o", str(out), str(ROOT / "oracle" / "radix_trace.cpp")], check=True)
    return out


@pytest.mark.parametrize("name", NAMES)
def test_trace_matches_reference_golden(trace_bin, name):
    got = subprocess.run([str(trace_bin), str(GOLDEN / f"radix_script_{name}.txt")], check=True,
                         capture_output=True, text=True).stdout
    want = (GOLDEN / f"radix_expected_{name}.txt").read_text()
    assert got.count("\n") == want.count("\n")
    for g, w in zip(got.splitlines(), want.splitlines()):
        assert g == w
    assert got == want


def test_golden_fixtures_exercise_the_interesting_cases():
    text = "".join((GOLDEN / f"radix_expected_{n}.txt").read_text() for n in NAMES)
    assert "hit=1" in text and "hit=0" in text
    assert "kv_pos=-1" in text                      # partial-edge / no-terminal lookups
    assert any(f"evicted={d}" in text for d in "123456789")
    assert "edge_offset=1" in text or "edge_offset=2" in text
    # config 4: first request misses (nothing cached), the other 23 hit exactly the 1024-id prefix
    c4 = (GOLDEN / "radix_expected_config4.txt").read_text()
    assert c4.count("hit=1 matched=1024") == 23 and c4.count("hit=0") == 1


@pytest.mark.skipif(not (REF / "tools" / "test_radix_tree.cpp").exists(),
                    reason="reference checkout not present on this machine")
@pytest.mark.parametrize("prog", ["test_radix_tree", "test_prefix_cache_full"])
def test_reference_own_tests_pass_on_these_headers(tmp_path, prog):
    """The reference test programs include its headers by relative path; pre-including this
    repository's headers (same include guards) makes them compile against these instead."""
    exe = tmp_path / prog
    inc = ROOT / "include" / "kuiper" / "base"
    subprocess.run(["g++", "-std=c++17", "-O2", "-pthread", "-include", str(inc / "radix_tree.h"),
                    "-include", str(inc / "prefix_cache.h"), "-o", str(exe),
                    str(REF / "tools" / f"{prog}.cpp")], check=True)
    res = subprocess.run([str(exe)], capture_output=True, text=True, timeout=120)
    assert res.returncode == 0, res.stdout[-2000:]
    assert "PASSED" in res.stdout or "7/7 tests passed" in res.stdout


@pytest.mark.skipif(not (ROOT / "oracle" / "_ref" / "radix_trace_ref").exists(),
                    reason="reference-compiled trace driver not built here")
def test_golden_files_are_what_the_reference_prints_today():
    for name in NAMES:
        out = subprocess.run([str(ROOT / "oracle" / "_ref" / "radix_trace_ref"),
                              str(GOLDEN / f"radix_script_{name}.txt")], check=True,
                             capture_output=True, text=True).stdout
        assert out == (GOLDEN / f"radix_expected_{name}.txt").read_text()
