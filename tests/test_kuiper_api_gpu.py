"""Runs the C++ test program of the kuiper-style layer API (tests/cpp/test_kuiper_api.cu):
op::MultiHeadAttention, FlashAttention{Decode,Prefill}Layer, KVCacheLayer, the misc and RoPE
layers, contiguous (reference) and paged modes, each against the CPU oracle."""
import subprocess

import pytest

pytestmark = pytest.mark.gpu


def test_layer_api_program(native_libs):
    from tests import buildtools
    exe = buildtools.build_cpp_tests()
    res = subprocess.run([str(exe)], capture_output=True, text=True, timeout=300)
    print(res.stdout[-3000:])
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-2000:]
    assert "0 failed" in res.stdout
