"""Binding of oracle/_ref/libref_cpu*.so: the reference project's own CPU kernels, compiled
unmodified against the glog / Armadillo stand-ins (oracle/Makefile, target `ref`), and the
seeded cases that pin the plain-C oracle to them.

Test infrastructure only.  The libraries exist where `make -C oracle ref REF=<checkout>` has
run; `load()` returns None elsewhere and the golden files under tests/golden/ (written from
these libraries by tests/golden/make_ref_cpu_golden.py) stand in for them.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent
REF_DIR = ROOT / "oracle" / "_ref"
GOLDEN = ROOT / "tests" / "golden" / "ref_cpu_golden.npz"


class RefCpu:
    def __init__(self, lib: C.CDLL):
        self.lib = lib
        f32p = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")
        i32 = C.c_int32
        sig = {
            "ref_mha": [i32] * 8 + [f32p] * 5,
            "ref_sin_cos_cache": [i32, i32, f32p, f32p],
            "ref_rope": [i32, i32, i32, f32p, f32p, i32, i32, f32p, f32p],
            "ref_rmsnorm": [i32, f32p, f32p, f32p],
            "ref_softmax": [f32p, i32],
            "ref_sequential_reductions": [],
        }
        for name, args in sig.items():
            fn = getattr(lib, name)
            fn.argtypes = args
            fn.restype = i32 if name == "ref_sequential_reductions" else None

    @property
    def sequential(self) -> bool:
        return bool(self.lib.ref_sequential_reductions())

    def sin_cos_cache(self, head_size, max_seq_len):
        s = np.empty((max_seq_len, head_size), np.float32)
        c = np.empty((max_seq_len, head_size), np.float32)
        self.lib.ref_sin_cos_cache(head_size, max_seq_len, s, c)
        return s, c

    def rope(self, pos, q, k, head_size, sin, cos):
        self.lib.ref_rope(q.shape[0], k.shape[0], head_size, q, k, pos, sin.shape[0], sin, cos)

    def mha(self, pos, head_num, layer_index, seq_len, kv_dim, kv_mul, head_size, layer_num, q, kc, vc):
        out = np.empty(head_num * head_size, np.float32)
        score = np.zeros(head_num * seq_len, np.float32)
        self.lib.ref_mha(pos, head_num, layer_index, seq_len, kv_dim, kv_mul, head_size, layer_num, out,
                         np.ascontiguousarray(q, np.float32), score, kc.reshape(-1), vc.reshape(-1))
        return out

    def rmsnorm(self, x, w):
        out = np.empty_like(x)
        self.lib.ref_rmsnorm(x.shape[0], np.ascontiguousarray(x), np.ascontiguousarray(w, np.float32), out)
        return out

    def softmax(self, x):
        y = np.ascontiguousarray(x, np.float32).copy()
        self.lib.ref_softmax(y, y.shape[0])
        return y


def load(sequential: bool):
    so = REF_DIR / ("libref_cpu_seq.so" if sequential else "libref_cpu.so")
    if not so.exists():
        return None
    return RefCpu(C.CDLL(str(so)))


# ---------------------------------------------------------------------------- the cases
# Each case is a function of (impl, seed) where impl offers sin_cos_cache / rope / mha /
# rmsnorm / softmax with the signatures above; `OracleAsImpl` adapts the plain-C oracle.
class OracleAsImpl:
    def __init__(self, oracle):
        self.o = oracle

    def sin_cos_cache(self, head_size, max_seq_len):
        return self.o.sin_cos_cache(head_size, max_seq_len, 1e6)

    def rope(self, pos, q, k, head_size, sin, cos):
        self.o.rope(pos, q, k, head_size, sin, cos)

    def mha(self, pos, head_num, layer_index, seq_len, kv_dim, kv_mul, head_size, layer_num, q, kc, vc):
        return self.o.mha(pos, head_num, layer_index, seq_len, kv_dim, kv_mul, head_size, q,
                          kc.reshape(-1), vc.reshape(-1))

    def rmsnorm(self, x, w):
        y = np.ascontiguousarray(x, np.float32).copy().reshape(1, -1)
        self.o.rmsnorm_heads(y, 1, y.shape[1], w, 1e-6)
        return y.reshape(-1)

    def softmax(self, x):
        y = np.ascontiguousarray(x, np.float32).copy()
        self.o.lib.orc_softmax_inplace(y, y.shape[0])
        return y


def case_config1(impl, seed=1):
    """Single-layer KV append + decode MHA at the Qwen2.5-1.5B attention shape: 12 Q heads,
    2 KV heads, head 128, 512 cached tokens + 1 new, fp32 N(0,1), RoPE theta 1e6 on the new
    q / k, contiguous cache.  Returns the rotated q, k and the [12*128] output."""
    H, HKV, D, S = 12, 2, 128, 520
    rng = np.random.default_rng(seed)
    kc = np.zeros((1, S, HKV * D), np.float32)
    vc = np.zeros((1, S, HKV * D), np.float32)
    kc[0, :512] = rng.standard_normal((512, HKV * D), np.float32)
    vc[0, :512] = rng.standard_normal((512, HKV * D), np.float32)
    q = rng.standard_normal(H * D, np.float32)
    k = rng.standard_normal(HKV * D, np.float32)
    v = rng.standard_normal(HKV * D, np.float32)
    sin, cos = impl.sin_cos_cache(D, S)
    impl.rope(512, q, k, D, sin, cos)
    kc[0, 512], vc[0, 512] = k, v
    out = impl.mha(512, H, 0, S, HKV * D, H // HKV, D, 1, q, kc, vc)
    return {"q_rot": q, "k_rot": k, "out": out}


def case_gqa_layer1(impl, seed=2):
    """Qwen3-8B head shape (32 / 8), second of two layers of a [2, 300, 1024] cache, 201 keys."""
    H, HKV, D, S, L = 32, 8, 128, 300, 2
    rng = np.random.default_rng(seed)
    kc = rng.standard_normal((L, S, HKV * D), np.float32)
    vc = rng.standard_normal((L, S, HKV * D), np.float32)
    q = rng.standard_normal(H * D, np.float32)
    return {"out": impl.mha(200, H, 1, S, HKV * D, H // HKV, D, L, q, kc, vc)}


def case_rope_chunk(impl, seed=3):
    """A 40-token chunk at positions 100..139, 4 Q heads / 2 KV heads, rotated row by row."""
    H, HKV, D, n, start = 4, 2, 128, 40, 100
    rng = np.random.default_rng(seed)
    q = rng.standard_normal((n, H * D), np.float32)
    k = rng.standard_normal((n, HKV * D), np.float32)
    sin, cos = impl.sin_cos_cache(D, start + n)
    for t in range(n):
        impl.rope(start + t, q[t], k[t], D, sin, cos)
    return {"q_rot": q, "k_rot": k, "sin_tail": sin[start:start + 8].copy(), "cos_tail": cos[start:start + 8].copy()}


def case_rmsnorm_softmax(impl, seed=4):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((6, 128), np.float32) * 3
    w = rng.standard_normal(128, np.float32)
    normed = np.stack([impl.rmsnorm(x[i], w) for i in range(6)])
    s = impl.softmax(rng.standard_normal(513, np.float32) * 4)
    return {"rmsnorm": normed, "softmax": s}


CASES = {"config1": case_config1, "gqa_layer1": case_gqa_layer1, "rope_chunk": case_rope_chunk,
         "rmsnorm_softmax": case_rmsnorm_softmax}
# outputs that involve no reduction: equal bit for bit whatever the summation order
EXACT_KEYS = {"q_rot", "k_rot", "sin_tail", "cos_tail"}


def run_all(impl) -> dict:
    out = {}
    for name, fn in CASES.items():
        for key, val in fn(impl).items():
            out[f"{name}.{key}"] = val
    return out
