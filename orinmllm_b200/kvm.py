"""ctypes binding of include/kpx_kvm.h (lib/libkuiper_b200.so): the host-side KV-cache
manager -- block pool, block tables, slot mappings, prefix sharing, copy-on-write."""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import capi

_P, _I32, _I64, _U64 = C.c_void_p, C.c_int32, C.c_int64, C.c_uint64
_LP = C.POINTER(capi.KvLayout)

SIGNATURES = {
    "kpx_kvm_create": (_P, [_I32, _I32, _U64, _I32, _I64, _I32]),
    "kpx_kvm_destroy": (None, [_P]),
    "kpx_kvm_add_sequence": (_I32, [_P]),
    "kpx_kvm_append": (C.c_int, [_P, _I32, _I32, _P]),
    "kpx_kvm_free_sequence": (C.c_int, [_P, _I32]),
    "kpx_kvm_seq_length": (_I32, [_P, _I32]),
    "kpx_kvm_seq_num_blocks": (_I32, [_P, _I32]),
    "kpx_kvm_block_table_row": (C.c_int, [_P, _I32, _P, _I32]),
    "kpx_kvm_num_free": (_I32, [_P]),
    "kpx_kvm_num_shared": (_I32, [_P]),
    "kpx_kvm_cow_events": (_I64, [_P]),
    "kpx_kvm_ref_counts": (C.c_int, [_P, _P, _I32]),
    "kpx_kvm_match_prefix": (C.c_int, [_P, _I32, _P, _I32, _P]),
    "kpx_kvm_insert_prefix": (C.c_int, [_P, _I32, _P, _I32]),
    "kpx_kvm_release_prefix": (C.c_int, [_P, _P, _I32]),
    "kpx_kvm_evict": (_I64, [_P, _I64]),
    "kpx_kvm_cached_tokens": (_I64, [_P]),
    "kpx_kvm_prefix_stats": (C.c_int, [_P, _P]),
    "kpx_kvm_pending": (C.c_int, [_P, _P, _P]),
    "kpx_kvm_take_pending": (C.c_int, [_P, _P, _P, _I32, _P, _P, _I32]),
    "kpx_kvm_flush_device": (C.c_int, [_P, _P, _P, _P, _P, _LP, _I32, _I64, _P, _I64, _P]),
}

_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        capi.lib()  # libkpx.so first (dependency, and it must exist)
        path = capi.LIB_DIR / "libkuiper_b200.so"
        if not path.exists():
            raise RuntimeError(f"{path} is missing: run python -m orinmllm_b200.build")
        handle = C.CDLL(str(path))
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype, fn.argtypes = res, args
        _lib = handle
    return _lib


def _i32(a):
    return np.ascontiguousarray(a, dtype=np.int32)


class KvManager:
    def __init__(self, num_blocks, block_size=16, seed=0, shuffle=True, max_cached_tokens=1 << 40,
                 min_prefix_length=4):
        self._h = lib().kpx_kvm_create(num_blocks, block_size, seed, int(shuffle), max_cached_tokens,
                                       min_prefix_length)
        if not self._h:
            raise ValueError("kpx_kvm_create refused the configuration")
        self.num_blocks, self.block_size = num_blocks, block_size

    def close(self):
        if self._h:
            lib().kpx_kvm_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def add_sequence(self) -> int:
        return lib().kpx_kvm_add_sequence(self._h)

    def append(self, seq, n) -> np.ndarray:
        slots = np.empty(max(n, 0), np.int64)
        capi.check(lib().kpx_kvm_append(self._h, seq, n, slots.ctypes.data), "kpx_kvm_append")
        return slots

    def try_append(self, seq, n):
        slots = np.empty(max(n, 0), np.int64)
        rc = lib().kpx_kvm_append(self._h, seq, n, slots.ctypes.data)
        return rc, slots

    def free_sequence(self, seq):
        capi.check(lib().kpx_kvm_free_sequence(self._h, seq), "kpx_kvm_free_sequence")

    def length(self, seq) -> int:
        return lib().kpx_kvm_seq_length(self._h, seq)

    def num_seq_blocks(self, seq) -> int:
        return lib().kpx_kvm_seq_num_blocks(self._h, seq)

    def block_table_row(self, seq, max_blocks) -> np.ndarray:
        row = np.empty(max_blocks, np.int32)
        capi.check(lib().kpx_kvm_block_table_row(self._h, seq, row.ctypes.data, max_blocks),
                   "kpx_kvm_block_table_row")
        return row

    def block_table(self, seqs, max_blocks=None) -> np.ndarray:
        if max_blocks is None:
            max_blocks = max([self.num_seq_blocks(s) for s in seqs] + [1])
        return np.stack([self.block_table_row(s, max_blocks) for s in seqs]) if seqs else np.zeros((0, max_blocks), np.int32)

    @property
    def num_free(self):
        return lib().kpx_kvm_num_free(self._h)

    @property
    def num_shared(self):
        return lib().kpx_kvm_num_shared(self._h)

    @property
    def cow_events(self):
        return lib().kpx_kvm_cow_events(self._h)

    def ref_counts(self) -> np.ndarray:
        out = np.empty(self.num_blocks, np.int32)
        capi.check(lib().kpx_kvm_ref_counts(self._h, out.ctypes.data, self.num_blocks), "kpx_kvm_ref_counts")
        return out

    def match_prefix(self, seq, tokens) -> int:
        t = _i32(tokens)
        m = C.c_int32(0)
        capi.check(lib().kpx_kvm_match_prefix(self._h, seq, t.ctypes.data, len(t), C.byref(m)),
                   "kpx_kvm_match_prefix")
        return m.value

    def insert_prefix(self, seq, tokens):
        t = _i32(tokens)
        capi.check(lib().kpx_kvm_insert_prefix(self._h, seq, t.ctypes.data, len(t)), "kpx_kvm_insert_prefix")

    def release_prefix(self, tokens):
        t = _i32(tokens)
        capi.check(lib().kpx_kvm_release_prefix(self._h, t.ctypes.data, len(t)), "kpx_kvm_release_prefix")

    def evict(self, target_tokens) -> int:
        return lib().kpx_kvm_evict(self._h, target_tokens)

    @property
    def cached_tokens(self):
        return lib().kpx_kvm_cached_tokens(self._h)

    def prefix_stats(self) -> dict:
        out = np.zeros(8, np.int64)
        capi.check(lib().kpx_kvm_prefix_stats(self._h, out.ctypes.data), "kpx_kvm_prefix_stats")
        keys = ["total_requests", "cache_hits", "cache_misses", "total_tokens_processed", "tokens_reused",
                "tokens_computed", "eviction_count", "tokens_evicted"]
        return dict(zip(keys, out.tolist()))

    def pending(self):
        a, b = C.c_int32(0), C.c_int32(0)
        lib().kpx_kvm_pending(self._h, C.byref(a), C.byref(b))
        return a.value, b.value

    def take_pending(self):
        nd, nc = self.pending()
        blocks, deltas = np.empty(nd, np.int32), np.empty(nd, np.int32)
        src, dst = np.empty(nc, np.int32), np.empty(nc, np.int32)
        capi.check(lib().kpx_kvm_take_pending(self._h, blocks.ctypes.data, deltas.ctypes.data, nd,
                                              src.ctypes.data, dst.ctypes.data, nc), "kpx_kvm_take_pending")
        return blocks, deltas, src, dst

    def flush_device(self, refcounts_dev, error_count_dev, k_pool, v_pool, layout, num_layers,
                     layer_stride, staging_dev, staging_bytes, stream=None):
        capi.check(lib().kpx_kvm_flush_device(self._h, capi.ptr(refcounts_dev), capi.ptr(error_count_dev),
                                              capi.ptr(k_pool), capi.ptr(v_pool), C.byref(layout), num_layers,
                                              layer_stride, capi.ptr(staging_dev), staging_bytes,
                                              capi._stream(stream)), "kpx_kvm_flush_device")
