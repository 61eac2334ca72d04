"""ctypes binding of include/kpx_sched.h (lib/libkuiper_b200.so): the request scheduler over
the paged KV cache -- admission by free blocks, prefix reuse, chunked prefill steps and batched
decode steps as plain arrays for the kernels."""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np

from . import kvm

_P, _I32, _I64 = C.c_void_p, C.c_int32, C.c_int64

SIGNATURES = {
    "kpx_sched_create": (_P, [_P, _I32, _I32, _I32, _I32, _I32]),
    "kpx_sched_destroy": (None, [_P]),
    "kpx_sched_submit": (_I32, [_P, _P, _I32, _I32, _I32]),
    "kpx_sched_submit_turn": (_I32, [_P, _P, _I32, _I32, _I32, _P, _I32]),
    "kpx_sched_set_end_tokens": (C.c_int, [_P, _P, _I32]),
    "kpx_sched_admit": (_I32, [_P]),
    "kpx_sched_next_prefill": (C.c_int, [_P]),
    "kpx_sched_prefill_shape": (C.c_int, [_P, _P, _P, _P]),
    "kpx_sched_prefill_arrays": (C.c_int, [_P, _P, _P, _P, _P, _P, _P, _P, _P, _I32]),
    "kpx_sched_complete_prefill": (C.c_int, [_P, _P, _I32]),
    "kpx_sched_next_decode": (C.c_int, [_P]),
    "kpx_sched_decode_shape": (C.c_int, [_P, _P, _P]),
    "kpx_sched_decode_arrays": (C.c_int, [_P, _P, _P, _P, _P, _P, _P, _I32]),
    "kpx_sched_complete_decode": (C.c_int, [_P, _P, _I32]),
    "kpx_sched_state": (_I32, [_P, _I32]),
    "kpx_sched_reused_tokens": (_I32, [_P, _I32]),
    "kpx_sched_tokens": (_I32, [_P, _I32, _P, _I32]),
    "kpx_sched_forget": (C.c_int, [_P, _I32]),
    "kpx_sched_num_waiting": (_I32, [_P]),
    "kpx_sched_num_running": (_I32, [_P]),
    "kpx_sched_stats": (C.c_int, [_P, _P]),
}

STATS_FIELDS = ("submitted", "admitted", "finished", "prompt_tokens", "reused_tokens", "prefilled_tokens",
                "decoded_tokens", "prefill_steps", "decode_steps", "admission_stalls", "peak_blocks_in_use",
                "gap_tokens")

_bound = False


def lib() -> C.CDLL:
    global _bound
    handle = kvm.lib()
    if not _bound:
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype, fn.argtypes = res, args
        _bound = True
    return handle


def _ptr(a):
    return a.ctypes.data_as(C.c_void_p)


@dataclass
class PrefillStep:
    request_ids: np.ndarray
    cu_q_lens: np.ndarray
    start_pos: np.ndarray
    positions: np.ndarray
    slot_mapping: np.ndarray
    token_ids: np.ndarray
    completes: np.ndarray
    block_table: np.ndarray


@dataclass
class DecodeStep:
    request_ids: np.ndarray
    seq_lens: np.ndarray
    positions: np.ndarray
    slot_mapping: np.ndarray
    token_ids: np.ndarray
    block_table: np.ndarray


class Scheduler:
    """base::KVScheduler on the pool and prefix cache of a KvManager."""

    def __init__(self, manager: kvm.KvManager, prefill_chunk=512, max_prefill_tokens=2048, max_prefill_rows=64,
                 max_decode_batch=256, use_prefix_cache=True):
        self.manager = manager  # keeps the pool alive
        self._h = lib().kpx_sched_create(manager._h, prefill_chunk, max_prefill_tokens, max_prefill_rows,
                                         max_decode_batch, int(use_prefix_cache))
        if not self._h:
            raise ValueError("kpx_sched_create refused the configuration")

    def close(self):
        if self._h:
            lib().kpx_sched_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def submit(self, prompt, max_new_tokens, also_register=0) -> int:
        p = np.ascontiguousarray(prompt, dtype=np.int32)
        rid = lib().kpx_sched_submit(self._h, _ptr(p), len(p), max_new_tokens, also_register)
        if rid < 0:
            raise ValueError("kpx_sched_submit refused the request")
        return rid

    def submit_turn(self, prompt, max_new_tokens, turn_suffix=(), also_register=0) -> int:
        """One turn of a conversation: at its end the last sampled token and `turn_suffix` are
        prefilled too and the whole history is registered (kpx_sched_submit_turn)."""
        p = np.ascontiguousarray(prompt, dtype=np.int32)
        sfx = np.ascontiguousarray(turn_suffix, dtype=np.int32)
        rid = lib().kpx_sched_submit_turn(self._h, _ptr(p), len(p), max_new_tokens, also_register,
                                          _ptr(sfx) if len(sfx) else None, len(sfx))
        if rid < 0:
            raise ValueError("kpx_sched_submit_turn refused the request")
        return rid

    def set_end_tokens(self, token_ids):
        """Sampled tokens that end a request early (kpx_sched_set_end_tokens); empty clears."""
        ids = np.ascontiguousarray(token_ids, dtype=np.int32)
        rc = lib().kpx_sched_set_end_tokens(self._h, _ptr(ids) if len(ids) else None, len(ids))
        if rc != 0:
            raise ValueError(f"kpx_sched_set_end_tokens: status {rc}")

    def admit(self) -> int:
        return lib().kpx_sched_admit(self._h)

    def next_prefill(self, min_table_width=0) -> PrefillStep | None:
        if not lib().kpx_sched_next_prefill(self._h):
            return None
        rows, toks, mb = C.c_int32(), C.c_int32(), C.c_int32()
        lib().kpx_sched_prefill_shape(self._h, C.byref(rows), C.byref(toks), C.byref(mb))
        r, t, w = rows.value, toks.value, max(mb.value, min_table_width, 1)
        s = PrefillStep(np.empty(r, np.int32), np.empty(r + 1, np.int32), np.empty(r, np.int32),
                        np.empty(t, np.int32), np.empty(t, np.int64), np.empty(t, np.int32),
                        np.empty(r, np.int32), np.empty((r, w), np.int32))
        rc = lib().kpx_sched_prefill_arrays(self._h, _ptr(s.request_ids), _ptr(s.cu_q_lens), _ptr(s.start_pos),
                                            _ptr(s.positions), _ptr(s.slot_mapping), _ptr(s.token_ids),
                                            _ptr(s.completes), _ptr(s.block_table), w)
        if rc != 0:
            raise RuntimeError(f"kpx_sched_prefill_arrays: status {rc}")
        return s

    def complete_prefill(self, sampled):
        a = np.ascontiguousarray(sampled, dtype=np.int32)
        rc = lib().kpx_sched_complete_prefill(self._h, _ptr(a), len(a))
        if rc != 0:
            raise RuntimeError(f"kpx_sched_complete_prefill: status {rc}")

    def next_decode(self, min_table_width=0) -> DecodeStep | None:
        if not lib().kpx_sched_next_decode(self._h):
            return None
        rows, mb = C.c_int32(), C.c_int32()
        lib().kpx_sched_decode_shape(self._h, C.byref(rows), C.byref(mb))
        r, w = rows.value, max(mb.value, min_table_width, 1)
        s = DecodeStep(np.empty(r, np.int32), np.empty(r, np.int32), np.empty(r, np.int32),
                       np.empty(r, np.int64), np.empty(r, np.int32), np.empty((r, w), np.int32))
        rc = lib().kpx_sched_decode_arrays(self._h, _ptr(s.request_ids), _ptr(s.seq_lens), _ptr(s.positions),
                                           _ptr(s.slot_mapping), _ptr(s.token_ids), _ptr(s.block_table), w)
        if rc != 0:
            raise RuntimeError(f"kpx_sched_decode_arrays: status {rc}")
        return s

    def complete_decode(self, sampled):
        a = np.ascontiguousarray(sampled, dtype=np.int32)
        rc = lib().kpx_sched_complete_decode(self._h, _ptr(a), len(a))
        if rc != 0:
            raise RuntimeError(f"kpx_sched_complete_decode: status {rc}")

    def state(self, rid) -> int:
        return lib().kpx_sched_state(self._h, rid)

    def reused_tokens(self, rid) -> int:
        return lib().kpx_sched_reused_tokens(self._h, rid)

    def tokens(self, rid) -> np.ndarray:
        n = lib().kpx_sched_tokens(self._h, rid, None, 0)
        if n < 0:
            raise KeyError(rid)
        out = np.empty(n, np.int32)
        lib().kpx_sched_tokens(self._h, rid, _ptr(out), n)
        return out

    def forget(self, rid):
        lib().kpx_sched_forget(self._h, rid)

    @property
    def num_waiting(self) -> int:
        return lib().kpx_sched_num_waiting(self._h)

    @property
    def num_running(self) -> int:
        return lib().kpx_sched_num_running(self._h)

    def stats(self) -> dict:
        out = np.zeros(12, np.int64)
        lib().kpx_sched_stats(self._h, _ptr(out))
        return dict(zip(STATS_FIELDS, (int(v) for v in out[:12])))
