"""ctypes binding of the C ABI in include/kpx.h (lib/libkpx.so).

This is a thin loader for test drivers, the benchmark and Python callers: every
function forwards raw device pointers to the native library and raises on a
non-zero status.  There is no Python or CPU implementation behind it: if the
native library has not been built, importing `lib()` raises.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

LIB_DIR = Path(__file__).resolve().parent / "lib"

KPX_F16, KPX_BF16, KPX_F32 = 0, 1, 2
KPX_OK = 0
KPX_ERR_UNIMPLEMENTED = 1
KPX_ERR_INTERNAL = 5
KPX_ERR_INVALID_ARGUMENT = 7
KPX_ERR_OUT_OF_BLOCKS = 8
KPX_ERR_CUDA = 9
KPX_ERR_WORKSPACE_TOO_SMALL = 10
KPX_ERR_DEVICE_TIMEOUT = 11
KPX_ERR_REFCOUNT = 12
KPX_ERR_NOT_FOUND = 13
KPX_ERR_STATIC_SCRATCH_LIMIT = 14


class KvLayout(C.Structure):
    """struct kpx_kv_layout"""
    _fields_ = [("dtype", C.c_int32), ("num_kv_heads", C.c_int32), ("head_size", C.c_int32),
                ("block_size", C.c_int32), ("block_stride", C.c_int64), ("head_stride", C.c_int64),
                ("token_stride", C.c_int64), ("num_blocks", C.c_int64)]


class KpxError(RuntimeError):
    def __init__(self, status: int, where: str):
        self.status = status
        super().__init__(f"{where}: status {status} ({status_string(status)})")


_P = C.c_void_p
_I32, _I64, _F32 = C.c_int32, C.c_int64, C.c_float
_LP = C.POINTER(KvLayout)

# name -> (restype, argtypes); must list every symbol include/kpx.h declares
SIGNATURES = {
    "kpx_status_string": (C.c_char_p, [C.c_int]),
    "kpx_abi_version": (C.c_int, []),
    "kpx_device_count": (C.c_int, []),
    "kpx_layout_paged": (C.c_int, [_LP, _I32, _I32, _I32, _I32]),
    "kpx_layout_contiguous": (C.c_int, [_LP, _I32, _I32, _I32, _I32]),
    "kpx_append": (C.c_int, [_P, _P, _LP, _P, _P, _P, _P, _I32, _I32, _P]),
    "kpx_rope_append": (C.c_int, [_P, _P, _P, _I32, _P, _I32, _P, _P, _P, _P, _LP, _P, _I32, _P]),
    "kpx_norm_rope_append": (C.c_int, [_P, _P, _P, _I32, _P, _P, _F32, _P, _I32, _P, _P, _P, _P, _LP, _P, _I32, _P]),
    "kpx_sin_cos_cache": (C.c_int, [_P, _P, _I32, _I32, _F32, _P]),
    "kpx_decode_workspace_bytes": (_I64, [_I32, _I32, _I32, _I32]),
    "kpx_paged_decode": (C.c_int, [_P, _P, _P, _P, _LP, _P, _I32, _P, _I32, _I32, _I32, _F32,
                                   _P, _I64, _P]),
    "kpx_paged_decode_overlapped": (C.c_int, [_P, _P, _P, _P, _LP, _P, _I32, _P, _I32, _I32, _I32, _F32,
                                              _P, _I64, _P]),
    "kpx_decode_plan_bytes": (_I64, []),
    "kpx_decode_plan": (C.c_int, [_P, _I64, _LP, _P, _I32, _P, _I32, _I32, _I32, _P]),
    "kpx_paged_decode_planned": (C.c_int, [_P, _P, _P, _P, _LP, _P, _I32, _P, _I32, _I32, _I32, _F32,
                                           _P, _I64, _P, _I32, _P]),
    "kpx_rope_append_decode": (C.c_int, [_P, _P, _P, _P, _P, _P, _P, _P, _LP, _P, _I32, _P, _I32, _I32, _F32,
                                         _P, _I64, _I32, _P]),
    "kpx_paged_decode_static": (C.c_int, [_P, _P, _P, _P, _LP, _P, _I32, _P, _I32, _I32, _I32, _F32, _P]),
    "kpx_workspace_init": (C.c_int, [_P, _I64, _P]),
    "kpx_workspace_status": (C.c_int, [_P, _P]),
    "kpx_prefill_workspace_bytes": (_I64, [_I32, _I32, _I32, _I32]),
    "kpx_paged_prefill": (C.c_int, [_P, _P, _P, _P, _LP, _P, _I32, _P, _P, _I32, _I32, _F32,
                                    _P, _I64, _P]),
    "kpx_cow_copy_blocks": (C.c_int, [_P, _P, _LP, _I32, _I64, _P, _P, _I32, _P]),
    "kpx_refcount_update": (C.c_int, [_P, _I32, _P, _P, _I32, _P, _P]),
}

_lib = None


def lib() -> C.CDLL:
    """Load lib/libkpx.so (once).  Raises if it has not been built."""
    global _lib
    if _lib is None:
        path = LIB_DIR / "libkpx.so"
        if not path.exists():
            raise RuntimeError(
                f"{path} is missing: build the CUDA library first "
                "(python -m orinmllm_b200.build); there is no fallback path")
        handle = C.CDLL(str(path))
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name, None)
            if fn is None:
                continue  # reported by the symbol test; callers of a missing symbol fail loudly
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def status_string(status: int) -> str:
    return lib().kpx_status_string(int(status)).decode()


def check(status: int, where: str) -> None:
    if status != KPX_OK:
        raise KpxError(status, where)


def ptr(t) -> int | None:
    """Device (or host) address of a torch tensor / numpy array / int / None."""
    if t is None:
        return None
    if isinstance(t, int):
        return t
    if hasattr(t, "data_ptr"):
        return t.data_ptr()
    if hasattr(t, "ctypes"):
        return t.ctypes.data
    raise TypeError(type(t))


def dtype_code(torch_dtype) -> int:
    import torch
    return {torch.float16: KPX_F16, torch.bfloat16: KPX_BF16, torch.float32: KPX_F32}[torch_dtype]


def layout_paged(dtype: int, kv_heads: int, head_size: int = 128, block_size: int = 16,
                 num_blocks: int = 0) -> KvLayout:
    lay = KvLayout()
    check(lib().kpx_layout_paged(C.byref(lay), dtype, kv_heads, head_size, block_size),
          "kpx_layout_paged")
    lay.num_blocks = num_blocks
    return lay


def layout_contiguous(dtype: int, kv_heads: int, head_size: int = 128, block_size: int = 16,
                      num_blocks: int = 0) -> KvLayout:
    lay = KvLayout()
    check(lib().kpx_layout_contiguous(C.byref(lay), dtype, kv_heads, head_size, block_size),
          "kpx_layout_contiguous")
    lay.num_blocks = num_blocks
    return lay


def _stream(stream) -> int | None:
    if stream is None:
        import torch
        return torch.cuda.current_stream().cuda_stream
    return int(stream)


def append(k_pool, v_pool, layout, k_src, v_src, slot_mapping=None, pos_dev=None, pos_bias=0,
           num_tokens=None, stream=None) -> None:
    if num_tokens is None:
        num_tokens = k_src.shape[0]
    check(lib().kpx_append(ptr(k_pool), ptr(v_pool), C.byref(layout), ptr(k_src), ptr(v_src),
                           ptr(slot_mapping), ptr(pos_dev), pos_bias, num_tokens, _stream(stream)),
          "kpx_append")


def rope_append(q, k, v, q_heads, positions, sin_cache, cos_cache, k_pool, v_pool, layout,
                slot_mapping, num_tokens, stream=None, pos_base=0) -> None:
    check(lib().kpx_rope_append(ptr(q), ptr(k), ptr(v), q_heads, ptr(positions), pos_base, ptr(sin_cache),
                                ptr(cos_cache), ptr(k_pool), ptr(v_pool), C.byref(layout),
                                ptr(slot_mapping), num_tokens, _stream(stream)), "kpx_rope_append")


def norm_rope_append(q, k, v, q_heads, q_norm_weight, k_norm_weight, norm_eps, positions, sin_cache, cos_cache,
                     k_pool, v_pool, layout, slot_mapping, num_tokens, stream=None, pos_base=0) -> None:
    check(lib().kpx_norm_rope_append(ptr(q), ptr(k), ptr(v), q_heads, ptr(q_norm_weight), ptr(k_norm_weight),
                                     norm_eps, ptr(positions), pos_base, ptr(sin_cache), ptr(cos_cache),
                                     ptr(k_pool), ptr(v_pool), C.byref(layout), ptr(slot_mapping), num_tokens,
                                     _stream(stream)), "kpx_norm_rope_append")


def sin_cos_cache(sin_cache, cos_cache, head_size, max_seq_len, theta, stream=None) -> None:
    check(lib().kpx_sin_cos_cache(ptr(sin_cache), ptr(cos_cache), head_size, max_seq_len, theta,
                                  _stream(stream)), "kpx_sin_cos_cache")


def decode_workspace_bytes(batch, num_q_heads, num_kv_heads, head_size=128) -> int:
    n = lib().kpx_decode_workspace_bytes(batch, num_q_heads, num_kv_heads, head_size)
    if n < 0:
        raise KpxError(KPX_ERR_INVALID_ARGUMENT, "kpx_decode_workspace_bytes")
    return n


def workspace_init(workspace, nbytes, stream=None) -> None:
    check(lib().kpx_workspace_init(ptr(workspace), nbytes, _stream(stream)), "kpx_workspace_init")


def workspace_status(workspace, stream=None) -> int:
    return lib().kpx_workspace_status(ptr(workspace), _stream(stream))


def paged_decode(out, q, k_pool, v_pool, layout, block_table, max_blocks_per_seq, seq_lens,
                 len_bias, batch, num_q_heads, scale, workspace, workspace_bytes,
                 stream=None) -> None:
    check(lib().kpx_paged_decode(ptr(out), ptr(q), ptr(k_pool), ptr(v_pool), C.byref(layout),
                                 ptr(block_table), max_blocks_per_seq, ptr(seq_lens), len_bias,
                                 batch, num_q_heads, scale, ptr(workspace), workspace_bytes,
                                 _stream(stream)), "kpx_paged_decode")


KPX_DECODE_OVERLAPPED = 1


def rope_append_decode(out, q, k_new, v_new, sin_cache, cos_cache, k_pool, v_pool, layout, block_table,
                       max_blocks_per_seq, positions, batch, num_q_heads, scale, workspace,
                       workspace_bytes, flags=0, stream=None) -> None:
    """One decode step of a layer in one launch (RoPE + append + attention)."""
    check(lib().kpx_rope_append_decode(ptr(out), ptr(q), ptr(k_new), ptr(v_new), ptr(sin_cache),
                                       ptr(cos_cache), ptr(k_pool), ptr(v_pool), C.byref(layout),
                                       ptr(block_table), max_blocks_per_seq, ptr(positions), batch,
                                       num_q_heads, scale, ptr(workspace), workspace_bytes, flags,
                                       _stream(stream)), "kpx_rope_append_decode")


def paged_decode_overlapped(out, q, k_pool, v_pool, layout, block_table, max_blocks_per_seq, seq_lens,
                            len_bias, batch, num_q_heads, scale, workspace, workspace_bytes,
                            stream=None) -> None:
    """kpx_paged_decode in the form for launches that overlap on the GPU (own workspace each)."""
    check(lib().kpx_paged_decode_overlapped(ptr(out), ptr(q), ptr(k_pool), ptr(v_pool), C.byref(layout),
                                            ptr(block_table), max_blocks_per_seq, ptr(seq_lens), len_bias,
                                            batch, num_q_heads, scale, ptr(workspace), workspace_bytes,
                                            _stream(stream)), "kpx_paged_decode_overlapped")


def decode_plan_bytes() -> int:
    return lib().kpx_decode_plan_bytes()


def decode_plan(plan, plan_bytes, layout, block_table, max_blocks_per_seq, seq_lens, len_bias, batch,
                num_q_heads, stream=None) -> None:
    """Works out once what every decode launch of a step would work out in its prologue."""
    check(lib().kpx_decode_plan(ptr(plan), plan_bytes, C.byref(layout), ptr(block_table), max_blocks_per_seq,
                                ptr(seq_lens), len_bias, batch, num_q_heads, _stream(stream)), "kpx_decode_plan")


def paged_decode_planned(out, q, k_pool, v_pool, layout, block_table, max_blocks_per_seq, seq_lens,
                         len_bias, batch, num_q_heads, scale, workspace, workspace_bytes, plan, flags=0,
                         stream=None) -> None:
    """kpx_paged_decode / _overlapped (by flags) with the step's plan."""
    check(lib().kpx_paged_decode_planned(ptr(out), ptr(q), ptr(k_pool), ptr(v_pool), C.byref(layout),
                                         ptr(block_table), max_blocks_per_seq, ptr(seq_lens), len_bias,
                                         batch, num_q_heads, scale, ptr(workspace), workspace_bytes,
                                         ptr(plan), flags, _stream(stream)), "kpx_paged_decode_planned")


def paged_decode_static(out, q, k_pool, v_pool, layout, block_table, max_blocks_per_seq, seq_lens,
                        len_bias, batch, num_q_heads, scale, stream=None) -> None:
    """Decode with the library's built-in scratch array (no workspace argument, no allocation)."""
    check(lib().kpx_paged_decode_static(ptr(out), ptr(q), ptr(k_pool), ptr(v_pool), C.byref(layout),
                                        ptr(block_table), max_blocks_per_seq, ptr(seq_lens),
                                        len_bias, batch, num_q_heads, scale, _stream(stream)),
          "kpx_paged_decode_static")


def prefill_workspace_bytes(total_q, num_q_heads, num_kv_heads, head_size=128) -> int:
    n = lib().kpx_prefill_workspace_bytes(total_q, num_q_heads, num_kv_heads, head_size)
    if n < 0:
        raise KpxError(KPX_ERR_INVALID_ARGUMENT, "kpx_prefill_workspace_bytes")
    return n


def paged_prefill(out, q, k_pool, v_pool, layout, block_table, max_blocks_per_seq, cu_q_lens_host,
                  start_pos_host, batch, num_q_heads, scale, workspace, workspace_bytes,
                  stream=None) -> None:
    check(lib().kpx_paged_prefill(ptr(out), ptr(q), ptr(k_pool), ptr(v_pool), C.byref(layout),
                                  ptr(block_table), max_blocks_per_seq, ptr(cu_q_lens_host),
                                  ptr(start_pos_host), batch, num_q_heads, scale, ptr(workspace),
                                  workspace_bytes, _stream(stream)), "kpx_paged_prefill")


def cow_copy_blocks(k_pool, v_pool, layout, num_layers, layer_stride, src_ids, dst_ids, n,
                    stream=None) -> None:
    check(lib().kpx_cow_copy_blocks(ptr(k_pool), ptr(v_pool), C.byref(layout), num_layers,
                                    layer_stride, ptr(src_ids), ptr(dst_ids), n, _stream(stream)),
          "kpx_cow_copy_blocks")


def refcount_update(refcounts, num_blocks, block_ids, deltas, n, error_count=None,
                    stream=None) -> None:
    check(lib().kpx_refcount_update(ptr(refcounts), num_blocks, ptr(block_ids), ptr(deltas), n,
                                    ptr(error_count), _stream(stream)), "kpx_refcount_update")
