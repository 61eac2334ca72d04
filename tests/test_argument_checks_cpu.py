"""Argument checks of the C ABI that happen on the host, before anything is launched: they can
be exercised without a GPU.  Device pointers here are made-up, suitably aligned numbers; a
call that got past the checks would return KPX_ERR_CUDA on a machine without a device and is
never made with them on a machine that has one."""
import ctypes as C

import numpy as np
import pytest

from orinmllm_b200 import capi

FAKE = 0x7F0000000000  # never dereferenced: every call below is refused first


@pytest.fixture(scope="module")
def lib(native_libs):
    return capi.lib()


def _prefill(lib, lay, cu, start, batch, out=FAKE, q=FAKE, kp=FAKE, vp=FAKE, table=FAKE, max_blocks=8,
             heads=8, ws=FAKE, ws_bytes=1 << 30):
    cu = np.ascontiguousarray(cu, np.int32)
    start = np.ascontiguousarray(start, np.int32)
    return lib.kpx_paged_prefill(out, q, kp, vp, C.byref(lay), table, max_blocks, cu.ctypes.data,
                                 start.ctypes.data, batch, heads, 0.1, ws, ws_bytes, None)


def test_prefill_refuses_what_the_tensor_core_path_would_fault_on(lib):
    lay = capi.layout_paged(capi.KPX_F16, 2, 128, 16, 64)
    bad = capi.KPX_ERR_INVALID_ARGUMENT
    cu, start = [0, 40, 100], [0, 16]
    assert _prefill(lib, lay, cu, start, 2, out=None) == bad
    assert _prefill(lib, lay, cu, start, 2, q=None) == bad
    assert _prefill(lib, lay, cu, start, 2, kp=None) == bad
    assert _prefill(lib, lay, cu, start, 2, vp=None) == bad
    assert _prefill(lib, lay, cu, start, 2, out=FAKE + 8) == bad            # 16-byte stores
    assert _prefill(lib, lay, cu, start, 2, q=FAKE + 2) == bad
    assert _prefill(lib, lay, cu, start, 2, kp=FAKE + 4) == bad
    assert _prefill(lib, lay, cu, start, 2, max_blocks=0) == bad            # a table needs a width
    assert _prefill(lib, lay, cu, start, 2, max_blocks=4) == bad            # row 1 ends at token 76: 5 blocks
    assert _prefill(lib, lay, cu, [0, 70], 2, max_blocks=8) == bad          # 70 + 60 tokens: 9 blocks
    assert _prefill(lib, lay, cu, start, 2, heads=7) == bad                 # not a multiple of the kv heads
    assert _prefill(lib, lay, [1, 40, 100], start, 2) == bad
    assert _prefill(lib, lay, [0, 50, 40], start, 2) == bad
    assert _prefill(lib, lay, cu, [0, -1], 2) == bad
    assert _prefill(lib, lay, cu, start, 2, ws=None) == bad
    assert _prefill(lib, lay, cu, start, 2, ws_bytes=1024) == capi.KPX_ERR_WORKSPACE_TOO_SMALL
    assert _prefill(lib, lay, [0], [], 0) == capi.KPX_OK                     # nothing to do


def test_decode_refuses_bad_arguments_on_the_host(lib):
    lay = capi.layout_paged(capi.KPX_F16, 2, 128, 16, 64)
    bad = capi.KPX_ERR_INVALID_ARGUMENT

    def decode(out=FAKE, q=FAKE, kp=FAKE, vp=FAKE, table=FAKE, max_blocks=8, lens=FAKE, bias=0, batch=3,
               heads=8, ws=FAKE, ws_bytes=1 << 30):
        return lib.kpx_paged_decode(out, q, kp, vp, C.byref(lay), table, max_blocks, lens, bias, batch, heads,
                                    0.1, ws, ws_bytes, None)

    assert decode(out=None) == bad and decode(q=None) == bad and decode(kp=None) == bad
    assert decode(out=FAKE + 4) == bad and decode(ws=FAKE + 8) == bad
    assert decode(max_blocks=0) == bad
    assert decode(heads=9) == bad
    assert decode(lens=None, bias=-1) == bad
    assert decode(lens=None, bias=8 * 16 + 1) == bad      # a fixed length the table rows cannot hold
    assert decode(ws_bytes=4096) == capi.KPX_ERR_WORKSPACE_TOO_SMALL
    assert decode(batch=0) == capi.KPX_OK
    lay2 = capi.layout_paged(capi.KPX_F16, 2, 64, 16, 64)
    assert lib.kpx_paged_decode(FAKE, FAKE, FAKE, FAKE, C.byref(lay2), FAKE, 8, FAKE, 0, 3, 8, 0.1, FAKE, 1 << 30,
                                None) == capi.KPX_ERR_UNIMPLEMENTED
