"""The C-ABI library loads without a GPU and exports every symbol include/kpx.h declares."""
import ctypes
import re
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def declared_symbols():
    text = (ROOT / "include" / "kpx.h").read_text()
    return sorted(set(re.findall(r"KPX_API\s+[\w\s\*]+?\b(kpx_\w+)\s*\(", text)))


def test_header_declares_entry_points():
    syms = declared_symbols()
    assert "kpx_append" in syms and "kpx_paged_decode" in syms and "kpx_paged_prefill" in syms
    assert len(syms) >= 15


def test_library_exports_every_declared_symbol(native_libs):
    handle = ctypes.CDLL(str(native_libs))
    missing = [s for s in declared_symbols() if not hasattr(handle, s)]
    assert not missing, f"declared in kpx.h but not exported: {missing}"


def test_binding_covers_every_declared_symbol(native_libs):
    from orinmllm_b200 import capi
    assert sorted(capi.SIGNATURES) == declared_symbols()
    assert capi.lib().kpx_abi_version() >= 1
    assert capi.status_string(0) == "ok"


def test_argument_validation_without_gpu(native_libs):
    # validation happens before any CUDA call, so these work on a CPU-only box
    from orinmllm_b200 import capi
    lay = capi.layout_paged(capi.KPX_F16, 8, 128, 16)
    assert (lay.block_stride, lay.head_stride, lay.token_stride) == (8 * 16 * 128, 16 * 128, 128)
    lay2 = capi.layout_contiguous(capi.KPX_F32, 2, 128, 16)
    assert (lay2.block_stride, lay2.head_stride, lay2.token_stride) == (16 * 256, 128, 256)
    L = capi.lib()
    assert L.kpx_append(None, None, ctypes.byref(lay), None, None, None, None, 0, 4, None) == capi.KPX_ERR_INVALID_ARGUMENT
    assert L.kpx_paged_decode(None, None, None, None, ctypes.byref(lay), None, 0, None, 0, 1, 32, 1.0, None, 0, None) == capi.KPX_ERR_INVALID_ARGUMENT
    assert capi.decode_workspace_bytes(64, 32, 8, 128) > 0
    assert L.kpx_decode_workspace_bytes(64, 32, 8, 96) < 0


def test_host_manager_library_exports_every_declared_symbol(native_libs):
    from orinmllm_b200 import build, kvm
    so = build.build_host()
    text = (ROOT / "include" / "kpx_kvm.h").read_text()
    declared = sorted(set(re.findall(r"KPX_API\s+[\w\s\*]+?\b(kpx_kvm_\w+)\s*\(", text)))
    assert len(declared) >= 20
    handle = ctypes.CDLL(str(so))
    assert not [s for s in declared if not hasattr(handle, s)]
    assert sorted(kvm.SIGNATURES) == declared


def test_scheduler_header_symbols_exported(native_libs):
    from orinmllm_b200 import build, sched
    so = build.build_host()
    text = (ROOT / "include" / "kpx_sched.h").read_text()
    declared = sorted(set(re.findall(r"KPX_API\s+[\w\s\*]+?\b(kpx_sched_\w+)\s*\(", text)))
    assert len(declared) >= 15
    handle = ctypes.CDLL(str(so))
    assert not [s for s in declared if not hasattr(handle, s)]
    assert sorted(sched.SIGNATURES) == declared


def test_scheduler_handles_reject_bad_arguments(native_libs):
    from orinmllm_b200 import sched
    lib = sched.lib()
    assert not lib.kpx_sched_create(None, 512, 2048, 64, 256, 1)
    assert lib.kpx_sched_submit(None, None, 0, 1, 0) == -1
    assert lib.kpx_sched_admit(None) == -1
    assert lib.kpx_sched_next_prefill(None) == 0 and lib.kpx_sched_next_decode(None) == 0
