"""CPU: the C-ABI library loads, exports every symbol the header declares, and its host-side
argument checks answer without touching a device."""
import ctypes
import os
import re

import pytest

import ubridge_b200 as ub
from ubridge_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    hdr = open(os.path.join(ROOT, "include", "ubridge_b200.h")).read()
    hdr = re.sub(r"/\*.*?\*/", "", hdr, flags=re.S)
    names = re.findall(r"\b([A-Za-z_][A-Za-z0-9_]*)\s*\(", hdr)
    skip = {"defined", "void"}
    return sorted({n for n in names if n not in skip})


def test_every_declared_symbol_is_exported():
    handle = ctypes.CDLL(_lib.LIB_PATH)
    declared = _declared_symbols()
    assert len(declared) > 60
    for name in declared:
        assert hasattr(handle, name), "declared in the header but not exported: " + name
    assert sorted(ub.EXPORTED_SYMBOLS) == declared


def test_status_strings_and_version():
    l = ub.lib()
    assert l.ub_version() >= 100
    assert ub.status_string(0) == "ok"
    assert "workspace" in ub.status_string(_lib.UB_ERR_WORKSPACE)


def test_registry_names_match_reference_tables():
    ex = ub.DeviceExecutor()
    for fmt in ("q8_0", "q4_k"):
        for dt in ("f16", "bf16", "f32"):
            assert ex.has_function("quant", "dequantize_block_%s_%s" % (fmt, dt))
    for dt in ("f16", "bf16", "f32"):
        assert ex.has_function("quant", "quantize_block_q8_0_" + dt)
        assert not ex.has_function("quant", "quantize_block_q4_k_" + dt)  # a stub in the reference too
    assert not ex.has_function("matmul", "dequantize_block_q8_0_f32")
    with pytest.raises(ub.UbridgeError) as ei:
        ex.get_function("quant", "no_such_kernel")
    assert ei.value.status == _lib.UB_ERR_UNSUPPORTED
    assert ub.lib().ub_launch(None, None, None, None) == _lib.UB_ERR_UNSUPPORTED


def test_host_side_argument_checks():
    l = ub.lib()
    one = ctypes.c_void_p(256)  # never dereferenced: the checks below fail first
    assert l.ub_dequant_q4k(one, one, 100, _lib.DTYPE_F32, None) == _lib.UB_ERR_INVALID_ARG      # not a block multiple
    assert l.ub_dequant_q8_0(one, one, 64, 99, None) == _lib.UB_ERR_INVALID_ARG                 # unknown dtype
    assert l.ub_dequant_q8_0(None, one, 64, _lib.DTYPE_F32, None) == _lib.UB_ERR_INVALID_ARG
    assert l.ub_dequant_q8_0(None, None, 0, _lib.DTYPE_F32, None) == _lib.UB_OK                  # empty is fine
    assert l.ub_qmatmul_q4k_bf16(one, one, one, 1, 8, 100, _lib.DTYPE_BF16, None, 0, None) == _lib.UB_ERR_INVALID_ARG
    assert l.ub_qmatmul_q4k_bf16(one, one, ctypes.c_void_p(260), 1, 8, 256, _lib.DTYPE_BF16, None, 0, None) \
        == _lib.UB_ERR_INVALID_ARG                                                               # weights not 16-byte aligned
    assert l.ub_qmatmul_q4k_f32(one, one, one, 64, 8, 256, _lib.DTYPE_F32, None, 0, None) == _lib.UB_ERR_WORKSPACE
    assert l.ub_qmatmul_workspace_bytes(1, 4096, 4096, 1) == 0
    assert l.ub_qmatmul_workspace_bytes(2048, 14336, 4096, 1) >= 2048 * (4096 + 14336) * 2
    assert l.ub_moe_layer_q4k(one, one, one, one, one, None, 4, 256, 256, 2, 1, 4, 1, None, 0, None) \
        == _lib.UB_ERR_WORKSPACE
    need = l.ub_moe_layer_q4k_workspace_bytes(256, 4096, 14336, 8, 2, 64)
    assert need >= 512 * (14336 + 4096) * 2
    l.topk_softmax_f32(one, one, one, 4, 5000, 2, 0, None)                                      # E beyond the reference's limit
    assert l.ub_last_status() == _lib.UB_ERR_INVALID_ARG
    l.moe_align_block_size(one, one, one, one, None, None, 0, 4, 1, 1, None)
    assert l.ub_last_status() == _lib.UB_ERR_INVALID_ARG


def test_no_device_calls_fail_cleanly_on_cpu():
    l = ub.lib()
    if l.ub_device_count() > 0:
        pytest.skip("a device is present")
    h = ctypes.c_void_p()
    assert l.ub_device_new(0, ctypes.byref(h)) == _lib.UB_ERR_INVALID_ARG
    with pytest.raises(ub.UbridgeError):
        ub.GcuDevice(0)


def test_missing_library_is_loud(monkeypatch, tmp_path):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "libubridge_b200.so"))
    with pytest.raises(RuntimeError, match="no fallback"):
        _lib.lib()


def test_product_never_imports_the_oracle():
    pkg = os.path.join(ROOT, "ubridge_b200")
    for dirpath, _dirs, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h", ".cpp")):
                text = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in text, os.path.join(dirpath, f)
