"""CPU checks of the drop-in boundary: the C-ABI library loads and exports what include/nvk.h declares."""
import ctypes
import os
import re

import pytest

from util import ROOT, entry, nvk


@pytest.fixture(scope="module")
def built():
    entry.build()
    return nvk()


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "nvk.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(nvk_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_expected_entry_points(built):
    assert set(_declared_symbols()) >= set(built.EXPORTED_SYMBOLS)


def test_library_exports_every_declared_symbol(built):
    lib = ctypes.CDLL(built.LIB_PATH)
    for name in _declared_symbols():
        assert hasattr(lib, name), f"libnvk.so does not export {name}"


def test_abi_version_and_error_channel(built):
    lib = built.lib()
    assert lib.nvk_abi_version() == 2
    # invalid arguments are rejected on the host, before any CUDA call
    rc = lib.nvk_store_kvcache(None, None, None, None, None, 3, ctypes.c_int64(1), ctypes.c_int64(4),
                               ctypes.c_int64(4), 2, None)
    assert rc == built.ERR_INVALID_ARGUMENT
    assert b"must be defined" in lib.nvk_last_error()
    one = ctypes.c_void_p(16)
    rc = lib.nvk_store_kvcache(one, one, one, one, one, 3, ctypes.c_int64(0), ctypes.c_int64(4),
                               ctypes.c_int64(4), 2, None)
    assert rc == built.ERR_INVALID_ARGUMENT
    assert b"at least one element" in lib.nvk_last_error()   # src/kernels/kvcache.cu:164-167
    rc = lib.nvk_store_kvcache(one, one, one, one, one, 2, ctypes.c_int64(1), ctypes.c_int64(4),
                               ctypes.c_int64(4), 2, None)
    assert rc == built.ERR_INVALID_ARGUMENT and b"int32 or int64" in lib.nvk_last_error()
    rc = lib.nvk_decode_attention_paged(one, one, one, one, 3, one, 3, ctypes.c_int64(1), ctypes.c_int64(1),
                                        ctypes.c_int64(1), 3, 2, 128, 256, ctypes.c_float(1.0), one, 1, None,
                                        ctypes.c_size_t(0), None)
    assert rc == built.ERR_INVALID_ARGUMENT and b"divisible" in lib.nvk_last_error()
    # index tensors carry a dtype code each: int32 (3) or int64 (4), nothing else
    rc = lib.nvk_decode_attention_paged(one, one, one, one, 3, one, 2, ctypes.c_int64(1), ctypes.c_int64(1),
                                        ctypes.c_int64(1), 4, 2, 128, 256, ctypes.c_float(1.0), one, 1, None,
                                        ctypes.c_size_t(0), None)
    assert rc == built.ERR_INVALID_ARGUMENT and b"int32 or int64" in lib.nvk_last_error()
    rc = lib.nvk_prefill_attention_varlen(one, None, None, one, one, one, 4, one, 5, one, 3, ctypes.c_int64(1),
                                          ctypes.c_int64(1), ctypes.c_int64(0), ctypes.c_int64(1), ctypes.c_int64(1), 0,
                                          4, 2, 128, 256, ctypes.c_float(1.0), one, 1, None)
    assert rc == built.ERR_INVALID_ARGUMENT and b"int32 or int64" in lib.nvk_last_error()
    rc = lib.nvk_prefill_status(None, None)
    assert rc == built.ERR_INVALID_ARGUMENT
    assert built.decode_attention_static_scratch_bytes() == 32 << 20


def test_workspace_size_depends_only_on_host_known_sizes(built):
    a = built.decode_attention_workspace_bytes(256, 32, 8, 128, 32, 256)
    b = built.decode_attention_workspace_bytes(256, 32, 8, 128, 32, 256)
    assert a == b and a > 0
    assert built.decode_attention_workspace_bytes(0, 32, 8, 128, 32, 256) == 0


def test_missing_library_fails_loudly(built, monkeypatch):
    monkeypatch.setattr(built, "_lib", None)
    monkeypatch.setattr(built, "LIB_PATH", os.path.join(ROOT, "does_not_exist", "libnvk.so"))
    with pytest.raises(built.NvkLibraryMissing):
        built.lib()
