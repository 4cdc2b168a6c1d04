"""CPU: the C-ABI library loads without a GPU and exports every symbol the header declares.
Only argument validation is exercised here — nothing is launched."""
import ctypes
import re
from pathlib import Path

import pytest

from nanopd_b200 import _lib

HEADERS = sorted((Path(__file__).resolve().parents[1] / "include").glob("*.h"))


def declared_symbols():
    names = set()
    for header in HEADERS:
        text = re.sub(r"/\*.*?\*/", "", header.read_text(), flags=re.S)
        names.update(re.findall(r"\b(npd_[a-z0-9_]+)\s*\(", text))
    return sorted(names)


def test_header_declares_the_four_kernels():
    names = declared_symbols()
    for want in ("npd_kv_store", "npd_paged_decode_attention", "npd_paged_prefill_attention", "npd_kv_migrate"):
        assert want in names


@pytest.mark.parametrize("name", declared_symbols())
def test_symbol_exported_and_bound(name):
    lib = _lib.load()
    assert hasattr(lib, name), f"{name} declared in the header but not exported"
    assert name in _lib.SIGNATURES, f"{name} has no ctypes signature"


def test_no_undeclared_bindings():
    assert sorted(_lib.SIGNATURES) == declared_symbols()


def test_version_and_error_string():
    lib = _lib.load()
    assert lib.npd_version() >= 100
    assert isinstance(lib.npd_last_error(), bytes)


def test_argument_errors_return_codes_without_touching_a_gpu():
    lib = _lib.load()
    # unsupported dtype code -> NPD_ERR_UNSUPPORTED before any CUDA call
    rc = lib.npd_kv_store(None, None, None, None, None, None, 1, 1, 128, 16, 1, 1, 2048, 128, 128, 1, 99, None, None)
    assert rc == _lib.NPD_ERR_UNSUPPORTED and b"dtype" in lib.npd_last_error()
    # head_dim outside the supported set
    rc = lib.npd_paged_decode_attention(None, None, None, None, None, None, 1.0, 1, 4, 4, 96, 16, 1, 1, 6144, 1,
                                        _lib.NPD_DTYPE_F16, None, 0, 0, None)
    assert rc == _lib.NPD_ERR_UNSUPPORTED and b"head_dim" in lib.npd_last_error()
    # q heads not a multiple of kv heads
    rc = lib.npd_paged_decode_attention(None, None, None, None, None, None, 1.0, 1, 5, 2, 128, 16, 1, 1, 4096, 1,
                                        _lib.NPD_DTYPE_BF16, None, 0, 0, None)
    assert rc == _lib.NPD_ERR_INVALID_ARG
    # migration with a block that is not a multiple of 16 bytes
    rc = lib.npd_kv_migrate(None, None, None, None, None, None, 1, 1, 3, 2, 3, 3, 1, 3, 3, 1, 0, None, None)
    assert rc == _lib.NPD_ERR_INVALID_ARG
    with pytest.raises(RuntimeError, match="nanopd_b200 error"):
        _lib.check(rc)


def test_workspace_size_is_reported_without_a_device():
    lib = _lib.load()
    small = lib.npd_decode_workspace_bytes(8, 12, 2, 128, 0)
    big = lib.npd_decode_workspace_bytes(4096, 32, 8, 128, 0)
    assert 0 < small <= big < (1 << 28)
    assert lib.npd_decode_workspace_bytes(8, 0, 2, 128, 0) == 0
