"""The C-ABI library builds, loads and exports what include/dsa_b200.h declares.
No kernel is launched here: only argument checks that return before any launch."""
import ctypes
import os
import re

import pytest

from llmdivedeep_b200 import _lib, build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "dsa_b200.h")


@pytest.fixture(scope="module")
def lib():
    build.build()
    return _lib.load()


def declared_symbols():
    src = open(HEADER).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(dsa_[a-z0-9_]+)\s*\(", src)))


def test_header_symbols_are_exported(lib):
    names = declared_symbols()
    assert "dsa_indexer_logits" in names and "dsa_topk_select" in names
    for n in names:
        assert hasattr(lib, n), f"{n} declared in dsa_b200.h but not exported"


def test_binding_table_matches_header(lib):
    assert sorted(_lib.SIGNATURES) == declared_symbols()


def test_version_and_empty_error(lib):
    assert lib.dsa_version() >= 100
    assert isinstance(lib.dsa_last_error_string(), bytes)


def test_argument_errors_come_back_as_codes(lib):
    # ld_logits < S
    rc = lib.dsa_indexer_logits(16, 16, 16, 16, 0, None, 16, 16, 8, 4, 16, 64, 128, 1, None, None)
    assert rc == -1 and b"ld_logits" in lib.dsa_last_error_string()
    # NULL pointer
    rc = lib.dsa_indexer_logits(None, 16, 16, 16, 0, None, 16, 16, 16, 4, 16, 64, 128, 1, None, None)
    assert rc == -5
    # misaligned q
    rc = lib.dsa_indexer_logits(8, 16, 16, 16, 0, None, 16, 16, 16, 4, 16, 64, 128, 1, None, None)
    assert rc == -2
    # bad weight dtype
    rc = lib.dsa_indexer_logits(16, 16, 16, 16, 7, None, 16, 16, 16, 4, 16, 64, 128, 1, None, None)
    assert rc == -5
    # empty problem is a no-op success
    assert lib.dsa_indexer_logits(None, None, None, None, 0, None, None, None, 0, 0, 0, 64, 128, 1, None, None) == 0
    assert lib.dsa_topk_select(None, 0, None, None, 0, 0, 0, None, None) == 0
    assert lib.dsa_topk_select(16, 4, None, None, 1, 8, 2, 16, None) == -1          # ld < S
    assert lib.dsa_topk_select(16, 8, None, None, 1, 8, 70000, 16, None) == -1      # k too large
    # workspace too small / missing
    assert lib.dsa_indexer_topk(16, 16, 16, 16, 0, None, 16, 512, 1024, 64, 128, 8, 16, None, 0, None, None) == -3
    assert lib.dsa_indexer_topk(16, 16, 16, 16, 0, None, 16, 512, 1024, 64, 128, 8, 16, 16, 1024, None, None) == -3
    assert lib.dsa_indexer_topk_workspace_bytes(4096, 65536) == 4096 * 65536 * 4
    assert lib.dsa_indexer_topk_workspace_bytes(3, 5) == 3 * 8 * 4


def test_missing_library_is_loud(monkeypatch, tmp_path):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        _lib.load()


def test_cpu_tensors_are_refused():
    import torch
    from llmdivedeep_b200 import ops
    x = torch.zeros(2, 8)
    with pytest.raises(_lib.DsaError):
        ops.topk_select(x, 2)
