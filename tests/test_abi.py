"""CPU tests of the drop-in boundary: the shared library loads and exports every symbol the
header declares, the ctypes table matches the header, and argument validation works without
a GPU (no kernel is launched here)."""
import ctypes
import os
import re

import pytest

from tests.conftest import ROOT


def _declared():
    text = open(os.path.join(ROOT, "include", "diffcache_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(dc_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported_and_bound():
    from diffcache_b200 import _lib

    lib = _lib.load()
    names = _declared()
    assert len(names) >= 20
    for name in names:
        assert hasattr(lib, name), f"{name} declared in the header but not exported"
        assert name in _lib.SIGNATURES, f"{name} has no ctypes signature"
    for name in _lib.SIGNATURES:
        assert name in names, f"{name} bound in ctypes but not declared in the header"
    assert lib.dc_version() >= 100


def test_every_declaration_cites_the_reference():
    text = open(os.path.join(ROOT, "include", "diffcache_b200.h")).read()
    assert text.count("lib.rs:") >= 10 and text.count("nsw.rs:") >= 5 and "diffcache.py:" in text


def test_argument_validation_without_gpu():
    from diffcache_b200 import _lib

    lib = _lib.load()
    h = ctypes.c_void_p()
    # q_heads not a multiple of kv_heads: the reference asserts (lib.rs:294)
    assert lib.dc_create(1, 30, 8, 128, 1024, 0, 0, ctypes.byref(h)) == -1
    assert b"multiple" in lib.dc_last_error()
    assert lib.dc_create(1, 32, 8, 96, 1024, 0, 0, ctypes.byref(h)) == -1
    assert lib.dc_ctx_len(None, None) == -1
    assert lib.dc_score_scan(None, 0, 1, 1, 128, 0, None, 0, 1, None, 0, None, 0) == -1
    assert lib.dc_topk_select(None, None, 0, 1, 1, 1, None, None, None, 0, None, 0) == -1
    assert lib.dc_merge_sorted_count(None, 2, 1, 8, 0, None, 0) == -1


def test_unknown_engine_option_is_rejected():
    from diffcache_b200 import DiffCacheGPU

    with pytest.raises(ValueError, match="Unknown option"):
        DiffCacheGPU(1, 32, 8, 128, bogus=1, device=0)


def test_product_does_not_import_the_oracle():
    pkg = os.path.join(ROOT, "diffcache_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                src = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in src.lower(), f"{f} mentions the oracle"
