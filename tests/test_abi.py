"""The C-ABI library: it loads, exports every symbol the header declares, its struct layouts
match the ctypes mirror, and it fails loudly (no CPU path) when no device is present.  No
compute is launched here."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "born_sampler.h")


def header_symbols():
    src = open(HEADER).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(born_[a-z0-9_]+)\s*\(", src)))


def test_header_declares_what_the_binding_expects():
    from born_b200 import _lib
    assert set(header_symbols()) == set(_lib.SYMBOLS)


def test_library_exports_every_declared_symbol(lib):
    for name in header_symbols():
        assert hasattr(lib, name), name


def test_struct_sizes_match_header(lib):
    from born_b200 import _lib
    assert C.sizeof(_lib.RowParams) == 32
    # the library checks struct_size itself; a wrong size must be rejected before anything else
    a = _lib.SampleArgs()
    a.struct_size = 4
    assert lib.born_sample(None, C.byref(a), None) == _lib.ERR_INVALID_ARGUMENT
    assert b"handle is NULL" in lib.born_last_error(None)


def test_version_string(lib):
    assert b"sm_100a" in lib.born_version()


def test_record_bytes(lib):
    assert lib.born_shard_record_bytes(64) == 32 + 64 * 8
    assert lib.born_shard_record_bytes(0) == -1


def test_create_rejects_bad_arguments(lib):
    from born_b200 import _lib
    h = C.c_void_p()
    assert lib.born_sampler_create(0, 0, 1000, 0, C.byref(h)) == _lib.ERR_INVALID_ARGUMENT
    assert lib.born_sampler_create(0, 8, 1 << 25, 0, C.byref(h)) == _lib.ERR_INVALID_ARGUMENT
    assert lib.born_sampler_create(0, 8, 1000, 0, None) == _lib.ERR_INVALID_ARGUMENT


def _no_gpu():
    try:
        import torch
        return not torch.cuda.is_available()
    except Exception:
        return True


@pytest.mark.skipif(not _no_gpu(), reason="only meaningful on a box without a GPU")
def test_no_device_is_an_error_not_a_fallback(lib):
    from born_b200 import Sampler, SamplerError, _lib
    h = C.c_void_p()
    rc = lib.born_sampler_create(0, 8, 1000, 0, C.byref(h))
    assert rc == _lib.ERR_NO_DEVICE and not h.value
    assert b"no CPU path" in lib.born_last_error(None)
    with pytest.raises(SamplerError):
        Sampler(device=0, max_batch=8, max_vocab=1000)


def test_product_does_not_import_the_oracle():
    pkg = os.path.join(ROOT, "born_b200")
    bad = re.compile(r"(from\s+oracle|import\s+oracle|libborn_oracle|oracle/|born_oracle\.)")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h", ".hpp")):
                text = open(os.path.join(dirpath, f)).read()
                assert not bad.search(text), f
