"""The C-ABI library builds, loads without a GPU and exports every symbol the public header
declares; the ctypes table covers the same set.  No compute calls here."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "catccos_b200.h")


def _declared():
    src = open(HEADER).read()
    names = set(re.findall(r"CATCCOS_API\s+[\w\s\*]+?\b(catccos_\w+)\s*\(", src))
    names |= set(re.findall(r"^CATCCOS_DECLARE_LAUNCH\((\w+)\);", src, flags=re.M))
    return names


@pytest.fixture(scope="module")
def library():
    from catccos_b200 import build as b
    b.build()                                   # no-op when the library is up to date
    from catccos_b200 import _lib
    return _lib


def test_header_declares_the_expected_families():
    names = _declared()
    assert {"catccos_shmem_init", "catccos_launch", "catccos_mx_quant", "LaunchMatmulAllReduceFP16",
            "LaunchAllGatherMatmulBF16", "LaunchMatmulReduceScatterBF16"} <= names


def test_every_declared_symbol_is_exported_and_bound(library):
    cdll = ctypes.CDLL(library.LIB_PATH)
    names = _declared()
    missing = [n for n in sorted(names) if not hasattr(cdll, n)]
    assert not missing, f"declared in the header but not exported: {missing}"
    unbound = sorted(names - set(library.SIGNATURES))
    assert not unbound, f"declared in the header but absent from the ctypes table: {unbound}"
    extra = sorted(set(library.SIGNATURES) - names)
    assert not extra, f"bound in ctypes but not declared in the header: {extra}"


def test_calls_fail_loudly_without_a_gpu_or_heap(library):
    import torch
    lib = library.lib()
    assert lib.catccos_shmem_n_pes() == 0
    til = library.CocTilingParams()
    til.m, til.k, til.n, til.rankSize = 128, 64, 256, 1
    rc = lib.catccos_launch(1, 27, None, 0, 0, None, None, None, ctypes.byref(til), 0, 0)
    assert rc == 2                                              # CATCCOS_ERR_NOT_INIT
    assert b"not initialised" in lib.catccos_last_error()
    if not torch.cuda.is_available():
        assert lib.catccos_shmem_init_emulated(2, 1 << 20) == 3  # CATCCOS_ERR_CUDA: no driver, no fallback
    assert lib.catccos_shmem_init(0, 2, 1 << 20, b"") == 1      # empty rendezvous string, as set_attr()
    # tiling struct layout: 17 uint32 fields
    assert ctypes.sizeof(library.CocTilingParams) == 17 * 4
