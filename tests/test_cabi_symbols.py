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


def test_error_behaviour_of_the_boundary_without_a_device():
    """What a caller sees before any device work: status codes and messages, as the reference's host code
    expects them (utils/shmem_init.h:16-39 rejects an empty ip_port; an unregistered (commType, dataType) pair
    gives no kernel, tests/dynamic_tiling/include/launch_map.h:31-39)."""
    import ctypes
    from catccos_b200 import KernelParams, lib, runtime as rt
    L = lib()
    t = rt.tiling(1024, 8192, 4096, 8)
    kp = KernelParams()
    assert L.catccos_launch(rt.ALLGATHER_MATMUL, rt.BF16, None, 0, 0, ctypes.byref(kp), None, None, ctypes.byref(t), 0, 0) == 2
    assert b"not initialised" in L.catccos_last_error()                       # CATCCOS_ERR_NOT_INIT
    assert L.catccos_launch(99, rt.BF16, None, 0, 0, ctypes.byref(kp), None, None, ctypes.byref(t), 0, 0) == 1
    assert b"no kernel registered for commType=99" in L.catccos_last_error()   # CATCCOS_ERR_INVALID
    assert L.catccos_shmem_init(0, 2, 1 << 20, b"") == 1 and b"ip_port" in L.catccos_last_error()
    assert L.catccos_shmem_init(3, 2, 1 << 20, b"tcp://127.0.0.1:1") == 1 and b"bad PE numbering" in L.catccos_last_error()
    assert not L.catccos_shmem_malloc(1024)
    assert L.catccos_shmem_my_pe() == -1 and L.catccos_shmem_n_pes() == 0


def test_buffer_sizes_of_the_benchmark_configurations():
    """Pure host arithmetic of catccos_symmetric_bytes / catccos_workspace_bytes: the dense and MXFP8 operators
    keep two halves of their region; everything fits the reference's 1004 MiB symmetric buffer."""
    import ctypes
    from catccos_b200 import lib, runtime as rt
    L = lib()

    def symm(comm, dt, m, k, n, ranks, **kw):
        t = rt.tiling(m, k, n, ranks, **kw)
        return L.catccos_symmetric_bytes(comm, dt, ctypes.byref(t)), L.catccos_workspace_bytes(comm, dt, ctypes.byref(t))

    assert symm(rt.ALLGATHER_MATMUL, rt.BF16, 1024, 8192, 4096, 8)[0] == 2 * 8 * 1024 * 8192 * 2
    assert symm(rt.MATMUL_REDUCE_SCATTER, rt.BF16, 8192, 2048, 8192, 8)[0] == 2 * 8192 * 8192 * 2
    assert symm(rt.MATMUL_ALLREDUCE, rt.FP16, 512, 1024, 2048, 2)[0] == 2 * (2 * 2 * 256 * 2048 * 2)
    assert symm(rt.ALLGATHER_MATMUL, rt.BF16, 1024, 8192, 4096, 1) == (0, 0)           # a single rank needs nothing
    s, w = symm(rt.FP8_MX_ALLGATHER_MATMUL, rt.BF16, 2048, 7168, 4096, 8)
    assert 2 * 8 * 2048 * 7168 < s <= 1004 << 20 and w > 0
    s, w = symm(rt.DISPATCH_FFN_COMBINE, rt.BF16, 4096, 7168, 4096, 8, topK=8, expertNum=256, epSize=8)
    assert 0 < s <= 1004 << 20 and w > 0
    assert symm(rt.MXFP8_MATMUL_REDUCE_SCATTER, rt.BF16, 8192, 2048, 8192, 8)[0] == 2 * 8192 * 8192 * 2
    assert L.catccos_fp4_gemm_workspace_bytes(1, 128, 256, 256) == 2048 + 4096 + 64    # atoms of A, of B, status words


def test_buffer_sizes_of_the_variants_and_fp4_operators():
    """The data-flow variants use the region of the operator they derive from; the MXFP4 operators gather half the
    code bytes of their MXFP8 twins with the same scale atoms."""
    import ctypes
    from catccos_b200 import lib, runtime as rt
    L = lib()

    def symm(comm, m, k, n, ranks, **kw):
        t = rt.tiling(m, k, n, ranks, **kw)
        return L.catccos_symmetric_bytes(comm, rt.BF16, ctypes.byref(t)), L.catccos_workspace_bytes(comm, rt.BF16, ctypes.byref(t))

    ag = symm(rt.ALLGATHER_MATMUL, 1024, 8192, 4096, 8)
    assert symm(rt.ALLGATHER_MATMUL_WITH_GATHER_RESULT, 1024, 8192, 4096, 8) == ag
    assert symm(rt.ALLGATHER_MATMUL_REMOTE_READ, 1024, 8192, 4096, 8) == ag
    assert symm(rt.ALLTOALL_MATMUL, 8 * 1024, 8192, 4096, 8) == ag                     # m = rows of every rank's A
    rs = symm(rt.MATMUL_REDUCE_SCATTER, 8192, 2048, 8192, 8)
    assert symm(rt.MATMUL_ALLTOALL, 8192, 2048, 8192, 8) == rs
    mxrs = symm(rt.MXFP8_MATMUL_REDUCE_SCATTER, 8192, 2048, 8192, 8)
    assert symm(rt.MXFP8_MATMUL_ALLTOALL, 8192, 2048, 8192, 8) == mxrs
    assert symm(rt.FP4_MX_MATMUL_REDUCE_SCATTER, 8192, 2048, 8192, 8) == mxrs          # partial tiles, not operands, are exchanged
    s8, w8 = symm(rt.FP8_MX_ALLGATHER_MATMUL, 2048, 7168, 4096, 8)
    s4, w4 = symm(rt.FP4_MX_ALLGATHER_MATMUL, 2048, 7168, 4096, 8)
    assert w4 == w8 and s8 - s4 == 2 * 8 * 2048 * 7168 // 2                            # half the code bytes in both halves
    kw = dict(expertNum=256, epSize=8)
    for c8, c4 in ((rt.FP8_MX_ALLTOALLV_GROUPED_MATMUL, rt.FP4_MX_ALLTOALLV_GROUPED_MATMUL),
                   (rt.FP8_MX_GROUPED_MATMUL_ALLTOALLV, rt.FP4_MX_GROUPED_MATMUL_ALLTOALLV)):
        a8, b8 = symm(c8, 4096, 7168, 4096, 8, **kw)
        a4, b4 = symm(c4, 4096, 7168, 4096, 8, **kw)
        assert 0 < a4 < a8 <= 1004 << 20 and b4 == b8 > 0
