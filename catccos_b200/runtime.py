"""Python-side helpers over the C-ABI: symmetric-heap lifetime and operator launches that take
torch CUDA tensors (device memory and streams only; no computation happens in torch)."""
import contextlib
import ctypes

import torch

from ._lib import CocTilingParams, KernelParams, check, lib

# CocCommType / CocDataType values (utils/info.h:46-93 of the reference)
MATMUL_ALLREDUCE = 0
ALLGATHER_MATMUL = 1
MATMUL_REDUCE_SCATTER = 3
ALLGATHER_MATMUL_WITH_GATHER_RESULT = 5
ALLGATHER_MATMUL_REMOTE_READ = 20
MXFP8_MATMUL_REDUCE_SCATTER = 18
MXFP8_MATMUL_ALLTOALL = 19
FP8_MX_ALLGATHER_MATMUL = 22
FP4_MX_ALLGATHER_MATMUL = 23
MX_QUANT_ALLGATHER = 24
FP8_MX_GROUPED_MATMUL_ALLTOALLV = 25
FP4_MX_GROUPED_MATMUL_ALLTOALLV = 26
FP8_MX_ALLTOALLV_GROUPED_MATMUL = 27
FP4_MX_ALLTOALLV_GROUPED_MATMUL = 28
FP4_MX_MATMUL_REDUCE_SCATTER = 30
DISPATCH_FFN_COMBINE = 32
ALLTOALL_MATMUL = 101
MATMUL_ALLTOALL = 102
FP16, BF16, FP8E4M3FN = 1, 27, 36

_DTYPE = {torch.float16: FP16, torch.bfloat16: BF16}


def shmem_init(my_pe, n_pes, local_mem_size, ip_port):
    check(lib().catccos_shmem_init(my_pe, n_pes, local_mem_size, ip_port.encode()))


def shmem_init_emulated(n_pes, local_mem_size):
    check(lib().catccos_shmem_init_emulated(n_pes, local_mem_size))


def shmem_finalize():
    check(lib().catccos_shmem_finalize())


def shmem_malloc(nbytes):
    p = lib().catccos_shmem_malloc(nbytes)
    if not p:
        raise MemoryError(lib().catccos_last_error().decode())
    return p


def shmem_free(ptr):
    lib().catccos_shmem_free(ptr)


@contextlib.contextmanager
def emulated_team(n_pes, local_mem_size):
    """All PEs on the current device of this process (development / single-GPU testing)."""
    shmem_init_emulated(n_pes, local_mem_size)
    try:
        yield
    finally:
        torch.cuda.synchronize()
        shmem_finalize()


def tiling(m, k, n, rank_size, **kw):
    t = CocTilingParams()
    t.m, t.k, t.n, t.rankSize = m, k, n, rank_size
    for key, val in kw.items():
        setattr(t, key, val)
    return t


def _stream_ptr(stream):
    s = stream if stream is not None else torch.cuda.current_stream()
    return ctypes.c_void_p(s.cuda_stream)


def symmetric_bytes(comm_type, dtype, til):
    return lib().catccos_symmetric_bytes(comm_type, dtype, ctypes.byref(til))


def last_status():
    words = (ctypes.c_int32 * 8)()
    rc = lib().catccos_last_status(words)
    return rc, list(words)


def launch(comm_type, a, b, c, symmetric, til, trans_a=0, trans_b=0, block_num=0, stream=None, dtype=None,
           custom=(), workspace=None):
    """One rank per process: catccos_launch (KernelDispatcher::GetKernelFunc + call)."""
    kp = KernelParams()
    kp.ptrA, kp.ptrB, kp.ptrC = a.data_ptr(), b.data_ptr(), c.data_ptr()
    arr = None
    if custom:
        arr = (ctypes.c_void_p * len(custom))(*[t.data_ptr() for t in custom])
        kp.customPtrs = ctypes.cast(arr, ctypes.POINTER(ctypes.c_void_p))
        kp.customCount = len(custom)
    dt = dtype if dtype is not None else _DTYPE[a.dtype]
    ws = ctypes.c_void_p(workspace.data_ptr()) if workspace is not None else None
    check(lib().catccos_launch(comm_type, dt, _stream_ptr(stream), block_num, 0, ctypes.byref(kp), ws,
                               ctypes.c_void_p(symmetric), ctypes.byref(til), trans_a, trans_b))


def launch_emulated(comm_type, a_list, b_list, c_list, symmetric, til, trans_a=0, trans_b=0, block_num=0,
                    stream=None, dtype=None, custom_lists=None, workspaces=None):
    """All ranks in one cooperative launch (needs shmem_init_emulated)."""
    n = len(a_list)
    kps = (KernelParams * n)()
    keep = []
    for i in range(n):
        kps[i].ptrA, kps[i].ptrB, kps[i].ptrC = a_list[i].data_ptr(), b_list[i].data_ptr(), c_list[i].data_ptr()
        if custom_lists:
            arr = (ctypes.c_void_p * len(custom_lists[i]))(*[t.data_ptr() for t in custom_lists[i]])
            keep.append(arr)
            kps[i].customPtrs = ctypes.cast(arr, ctypes.POINTER(ctypes.c_void_p))
            kps[i].customCount = len(custom_lists[i])
    dt = dtype if dtype is not None else _DTYPE[a_list[0].dtype]
    ws = None
    if workspaces is not None:
        ws = (ctypes.c_void_p * n)(*[w.data_ptr() for w in workspaces])
    check(lib().catccos_launch_emulated(comm_type, dt, _stream_ptr(stream), block_num, kps, ws,
                                        ctypes.c_void_p(symmetric), ctypes.byref(til), trans_a, trans_b))
