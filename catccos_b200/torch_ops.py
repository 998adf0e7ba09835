"""`torch.ops.catccos.*` on CUDA tensors.

Mirrors the reference's TORCH_LIBRARY (examples/torch_binding/src/torch_bindings.cpp:85-240):
`init(rank_id, rank_size, local_mem_size, ip_port) -> int`, `allgather_matmul(a, b, rank_size)
-> Tensor`, `finalize() -> int`, with the same argument checks, the symmetric buffer allocated at
the first operator call and kept for later calls (:46-68), a stream synchronise before it is freed
(:206-213) and Meta kernels for shape inference (torch_bindings_meta.cpp:17-36).  The reference
binds AllGather-Matmul for float16 only; here bfloat16 is accepted too and Matmul-ReduceScatter
and Matmul-AllReduce are bound the same way.  All computation happens in the CUDA library
(`catccos_launch`); torch supplies tensors and the current stream.

Importing this module registers the operators; importing it twice is harmless.
"""
import threading

import torch

from . import runtime as rt

# examples/allgather_matmul/scripts/allgather_matmul.py passes the reference's SHMEM_BUFF_BYTES worth of
# local memory; the operators here size the symmetric buffer from the largest shape seen so far
_LOCK = threading.Lock()


class _State:
    def __init__(self):
        self.initialized = False
        self.rank_id = -1
        self.rank_size = 0
        self.local_mem_size = 0
        self.symm_ptr = None
        self.symm_bytes = 0


_STATE = _State()
_LIB = None


def _define():
    global _LIB
    if _LIB is not None:
        return
    lib = torch.library.Library("catccos", "DEF")
    lib.define("init(int rank_id, int rank_size, int local_mem_size, str ip_port) -> int")
    lib.define("allgather_matmul(Tensor a, Tensor b, int rank_size) -> Tensor")
    lib.define("matmul_reduce_scatter(Tensor a, Tensor b, int rank_size) -> Tensor")
    lib.define("matmul_allreduce(Tensor a, Tensor b, int rank_size) -> Tensor")
    lib.define("allgather_matmul_remote_read(Tensor a, Tensor b, int rank_size) -> Tensor")
    lib.define("allgather_matmul_with_gather_result(Tensor a, Tensor b, int rank_size) -> (Tensor, Tensor)")
    lib.define("alltoall_matmul(Tensor a, Tensor b, int rank_size) -> Tensor")
    lib.define("matmul_alltoall(Tensor a, Tensor b, int rank_size) -> Tensor")
    lib.define("finalize() -> int")
    lib.impl("init", _init, "CompositeExplicitAutograd")
    lib.impl("finalize", _finalize, "CompositeExplicitAutograd")
    lib.impl("allgather_matmul", _allgather_matmul, "CUDA")
    lib.impl("matmul_reduce_scatter", _matmul_reduce_scatter, "CUDA")
    lib.impl("matmul_allreduce", _matmul_allreduce, "CUDA")
    lib.impl("allgather_matmul", _allgather_matmul_meta, "Meta")
    lib.impl("matmul_reduce_scatter", _matmul_reduce_scatter_meta, "Meta")
    lib.impl("matmul_allreduce", _matmul_allreduce_meta, "Meta")
    for name, cuda, meta in (("allgather_matmul_remote_read", _allgather_matmul_remote_read, _allgather_matmul_meta),
                             ("allgather_matmul_with_gather_result", _allgather_matmul_with_gather_result,
                              _allgather_matmul_with_gather_result_meta),
                             ("alltoall_matmul", _alltoall_matmul, _matmul_allreduce_meta),
                             ("matmul_alltoall", _matmul_alltoall, _matmul_allreduce_meta)):
        lib.impl(name, cuda, "CUDA")
        lib.impl(name, meta, "Meta")
    _LIB = lib


def _check(cond, msg):
    if not cond:
        raise RuntimeError(msg)


def _init(rank_id, rank_size, local_mem_size, ip_port):
    with _LOCK:
        if _STATE.initialized:
            return 0
        _check(rank_id >= 0, f"invalid rank_id: {rank_id}")
        _check(rank_size > 0, f"invalid rank_size: {rank_size}")
        _check(local_mem_size > 0, f"invalid local_mem_size: {local_mem_size}")
        _check(len(ip_port) > 0, "ip_port is empty")
        rt.shmem_init(rank_id, rank_size, local_mem_size, ip_port)
        _STATE.initialized = True
        _STATE.rank_id = rank_id
        _STATE.rank_size = rank_size
        _STATE.local_mem_size = local_mem_size
        return 0


def _finalize():
    with _LOCK:
        if not _STATE.initialized:
            return 0
        if _STATE.symm_ptr is not None:
            torch.cuda.current_stream().synchronize()
            rt.shmem_free(_STATE.symm_ptr)
            _STATE.symm_ptr = None
            _STATE.symm_bytes = 0
        rt.shmem_finalize()
        _STATE.initialized = False
        _STATE.rank_id = -1
        _STATE.rank_size = 0
        return 0


def _symm(nbytes):
    """The cached symmetric buffer, allocated on first use with everything the heap has left."""
    _check(_STATE.initialized, "catccos TORCH_LIBRARY not initialized, call torch.ops.catccos.init(...) first")
    if _STATE.symm_ptr is None:
        want = max(int(nbytes), 1024)
        # take the whole heap (minus slack for alignment) so that later, larger shapes fit as well
        whole = _STATE.local_mem_size - (1 << 20)
        size = max(want, whole) if whole > want else want
        _STATE.symm_ptr = rt.shmem_malloc(size)
        _STATE.symm_bytes = size
    _check(_STATE.symm_bytes >= nbytes,
           f"existing symm buffer too small, existing={_STATE.symm_bytes}, required={nbytes}")
    return _STATE.symm_ptr


def _check_operands(a, b, rank_size):
    _check(_STATE.initialized, "catccos TORCH_LIBRARY not initialized, call torch.ops.catccos.init(...) first")
    _check(rank_size == _STATE.rank_size, f"rank_size mismatch: input={rank_size}, initialized={_STATE.rank_size}")
    _check(a.dtype in (torch.float16, torch.bfloat16), f"Only float16 / bfloat16 supported for a, got {a.dtype}")
    _check(b.dtype == a.dtype, f"a and b must have the same dtype, got {a.dtype} and {b.dtype}")
    _check(a.is_cuda and b.is_cuda, f"Only CUDA supported, got {a.device} and {b.device}")
    _check(a.device == b.device, "a and b must be on same device")
    _check(a.dim() == 2, f"a must be 2D, got dim={a.dim()}")
    _check(b.dim() == 2, f"b must be 2D, got dim={b.dim()}")
    _check(b.size(0) == a.size(1), f"A/K shape mismatch, a.size(1)={a.size(1)}, b.size(0)={b.size(0)}")


def _run(comm, a, b, out_rows, rank_size, custom=None):
    _check_operands(a, b, rank_size)
    m, k, n = a.size(0), a.size(1), b.size(1)
    a_c, b_c = a.contiguous(), b.contiguous()
    c = torch.empty((out_rows, n), dtype=a.dtype, device=a.device)
    til = rt.tiling(m, k, n, rank_size)
    need = rt.symmetric_bytes(comm, rt._DTYPE[a.dtype], til)
    with torch.cuda.device(a.device):
        symm = _symm(need) if rank_size > 1 else 0
        rt.launch(comm, a_c, b_c, c, symm, til, custom=custom)
    return c


def _allgather_matmul(a, b, rank_size):
    """C[rank_size * m, n]: rows s*m .. (s+1)*m are A_s @ B (torch_bindings.cpp:122-200)."""
    return _run(rt.ALLGATHER_MATMUL, a, b, a.size(0) * rank_size, rank_size)


def _matmul_reduce_scatter(a, b, rank_size):
    """D[m / rank_size, n]: this rank's rows of sum_r A_r @ B_r
    (examples/matmul_reduce_scatter/matmul_reduce_scatter_host.h:17-91)."""
    _check(a.size(0) % rank_size == 0, f"m ({a.size(0)}) must be divisible by rank_size ({rank_size})")
    return _run(rt.MATMUL_REDUCE_SCATTER, a, b, a.size(0) // rank_size, rank_size)


def _matmul_allreduce(a, b, rank_size):
    """D[m, n] = sum_r A_r @ B_r on every rank (examples/matmul_allreduce/matmul_allreduce_host.h:17-96)."""
    return _run(rt.MATMUL_ALLREDUCE, a, b, a.size(0), rank_size)


def _allgather_matmul_remote_read(a, b, rank_size):
    """The same product with the remote-read data flow (examples/allgather_matmul_remote_read)."""
    return _run(rt.ALLGATHER_MATMUL_REMOTE_READ, a, b, a.size(0) * rank_size, rank_size)


def _allgather_matmul_with_gather_result(a, b, rank_size):
    """(C, gathered A [rank_size * m, k]) (examples/allgather_matmul_with_gather_result)."""
    gathered = torch.empty((a.size(0) * rank_size, a.size(1)), dtype=a.dtype, device=a.device)
    c = _run(rt.ALLGATHER_MATMUL_WITH_GATHER_RESULT, a, b, a.size(0) * rank_size, rank_size, custom=[gathered])
    return c, gathered


def _alltoall_matmul(a, b, rank_size):
    """C[m, n]: block j of every rank's A (rank order) times this rank's B (examples/ascend950_alltoall_matmul)."""
    _check(a.size(0) % rank_size == 0, f"m ({a.size(0)}) must be divisible by rank_size ({rank_size})")
    return _run(rt.ALLTOALL_MATMUL, a, b, a.size(0), rank_size)


def _matmul_alltoall(a, b, rank_size):
    """C[m, n]: row block j of every rank's A_i @ B_i, in rank order (examples/ascend950_matmul_alltoall)."""
    _check(a.size(0) % rank_size == 0, f"m ({a.size(0)}) must be divisible by rank_size ({rank_size})")
    return _run(rt.MATMUL_ALLTOALL, a, b, a.size(0), rank_size)


def _allgather_matmul_with_gather_result_meta(a, b, rank_size):
    return a.new_empty((a.size(0) * rank_size, b.size(1))), a.new_empty((a.size(0) * rank_size, a.size(1)))


def _allgather_matmul_meta(a, b, rank_size):
    return a.new_empty((a.size(0) * rank_size, b.size(1)))


def _matmul_reduce_scatter_meta(a, b, rank_size):
    return a.new_empty((a.size(0) // rank_size, b.size(1)))


def _matmul_allreduce_meta(a, b, rank_size):
    return a.new_empty((a.size(0), b.size(1)))


_define()
