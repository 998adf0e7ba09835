"""Parity of the f16/bf16 fused operators (CUDA, through the C-ABI) against the CPU oracle.

World sizes > 1 run as emulated PEs: all ranks inside one cooperative launch on one GPU, using
the same kernels, flags and peer stores as the one-process-per-GPU path."""
import pytest
import torch

from oracle import dense, inputs
from tests.gpu_util import assert_close_to_golden, assert_reduced_close, dev

pytestmark = pytest.mark.gpu

TOL = 1e-2   # max relative error for f16/bf16 against the fp32-accumulated golden


def _rt():
    from catccos_b200 import runtime
    return runtime


def _run_emulated(comm, world, a_list, b_list, out_shape, m, k, n, trans_b, dtype):
    rt = _rt()
    til = rt.tiling(m, k, n, world)
    need = rt.symmetric_bytes(comm, rt.BF16, til)
    with rt.emulated_team(world, max(need, 1 << 20)):
        symm = rt.shmem_malloc(max(need, 1024))
        a_d = [dev(a) for a in a_list]
        b_d = [dev(b.t() if trans_b else b) for b in b_list]
        c_d = [torch.full(out_shape, float("nan"), dtype=dtype, device="cuda") for _ in range(world)]
        # twice: the second launch exercises flag epochs and buffer reuse
        for _ in range(2):
            rt.launch_emulated(comm, a_d, b_d, c_d, symm, til, trans_b=1 if trans_b else 0)
        rc, words = rt.last_status()
        assert rc == 0, words
        return [c.cpu() for c in c_d]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("trans_b", [0, 1])
@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (256, 512, 256), (200, 264, 136), (1024, 2048, 1024), (8, 8, 8)])
def test_single_rank_gemm(dtype, trans_b, m, n, k):
    """World size 1: AllGather-Matmul degenerates to the plain tcgen05 GEMM."""
    rt = _rt()
    a, b = inputs.allgather_matmul_inputs(1, m, k, n, dtype)
    gold = dense.golden_allgather_matmul(a, b)[0]
    out = _run_emulated(rt.ALLGATHER_MATMUL, 1, a, b, (m, n), m, k, n, trans_b, dtype)[0]
    assert_close_to_golden(out, gold, k, TOL, f"gemm {m}x{n}x{k}")


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("trans_b", [0, 1])
@pytest.mark.parametrize("m_local,n,k", [(128, 256, 128), (320, 520, 192), (100, 256, 64)])
def test_allgather_matmul(world, trans_b, m_local, n, k):
    rt = _rt()
    a, b = inputs.allgather_matmul_inputs(world, m_local, k, n, torch.bfloat16)
    gold = dense.golden_allgather_matmul(a, b)
    outs = _run_emulated(rt.ALLGATHER_MATMUL, world, a, b, (world * m_local, n), m_local, k, n, trans_b,
                         torch.bfloat16)
    for r in range(world):
        assert_close_to_golden(outs[r], gold[r], k, TOL, f"agmm rank {r}")


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("trans_b", [0, 1])
@pytest.mark.parametrize("m,n,k", [(512, 256, 128), (1024, 520, 192)])
def test_matmul_reduce_scatter(world, trans_b, m, n, k):
    rt = _rt()
    a, b = inputs.matmul_reduce_scatter_inputs(world, m, k, n, torch.bfloat16)
    partials = [dense.matmul_fp32(x, y) for x, y in zip(a, b)]
    outs = _run_emulated(rt.MATMUL_REDUCE_SCATTER, world, a, b, (m // world, n), m, k, n, trans_b, torch.bfloat16)
    mr = m // world
    for r in range(world):
        assert_reduced_close(outs[r], [p[r * mr:(r + 1) * mr] for p in partials], k, TOL, f"mmrs rank {r}")


@pytest.mark.parametrize("comm_name", ["ALLGATHER_MATMUL", "MATMUL_REDUCE_SCATTER"])
def test_back_to_back_launches_with_new_inputs(comm_name):
    """Three launches of one operator without a sync in between, each with its own inputs: the
    operator alternates between the two halves of its symmetric region, and a launch may start
    writing a peer's half while that peer still reads the other one."""
    rt = _rt()
    world, k, n = 4, 192, 520
    comm = getattr(rt, comm_name)
    ag = comm_name == "ALLGATHER_MATMUL"
    m = 320 if ag else 1024
    til = rt.tiling(m, k, n, world)
    need = rt.symmetric_bytes(comm, rt.BF16, til)
    rounds = []
    for i in range(3):
        if ag:
            a, b = inputs.allgather_matmul_inputs(world, m, k, n, torch.bfloat16)
        else:
            a, b = inputs.matmul_reduce_scatter_inputs(world, m, k, n, torch.bfloat16)
        a = [x.roll(7 * i, 0) * (-1) ** i for x in a]     # the generators seed by rank only: make the launches differ
        rounds.append((a, b))
    out_shape = (world * m, n) if ag else (m // world, n)
    with rt.emulated_team(world, max(need, 1 << 20)):
        symm = rt.shmem_malloc(max(need, 1024))
        outs = []
        keep = []
        for a, b in rounds:
            a_d = [dev(x) for x in a]
            b_d = [dev(x) for x in b]
            c_d = [torch.full(out_shape, float("nan"), dtype=torch.bfloat16, device="cuda") for _ in range(world)]
            rt.launch_emulated(comm, a_d, b_d, c_d, symm, til, trans_b=0)
            keep.append((a_d, b_d))
            outs.append(c_d)
        rc, words = rt.last_status()
        assert rc == 0, words
        outs = [[c.cpu() for c in c_d] for c_d in outs]
    for i, (a, b) in enumerate(rounds):
        if ag:
            gold = dense.golden_allgather_matmul(a, b)
            for r in range(world):
                assert_close_to_golden(outs[i][r], gold[r], k, TOL, f"launch {i} rank {r}")
        else:
            partials = [dense.matmul_fp32(x, y) for x, y in zip(a, b)]
            mr = m // world
            for r in range(world):
                assert_reduced_close(outs[i][r], [p[r * mr:(r + 1) * mr] for p in partials], k, TOL,
                                     f"launch {i} rank {r}")


@pytest.mark.parametrize("world,m,n,k,dtype", [
    (2, 512, 2048, 1024, torch.float16),      # benchmark configuration 1
    (4, 300, 264, 128, torch.float16),        # ragged rows per rank
    (8, 1024, 512, 64, torch.bfloat16),
])
def test_matmul_allreduce(world, m, n, k, dtype):
    rt = _rt()
    if dtype == torch.float16:
        a, b = inputs.matmul_allreduce_inputs(world, m, k, n, dtype)
    else:
        # bf16 partials carry 8 bits: use the activation x weight magnitudes of the bf16 configurations
        a, b = inputs.matmul_reduce_scatter_inputs(world, m, k, n, dtype)
    partials = [dense.matmul_fp32(x, y) for x, y in zip(a, b)]
    outs = _run_emulated(rt.MATMUL_ALLREDUCE, world, a, b, (m, n), m, k, n, 0, dtype)
    for r in range(world):
        assert_reduced_close(outs[r], partials, k, TOL, f"mmar rank {r}")
    # every rank must hold bit-identical results (deterministic reduction, then broadcast)
    for r in range(1, world):
        assert torch.equal(outs[0], outs[r])


@pytest.mark.parametrize("comm_name,world,m,n,k,dtype", [
    ("mmar", 2, 512, 2048, 1024, torch.float16),
    ("mmar", 8, 512, 512, 256, torch.bfloat16),
    ("mmrs", 4, 512, 512, 2048, torch.bfloat16),
])
def test_reduce_ops_with_the_reference_data_model(comm_name, world, m, n, k, dtype):
    """The reference's generator gives every rank the same A and B (examples/utils/gen_data.py:42-51);
    on such data the reference's own gate has to pass strictly."""
    rt = _rt()
    a1, b1 = inputs.matmul_allreduce_inputs(1, m, k, n, dtype)
    a, b = a1 * world, b1 * world
    gold = dense.golden_matmul_allreduce(a, b)
    if comm_name == "mmar":
        outs = _run_emulated(rt.MATMUL_ALLREDUCE, world, a, b, (m, n), m, k, n, 0, dtype)
        golds = [gold] * world
    else:
        outs = _run_emulated(rt.MATMUL_REDUCE_SCATTER, world, a, b, (m // world, n), m, k, n, 0, dtype)
        golds = dense.golden_matmul_reduce_scatter(a, b)
    for r in range(world):
        assert_close_to_golden(outs[r], golds[r], k, TOL, f"{comm_name} rank {r}", strict_reference=True)


def test_bounded_wait_reports_and_context_survives():
    """A wait on a flag that nothing sets runs out, the status words say where, and the context
    keeps working."""
    import ctypes
    rt = _rt()
    from catccos_b200 import lib
    with rt.emulated_team(1, 1 << 20):
        assert lib().catccos_debug_wait_unset_flag(ctypes.c_void_p(torch.cuda.current_stream().cuda_stream), 50) == 0
        rc, words = rt.last_status()
        assert rc == 6 and words[0] == 1 and words[1] == 10, (rc, words)
        assert lib().catccos_reset_status() == 0
        rc, words = rt.last_status()
        assert rc == 0
        x = torch.ones(4, device="cuda")
        assert float(x.sum()) == 4.0


def test_partials_beyond_the_fp16_exchange_range_are_reported(monkeypatch):
    """The reduce family sends its partial tiles as fp16 (11-bit mantissa) by default.  A partial
    product beyond 65504 does not fit: the launch finishes, the status words say so
    (CATCCOS_ERR_RANGE), and CATCCOS_RS_EXCHANGE=native, which sends partials in the bf16 output
    type as the reference does, computes the same operator correctly."""
    from catccos_b200 import lib
    rt = _rt()
    world, m, n, k = 2, 512, 256, 128
    a = [torch.full((m, k), 300.0, dtype=torch.bfloat16) for _ in range(world)]
    b = [torch.full((k, n), 100.0 + r, dtype=torch.bfloat16) for r in range(world)]     # partials of about 3.8e6
    gold = dense.golden_matmul_reduce_scatter(a, b)
    til = rt.tiling(m, k, n, world)
    need = rt.symmetric_bytes(rt.MATMUL_REDUCE_SCATTER, rt.BF16, til)

    def run():
        with rt.emulated_team(world, max(need, 1 << 20)):
            symm = rt.shmem_malloc(max(need, 1024))
            c_d = [torch.zeros((m // world, n), dtype=torch.bfloat16, device="cuda") for _ in range(world)]
            rt.launch_emulated(rt.MATMUL_REDUCE_SCATTER, [dev(x) for x in a], [dev(x) for x in b], c_d, symm, til)
            rc, words = rt.last_status()
            assert lib().catccos_reset_status() == 0
            return rc, words, [c.cpu() for c in c_d]

    monkeypatch.delenv("CATCCOS_RS_EXCHANGE", raising=False)
    rc, words, _ = run()
    assert rc == 7 and words[0] == 5, (rc, words)
    assert b"fp16 range" in lib().catccos_last_error()
    monkeypatch.setenv("CATCCOS_RS_EXCHANGE", "native")
    rc, words, outs = run()
    assert rc == 0, words
    for r in range(world):
        assert_close_to_golden(outs[r], gold[r], k, TOL, f"native exchange rank {r}")
