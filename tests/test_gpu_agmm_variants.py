"""Data-flow variants of AllGather-Matmul through the C-ABI: the product against the CPU oracle, the
gathered A (gather-result variant) bit for bit against the concatenation of every rank's A.  World
sizes > 1 run as emulated PEs (all ranks inside one cooperative launch)."""
import pytest
import torch

from oracle import dense, inputs
from tests.gpu_util import assert_close_to_golden, dev

pytestmark = pytest.mark.gpu
TOL = 1e-2


def _run(comm, world, a_list, b_list, m, k, n, trans_b, dtype, gather, launches=2):
    from catccos_b200 import runtime as rt
    til = rt.tiling(m, k, n, world)
    need = rt.symmetric_bytes(comm, rt.BF16, til)
    with rt.emulated_team(world, max(need, 1 << 20)):
        symm = rt.shmem_malloc(max(need, 1024))
        b_d = [dev(b.t() if trans_b else b) for b in b_list]
        c_d = [torch.full((world * m, n), float("nan"), dtype=dtype, device="cuda") for _ in range(world)]
        g_d = [torch.full((world * m, k), float("nan"), dtype=dtype, device="cuda") for _ in range(world)] if gather else None
        for it in range(launches):
            # new values of A on every launch: what a launch leaves in the symmetric region must not leak into the next
            a_d = [dev(a if it == launches - 1 else a * 0.5) for a in a_list]
            rt.launch_emulated(comm, a_d, b_d, c_d, symm, til, trans_b=1 if trans_b else 0,
                               custom_lists=[[g] for g in g_d] if gather else None)
        rc, words = rt.last_status()
        assert rc == 0, words
        return [c.cpu() for c in c_d], ([g.cpu() for g in g_d] if gather else None)


@pytest.mark.parametrize("world", [1, 2, 4, 8])
@pytest.mark.parametrize("m_local,n,k,trans_b,dtype", [(128, 256, 128, 0, torch.bfloat16), (320, 520, 192, 1, torch.float16),
                                                        (100, 256, 64, 0, torch.bfloat16)])
def test_allgather_matmul_with_gather_result(world, m_local, n, k, trans_b, dtype):
    from catccos_b200 import runtime as rt
    a, b = inputs.allgather_matmul_inputs(world, m_local, k, n, dtype)
    gold = dense.golden_allgather_matmul(a, b)
    outs, gathered = _run(rt.ALLGATHER_MATMUL_WITH_GATHER_RESULT, world, a, b, m_local, k, n, trans_b, dtype, True)
    want = torch.cat(a, dim=0)
    for r in range(world):
        assert_close_to_golden(outs[r], gold[r], k, TOL, f"agmm+gather rank {r}")
        assert torch.equal(gathered[r].view(torch.int16), want.view(torch.int16)), f"rank {r}: gathered A differs"


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("m_local,n,k,trans_b,dtype", [(128, 256, 128, 0, torch.bfloat16), (320, 520, 192, 1, torch.float16),
                                                        (100, 256, 64, 0, torch.bfloat16), (1024, 512, 1024, 0, torch.bfloat16)])
def test_allgather_matmul_remote_read(world, m_local, n, k, trans_b, dtype):
    from catccos_b200 import runtime as rt
    if world * m_local > 4096:
        pytest.skip("one shape at world 8 is enough for the large case")
    a, b = inputs.allgather_matmul_inputs(world, m_local, k, n, dtype)
    gold = dense.golden_allgather_matmul(a, b)
    outs, _ = _run(rt.ALLGATHER_MATMUL_REMOTE_READ, world, a, b, m_local, k, n, trans_b, dtype, False, launches=3)
    for r in range(world):
        assert_close_to_golden(outs[r], gold[r], k, TOL, f"remote-read agmm rank {r}")


def test_variants_need_the_pair_kernel(monkeypatch):
    from catccos_b200 import runtime as rt, CatccosError
    monkeypatch.setenv("CATCCOS_TWO_CTA", "0")
    a, b = inputs.allgather_matmul_inputs(2, 128, 64, 256, torch.bfloat16)
    with pytest.raises(CatccosError, match="CTA-pair kernel"):
        _run(rt.ALLGATHER_MATMUL_REMOTE_READ, 2, a, b, 128, 64, 256, 0, torch.bfloat16, False)


@pytest.mark.parametrize("world", [1, 2, 4, 8])
@pytest.mark.parametrize("chunk,n,k,trans_b,dtype", [(128, 256, 128, 0, torch.bfloat16), (320, 520, 192, 1, torch.float16),
                                                      (100, 256, 64, 0, torch.bfloat16)])
def test_alltoall_matmul(world, chunk, n, k, trans_b, dtype):
    """AllToAll-Matmul: rank j ends up with block j of every rank's A (in rank order) times its own B
    (examples/ascend950_alltoall_matmul/scripts/gen_data.py:19-86)."""
    from catccos_b200 import runtime as rt
    m = chunk * world
    a, b = inputs.allgather_matmul_inputs(world, m, k, n, dtype)          # every rank: A [m, k], B [k, n]
    til = rt.tiling(m, k, n, world)
    need = rt.symmetric_bytes(rt.ALLTOALL_MATMUL, rt.BF16, til)
    with rt.emulated_team(world, max(need, 1 << 20)):
        symm = rt.shmem_malloc(max(need, 1024))
        a_d = [dev(x) for x in a]
        b_d = [dev(x.t() if trans_b else x) for x in b]
        c_d = [torch.full((m, n), float("nan"), dtype=dtype, device="cuda") for _ in range(world)]
        for _ in range(2):
            rt.launch_emulated(rt.ALLTOALL_MATMUL, a_d, b_d, c_d, symm, til, trans_b=1 if trans_b else 0)
        rc, words = rt.last_status()
        assert rc == 0, words
        outs = [c.cpu() for c in c_d]
    for j in range(world):
        assembled = torch.cat([a[i][j * chunk:(j + 1) * chunk] for i in range(world)], dim=0)
        gold = dense.matmul_fp32(assembled, b[j])
        assert_close_to_golden(outs[j], gold, k, TOL, f"alltoall-matmul rank {j}")


@pytest.mark.parametrize("world", [1, 2, 4, 8])
@pytest.mark.parametrize("chunk,n,k,trans_b,dtype", [(128, 256, 128, 0, torch.bfloat16), (320, 520, 192, 1, torch.float16),
                                                      (100, 264, 64, 0, torch.bfloat16)])
def test_matmul_alltoall(world, chunk, n, k, trans_b, dtype):
    """Matmul-AllToAll: C_i = A_i x B_i on every rank, then rank j holds row block j of every C_i in rank order
    (examples/ascend950_matmul_alltoall/scripts/gen_data.py:19-89)."""
    from catccos_b200 import runtime as rt
    m = chunk * world
    a, b = inputs.matmul_reduce_scatter_inputs(world, m, k, n, dtype)       # every rank: A [m, k], B [k, n]
    til = rt.tiling(m, k, n, world)
    need = rt.symmetric_bytes(rt.MATMUL_ALLTOALL, rt.BF16, til)
    with rt.emulated_team(world, max(need, 1 << 20)):
        symm = rt.shmem_malloc(max(need, 1024))
        a_d = [dev(x) for x in a]
        b_d = [dev(x.t() if trans_b else x) for x in b]
        c_d = [torch.full((m, n), float("nan"), dtype=dtype, device="cuda") for _ in range(world)]
        for _ in range(2):
            rt.launch_emulated(rt.MATMUL_ALLTOALL, a_d, b_d, c_d, symm, til, trans_b=1 if trans_b else 0)
        rc, words = rt.last_status()
        assert rc == 0, words
        outs = [c.cpu() for c in c_d]
    full = [dense.matmul_fp32(x, y) for x, y in zip(a, b)]
    for j in range(world):
        gold = torch.cat([full[i][j * chunk:(j + 1) * chunk] for i in range(world)], dim=0)
        assert_close_to_golden(outs[j], gold, k, TOL, f"matmul-alltoall rank {j}")
