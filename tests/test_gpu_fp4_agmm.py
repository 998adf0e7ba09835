"""MXFP4 AllGather-Matmul (Ascend950Fp4MxAllGatherMatmul) through the C-ABI: the reference generator's own files
(tests/golden/fp4_agmm.npz) and seeded random cases against the CPU oracle, world sizes 1/2/4/8 as emulated PEs.
Tolerance 5e-2 of max(1, |golden|) (FP4)."""
import ctypes
import os

import numpy as np
import pytest
import torch

from oracle import dense, mxquant, verify

pytestmark = pytest.mark.gpu
TOL_FP4 = 5e-2


def _run(world, m, n, k, a_codes, a_scales, b_codes, b_scales, out=torch.bfloat16, launches=2):
    """a_codes[r]: [m, k/2] packed e2m1; b_codes[r]: [n, k/2] (B^T); scales: E8M0 [rows, even(k/32)]."""
    from catccos_b200 import runtime as rt, lib
    til = rt.tiling(m, k, n, world)
    comm = rt.FP4_MX_ALLGATHER_MATMUL
    code = rt.BF16 if out == torch.bfloat16 else rt.FP16
    need = rt.symmetric_bytes(comm, code, til)
    ws_bytes = lib().catccos_workspace_bytes(comm, code, ctypes.byref(til))
    assert ws_bytes > 0
    dev = lambda x: torch.from_numpy(np.ascontiguousarray(x)).cuda()
    with rt.emulated_team(world, max(need, 1 << 20) + (1 << 20)):
        symm = rt.shmem_malloc(max(need, 1024))
        a_d, b_d = [dev(x) for x in a_codes], [dev(x) for x in b_codes]
        as_d, bs_d = [dev(x) for x in a_scales], [dev(x) for x in b_scales]
        c_d = [torch.full((world * m, n), float("nan"), dtype=out, device="cuda") for _ in range(world)]
        ws = [torch.zeros(ws_bytes, dtype=torch.uint8, device="cuda") for _ in range(world)]
        for _ in range(launches):
            rt.launch_emulated(comm, a_d, b_d, c_d, symm, til, trans_b=1, dtype=code,
                               custom_lists=[[as_d[r], bs_d[r]] for r in range(world)], workspaces=ws)
        rc, words = rt.last_status()
        assert rc == 0, words
        return [c.cpu().to(torch.float32) for c in c_d]


def test_on_the_reference_fixture(golden_dir):
    f = np.load(os.path.join(golden_dir, "fp4_agmm.npz"))
    world, m, n, k = [int(v) for v in f["shape"]]
    outs = _run(world, m, n, k, [f[f"a{r}"] for r in range(world)], [f[f"a_scale{r}"] for r in range(world)],
                [f[f"b{r}"] for r in range(world)], [f[f"b_scale{r}"] for r in range(world)])
    for r in range(world):
        err = verify.max_rel_err(outs[r], torch.from_numpy(f[f"golden{r}"]))
        assert err <= TOL_FP4, f"rank {r}: {err}"


@pytest.mark.parametrize("world,m,n,k,out", [(1, 200, 272, 320, torch.bfloat16), (2, 128, 256, 256, torch.float16),
                                             (4, 320, 528, 448, torch.bfloat16), (8, 100, 256, 64, torch.bfloat16),
                                             (2, 1024, 1024, 4096, torch.bfloat16)])
def test_random(world, m, n, k, out):
    rng = np.random.default_rng(1000 + world + m + k)
    a_codes, a_scales, a_deq, b_codes, b_scales, b_deq = [], [], [], [], [], []
    for r in range(world):
        _, pa, sa, da = mxquant.quantize_mx_e2m1(rng.standard_normal((m, k)).astype(np.float32))
        _, pb, sb, db = mxquant.quantize_mx_e2m1((rng.standard_normal((n, k)) * 0.05).astype(np.float32))
        a_codes.append(pa); a_scales.append(sa); a_deq.append(da)
        b_codes.append(pb); b_scales.append(sb); b_deq.append(np.ascontiguousarray(db.T))
    gold = dense.golden_fp4_allgather_matmul(a_deq, b_deq)
    outs = _run(world, m, n, k, a_codes, a_scales, b_codes, b_scales, out)
    for r in range(world):
        err = verify.max_rel_err(outs[r], gold[r])
        assert err <= TOL_FP4, f"rank {r}: {err}"


def test_needs_k_major_operands():
    from catccos_b200 import runtime as rt, lib, CatccosError
    til = rt.tiling(128, 128, 128, 1)
    z = lambda *s: torch.zeros(s, dtype=torch.uint8, device="cuda")
    with rt.emulated_team(1, 1 << 20):
        ws = z(lib().catccos_workspace_bytes(rt.FP4_MX_ALLGATHER_MATMUL, rt.BF16, ctypes.byref(til)))
        c = torch.zeros((128, 128), dtype=torch.bfloat16, device="cuda")
        with pytest.raises(CatccosError, match="K-major"):
            rt.launch_emulated(rt.FP4_MX_ALLGATHER_MATMUL, [z(128, 64)], [z(128, 64)], [c], rt.shmem_malloc(1024), til,
                               trans_b=0, dtype=rt.BF16, custom_lists=[[z(128, 4), z(128, 4)]], workspaces=[ws])


@pytest.mark.parametrize("world,rows_per_rank,n,k,out", [(1, 128, 256, 256, torch.bfloat16), (2, 128, 272, 320, torch.float16),
                                                         (4, 256, 528, 448, torch.bfloat16), (8, 128, 256, 64, torch.bfloat16),
                                                         (2, 512, 1024, 2048, torch.bfloat16)])
def test_mxfp4_matmul_reduce_scatter(world, rows_per_rank, n, k, out):
    """MXFP4 Matmul-ReduceScatter (Ascend950Fp4MxMatmulReduceScatter): D_r = rows r of sum_s dequant(A_s) x dequant(B_s)
    (examples/utils/gen_data_fp4_mx.py:755-818), operands K-major."""
    from catccos_b200 import runtime as rt, lib
    from tests.gpu_util import assert_reduced_close
    m = rows_per_rank * world
    rng = np.random.default_rng(2000 + world + m + k)
    a_codes, a_scales, b_codes, b_scales, partials = [], [], [], [], []
    for r in range(world):
        _, pa, sa, da = mxquant.quantize_mx_e2m1(rng.standard_normal((m, k)).astype(np.float32))
        _, pb, sb, db = mxquant.quantize_mx_e2m1((rng.standard_normal((n, k)) * 0.05).astype(np.float32))
        a_codes.append(pa); a_scales.append(sa); b_codes.append(pb); b_scales.append(sb)
        partials.append(torch.from_numpy(da) @ torch.from_numpy(np.ascontiguousarray(db.T)))
    til = rt.tiling(m, k, n, world)
    comm = rt.FP4_MX_MATMUL_REDUCE_SCATTER
    code = rt.BF16 if out == torch.bfloat16 else rt.FP16
    need = rt.symmetric_bytes(comm, code, til)
    ws_bytes = lib().catccos_workspace_bytes(comm, code, ctypes.byref(til))
    dev = lambda x: torch.from_numpy(np.ascontiguousarray(x)).cuda()
    with rt.emulated_team(world, max(need, 1 << 20) + (1 << 20)):
        symm = rt.shmem_malloc(max(need, 1024))
        a_d, b_d = [dev(x) for x in a_codes], [dev(x) for x in b_codes]
        as_d, bs_d = [dev(x) for x in a_scales], [dev(x) for x in b_scales]
        c_d = [torch.full((rows_per_rank, n), float("nan"), dtype=out, device="cuda") for _ in range(world)]
        ws = [torch.zeros(ws_bytes, dtype=torch.uint8, device="cuda") for _ in range(world)]
        for _ in range(2):
            rt.launch_emulated(comm, a_d, b_d, c_d, symm, til, trans_b=1, dtype=code,
                               custom_lists=[[as_d[r], bs_d[r]] for r in range(world)], workspaces=ws)
        rc, words = rt.last_status()
        assert rc == 0, words
        outs = [c.cpu() for c in c_d]
    for r in range(world):
        rows = slice(r * rows_per_rank, (r + 1) * rows_per_rank)
        assert_reduced_close(outs[r], [p[rows] for p in partials], k, TOL_FP4, f"mxfp4 mmrs rank {r}")
