"""MXFP8 Matmul-ReduceScatter (e5m2 codes, as the reference's example feeds; tolerance 2e-2)
against the CPU oracle, through the C-ABI, world sizes 1/2/4 as emulated PEs."""
import ctypes
import os

import numpy as np
import pytest
import torch

from oracle import dense, mxquant
from tests.gpu_util import assert_reduced_close, dev

pytestmark = pytest.mark.gpu
TOL_MX = 2e-2


def _inputs(world, m, k, n, trans_b):
    a_codes, a_scales, b_codes, b_scales, b_dev, bs_dev = [], [], [], [], [], []
    for r in range(world):
        g = torch.Generator().manual_seed(700 + r)
        act = torch.randn((m, k), generator=g).numpy()
        w = (torch.randn((k, n), generator=g) * 0.02).numpy()
        ac, asc, _ = mxquant.quantize_mx_e5m2(act)
        bct, bsct, _ = mxquant.quantize_mx_e5m2(np.ascontiguousarray(w.T))      # blocks along k: [n, k], [n, even(k/32)]
        bc, bsc = np.ascontiguousarray(bct.T), np.ascontiguousarray(bsct.T)       # [k, n], [even(k/32), n]
        a_codes.append(ac); a_scales.append(asc); b_codes.append(bc); b_scales.append(bsc)
        if trans_b:
            b_dev.append(bct)
            bs_dev.append(bsct)
        else:
            b_dev.append(bc)
            bs_dev.append(np.ascontiguousarray(bsc.reshape(bsc.shape[0] // 2, 2, n).transpose(0, 2, 1)))   # [k/64, n, 2]
    return a_codes, a_scales, b_codes, b_scales, b_dev, bs_dev


@pytest.mark.parametrize("world", [1, 2, 4])
@pytest.mark.parametrize("trans_b", [1, 0])
@pytest.mark.parametrize("rows_per_rank,n,k,out", [(128, 256, 128, torch.bfloat16), (256, 520, 448, torch.bfloat16),
                                                    (384, 1024, 1024, torch.float16)])
def test_mx_matmul_reduce_scatter(world, trans_b, rows_per_rank, n, k, out):
    from catccos_b200 import runtime as rt, lib
    if n % 16:
        n = n // 16 * 16
    m = rows_per_rank * world
    a_codes, a_scales, b_codes, b_scales, b_dev, bs_dev = _inputs(world, m, k, n, trans_b)
    partials = []
    for r in range(world):
        a = mxquant.dequant_mx(a_codes[r], a_scales[r], "e5m2")
        b = mxquant.dequant_mx(np.ascontiguousarray(b_codes[r].T), np.ascontiguousarray(b_scales[r].T), "e5m2").T
        partials.append(torch.from_numpy(a) @ torch.from_numpy(np.ascontiguousarray(b)))
    gold = dense.golden_mx_matmul_reduce_scatter(a_codes, a_scales, b_codes, b_scales, "e5m2")
    til = rt.tiling(m, k, n, world)
    code = rt.BF16 if out == torch.bfloat16 else rt.FP16
    need = rt.symmetric_bytes(rt.MXFP8_MATMUL_REDUCE_SCATTER, code, til)
    ws_bytes = lib().catccos_workspace_bytes(rt.MXFP8_MATMUL_REDUCE_SCATTER, code, ctypes.byref(til))
    with rt.emulated_team(world, max(need, 1 << 20)):
        symm = rt.shmem_malloc(max(need, 1024))
        a_d = [dev(torch.from_numpy(x)) for x in a_codes]
        b_d = [dev(torch.from_numpy(x)) for x in b_dev]
        as_d = [dev(torch.from_numpy(x)) for x in a_scales]
        bs_d = [dev(torch.from_numpy(x)) for x in bs_dev]
        c_d = [torch.full((rows_per_rank, n), float("nan"), dtype=out, device="cuda") for _ in range(world)]
        ws = [torch.zeros(ws_bytes, dtype=torch.uint8, device="cuda") for _ in range(world)]
        for _ in range(2):
            rt.launch_emulated(rt.MXFP8_MATMUL_REDUCE_SCATTER, a_d, b_d, c_d, symm, til, trans_b=trans_b, dtype=code,
                               custom_lists=[[as_d[r], bs_d[r]] for r in range(world)], workspaces=ws)
        rc, words = rt.last_status()
        assert rc == 0, words
        outs = [c.cpu() for c in c_d]
    for r in range(world):
        rows = slice(r * rows_per_rank, (r + 1) * rows_per_rank)
        assert torch.allclose(sum(p[rows] for p in partials), gold[r], rtol=1e-5, atol=1e-4)
        assert_reduced_close(outs[r], [p[rows] for p in partials], k, TOL_MX, f"mx mmrs rank {r}")


def test_rows_per_rank_must_be_a_multiple_of_128():
    from catccos_b200 import runtime as rt, CatccosError
    world, m, k, n = 2, 192, 128, 256
    til = rt.tiling(m, k, n, world)
    with rt.emulated_team(world, 1 << 22):
        symm = rt.shmem_malloc(1 << 20)
        z = [torch.zeros((m, k), dtype=torch.uint8, device="cuda") for _ in range(world)]
        zb = [torch.zeros((n, k), dtype=torch.uint8, device="cuda") for _ in range(world)]
        c = [torch.zeros((m // world, n), dtype=torch.bfloat16, device="cuda") for _ in range(world)]
        s = [torch.zeros((m, 4), dtype=torch.uint8, device="cuda") for _ in range(world)]
        with pytest.raises(CatccosError, match="multiple of 128"):
            rt.launch_emulated(rt.MXFP8_MATMUL_REDUCE_SCATTER, z, zb, c, symm, til, trans_b=1, dtype=rt.BF16,
                               custom_lists=[[s[r], s[r]] for r in range(world)], workspaces=s)


@pytest.mark.parametrize("world", [1, 2, 4, 8])
@pytest.mark.parametrize("trans_b,rows_per_rank,n,k,out", [(0, 128, 256, 128, torch.bfloat16), (1, 256, 528, 448, torch.float16)])
def test_mx_matmul_alltoall(world, trans_b, rows_per_rank, n, k, out):
    """MXFP8 Matmul-AllToAll (e4m3 codes): C_i = A_i x B_i on dequantised operands, row block j of every C_i on rank j
    in rank order (row-block form of examples/ascend950_mxfp8_matmul_alltoall/scripts/gen_data_slice_m.py)."""
    from catccos_b200 import runtime as rt, lib
    from oracle import verify
    m = rows_per_rank * world
    a_codes, a_scales, b_dev, bs_dev, full = [], [], [], [], []
    for r in range(world):
        g = torch.Generator().manual_seed(900 + r)
        act = torch.randn((m, k), generator=g).numpy()
        w = (torch.randn((k, n), generator=g) * 0.02).numpy()
        ac, asc, a_deq = mxquant.quantize_mx_e4m3(act, "rne")
        bct, bsct, bt_deq = mxquant.quantize_mx_e4m3(np.ascontiguousarray(w.T), "rne")     # [n, k] blocks along k
        a_codes.append(ac); a_scales.append(asc)
        if trans_b:
            b_dev.append(bct); bs_dev.append(bsct)
        else:
            bsc = np.ascontiguousarray(bsct.T)
            b_dev.append(np.ascontiguousarray(bct.T))
            bs_dev.append(np.ascontiguousarray(bsc.reshape(bsc.shape[0] // 2, 2, n).transpose(0, 2, 1)))
        full.append(torch.from_numpy(a_deq) @ torch.from_numpy(np.ascontiguousarray(bt_deq.T)))
    til = rt.tiling(m, k, n, world)
    code = rt.BF16 if out == torch.bfloat16 else rt.FP16
    need = rt.symmetric_bytes(rt.MXFP8_MATMUL_ALLTOALL, code, til)
    ws_bytes = lib().catccos_workspace_bytes(rt.MXFP8_MATMUL_ALLTOALL, code, ctypes.byref(til))
    with rt.emulated_team(world, max(need, 1 << 20)):
        symm = rt.shmem_malloc(max(need, 1024))
        a_d = [dev(torch.from_numpy(x)) for x in a_codes]
        b_d = [dev(torch.from_numpy(x)) for x in b_dev]
        as_d = [dev(torch.from_numpy(x)) for x in a_scales]
        bs_d = [dev(torch.from_numpy(x)) for x in bs_dev]
        c_d = [torch.full((m, n), float("nan"), dtype=out, device="cuda") for _ in range(world)]
        ws = [torch.zeros(ws_bytes, dtype=torch.uint8, device="cuda") for _ in range(world)]
        for _ in range(2):
            rt.launch_emulated(rt.MXFP8_MATMUL_ALLTOALL, a_d, b_d, c_d, symm, til, trans_b=trans_b, dtype=code,
                               custom_lists=[[as_d[r], bs_d[r]] for r in range(world)], workspaces=ws)
        rc, words = rt.last_status()
        assert rc == 0, words
        outs = [c.cpu().to(torch.float32) for c in c_d]
    for j in range(world):
        gold = torch.cat([full[i][j * rows_per_rank:(j + 1) * rows_per_rank] for i in range(world)], dim=0)
        err = verify.max_rel_err(outs[j], gold)
        assert err <= TOL_MX, f"mx matmul-alltoall rank {j}: {err}"
