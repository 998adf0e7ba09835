"""Block-scaled FP4 GEMM (MXFP4 as in the reference's FP4 operators, and NVFP4) against the CPU oracle,
max relative error 5e-2 normalised by max(1, |golden|)."""
import ctypes
import os

import numpy as np
import pytest
import torch

from oracle import mxquant, verify

pytestmark = pytest.mark.gpu
TOL_FP4 = 5e-2


def _run(fmt, packed_a, scale_a, packed_bt, scale_bt, alpha, m, n, k, out=torch.bfloat16):
    from catccos_b200 import lib, check
    dev = lambda x: torch.from_numpy(np.ascontiguousarray(x)).cuda()
    a, b, sa, sb = dev(packed_a), dev(packed_bt), dev(scale_a), dev(scale_bt)
    c = torch.full((m, n), float("nan"), dtype=out, device="cuda")
    ws = torch.zeros(lib().catccos_fp4_gemm_workspace_bytes(fmt, m, n, k), dtype=torch.uint8, device="cuda")
    code = 27 if out == torch.bfloat16 else 1
    check(lib().catccos_fp4_gemm(ctypes.c_void_p(torch.cuda.current_stream().cuda_stream), fmt, code,
                                 ctypes.c_void_p(a.data_ptr()), ctypes.c_void_p(b.data_ptr()), ctypes.c_void_p(c.data_ptr()),
                                 ctypes.c_void_p(sa.data_ptr()), ctypes.c_void_p(sb.data_ptr()), ctypes.c_float(alpha), m, n, k,
                                 ctypes.c_void_p(ws.data_ptr()), 0))
    torch.cuda.synchronize()
    return c.cpu()


def test_mxfp4_on_the_reference_fixture(golden_dir):
    f = np.load(os.path.join(golden_dir, "fp4_agmm.npz"))
    world, m, n, k = [int(v) for v in f["shape"]]
    for r in range(world):
        out = _run(0, f[f"a{r}"], f[f"a_scale{r}"], f[f"b{r}"], f[f"b_scale{r}"], 1.0, m, n, k)
        gold = torch.from_numpy(f[f"golden{r}"][r * m:(r + 1) * m])          # rank r's own rows of its gathered product
        assert verify.max_rel_err(out, gold) <= TOL_FP4


@pytest.mark.parametrize("m,n,k", [(128, 256, 256), (200, 264, 320), (1024, 2048, 4096)])
def test_mxfp4_random(m, n, k):
    g = torch.Generator().manual_seed(m + n + k)
    a = torch.randn((m, k), generator=g).numpy()
    bt = (torch.randn((n, k), generator=g) * 0.05).numpy()
    _, pa, sa, da = mxquant.quantize_mx_e2m1(a)
    _, pb, sb, db = mxquant.quantize_mx_e2m1(bt)
    gold = torch.from_numpy(da) @ torch.from_numpy(db).T
    out = _run(0, pa, sa, pb, sb, 1.0, m, n, k)
    assert verify.max_rel_err(out, gold) <= TOL_FP4


@pytest.mark.parametrize("m,n,k,out", [(128, 256, 256, torch.bfloat16), (200, 264, 320, torch.float16),
                                       (1024, 2048, 4096, torch.bfloat16)])
def test_nvfp4_random(m, n, k, out):
    g = torch.Generator().manual_seed(7 * m + n + k)
    a = torch.randn((m, k), generator=g).numpy()
    bt = (torch.randn((n, k), generator=g) * 0.05).numpy()
    _, pa, sa, ta, da = mxquant.quantize_nvfp4(a)
    _, pb, sb, tb, db = mxquant.quantize_nvfp4(bt)
    gold = torch.from_numpy(da) @ torch.from_numpy(db).T
    got = _run(1, pa, sa, pb, sb, float(ta) * float(tb), m, n, k, out)
    assert verify.max_rel_err(got, gold) <= TOL_FP4
