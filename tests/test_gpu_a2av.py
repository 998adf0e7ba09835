"""Standalone MXFP8 AllToAllV-GroupedMatmul and GroupedMatmul-AllToAllV through the C-ABI against the
reference's own generator output (tests/golden/alltoallv_gmm.npz) and against the CPU oracle on
larger random cases; world sizes 2/4/8 as emulated PEs.  Tolerance 2e-2 (MXFP8)."""
import ctypes
import os

import numpy as np
import pytest
import torch

from oracle import moe, mxquant, verify

pytestmark = pytest.mark.gpu
TOL_MX = 2e-2


def _run(comm, world, m, n, k, experts, a_codes, a_scales, b_codes, b_scales, local_tokens, out_dtype=torch.float16):
    """One emulated launch (twice, for flag epochs); returns every rank's [world*m, n] output as fp32."""
    from catccos_b200 import runtime as rt, lib
    til = rt.tiling(m, k, n, world, expertNum=experts, epSize=world)
    code = rt.FP16 if out_dtype == torch.float16 else rt.BF16
    need = rt.symmetric_bytes(comm, code, til)
    ws_bytes = lib().catccos_workspace_bytes(comm, code, ctypes.byref(til))
    assert need > 0 and ws_bytes > 0
    dev = lambda x: torch.from_numpy(np.ascontiguousarray(x)).cuda()
    with rt.emulated_team(world, need + (1 << 20)):
        symm = rt.shmem_malloc(need)
        a_d = [dev(x) for x in a_codes]
        b_d = [dev(x) for x in b_codes]
        as_d = [dev(x) for x in a_scales]
        bs_d = [dev(x) for x in b_scales]
        lt_d = [dev(np.asarray(x, dtype=np.int32)) for x in local_tokens]
        gt_d = [torch.zeros(world * (experts // world), dtype=torch.int32, device="cuda") for _ in range(world)]
        c_d = [torch.full((world * m, n), float("nan"), dtype=out_dtype, device="cuda") for _ in range(world)]
        ws = [torch.zeros(ws_bytes, dtype=torch.uint8, device="cuda") for _ in range(world)]
        for _ in range(2):
            rt.launch_emulated(comm, a_d, b_d, c_d, symm, til, dtype=code,
                               custom_lists=[[as_d[r], bs_d[r], lt_d[r], gt_d[r]] for r in range(world)], workspaces=ws)
        rc, words = rt.last_status()
        assert rc == 0, words
        return [c.cpu().to(torch.float32) for c in c_d]


def _check(out, gold_rows, what):
    rows = gold_rows.shape[0]
    err = verify.max_rel_err(out[:rows], torch.from_numpy(np.ascontiguousarray(gold_rows)))
    assert err <= TOL_MX, f"{what}: max relative error {err}"
    assert not out[rows:].any(), f"{what}: rows past the real count must stay zero"


def test_alltoallv_grouped_matmul_on_the_reference_fixture(golden_dir):
    from catccos_b200 import runtime as rt
    f = np.load(os.path.join(golden_dir, "alltoallv_gmm.npz"))
    world, m, n, k, experts = [int(v) for v in f["shape"]]
    outs = _run(rt.FP8_MX_ALLTOALLV_GROUPED_MATMUL, world, m, n, k, experts,
                [f[f"d_a{r}"] for r in range(world)], [f[f"d_a_scale{r}"].reshape(m, -1) for r in range(world)],
                [f[f"d_b{r}"] for r in range(world)], [f[f"d_b_scale{r}"] for r in range(world)],
                [f[f"d_local_tokens{r}"] for r in range(world)])
    for r in range(world):
        rows = int(f[f"d_global_tokens{r}"].sum())
        _check(outs[r], f[f"d_golden{r}"][:rows], f"dispatch-GMM rank {r}")


def test_grouped_matmul_alltoallv_on_the_reference_fixture(golden_dir):
    from catccos_b200 import runtime as rt
    f = np.load(os.path.join(golden_dir, "alltoallv_gmm.npz"))
    world, _, n, k, experts = [int(v) for v in f["shape"]]
    m = int(f["c_m"][0])
    outs = _run(rt.FP8_MX_GROUPED_MATMUL_ALLTOALLV, world, m, n, k, experts,
                [f[f"c_a{r}"] for r in range(world)], [f[f"c_a_scale{r}"].reshape(m, -1) for r in range(world)],
                [f[f"c_b{r}"] for r in range(world)], [f[f"c_b_scale{r}"] for r in range(world)],
                [f[f"c_local_tokens{r}"] for r in range(world)])
    for r in range(world):
        rows = int(f[f"c_local_tokens{r}"].sum())
        _check(outs[r], f[f"c_golden{r}"][:rows], f"GMM-combine rank {r}")


def _random_case(world, m, n, k, experts, seed):
    """Seeded operands in the operators' own layouts plus their dequantised fp32 twins."""
    rng = np.random.default_rng(seed)
    epr = experts // world
    counts = np.zeros((world, experts), dtype=np.int32)
    for r in range(world):
        w = rng.dirichlet(np.full(experts, 0.6))
        c = np.floor(w * m).astype(np.int32)
        c[rng.integers(0, experts)] += m - int(c.sum()) - int(rng.integers(0, 3))      # up to 2 rows unused
        counts[r] = np.maximum(c, 0)
    b_codes, b_scales, w_deq = [], [], []
    for r in range(world):
        cs, ss, ds = [], [], []
        for le in range(epr):
            w = (rng.standard_normal((k, n)) * 0.05).astype(np.float32)
            c, s, d = mxquant.quantize_mx_e4m3_axis0(w, "rne")                 # codes [k, n], scales [k/32(+pad), n]
            cs.append(c)
            ss.append(np.ascontiguousarray(s[:k // 32].reshape(k // 64, 2, n).transpose(0, 2, 1)))   # [k/64, n, 2]
            ds.append(d)
        b_codes.append(np.stack(cs)); b_scales.append(np.stack(ss)); w_deq.append(ds)
    return counts, b_codes, b_scales, w_deq


@pytest.mark.parametrize("world,m,n,k,experts,out", [(2, 300, 272, 320, 4, torch.bfloat16), (4, 520, 1024, 512, 8, torch.float16),
                                                      (8, 200, 256, 192, 32, torch.bfloat16)])
def test_alltoallv_grouped_matmul_random(world, m, n, k, experts, out):
    from catccos_b200 import runtime as rt
    counts, b_codes, b_scales, w_deq = _random_case(world, m, n, k, experts, 11 + world)
    rng = np.random.default_rng(99)
    a_codes, a_scales, a_deq = [], [], []
    for r in range(world):
        x = rng.standard_normal((m, k)).astype(np.float32)
        c, s, d = mxquant.quantize_mx_e4m3(x, "rne")
        a_codes.append(c); a_scales.append(s[:, :k // 32].copy()); a_deq.append(d)
    gold, blocks = moe.alltoallv_grouped_matmul(a_deq, w_deq, counts, world, experts // world)
    outs = _run(rt.FP8_MX_ALLTOALLV_GROUPED_MATMUL, world, m, n, k, experts, a_codes, a_scales, b_codes, b_scales,
                list(counts), out)
    for r in range(world):
        assert gold[r].shape[0] == sum(blocks[r])
        _check(outs[r], gold[r], f"dispatch-GMM rank {r}")


@pytest.mark.parametrize("world,m,n,k,experts,out", [(2, 300, 272, 320, 4, torch.float16), (4, 520, 1024, 512, 8, torch.bfloat16),
                                                      (8, 200, 256, 192, 32, torch.float16)])
def test_grouped_matmul_alltoallv_random(world, m, n, k, experts, out):
    from catccos_b200 import runtime as rt
    epr = experts // world
    counts, b_codes, b_scales, w_deq = _random_case(world, m // world, n, k, experts, 23 + world)   # rows every rank contributes
    rng = np.random.default_rng(7)
    a_codes, a_scales, a_deq = [], [], []
    for o in range(world):
        held = int(counts[:, o * epr:(o + 1) * epr].sum())        # rows owner o holds (local expert major, source minor)
        assert held <= m
        x = rng.standard_normal((m, k)).astype(np.float32)
        c, s, d = mxquant.quantize_mx_e4m3(x, "rne")
        a_codes.append(c); a_scales.append(s[:, :k // 32].copy()); a_deq.append(d)
    gold = moe.grouped_matmul_alltoallv(a_deq, w_deq, counts, world, epr)
    outs = _run(rt.FP8_MX_GROUPED_MATMUL_ALLTOALLV, world, m, n, k, experts, a_codes, a_scales, b_codes, b_scales,
                list(counts), out)
    for r in range(world):
        assert gold[r].shape[0] == int(counts[r].sum())
        _check(outs[r], gold[r], f"GMM-combine rank {r}")


def test_argument_errors():
    from catccos_b200 import runtime as rt, CatccosError
    world, m, n, k, experts = 2, 64, 64, 96, 4                      # k % 64 != 0
    z = lambda *s: np.zeros(s, dtype=np.uint8)
    with pytest.raises(CatccosError, match="k % 64"):
        _run(rt.FP8_MX_ALLTOALLV_GROUPED_MATMUL, world, m, n, k, experts, [z(m, k)] * 2, [z(m, k // 32)] * 2,
             [z(2, k, n)] * 2, [z(2, 2, n, 2)] * 2, [np.zeros(experts, np.int32)] * 2)


# ---- MXFP4 forms (Ascend950Fp4MxAllToAllVGroupedMatmul / Ascend950Fp4MxGroupedMatmulAllToAllV), tolerance 5e-2 ----
TOL_FP4 = 5e-2


def _fp4_case(world, rows, n, k, experts, seed):
    rng = np.random.default_rng(seed)
    epr = experts // world
    counts = np.zeros((world, experts), dtype=np.int32)
    for r in range(world):
        w = rng.dirichlet(np.full(experts, 0.6))
        c = np.floor(w * rows).astype(np.int32)
        c[rng.integers(0, experts)] += rows - int(c.sum()) - int(rng.integers(0, 3))
        counts[r] = np.maximum(c, 0)
    b_codes, b_scales, w_deq = [], [], []
    for r in range(world):
        cs, ss, ds = [], [], []
        for le in range(epr):
            wt = (rng.standard_normal((n, k)) * 0.05).astype(np.float32)          # K-major weights [n, k]
            _, pk, sc, dq = mxquant.quantize_mx_e2m1(wt)
            cs.append(pk); ss.append(sc[:, :k // 32].copy()); ds.append(np.ascontiguousarray(dq.T))
        b_codes.append(np.stack(cs)); b_scales.append(np.stack(ss)); w_deq.append(ds)
    return rng, counts, b_codes, b_scales, w_deq


def _check_fp4(out, gold_rows, what):
    rows = gold_rows.shape[0]
    err = verify.max_rel_err(out[:rows], torch.from_numpy(np.ascontiguousarray(gold_rows)))
    assert err <= TOL_FP4, f"{what}: max relative error {err}"
    assert not out[rows:].any(), f"{what}: rows past the real count must stay zero"


@pytest.mark.parametrize("world,m,n,k,experts,out", [(2, 300, 272, 256, 4, torch.bfloat16), (4, 520, 1024, 512, 8, torch.float16),
                                                      (8, 200, 256, 768, 32, torch.bfloat16)])
def test_fp4_alltoallv_grouped_matmul_random(world, m, n, k, experts, out):
    from catccos_b200 import runtime as rt
    rng, counts, b_codes, b_scales, w_deq = _fp4_case(world, m, n, k, experts, 311 + world)
    a_codes, a_scales, a_deq = [], [], []
    for r in range(world):
        _, pk, sc, dq = mxquant.quantize_mx_e2m1(rng.standard_normal((m, k)).astype(np.float32))
        a_codes.append(pk); a_scales.append(sc[:, :k // 32].copy()); a_deq.append(dq)
    gold, blocks = moe.alltoallv_grouped_matmul(a_deq, w_deq, counts, world, experts // world)
    outs = _run(rt.FP4_MX_ALLTOALLV_GROUPED_MATMUL, world, m, n, k, experts, a_codes, a_scales, b_codes, b_scales,
                list(counts), out)
    for r in range(world):
        assert gold[r].shape[0] == sum(blocks[r])
        _check_fp4(outs[r], gold[r], f"fp4 dispatch-GMM rank {r}")


@pytest.mark.parametrize("world,m,n,k,experts,out", [(2, 300, 272, 256, 4, torch.float16), (4, 520, 1024, 512, 8, torch.bfloat16),
                                                      (8, 200, 256, 768, 32, torch.float16)])
def test_fp4_grouped_matmul_alltoallv_random(world, m, n, k, experts, out):
    from catccos_b200 import runtime as rt
    epr = experts // world
    rng, counts, b_codes, b_scales, w_deq = _fp4_case(world, m // world, n, k, experts, 523 + world)
    a_codes, a_scales, a_deq = [], [], []
    for o in range(world):
        assert int(counts[:, o * epr:(o + 1) * epr].sum()) <= m
        _, pk, sc, dq = mxquant.quantize_mx_e2m1(rng.standard_normal((m, k)).astype(np.float32))
        a_codes.append(pk); a_scales.append(sc[:, :k // 32].copy()); a_deq.append(dq)
    gold = moe.grouped_matmul_alltoallv(a_deq, w_deq, counts, world, epr)
    outs = _run(rt.FP4_MX_GROUPED_MATMUL_ALLTOALLV, world, m, n, k, experts, a_codes, a_scales, b_codes, b_scales,
                list(counts), out)
    for r in range(world):
        assert gold[r].shape[0] == int(counts[r].sum())
        _check_fp4(outs[r], gold[r], f"fp4 GMM-combine rank {r}")


def test_fp4_needs_k_multiple_of_256():
    from catccos_b200 import runtime as rt, CatccosError
    world, m, n, k, experts = 2, 64, 64, 320, 4
    z = lambda *s: np.zeros(s, dtype=np.uint8)
    with pytest.raises(CatccosError, match="k % 256"):
        _run(rt.FP4_MX_ALLTOALLV_GROUPED_MATMUL, world, m, n, k, experts, [z(m, k // 2)] * 2, [z(m, k // 32)] * 2,
             [z(2, n, k // 2)] * 2, [z(2, n, k // 32)] * 2, [np.zeros(experts, np.int32)] * 2)
