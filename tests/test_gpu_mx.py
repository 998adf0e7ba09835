"""MX quantisation (bit-exact) and the MXFP8 AllGather-Matmul (tolerance 2e-2) against the CPU
oracle, through the C-ABI."""
import ctypes
import os

import numpy as np
import pytest
import torch

from oracle import dense, mxquant
from tests.gpu_util import dev

pytestmark = pytest.mark.gpu
TOL_MX = 2e-2


def _quant_gpu(x_bf16):
    from catccos_b200 import lib, check
    rows, k = x_bf16.shape
    nb = k // 32
    xd = x_bf16.cuda().contiguous()
    codes = torch.zeros((rows, k), dtype=torch.uint8, device="cuda")
    scales = torch.zeros((rows, (nb + 1) // 2 * 2), dtype=torch.uint8, device="cuda")
    atoms = torch.zeros(lib().catccos_sf_atoms_bytes(rows, k), dtype=torch.uint8, device="cuda")
    check(lib().catccos_mx_quant(ctypes.c_void_p(torch.cuda.current_stream().cuda_stream), ctypes.c_void_p(xd.data_ptr()),
                                 ctypes.c_void_p(codes.data_ptr()), ctypes.c_void_p(scales.data_ptr()),
                                 ctypes.c_void_p(atoms.data_ptr()), rows, k))
    torch.cuda.synchronize()
    return codes.cpu().numpy(), scales.cpu().numpy(), atoms.cpu().numpy()


def _atoms_ref(scales, rows, k):
    nb = k // 32
    kb4 = (k + 127) // 128
    out = np.full(((rows + 127) // 128) * kb4 * 512, 127, dtype=np.uint8)
    r, kb = np.meshgrid(np.arange(rows), np.arange(nb), indexing="ij")
    off = ((r >> 7) * kb4 + (kb >> 2)) * 512 + (r & 31) * 16 + ((r >> 5) & 3) * 4 + (kb & 3)
    out[off.reshape(-1)] = scales[:, :nb].reshape(-1)
    return out


def test_mx_quant_bit_exact_on_reference_fixture(golden_dir):
    f = np.load(os.path.join(golden_dir, "mx_quant.npz"))
    x = torch.from_numpy(f["x"]).to(torch.bfloat16)          # fixture values are bf16-exact
    codes, scales, atoms = _quant_gpu(x)
    assert np.array_equal(codes, f["native_codes"])           # the reference's own RNE output
    assert np.array_equal(scales, f["native_scale"])
    assert np.array_equal(atoms, _atoms_ref(scales, *x.shape))


@pytest.mark.parametrize("rows,k,std", [(256, 7168, 1.0), (1000, 2048, 0.02), (33, 96, 30.0), (4096, 1024, 1.0)])
def test_mx_quant_bit_exact_random(rows, k, std):
    g = torch.Generator().manual_seed(rows + k)
    x = (torch.randn((rows, k), generator=g) * std).to(torch.bfloat16)
    x[0, :32] = 0
    x[1, 5] = float("inf")
    x[2, 7] = float("nan")
    x[3, :64] = 1e-20
    codes, scales, atoms = _quant_gpu(x)
    rc, rs, _ = mxquant.quantize_mx_e4m3(x.to(torch.float32).numpy(), "rne")
    assert np.array_equal(scales, rs)
    assert np.array_equal(codes, rc)
    assert np.array_equal(atoms, _atoms_ref(scales, rows, k))


def _mx_inputs(world, m, k, n, trans_b):
    a_codes, a_scales, b_codes, b_scales_kn, b_dev, bs_dev = [], [], [], [], [], []
    for r in range(world):
        g = torch.Generator().manual_seed(50 + r)
        act = torch.randn((m, k), generator=g).to(torch.bfloat16).to(torch.float32).numpy()
        w = (torch.randn((k, n), generator=g) * 0.02).to(torch.bfloat16).to(torch.float32).numpy()
        ac, asc, _ = mxquant.quantize_mx_e4m3(act, "rne")
        bc, bsc, _ = mxquant.quantize_mx_e4m3_axis0(w, "rne")         # codes [k,n], scales [even(k/32), n]
        a_codes.append(ac); a_scales.append(asc); b_codes.append(bc); b_scales_kn.append(bsc)
        if trans_b:
            b_dev.append(np.ascontiguousarray(bc.T))                   # [n, k]
            bs_dev.append(np.ascontiguousarray(bsc.T))                 # [n, even(k/32)]
        else:
            b_dev.append(bc)                                           # [k, n]
            bs_dev.append(np.ascontiguousarray(bsc.reshape(bsc.shape[0] // 2, 2, n).transpose(0, 2, 1)))  # [k/64, n, 2]
    return a_codes, a_scales, b_codes, b_scales_kn, b_dev, bs_dev


@pytest.mark.parametrize("world", [1, 2, 4])
@pytest.mark.parametrize("trans_b", [0, 1])
@pytest.mark.parametrize("m,n,k,out", [(128, 256, 128, torch.bfloat16), (320, 384, 448, torch.bfloat16),
                                        (256, 512, 1024, torch.float16)])
def test_mx_allgather_matmul(world, trans_b, m, n, k, out):
    from catccos_b200 import runtime as rt, lib
    a_codes, a_scales, b_codes, b_scales_kn, b_dev, bs_dev = _mx_inputs(world, m, k, n, trans_b)
    gold = dense.golden_mx_allgather_matmul(a_codes, a_scales, b_codes, b_scales_kn)
    til = rt.tiling(m, k, n, world)
    code = rt.BF16 if out == torch.bfloat16 else rt.FP16
    need = rt.symmetric_bytes(rt.FP8_MX_ALLGATHER_MATMUL, code, til)
    ws_bytes = lib().catccos_workspace_bytes(rt.FP8_MX_ALLGATHER_MATMUL, code, ctypes.byref(til))
    with rt.emulated_team(world, max(need, 1 << 20)):
        symm = rt.shmem_malloc(max(need, 1024))
        a_d = [dev(torch.from_numpy(x)) for x in a_codes]
        b_d = [dev(torch.from_numpy(x)) for x in b_dev]
        as_d = [dev(torch.from_numpy(x)) for x in a_scales]
        bs_d = [dev(torch.from_numpy(x)) for x in bs_dev]
        c_d = [torch.full((world * m, n), float("nan"), dtype=out, device="cuda") for _ in range(world)]
        ws = [torch.zeros(ws_bytes, dtype=torch.uint8, device="cuda") for _ in range(world)]
        for _ in range(2):
            rt.launch_emulated(rt.FP8_MX_ALLGATHER_MATMUL, a_d, b_d, c_d, symm, til, trans_b=trans_b, dtype=code,
                               custom_lists=[[as_d[r], bs_d[r]] for r in range(world)], workspaces=ws)
        rc, words = rt.last_status()
        assert rc == 0, words
        outs = [c.cpu() for c in c_d]
    from oracle import verify
    for r in range(world):
        err = verify.max_rel_err(outs[r], gold[r])
        assert err <= TOL_MX, f"rank {r}: max relative error {err}"


@pytest.mark.parametrize("world", [1, 2, 4, 8])
@pytest.mark.parametrize("m,n", [(128, 256), (200, 7168), (64, 96)])
def test_mx_quant_allgather_bit_exact(world, m, n):
    """MxQuantAllGather: every rank ends with all ranks' codes and scales, byte for byte as the golden
    (the reference compares these outputs bytewise: examples/ascend950_mx_quant_allgather/scripts/run.sh)."""
    from catccos_b200 import runtime as rt
    if world > 1 and (m * n) % 16:
        pytest.skip("rows per rank not a multiple of 16 bytes")
    xs = [(torch.randn((m, n), generator=torch.Generator().manual_seed(900 + r)) * (0.5 + r)).to(torch.bfloat16)
          for r in range(world)]
    gold_c, gold_s = [], []
    for x in xs:
        c, s, _ = mxquant.quantize_mx_e4m3(x.to(torch.float32).numpy(), "rne")
        gold_c.append(c); gold_s.append(s)
    gold_c, gold_s = np.concatenate(gold_c), np.concatenate(gold_s)
    sld = gold_s.shape[1]
    if world > 1 and (m * sld) % 16:
        pytest.skip("scale rows per rank not a multiple of 16 bytes")
    til = rt.tiling(m, 1, n, world)
    need = rt.symmetric_bytes(rt.MX_QUANT_ALLGATHER, rt.FP8E4M3FN, til)
    with rt.emulated_team(world, max(need, 1 << 20)):
        symm = rt.shmem_malloc(max(need, 1024))
        x_d = [dev(x) for x in xs]
        s_d = [torch.zeros((world * m, sld), dtype=torch.uint8, device="cuda") for _ in range(world)]
        c_d = [torch.zeros((world * m, n), dtype=torch.uint8, device="cuda") for _ in range(world)]
        for _ in range(2):
            rt.launch_emulated(rt.MX_QUANT_ALLGATHER, x_d, s_d, c_d, symm, til, dtype=rt.FP8E4M3FN)
        rc, words = rt.last_status()
        assert rc == 0, words
        for r in range(world):
            assert np.array_equal(c_d[r].cpu().numpy(), gold_c), f"codes on rank {r}"
            assert np.array_equal(s_d[r].cpu().numpy(), gold_s), f"scales on rank {r}"
