"""Dense goldens: Matmul-AllReduce, AllGather-Matmul, Matmul-ReduceScatter.

Test infrastructure only (see package docstring).
"""
import torch


def matmul_fp32(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """fp32-accumulated product of low-precision operands.

    Follows examples/utils/gen_data.py:45-53 (`torch.matmul(a.to(float32),
    b.to(float32))`)."""
    return torch.matmul(a.to(torch.float32), b.to(torch.float32))


def golden_matmul_allreduce(a_list, b_list) -> torch.Tensor:
    """D = sum_r A_r @ B_r, fp32, identical on every rank.

    examples/utils/gen_data.py:66-70 (sum over ranks of the per-rank product)."""
    out = matmul_fp32(a_list[0], b_list[0])
    for a, b in zip(a_list[1:], b_list[1:]):
        out = out + matmul_fp32(a, b)
    return out


def golden_matmul_reduce_scatter(a_list, b_list):
    """Per-rank row block of the all-reduced product.

    examples/utils/gen_data.py:66-70 builds the summed [M,N] golden; the
    operator writes rank r's rows [r*M/R,(r+1)*M/R) at byte offset r*size
    (examples/matmul_reduce_scatter/matmul_reduce_scatter_host.h:70)."""
    full = golden_matmul_allreduce(a_list, b_list)
    r = len(a_list)
    m = full.shape[0] // r
    return [full[i * m:(i + 1) * m].contiguous() for i in range(r)]


def golden_allgather_matmul(a_list, b_list):
    """C_r = cat(A_0..A_{R-1}) @ B_r, fp32, one output per rank.

    examples/utils/gen_data_allgather_matmul.py:54-64 (per-rank distinct A and
    B); examples/utils/gen_data.py:63-65 is the same-B special case."""
    gathered = torch.cat([a.to(torch.float32) for a in a_list], dim=0)
    return [torch.matmul(gathered, b.to(torch.float32)) for b in b_list]


def golden_mx_allgather_matmul(a_codes_list, a_scales_list, b_codes_list, b_scales_list):
    """MXFP8 AllGather-Matmul golden: C_r = cat_s(dequant(A_s)) @ dequant(B_r) in fp32.

    examples/utils/gen_data_fp8_mx_allgather_matmul.py:645-669 (`matmul(allgathered_a, b_fp32)` on
    the dequantised operands).  a_codes: uint8 [m,k] with scales [m, >=k/32]; b_codes: uint8 [k,n]
    with scales [>=k/32, n] (blocks of 32 along k for both operands)."""
    import numpy as np
    from . import mxquant
    a = np.concatenate([mxquant.dequant_mx_e4m3(c, s) for c, s in zip(a_codes_list, a_scales_list)], axis=0)
    outs = []
    for bc, bs in zip(b_codes_list, b_scales_list):
        b = mxquant.dequant_mx_e4m3(np.ascontiguousarray(bc.T), np.ascontiguousarray(bs.T)).T
        outs.append(torch.matmul(torch.from_numpy(a), torch.from_numpy(np.ascontiguousarray(b))))
    return outs


def golden_mx_matmul_reduce_scatter(a_codes_list, a_scales_list, b_codes_list, b_scales_list, fmt="e5m2"):
    """MXFP8 Matmul-ReduceScatter golden: D = sum_r dequant(A_r) @ dequant(B_r) in fp32, rows
    chunked over the ranks.

    examples/ascend950_mxfp8_matmul_reduce_scatter/scripts/gen_data_mxfp8_mmrs.py:333-335 (per-rank
    `a_fp32 @ b_fp32` on the dequantised operands) and :375-385 (sum over ranks, `torch.chunk` along
    rows).  a_codes: uint8 [M,k] with scales [M, >=k/32]; b_codes: uint8 [k,N] with scales
    [>=k/32, N]; blocks of 32 along k for both; `fmt` "e5m2" (what that example feeds) or "e4m3"."""
    import numpy as np
    from . import mxquant
    total = None
    for ac, asc, bc, bsc in zip(a_codes_list, a_scales_list, b_codes_list, b_scales_list):
        a = mxquant.dequant_mx(ac, asc, fmt)
        b = mxquant.dequant_mx(np.ascontiguousarray(bc.T), np.ascontiguousarray(bsc.T), fmt).T
        c = torch.matmul(torch.from_numpy(a), torch.from_numpy(np.ascontiguousarray(b)))
        total = c if total is None else total + c
    return list(torch.chunk(total, len(a_codes_list), dim=0))


def golden_fp4_allgather_matmul(a_list, b_list):
    """FP4 AllGather-Matmul golden on operands that are already dequantised to fp32 (MXFP4:
    mxquant.dequant_mxfp4, NVFP4: mxquant.dequant_nvfp4): C_r = cat_s(A_s) @ B_r in fp32, as
    examples/utils/gen_data_fp4_mx_allgather_matmul.py:665-677 does for MXFP4.  a_list[s]: [m, k],
    b_list[r]: [k, n]."""
    import numpy as np
    gathered = torch.from_numpy(np.concatenate(a_list, axis=0))
    return [torch.matmul(gathered, torch.from_numpy(np.ascontiguousarray(b))) for b in b_list]
