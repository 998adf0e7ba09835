"""The allocation-free GEMM entry point (catccos_gemm_no_alloc) against the regular launcher.

For users whose code cannot allocate device memory at the call site (a plugin inside a host
runtime that owns all device memory, latency-critical loops that cannot take an allocation's
implicit synchronisation): the entry point keeps its scratch in a fixed array inside the
library.  Checked here through the C-ABI, two calls in a row, bit for bit against
catccos_launch_emulated on the same inputs (same kernel, so no tolerance is needed) and within
1e-2 of the fp32 CPU golden, plus the documented size limit.  Collected last on purpose.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _call(lib, a, b, c, m, n, k, dtype_code, trans_b, block_num=0):
    return lib.catccos_gemm_no_alloc(
        ctypes.c_void_p(torch.cuda.current_stream().cuda_stream), ctypes.c_void_p(a.data_ptr()),
        ctypes.c_void_p(b.data_ptr()), ctypes.c_void_p(c.data_ptr()), m, n, k, dtype_code, trans_b, block_num)


@pytest.mark.parametrize("dtype,trans_b", [(torch.bfloat16, 0), (torch.float16, 1)])
def test_no_alloc_gemm_matches_regular_launcher(dtype, trans_b):
    from catccos_b200 import lib, runtime as rt
    l = lib()
    m, n, k = 520, 776, 392
    g = torch.Generator().manual_seed(5)
    a = torch.randn((m, k), generator=g).to(dtype).cuda()
    b = (torch.randn((n, k) if trans_b else (k, n), generator=g) * 0.05).to(dtype).cuda()
    code = rt.BF16 if dtype == torch.bfloat16 else rt.FP16

    # two calls in a row through the new entry point (no symmetric heap exists at this point)
    outs = []
    for _ in range(2):
        c = torch.full((m, n), float("nan"), dtype=dtype, device="cuda")
        assert _call(l, a, b, c, m, n, k, code, trans_b) == 0, l.catccos_last_error()
        words = (ctypes.c_int32 * 8)()
        assert l.catccos_gemm_no_alloc_status(words, None, 0) == 0, list(words)
        outs.append(c)
    assert torch.equal(outs[0], outs[1])

    # the existing entry point on the same inputs
    with rt.emulated_team(1, 1 << 20):
        ref = torch.full((m, n), float("nan"), dtype=dtype, device="cuda")
        rt.launch_emulated(rt.ALLGATHER_MATMUL, [a], [b], [ref], 0, rt.tiling(m, k, n, 1), trans_b=trans_b)
        rc, words = rt.last_status()
        assert rc == 0, words
    assert not torch.isnan(ref.float()).any()
    assert torch.equal(outs[0], ref) and torch.equal(outs[1], ref)

    # and the CPU golden of the product (fp32 accumulation), as for the other dense operators
    from oracle import dense, verify
    bf = b.cpu().t() if trans_b else b.cpu()
    assert verify.max_rel_err(outs[1].cpu(), dense.matmul_fp32(a.cpu(), bf)) <= 1e-2


def test_no_alloc_gemm_rejects_what_it_cannot_hold():
    from catccos_b200 import lib, runtime as rt
    l = lib()
    a = torch.zeros((128, 64), dtype=torch.bfloat16, device="cuda")
    b = torch.zeros((64, 256), dtype=torch.bfloat16, device="cuda")
    c = torch.zeros((128, 256), dtype=torch.bfloat16, device="cuda")
    assert _call(l, a, b, c, 128, 256, 60, rt.BF16, 0) == 1          # k not a multiple of 8
    assert _call(l, a, b, c, 128, 256, 64, rt.INT8 if hasattr(rt, "INT8") else 2, 0) == 1
    assert b"16-byte" in l.catccos_last_error() or b"FP16" in l.catccos_last_error()
    # trace read-back beyond the array's 256 CTA slots is refused
    assert l.catccos_gemm_no_alloc_status(None, None, 257) == 1
    # a normal call still works afterwards, with a capped grid, and leaves a trace
    assert _call(l, a, b, c, 128, 256, 64, rt.BF16, 0, 4) == 0
    trace = (ctypes.c_uint64 * (4 * 16))()
    assert l.catccos_gemm_no_alloc_status(None, trace, 4) == 0
    assert trace[0] > 0 and trace[1] >= trace[0]                     # CTA 0: start and end stamps
