"""Parity at the full sizes of the benchmark configurations 2-5 (through the C-ABI, against the CPU
oracle).  Configurations 2-4 run their eight ranks as emulated PEs on one GPU (about 3 GB); the MoE
runs one rank at its full per-rank size (4096 tokens, 32 local experts, top-8 Zipf routing).

What is compared: the whole output where the fp32 CPU golden takes seconds (configurations 2 and
3), a seeded sample of 512 rows per source rank for the MXFP8 AllGather-Matmul, and for the MoE
the routing tables bit for bit, a sample of dispatched rows bit for bit and the final output of a
token sample that reaches every local expert."""
import ctypes

import numpy as np
import pytest
import torch

from oracle import dense, inputs, moe, mxquant, verify
from tests.gpu_util import dev

pytestmark = pytest.mark.gpu
WORLD = 8


def _rows(n_rows, count, seed):
    g = torch.Generator().manual_seed(seed)
    idx = torch.randperm(n_rows, generator=g)[:count]
    idx[0], idx[-1] = 0, n_rows - 1
    return torch.unique(idx)


def _lut_dequant(codes, scales):
    """uint8 e4m3 codes [r, k] and E8M0 bytes [r, >= k/32] -> fp32 [r, k]: the oracle's decoding
    (mxquant.e4m3_to_f32) as a 256-entry table, so that full-size weights take milliseconds."""
    lut = torch.from_numpy(mxquant.e4m3_to_f32(np.arange(256, dtype=np.uint8)))
    r, k = codes.shape
    v = lut[codes.to(torch.int64)].view(r, k // 32, 32)
    return (v * torch.exp2(scales[:, :k // 32].to(torch.float32) - 127.0)[:, :, None]).view(r, k)


def _quant_gpu(x_bf16_dev):
    from catccos_b200 import lib, check
    rows, k = x_bf16_dev.shape
    codes = torch.empty((rows, k), dtype=torch.uint8, device="cuda")
    scales = torch.empty((rows, (k // 32 + 1) // 2 * 2), dtype=torch.uint8, device="cuda")
    check(lib().catccos_mx_quant(ctypes.c_void_p(torch.cuda.current_stream().cuda_stream),
                                 ctypes.c_void_p(x_bf16_dev.data_ptr()), ctypes.c_void_p(codes.data_ptr()),
                                 ctypes.c_void_p(scales.data_ptr()), None, rows, k))
    return codes, scales


def test_allgather_matmul_bf16_configuration_2():
    """allgather_matmul bf16, world 8: A_local [1024, 8192], B [8192, 4096] per rank; K = 8192
    accumulation, 512 pair tiles per rank, every element of every rank's [8192, 4096] output."""
    from catccos_b200 import runtime as rt
    m, k, n = 1024, 8192, 4096
    a, b = inputs.allgather_matmul_inputs(WORLD, m, k, n, torch.bfloat16)
    til = rt.tiling(m, k, n, WORLD)
    need = rt.symmetric_bytes(rt.ALLGATHER_MATMUL, rt.BF16, til)
    with rt.emulated_team(WORLD, need + (1 << 20)):
        symm = rt.shmem_malloc(need)
        a_d, b_d = [dev(x) for x in a], [dev(x) for x in b]
        c_d = [torch.full((WORLD * m, n), float("nan"), dtype=torch.bfloat16, device="cuda") for _ in range(WORLD)]
        for _ in range(2):
            rt.launch_emulated(rt.ALLGATHER_MATMUL, a_d, b_d, c_d, symm, til)
        rc, words = rt.last_status()
        assert rc == 0, words
        outs = [c.cpu() for c in c_d]
    gathered = torch.cat([x.to(torch.float32) for x in a], dim=0)
    for r in range(WORLD):
        gold = torch.matmul(gathered, b[r].to(torch.float32))
        err = verify.max_rel_err(outs[r], gold)
        assert err <= 1e-2, f"rank {r}: max relative error {err}"
        ok, precision, eb = verify.reference_check(outs[r], gold, k)
        assert ok, f"rank {r}: reference gate failed (precision {precision:.4f}%, eb {eb:.2f}%)"


def test_matmul_reduce_scatter_bf16_configuration_3():
    """matmul_reduce_scatter bf16, world 8: A [8192, 2048], B [2048, 8192] per rank, summed and
    row-scattered to [1024, 8192] per rank; every element, with the reduce family's tolerance
    (reference rtol widened by the round-off of each exchanged 16-bit partial)."""
    from catccos_b200 import runtime as rt
    m, k, n = 8192, 2048, 8192
    a, b = inputs.matmul_reduce_scatter_inputs(WORLD, m, k, n, torch.bfloat16)
    til = rt.tiling(m, k, n, WORLD)
    need = rt.symmetric_bytes(rt.MATMUL_REDUCE_SCATTER, rt.BF16, til)
    with rt.emulated_team(WORLD, need + (1 << 20)):
        symm = rt.shmem_malloc(need)
        a_d, b_d = [dev(x) for x in a], [dev(x) for x in b]
        c_d = [torch.full((m // WORLD, n), float("nan"), dtype=torch.bfloat16, device="cuda") for _ in range(WORLD)]
        for _ in range(2):
            rt.launch_emulated(rt.MATMUL_REDUCE_SCATTER, a_d, b_d, c_d, symm, til)
        rc, words = rt.last_status()
        assert rc == 0, words
        out = torch.cat([c.cpu() for c in c_d], dim=0)
    gold = torch.zeros((m, n), dtype=torch.float32)
    slack = torch.zeros((m, n), dtype=torch.float32)
    for x, y in zip(a, b):
        part = dense.matmul_fp32(x, y)
        gold += part
        slack += part.abs()
    err = verify.max_rel_err(out, gold)
    assert err <= 1e-2, f"max relative error {err}"
    bound = verify.get_rtol(torch.bfloat16, k) * torch.clamp(gold.abs(), min=1.0) + slack * 2.0 ** -8
    bad = int(((out.to(torch.float32) - gold).abs() > bound).sum())
    assert bad == 0, f"{bad} elements beyond the widened reference tolerance"
    _, _, eb = verify.reference_check(out, gold, k)
    assert eb <= 100, f"mean bias {eb:.1f}% of the reference bound"


def test_mxfp8_allgather_matmul_configuration_4():
    """MXFP8 allgather_matmul, world 8: activations [2048, 7168] per rank and weights [7168, 4096]
    quantised to e4m3 + E8M0 per 32 along K (on the GPU, checked bit for bit against the oracle on a
    row sample), bf16 output [16384, 4096]; 512 sampled rows per source rank on every rank."""
    from catccos_b200 import runtime as rt, lib
    m, k, n = 2048, 7168, 4096
    kb = k // 32
    til = rt.tiling(m, k, n, WORLD)
    need = rt.symmetric_bytes(rt.FP8_MX_ALLGATHER_MATMUL, rt.BF16, til)
    ws_bytes = lib().catccos_workspace_bytes(rt.FP8_MX_ALLGATHER_MATMUL, rt.BF16, ctypes.byref(til))
    a_c, a_s, w_ct, w_st = [], [], [], []
    for r in range(WORLD):
        act = inputs.normal((m, k), torch.bfloat16, 4000 + r).cuda()
        w_t = inputs.normal((n, k), torch.bfloat16, 5000 + r, 0.02).cuda()       # [n, k]: blocks along k
        c, s = _quant_gpu(act)
        a_c.append(c); a_s.append(s)
        c, s = _quant_gpu(w_t)
        w_ct.append(c); w_st.append(s)
        idx = _rows(m, 64, 60 + r)
        qc, qs, _ = mxquant.quantize_mx_e4m3(act[idx.cuda()].cpu().to(torch.float32).numpy(), "rne")
        assert np.array_equal(qc, a_c[r][idx.cuda()].cpu().numpy()) and np.array_equal(qs, a_s[r][idx.cuda()].cpu().numpy())
    with rt.emulated_team(WORLD, need + (1 << 20)):
        symm = rt.shmem_malloc(need)
        b_d = [c.t().contiguous() for c in w_ct]                                  # [k, n]
        bs_d = [s[:, :kb].t().contiguous().reshape(kb // 2, 2, n).permute(0, 2, 1).contiguous() for s in w_st]
        as_d = [s[:, :kb].contiguous() for s in a_s]
        c_d = [torch.full((WORLD * m, n), float("nan"), dtype=torch.bfloat16, device="cuda") for _ in range(WORLD)]
        ws = [torch.zeros(ws_bytes, dtype=torch.uint8, device="cuda") for _ in range(WORLD)]
        for _ in range(2):
            rt.launch_emulated(rt.FP8_MX_ALLGATHER_MATMUL, a_c, b_d, c_d, symm, til, dtype=rt.BF16,
                               custom_lists=[[as_d[r], bs_d[r]] for r in range(WORLD)], workspaces=ws)
        rc, words = rt.last_status()
        assert rc == 0, words
        samples = [_rows(m, 512, 70 + s) for s in range(WORLD)]
        rows_all = torch.cat([s * m + samples[s] for s in range(WORLD)])
        outs = [c[rows_all.cuda()].cpu() for c in c_d]
    a_deq = torch.cat([_lut_dequant(a_c[s][samples[s].cuda()].cpu(), a_s[s][samples[s].cuda()].cpu()) for s in range(WORLD)])
    for r in range(WORLD):
        gold = torch.matmul(a_deq, _lut_dequant(w_ct[r].cpu(), w_st[r].cpu()).t())
        err = verify.max_rel_err(outs[r], gold)
        assert err <= 2e-2, f"rank {r}: max relative error {err}"


def _up(v, a):
    return (v + a - 1) // a * a


def test_moe_configuration_5_one_rank():
    """MoE at the full per-rank size: 4096 tokens, hidden 7168, 32 local experts with FFN 2048
    (n = 4096 up/gate columns), top-8 routing with a Zipf(1.1) bias, MXFP8 weights.  Routing tables
    bit for bit, a sample of dispatched rows bit for bit, and the output of 192 sampled tokens
    (every expert is reached) within 2e-2 of the golden pipeline."""
    from catccos_b200 import runtime as rt, lib
    m, k, n, top_k, experts = 4096, 7168, 4096, 8, 32
    x = inputs.normal((m, k), torch.bfloat16, 77)
    ids, probs = inputs.zipf_topk_routing(m, experts, top_k, 78)
    w1q = torch.empty((experts, n, k), dtype=torch.uint8, device="cuda")
    w1s = torch.empty((experts, n, k // 32), dtype=torch.uint8, device="cuda")
    w2q = torch.empty((experts, k, n // 2), dtype=torch.uint8, device="cuda")
    w2s = torch.empty((experts, k, (n // 2) // 32), dtype=torch.uint8, device="cuda")
    g = torch.Generator(device="cuda").manual_seed(79)
    for e in range(experts):
        w = (torch.randn((n, k), generator=g, device="cuda") * 0.02).to(torch.bfloat16)
        c, s = _quant_gpu(w)
        w1q[e], w1s[e] = c, s[:, :k // 32]
        w = (torch.randn((k, n // 2), generator=g, device="cuda") * 0.02).to(torch.bfloat16)
        c, s = _quant_gpu(w)
        w2q[e], w2s[e] = c, s[:, :(n // 2) // 32]
    til = rt.tiling(m, k, n, 1, topK=top_k, expertNum=experts, epSize=1)
    need = rt.symmetric_bytes(rt.DISPATCH_FFN_COMBINE, rt.BF16, til)
    ws_bytes = lib().catccos_workspace_bytes(rt.DISPATCH_FFN_COMBINE, rt.BF16, ctypes.byref(til))
    with rt.emulated_team(1, need + (1 << 20)):
        symm = rt.shmem_malloc(need)
        x_d = dev(x)
        idx_d = dev(torch.from_numpy(ids.astype(np.int32)))
        pr_d = dev(torch.from_numpy(probs.astype(np.float32)))
        out_d = torch.full((m, k), float("nan"), dtype=torch.bfloat16, device="cuda")
        ws = torch.zeros(ws_bytes, dtype=torch.uint8, device="cuda")
        for _ in range(2):
            rt.launch_emulated(rt.DISPATCH_FFN_COMBINE, [x_d], [w1q], [out_d], symm, til, dtype=rt.BF16,
                               custom_lists=[[w2q, idx_d, pr_d, w1s, w2s]], workspaces=[ws])
        rc, words = rt.last_status()
        assert rc == 0, words
        out = out_d.cpu()
        # routing tables and receive rows (layout as in tests/test_gpu_moe.py)
        rows_cap = _up(min(max(2 * m * top_k, 16384), m * top_k) + experts * 128, 128)
        sld = _up(k // 32, 2)
        idx_bytes = _up(m * top_k * 4, 1024)
        counts_bytes = _up(experts * 4, 1024)
        w_host = ws[:idx_bytes + 8 * 512 * 4].cpu().numpy()
        eri = w_host[:m * top_k * 4].view(np.int32).copy()
        counts = w_host[idx_bytes:idx_bytes + 8 * 512 * 4].view(np.int32).reshape(8, 512)[0, :experts].copy()
        nbytes = counts_bytes + _up(rows_cap * k, 1024) + _up(rows_cap * sld, 1024)
        h = np.empty(nbytes, dtype=np.uint8)
        assert lib().catccos_shmem_get_host(h.ctypes.data_as(ctypes.c_void_p), ctypes.c_void_p(symm), 0, nbytes) == 0
    codes = h[counts_bytes:counts_bytes + rows_cap * k].reshape(rows_cap, k)
    scales = h[counts_bytes + _up(rows_cap * k, 1024):][:rows_cap * sld].reshape(rows_cap, sld)

    sorted_src, gold_counts = moe.moe_init_routing(ids, experts)
    assert np.array_equal(counts, gold_counts), "tokens per expert differ"
    inv = moe.expanded_row_idx_src_to_dst(sorted_src)
    assert np.array_equal(eri, inv), "expandedRowIdx differs"
    # dispatched rows: permuted row d sits at its expert's 128-aligned segment start + offset inside the expert
    seg_start = np.concatenate([[0], np.cumsum(_up(gold_counts.astype(np.int64), 128))[:-1]])
    first = np.concatenate([[0], np.cumsum(gold_counts.astype(np.int64))[:-1]])
    sample = np.unique(np.concatenate([[0, m * top_k - 1], np.random.default_rng(5).integers(0, m * top_k, 2048)]))
    flat_expert = ids.reshape(-1)[sorted_src[sample]]
    dev_row = seg_start[flat_expert] + (sample - first[flat_expert])
    qc, qs, _ = mxquant.quantize_mx_e4m3(x[torch.from_numpy(sorted_src[sample].astype(np.int64) // top_k)]
                                         .to(torch.float32).numpy(), "rne")
    assert np.array_equal(codes[dev_row], qc), "dispatched codes differ"
    assert np.array_equal(scales[dev_row], qs), "dispatched scales differ"

    # final output of sampled tokens through the golden stages
    toks = _rows(m, 192, 81).numpy()
    for e in np.setdiff1d(np.arange(experts), np.unique(ids[toks])):      # every expert at least once
        toks = np.append(toks, np.nonzero((ids == e).any(axis=1))[0][:1])
    toks = np.unique(toks)
    _, _, x_deq = mxquant.quantize_mx_e4m3(x[torch.from_numpy(toks)].to(torch.float32).numpy(), "rne")
    rows_back = np.zeros((len(toks), top_k, k), dtype=np.float32)
    for e in range(experts):
        t_sel, k_sel = np.nonzero(ids[toks] == e)
        if len(t_sel) == 0:
            continue
        w1 = _lut_dequant(w1q[e].cpu(), w1s[e].cpu())
        w2 = _lut_dequant(w2q[e].cpu(), w2s[e].cpu())
        c1 = torch.matmul(torch.from_numpy(x_deq[t_sel]), w1.t()).to(torch.bfloat16).to(torch.float32).numpy()
        _, _, g_deq = mxquant.quantize_mx_e4m3(moe.swiglu_bf16(c1), "rne")
        rows_back[t_sel, k_sel] = torch.matmul(torch.from_numpy(g_deq), w2.t()).to(torch.bfloat16).to(torch.float32).numpy()
    acc = np.zeros((len(toks), k), dtype=np.float32)
    for j in range(top_k):
        acc = (acc + rows_back[:, j] * probs[toks, j:j + 1].astype(np.float32)).astype(np.float32)
    gold = torch.from_numpy(mxquant.bf16_bits_to_f32(mxquant.f32_to_bf16_bits(acc)).reshape(acc.shape))
    err = verify.max_rel_err(out[torch.from_numpy(toks)], gold)
    assert err <= 2e-2, f"max relative error {err}"
