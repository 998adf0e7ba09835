"""MoE dispatch -> grouped GEMM -> SwiGLU -> grouped GEMM -> combine through the C-ABI against the
CPU oracle: routing and the dispatched (quantised, permuted) rows bit-exactly, the final output
within the MXFP8 tolerance."""
import ctypes
import os

import numpy as np
import pytest
import torch

from oracle import inputs, moe, mxquant, verify
from tests.gpu_util import dev

pytestmark = pytest.mark.gpu
TOL_MX = 2e-2


def _up(v, a):
    return (v + a - 1) // a * a


def _rows_cap(world, m, top_k, el):
    cap = max(2 * m * top_k, 16384)
    cap = min(cap, world * m * top_k) + el * 128
    return _up(cap, 128)


def _run(world, m, k, n, top_k, experts, xs, idxs, probs, w1q, w1s, w2q, w2s):
    from catccos_b200 import runtime as rt, lib
    til = rt.tiling(m, k, n, world, topK=top_k, expertNum=experts, epSize=world)
    need = rt.symmetric_bytes(rt.DISPATCH_FFN_COMBINE, rt.BF16, til)
    ws_bytes = lib().catccos_workspace_bytes(rt.DISPATCH_FFN_COMBINE, rt.BF16, ctypes.byref(til))
    assert need > 0 and ws_bytes > 0
    with rt.emulated_team(world, need + (1 << 20)):
        symm = rt.shmem_malloc(need)
        x_d = [dev(torch.from_numpy(x).to(torch.bfloat16)) for x in xs]
        w1_d = [dev(torch.from_numpy(w)) for w in w1q]
        w2_d = [dev(torch.from_numpy(w)) for w in w2q]
        w1s_d = [dev(torch.from_numpy(w)) for w in w1s]
        w2s_d = [dev(torch.from_numpy(w)) for w in w2s]
        idx_d = [dev(torch.from_numpy(i.astype(np.int32))) for i in idxs]
        pr_d = [dev(torch.from_numpy(p.astype(np.float32))) for p in probs]
        out_d = [torch.full((m, k), float("nan"), dtype=torch.bfloat16, device="cuda") for _ in range(world)]
        ws = [torch.zeros(ws_bytes, dtype=torch.uint8, device="cuda") for _ in range(world)]
        for _ in range(2):
            rt.launch_emulated(rt.DISPATCH_FFN_COMBINE, x_d, w1_d, out_d, symm, til, dtype=rt.BF16,
                               custom_lists=[[w2_d[r], idx_d[r], pr_d[r], w1s_d[r], w2s_d[r]] for r in range(world)],
                               workspaces=ws)
        rc, words = rt.last_status()
        assert rc == 0, words
        outs = [o.cpu().to(torch.float32).numpy() for o in out_d]
        # internals for the bit-exact checks: expanded row index and counts (workspace), receive rows (heap)
        el = experts // world
        rows_cap = _rows_cap(world, m, top_k, el)
        sld = _up(k // 32, 2)
        idx_bytes = _up(m * top_k * 4, 1024)
        counts_bytes = _up(world * experts * 4, 1024)
        internals = []
        for r in range(world):
            w = ws[r].cpu().numpy()
            eri = w[:m * top_k * 4].view(np.int32).copy()
            counts = w[idx_bytes:idx_bytes + 8 * 512 * 4].view(np.int32).reshape(8, 512)[:world, :experts].copy()
            combine_off = counts_bytes + _up(rows_cap * k, 1024) + _up(rows_cap * sld, 1024)
            nbytes = combine_off + m * top_k * k * 2
            h = np.empty(nbytes, dtype=np.uint8)
            assert lib().catccos_shmem_get_host(h.ctypes.data_as(ctypes.c_void_p), ctypes.c_void_p(symm), r, nbytes) == 0
            codes = h[counts_bytes:counts_bytes + rows_cap * k].reshape(rows_cap, k)
            sc = h[counts_bytes + _up(rows_cap * k, 1024):][:rows_cap * sld].reshape(rows_cap, sld)
            combine = h[combine_off:combine_off + m * top_k * k * 2].view(np.uint16).reshape(m * top_k, k).copy()
            internals.append((eri, counts, codes, sc, combine))
        return outs, internals


def _oracle(world, epr, xs, idxs, probs, w1q, w1s, w2q, w2s):
    return moe.dispatch_ffn_combine(xs, idxs, probs, w1q, w1s, w2q, w2s, world, epr, return_intermediates=True)


def _check_bit_exact_parts(world, epr, top_k, inter, internals):
    counts_all = inter["counts"]
    for r in range(world):
        eri, counts, codes, sc, _ = internals[r]
        assert np.array_equal(counts, counts_all), "tokens per expert (all-gathered) differ"
        assert np.array_equal(eri, moe.expanded_row_idx_src_to_dst(inter["sorted_src"][r])), "expandedRowIdx differs"
        # dispatched rows: golden receive order, every local expert's segment starting on a multiple of 128
        q, s, _ = mxquant.quantize_mx_e4m3(inter["recv"][r], "rne")
        pos, base = 0, 0
        for n_rows in inter["blocks"][r]:
            assert np.array_equal(codes[base:base + n_rows], q[pos:pos + n_rows]), "dispatched codes differ"
            assert np.array_equal(sc[base:base + n_rows], s[pos:pos + n_rows]), "dispatched scales differ"
            pos += n_rows
            base += _up(n_rows, 128)


def test_moe_on_the_reference_fixture(golden_dir):
    f = np.load(os.path.join(golden_dir, "moe.npz"))
    m, k, n, top_k, e_num, ep = [int(v) for v in f["e2e_shape"]]
    epr = e_num // ep
    xs = [mxquant.bf16_bits_to_f32(f[f"e2e_x{r}"]).reshape(m, k) for r in range(ep)]
    idxs = [f[f"e2e_idx{r}"] for r in range(ep)]
    probs = [f[f"e2e_probs{r}"] for r in range(ep)]
    w1q = [f[f"e2e_w1q{r}"] for r in range(ep)]
    w1s = [f[f"e2e_w1s{r}"] for r in range(ep)]
    w2q = [f[f"e2e_w2q{r}"] for r in range(ep)]
    w2s = [f[f"e2e_w2s{r}"] for r in range(ep)]
    outs, internals = _run(ep, m, k, n, top_k, e_num, xs, idxs, probs, w1q, w1s, w2q, w2s)
    gold, inter = _oracle(ep, epr, xs, idxs, probs, w1q, w1s, w2q, w2s)
    _check_bit_exact_parts(ep, epr, top_k, inter, internals)
    for r in range(ep):
        ref = mxquant.bf16_bits_to_f32(f[f"e2e_out{r}"]).reshape(m, k)       # the reference's own output file
        for name, g in (("oracle", gold[r]), ("reference file", ref)):
            err = verify.max_rel_err(torch.from_numpy(outs[r]), torch.from_numpy(g))
            assert err <= TOL_MX, f"rank {r} vs {name}: {err}"


@pytest.mark.parametrize("world,m,k,n,top_k,experts", [
    (1, 96, 256, 512, 2, 4),
    (2, 200, 512, 1024, 4, 8),
    (4, 128, 768, 512, 8, 32),
    (8, 64, 256, 512, 2, 16),
])
def test_moe_zipf_routing(world, m, k, n, top_k, experts):
    epr = experts // world
    xs, idxs, probs, w1q, w1s, w2q, w2s = [], [], [], [], [], [], []
    for r in range(world):
        xs.append(inputs.bf16_as_f32(inputs.normal((m, k), torch.bfloat16, 10 + r)))
        ids, pr = inputs.zipf_topk_routing(m, experts, top_k, 100 + r)
        idxs.append(ids); probs.append(pr)
        q1, s1, q2, s2 = [], [], [], []
        for e in range(epr):
            w1 = inputs.bf16_as_f32(inputs.normal((k, n), torch.bfloat16, 1000 + r * 64 + e, 0.02))
            w2 = inputs.bf16_as_f32(inputs.normal((n // 2, k), torch.bfloat16, 5000 + r * 64 + e, 0.02))
            c, s, _ = mxquant.quantize_mx_e4m3_axis0(w1, "rne")      # [k, n], scales [k/32(+pad), n]
            q1.append(np.ascontiguousarray(c.T)); s1.append(np.ascontiguousarray(s[:k // 32].T))
            c, s, _ = mxquant.quantize_mx_e4m3_axis0(w2, "rne")
            q2.append(np.ascontiguousarray(c.T)); s2.append(np.ascontiguousarray(s[:(n // 2) // 32].T))
        w1q.append(np.stack(q1)); w1s.append(np.stack(s1)); w2q.append(np.stack(q2)); w2s.append(np.stack(s2))
    outs, internals = _run(world, m, k, n, top_k, experts, xs, idxs, probs, w1q, w1s, w2q, w2s)
    gold, inter = _oracle(world, epr, xs, idxs, probs, w1q, w1s, w2q, w2s)
    _check_bit_exact_parts(world, epr, top_k, inter, internals)
    for r in range(world):
        err = verify.max_rel_err(torch.from_numpy(outs[r]), torch.from_numpy(gold[r]))
        assert err <= TOL_MX, f"rank {r}: {err}"
    _check_unpermute_bit_exact(world, probs, outs, internals)


def _check_unpermute_bit_exact(world, probs, outs, internals):
    """The un-permute kernel alone: the rows the combine stage left in this rank's buffer, weighted and summed by
    the oracle in the kernel's order of operations (fp32 multiply, fp32 add, top-k order, one bf16 rounding),
    must give the operator's output bit for bit."""
    for r in range(world):
        eri, _, _, _, combine = internals[r]
        rows = mxquant.bf16_bits_to_f32(combine)
        want = moe.unpermute_fp32(rows, eri, np.asarray(probs[r], dtype=np.float32))
        assert np.array_equal(want.view(np.uint32), outs[r].view(np.uint32)), f"rank {r}: un-permute differs from the oracle"
