"""The CPU oracle against fixtures produced by the reference's own Python golden
code (tests/golden/make_golden.py) and against the reference's known-answer
vectors.  CPU only."""
import os

import numpy as np
import torch

from oracle import dense, moe, mxquant, swizzle, verify


def _load(golden_dir, name):
    return np.load(os.path.join(golden_dir, name))


# ---------------------------------------------------------------- MX quant --
def test_mx_e4m3_rne_bit_exact(golden_dir):
    f = _load(golden_dir, "mx_quant.npz")
    codes, scale, deq = mxquant.quantize_mx_e4m3(f["x"], "rne")
    assert np.array_equal(codes, f["native_codes"])
    assert np.array_equal(scale, f["native_scale"])
    assert np.array_equal(deq, f["native_dequant"])


def test_mx_e4m3_lut_bit_exact(golden_dir):
    f = _load(golden_dir, "mx_quant.npz")
    codes, scale, deq = mxquant.quantize_mx_e4m3(f["x"], "lut")
    assert np.array_equal(codes, f["lut_codes"])
    assert np.array_equal(scale, f["lut_scale"])
    assert np.array_equal(deq, f["lut_dequant"])
    # the two backends differ only on exact ties
    assert (f["lut_codes"] != f["native_codes"]).sum() > 0


def test_mx_e4m3_axis0_bit_exact(golden_dir):
    f = _load(golden_dir, "mx_quant.npz")
    for backend, mode in (("native", "rne"), ("lut", "lut")):
        codes, scale, _ = mxquant.quantize_mx_e4m3_axis0(f["axis0_x"], mode)
        assert np.array_equal(codes, f[f"{backend}_axis0_codes"])
        assert np.array_equal(scale, f[f"{backend}_axis0_scale"])


def test_mx_edge_cases(golden_dir):
    f = _load(golden_dir, "mx_quant.npz")
    _, scale, _ = mxquant.quantize_mx_e4m3(f["x"], "rne")
    assert (scale[0, :5] == 127).all()            # all-zero blocks -> exp 0
    assert scale[1, 0] == 127                     # amax < 1e-12 -> exp 0
    assert scale[2, 0] == 127                     # 2^-120 is below 1e-12 too -> exp 0
    x = np.full((1, 32), 2.0 ** -30, dtype=np.float32)
    assert mxquant.quantize_mx_e4m3(x)[1][0, 0] == 127 - 30 - 8
    assert (scale[:, 5] == 127).all()             # odd block count padded with 1.0


def test_mx_e2m1_bit_exact(golden_dir):
    f = _load(golden_dir, "mx_quant.npz")
    idx, packed, scale, deq = mxquant.quantize_mx_e2m1(f["fp4_x"])
    assert np.array_equal(idx, f["fp4_idx"])
    assert np.array_equal(packed, f["fp4_packed"])
    assert np.array_equal(scale, f["fp4_scale"])
    assert np.array_equal(deq, f["fp4_dequant"])


def test_e4m3_rne_matches_torch_cast_everywhere():
    allc = np.arange(256, dtype=np.uint8)
    vals = mxquant.e4m3_to_f32(allc)
    finite = vals[np.isfinite(vals)]
    mids = np.sort(np.unique(finite))
    probe = np.concatenate([mids, (mids[:-1] + mids[1:]) / 2, np.nextafter(((mids[:-1] + mids[1:]) / 2).astype(np.float32), np.float32(1e9)),
                            np.nextafter(((mids[:-1] + mids[1:]) / 2).astype(np.float32), np.float32(-1e9))]).astype(np.float32)
    ref = torch.from_numpy(probe).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    assert np.array_equal(mxquant.f32_to_e4m3_rne(probe), ref)


def test_bf16_round_trip():
    x = (np.random.default_rng(0).standard_normal(4096) * 100).astype(np.float32)
    ref = torch.from_numpy(x).to(torch.bfloat16).view(torch.uint16).numpy()
    assert np.array_equal(mxquant.f32_to_bf16_bits(x), ref)


# ------------------------------------------------------------------- dense --
def test_dense_goldens(golden_dir):
    f = _load(golden_dir, "dense.npz")
    a = [torch.from_numpy(f[f"mmar_a{r}"]) for r in range(2)]
    b = [torch.from_numpy(f[f"mmar_b{r}"]) for r in range(2)]
    assert np.array_equal(dense.golden_matmul_allreduce(a, b).numpy(), f["mmar_golden"])
    rs = dense.golden_matmul_reduce_scatter(a, b)
    assert np.array_equal(torch.cat(rs).numpy(), f["mmar_golden"])
    a = [torch.from_numpy(f[f"agmm_a{r}"]).view(torch.bfloat16) for r in range(2)]
    b = [torch.from_numpy(f[f"agmm_b{r}"]).view(torch.bfloat16) for r in range(2)]
    for r, g in enumerate(dense.golden_allgather_matmul(a, b)):
        assert np.array_equal(g.numpy(), f[f"agmm_golden{r}"])


def test_verifier_decisions(golden_dir):
    f = _load(golden_dir, "verify.npz")
    golden = torch.from_numpy(f["golden"])
    for dt, k, name, act, ok in zip(f["dtypes"], f["ks"], f["names"], f["actual"], f["ok"]):
        dtype = {"bfloat16": torch.bfloat16, "float16": torch.float16}[str(dt)]
        got, _, _ = verify.reference_check(torch.from_numpy(act).to(dtype), golden, int(k))
        assert got == bool(ok), (dt, k, name)


# ---------------------------------------------------------------- swizzle --
def test_comm_swizzle_tables(golden_dir):
    f = _load(golden_dir, "comm_swizzle.npz")
    for ci, (gr, gc, gk, sr, sc, direction, det) in enumerate(f["configs"]):
        table = f[f"table{ci}"]
        for i, (data, rank) in enumerate(table):
            row, col, rk = swizzle.block_comm_swizzle_coord(gr, gc, gk, sr, sc, i, int(direction), bool(det))
            assert (row * gc + col, rk) == (data, rank), (ci, i)


def test_comm_swizzle_worked_example():
    # docs/comm_swizzle/comm_swizzle_algorithm.md:87-95, gridShape=(2,2,4), coreSplit=(2,2)
    want = [(0, 0, 0), (0, 1, 1), (0, 0, 2), (0, 1, 3)]
    assert [swizzle.comm_swizzle_coord(2, 2, 4, 2, 2, i) for i in range(4)] == want


def test_matrix_swizzle_is_a_serpentine_permutation():
    for rows, cols, off in ((5, 3, 2), (8, 16, 7), (1, 9, 7), (9, 1, 3)):
        seen = [swizzle.matrix_swizzle_coord(rows, cols, i, off) for i in range(rows * cols)]
        assert sorted(seen) == [(r, c) for r in range(rows) for c in range(cols)]
    # first group walks columns forward, second group backward
    assert swizzle.matrix_swizzle_coord(4, 3, 0, 2) == (0, 0)
    assert swizzle.matrix_swizzle_coord(4, 3, 6, 2) == (2, 2)


def test_alltoallv_gmm_scheduler_known_answer():
    # tests/comm_block_scheduler_alltoallv_gmm/test_comm_block_scheduler_alltoallv_gmm.cpp:94-101
    expected = [1, 3, 0, 0, 42, 1, 1, 4, 4, 0, 0, 4, 0, 10, 2, 3]
    t = np.arange(1, 33)
    got = []
    prev, loops, offs = moe.set_comm_core(t, 2, 4, 2, 1, 3)
    got += [1, 3, 0, 0, prev, loops, offs[0], offs[1]]
    prev, loops, offs = moe.set_comm_core(t, 2, 4, 2, 4, 6)
    got += [4, prev, loops, offs[0]]
    prev, loops, offs = moe.set_comm_core(t, 2, 4, 2, 0, 3)
    got += [0, prev, loops, offs[1]]
    assert got == expected
    cs = moe.cumsum_mm(t, 2, 4, 2)
    assert cs.tolist() == [[5, 6], [18, 20], [39, 42], [68, 72]]


# -------------------------------------------------------------------- MoE --
def test_moe_subfunctions(golden_dir):
    f = _load(golden_dir, "moe.npz")
    ep, epr, top_k = 3, 2, 2
    srcs, counts, routed = [], [], []
    for r in range(ep):
        s, c = moe.moe_init_routing(f[f"sub_idx{r}"], ep * epr)
        assert np.array_equal(s, f[f"sub_rowidx{r}"])
        assert np.array_equal(c, f[f"sub_tokens{r}"])
        rt = moe.permute_rows(f[f"sub_x{r}"], s, top_k)
        assert np.array_equal(rt, f[f"sub_routed{r}"])
        srcs.append(s); counts.append(c); routed.append(rt)
    recv, blocks = moe.alltoallv_dispatch(routed, np.stack(counts), ep, epr)
    for r in range(ep):
        assert np.array_equal(recv[r], f[f"sub_recv{r}"])
        assert blocks[r] == f[f"sub_blocks{r}"].tolist()
    back = moe.alltoallv_combine(recv, np.stack(counts), ep, epr)
    for r in range(ep):
        assert np.array_equal(back[r], f[f"sub_back{r}"])
        assert np.array_equal(back[r], routed[r])          # dispatch then combine is the identity
        ref = moe.unpermute_reference_cpu(back[r], srcs[r], f[f"sub_probs{r}"])
        assert np.array_equal(ref, f[f"sub_combine{r}"])
        mine = moe.unpermute_fp32(back[r], moe.expanded_row_idx_src_to_dst(srcs[r]), f[f"sub_probs{r}"])
        assert np.allclose(mine, ref, rtol=2 ** -6, atol=2 ** -6)
    assert np.array_equal(moe.swiglu_bf16(f["swiglu_in"]), f["swiglu_out"])


def test_moe_full_pipeline(golden_dir):
    f = _load(golden_dir, "moe.npz")
    m, k, n, top_k, e_num, ep = [int(v) for v in f["e2e_shape"]]
    epr = e_num // ep
    xs = [mxquant.bf16_bits_to_f32(f[f"e2e_x{r}"]).reshape(m, k) for r in range(ep)]
    outs, inter = moe.dispatch_ffn_combine(
        xs, [f[f"e2e_idx{r}"] for r in range(ep)], [f[f"e2e_probs{r}"] for r in range(ep)],
        [f[f"e2e_w1q{r}"] for r in range(ep)], [f[f"e2e_w1s{r}"] for r in range(ep)],
        [f[f"e2e_w2q{r}"] for r in range(ep)], [f[f"e2e_w2s{r}"] for r in range(ep)],
        ep, epr, return_intermediates=True)
    for r in range(ep):
        assert np.array_equal(inter["sorted_src"][r], f[f"e2e_rowidx{r}"])
        # GEMM2 output rows (bf16) before the combine all-to-all: bit-exact
        assert np.array_equal(mxquant.f32_to_bf16_bits(inter["gmm2"][r]).reshape(-1), f[f"e2e_gmm2{r}"].reshape(-1))
        assert np.array_equal(mxquant.f32_to_bf16_bits(inter["back"][r]).reshape(-1), f[f"e2e_back{r}"].reshape(-1))
        ref = mxquant.bf16_bits_to_f32(f[f"e2e_out{r}"]).reshape(m, k)
        # final weighted sum: fp32 accumulate (device definition) vs the reference's bf16 CPU fallback
        err = np.abs(outs[r] - ref) / np.maximum(1.0, np.abs(ref))
        assert err.max() <= 2 ** -6


def test_mx_e5m2_quantiser_bit_exact(golden_dir):
    """e5m2 codes and E8M0 scales of the MXFP8 Matmul-ReduceScatter example's generator."""
    f = _load(golden_dir, "mx_mmrs.npz")
    codes, scale, _ = mxquant.quantize_mx_e5m2(f["q_x"])
    assert np.array_equal(codes, f["q_codes"])
    assert np.array_equal(scale, f["q_scale"])
    # every finite e5m2 value survives a decode / encode round trip
    allc = np.array([c for c in range(256) if (c & 0x7C) != 0x7C], dtype=np.uint8)
    back = mxquant.f32_to_e5m2_nearest(mxquant.e5m2_to_f32(allc))
    assert np.array_equal(back & 0x7F, allc & 0x7F)


def test_mx_matmul_reduce_scatter_golden(golden_dir):
    f = _load(golden_dir, "mx_mmrs.npz")
    m, k, n, world = [int(v) for v in f["shape"]]
    a = [f[f"a{r}"] for r in range(world)]
    a_s = [f[f"a_scale{r}"].reshape(m, -1) for r in range(world)]
    b = [np.ascontiguousarray(f[f"b{r}"].T) for r in range(world)]                       # files hold B^T (transB = 1)
    b_s = [np.ascontiguousarray(f[f"b_scale{r}"].reshape(n, -1).T) for r in range(world)]
    outs = dense.golden_mx_matmul_reduce_scatter(a, a_s, b, b_s, "e5m2")
    mine = torch.cat(outs, dim=0).numpy()
    assert mine.shape == f["golden"].shape
    assert np.allclose(mine, f["golden"], rtol=1e-5, atol=1e-4)
    low = mxquant.bf16_bits_to_f32(f["golden_low"]).reshape(m, n)
    assert np.abs(mine - low).max() <= 2 ** -6 * max(1.0, np.abs(mine).max())


def _a2av_operands(f, prefix, world, experts, m, k, n):
    epr = experts // world
    a = [mxquant.dequant_mx(f[f"{prefix}_a{r}"], f[f"{prefix}_a_scale{r}"].reshape(m, -1), "e4m3") for r in range(world)]
    w = []
    for r in range(world):
        per = []
        for le in range(epr):
            codes = f[f"{prefix}_b{r}"][le]                                                # [k, n]
            sc = f[f"{prefix}_b_scale{r}"][le].transpose(0, 2, 1).reshape(-1, n)           # [k/64, n, 2] -> [k/32, n]
            per.append(np.ascontiguousarray(
                mxquant.dequant_mx(np.ascontiguousarray(codes.T), np.ascontiguousarray(sc.T), "e4m3").T))
        w.append(per)
    return a, w


def test_alltoallv_grouped_matmul_golden(golden_dir):
    f = _load(golden_dir, "alltoallv_gmm.npz")
    world, m, n, k, experts = [int(v) for v in f["shape"]]
    a, w = _a2av_operands(f, "d", world, experts, m, k, n)
    counts = np.stack([f[f"d_local_tokens{r}"] for r in range(world)])
    outs, blocks = moe.alltoallv_grouped_matmul(a, w, counts, world, experts // world)
    for r in range(world):
        assert blocks[r] == f[f"d_global_tokens{r}"].sum(axis=0).tolist()
        rows = outs[r].shape[0]
        assert np.allclose(outs[r], f[f"d_golden{r}"][:rows], rtol=1e-5, atol=1e-4)
        assert not f[f"d_golden{r}"][rows:].any()


def test_grouped_matmul_alltoallv_golden(golden_dir):
    f = _load(golden_dir, "alltoallv_gmm.npz")
    world, _, n, k, experts = [int(v) for v in f["shape"]]
    m2 = int(f["c_m"][0])
    a, w = _a2av_operands(f, "c", world, experts, m2, k, n)
    counts = np.stack([f[f"c_local_tokens{r}"] for r in range(world)])
    back = moe.grouped_matmul_alltoallv(a, w, counts, world, experts // world)
    for r in range(world):
        rows = back[r].shape[0]
        assert rows == int(counts[r].sum())
        assert np.allclose(back[r], f[f"c_golden{r}"][:rows], rtol=1e-5, atol=1e-4)


def test_mxfp4_allgather_matmul_golden(golden_dir):
    """MXFP4 operands (packed e2m1, E8M0 per 32) of the reference's FP4 AllGather-Matmul generator."""
    f = _load(golden_dir, "fp4_agmm.npz")
    world, m, n, k = [int(v) for v in f["shape"]]
    a = [mxquant.dequant_mxfp4(f[f"a{r}"], f[f"a_scale{r}"], k) for r in range(world)]
    b = [np.ascontiguousarray(mxquant.dequant_mxfp4(f[f"b{r}"], f[f"b_scale{r}"], k).T) for r in range(world)]   # files hold B^T
    outs = dense.golden_fp4_allgather_matmul(a, b)
    for r in range(world):
        assert np.allclose(outs[r].numpy(), f[f"golden{r}"], rtol=1e-5, atol=1e-5)


def test_nvfp4_definition_round_trips():
    """NVFP4 is not in the reference (parity unpinned): check the definition against itself — values on
    the e2m1 x e4m3 grid survive quantisation exactly, everything else lands within half a step."""
    rng = np.random.default_rng(3)
    x = rng.standard_normal((8, 64)).astype(np.float32) * 3
    idx, packed, sb, ts, deq = mxquant.quantize_nvfp4(x)
    assert packed.shape == (8, 32) and sb.shape == (8, 4)
    assert np.array_equal(mxquant.dequant_nvfp4(packed, sb, ts, 64), deq)
    idx2, packed2, sb2, ts2, deq2 = mxquant.quantize_nvfp4(deq)       # grid values: a fixed point
    assert np.allclose(deq2, deq, rtol=0, atol=1e-6 * np.abs(deq).max())
    sval = np.repeat(mxquant.e4m3_to_f32(sb) * ts, 16, axis=1)
    assert (np.abs(deq - x) <= 1.0 * sval + 1e-6).all()              # largest e2m1 step is 2 (between 4 and 6): half of it
    # ties go to the even code: 2.5 -> 2, 3.5 -> 4 (in units of the block scale)
    assert mxquant._e2m1_rne_index(np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0])).tolist() == [0, 2, 2, 4, 4, 6, 6]
