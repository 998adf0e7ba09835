#!/usr/bin/env python3
"""Regenerates the golden fixtures in this directory from the reference's own
Python host-golden code.

Run where the reference checkout is available:
    python tests/golden/make_golden.py /path/to/reference
It imports the reference's `examples/utils/*.py` (unmodified), feeds them small
seeded inputs and stores inputs + outputs as `.npz`.  The fixtures travel with
the repository; the reference does not.  Nothing in the test-suite imports this
script.
"""
import ast
import contextlib
import importlib
import io
import os
import subprocess
import sys
import tempfile

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _import_ref(name, backend=None):
    if backend is not None:
        os.environ["GEN_DATA_QUANT_BACKEND"] = backend
    if name in sys.modules:
        return importlib.reload(sys.modules[name])
    return importlib.import_module(name)


def mx_quant_fixture():
    rng = np.random.default_rng(1234)
    m, k = 24, 160                                   # 5 blocks per row -> padded to 6 scales
    x = (rng.standard_normal((m, k)) * rng.choice([1e-3, 0.1, 1.0, 30.0, 4000.0], size=(m, 1))).astype(np.float32)
    x = torch.from_numpy(x).to(torch.bfloat16).to(torch.float32).numpy()     # bf16-valued
    x[0, :] = 0.0                                     # all-zero row
    x[1, :32] = 1e-13                                 # amax < 1e-12 block
    x[2, :32] = 2.0 ** -120                           # tiny exponent block
    x[3, 0] = 3.0e38                                  # near fp32 max (bf16 representable after rounding)
    x[3] = torch.from_numpy(x[3]).to(torch.bfloat16).to(torch.float32).numpy()
    # exact rounding ties after scaling: amax 256 -> scale 1, values k+0.5 ulp
    x[4, :32] = np.array([256.0] + [1.0625, 1.1875, 2.125, 2.375, 17.0, 19.0, 0.001953125 * 1.5] * 4 + [0.0] * 3,
                         dtype=np.float32)
    x[5, :32] = -x[4, :32]
    out = {"x": x}
    for backend in ("native", "lut"):
        mod = _import_ref("gen_mx_quant_allgather_data", backend)
        q, s, d = mod._quantize_fp8(torch.from_numpy(x), "E4M3", 1)
        out[f"{backend}_codes"] = q.view(torch.uint8).numpy()
        out[f"{backend}_scale"] = s.to(torch.float8_e8m0fnu).view(torch.uint8).numpy()
        out[f"{backend}_dequant"] = d.numpy()
        xt = np.ascontiguousarray(x[:, :128].T)       # [128, 24]: blocks along axis 0
        q0, s0, d0 = mod._quantize_fp8(torch.from_numpy(xt), "E4M3", 0)
        out[f"{backend}_axis0_codes"] = q0.view(torch.uint8).numpy()
        out[f"{backend}_axis0_scale"] = s0.to(torch.float8_e8m0fnu).view(torch.uint8).numpy()
    out["axis0_x"] = xt
    # MXFP4 e2m1
    mod = _import_ref("gen_mx_quant_allgather_data", "lut")
    x4 = x[6:, :96].copy()
    q4, s4, d4 = mod._quantize(torch.from_numpy(x4), "E2M1", 1)
    _, idx4 = mod._quantize_to_fp4_lut(q4, "E2M1")
    out["fp4_x"] = x4
    out["fp4_idx"] = idx4.numpy()
    out["fp4_packed"] = mod._pack_fp4_nibbles(idx4).numpy()
    out["fp4_scale"] = s4.to(torch.float8_e8m0fnu).view(torch.uint8).numpy()
    out["fp4_dequant"] = d4.numpy()
    np.savez_compressed(os.path.join(HERE, "mx_quant.npz"), **out)


def verify_fixture():
    vr = _import_ref("verify_result")
    ut = _import_ref("utils")
    g = torch.Generator().manual_seed(7)
    golden = torch.randn(4096, generator=g) * 8
    cases = []
    for dtype, k in ((torch.bfloat16, 4096), (torch.bfloat16, 512), (torch.float16, 1024), (torch.float16, 8192)):
        rtol = ut.get_rtol(dtype, k)
        good = golden.to(dtype)
        bad = good.clone()
        bad[17] = bad[17] + (2.5 * rtol * max(1.0, abs(float(golden[17]))))
        biased = (golden * (1 + 0.9 * rtol)).to(dtype)
        for name, act in (("good", good), ("bad", bad), ("biased", biased)):
            with contextlib.redirect_stdout(io.StringIO()):
                ok = vr.precision_performance_analysis(vr.OpTypes.COMPUTE_FLOAT, [golden], [act], rtol)
            cases.append((str(dtype).split(".")[-1], k, name, act.to(torch.float32).numpy(), bool(ok)))
    np.savez_compressed(os.path.join(HERE, "verify.npz"), golden=golden.numpy(),
                        dtypes=np.array([c[0] for c in cases]), ks=np.array([c[1] for c in cases]),
                        names=np.array([c[2] for c in cases]), actual=np.stack([c[3] for c in cases]),
                        ok=np.array([c[4] for c in cases]))


def dense_fixture(ref_root):
    utils_dir = os.path.join(ref_root, "examples", "utils")
    out = {}
    with tempfile.TemporaryDirectory() as td:
        # matmul-allreduce / reduce-scatter flavour: gen_data.py, 2 ranks, fp16
        subprocess.check_call([sys.executable, os.path.join(utils_dir, "gen_data.py"), "mmar", "float16", "2",
                               "24", "40", "64", "0", "0", td], stdout=subprocess.DEVNULL)
        for r in range(2):
            out[f"mmar_a{r}"] = np.fromfile(os.path.join(td, f"rank_{r}_a.bin"), dtype=np.float16).reshape(24, 64)
            out[f"mmar_b{r}"] = np.fromfile(os.path.join(td, f"rank_{r}_b.bin"), dtype=np.float16).reshape(64, 40)
        out["mmar_golden"] = np.fromfile(os.path.join(td, "golden.bin"), dtype=np.float32).reshape(24, 40)
    with tempfile.TemporaryDirectory() as td:
        subprocess.check_call([sys.executable, os.path.join(utils_dir, "gen_data_allgather_matmul.py"), "agmm", "bf16",
                               "2", "16", "40", "64", "0", "0", td], stdout=subprocess.DEVNULL)
        for r in range(2):
            out[f"agmm_a{r}"] = np.fromfile(os.path.join(td, f"rank_{r}_a.bin"), dtype=np.uint16).reshape(16, 64)
            out[f"agmm_b{r}"] = np.fromfile(os.path.join(td, f"rank_{r}_b.bin"), dtype=np.uint16).reshape(64, 40)
            out[f"agmm_golden{r}"] = np.fromfile(os.path.join(td, f"golden_{r}.bin"), dtype=np.float32).reshape(32, 40)
    np.savez_compressed(os.path.join(HERE, "dense.npz"), **out)


def swizzle_fixture(ref_root):
    src = open(os.path.join(ref_root, "docs", "comm_swizzle", "comm_swizzle_animation.py")).read()
    fn = [n for n in ast.parse(src).body if isinstance(n, ast.FunctionDef) and n.name == "comm_swizzle_get_coord"][0]
    code = compile(ast.Module(body=[fn], type_ignores=[]), "comm_swizzle_animation.py", "exec")
    configs = [(2, 2, 4, 2, 2, 0, False), (4, 4, 4, 8, 1, 0, False), (5, 1, 8, 20, 1, 0, False),
               (3, 2, 8, 4, 2, 0, True), (7, 1, 2, 3, 1, 0, False), (4, 2, 4, 2, 2, 1, False)]
    out = {"configs": np.array([[int(v) for v in c] for c in configs])}
    for ci, (gr, gc, gk, sr, sc, direction, det) in enumerate(configs):
        env = dict(SWIZZLE_DIRECTION=direction, CORE_SPLIT_ROW=sr, CORE_SPLIT_COL=sc, IS_DETERMINISTIC=False,
                   GRID_ROW=gr, GRID_COL=gc, GRID_RANK=gk, IS_RANK_SHIFT=True)
        # The script folds coreSplit to (row*col,1) in deterministic mode before calling;
        # the C++ template receives the split as given and only pins the group height.
        env["IS_DETERMINISTIC"] = det
        exec(code, env)
        total = gr * gc * gk
        out[f"table{ci}"] = np.array([env["comm_swizzle_get_coord"](i) for i in range(total)])
    np.savez_compressed(os.path.join(HERE, "comm_swizzle.npz"), **out)


def moe_fixture():
    gm = _import_ref("gen_data_moe")
    _import_ref("gen_mx_quant_allgather_data", "lut")
    out = {}
    # sub-functions on tiny inputs
    g = torch.Generator().manual_seed(3)
    ep, epr, top_k, m, k = 3, 2, 2, 7, 8
    e_num = ep * epr
    xs = [torch.randn((m, k), generator=g).to(torch.bfloat16) for _ in range(ep)]
    idx = [torch.argsort(torch.rand((m, e_num), generator=g), dim=-1)[:, :top_k].to(torch.int32) for _ in range(ep)]
    probs = [torch.softmax(torch.randn((m, top_k), generator=g), dim=-1) for _ in range(ep)]
    routed, rows, toks = [], [], []
    for r in range(ep):
        a, row_idx, t = gm.moe_init_routing_cpu(xs[r], idx[r], e_num, 0)
        routed.append(a.unsqueeze(0)); rows.append(row_idx); toks.append(t)
    with contextlib.redirect_stdout(io.StringIO()):
        recv, blocks = gm.alltoallv1(routed, toks, ep, epr, k, m * top_k * ep, 1)
        back = gm.alltoallv2(recv, toks, ep, epr, k)
        comb = [gm.unpermute_cpu(back[r], rows[r], probs[r]) for r in range(ep)]
    for r in range(ep):
        out[f"sub_x{r}"] = xs[r].to(torch.float32).numpy()
        out[f"sub_idx{r}"] = idx[r].numpy()
        out[f"sub_probs{r}"] = probs[r].numpy()
        out[f"sub_routed{r}"] = routed[r][0].to(torch.float32).numpy()
        out[f"sub_rowidx{r}"] = rows[r].numpy()
        out[f"sub_tokens{r}"] = toks[r].numpy()
        out[f"sub_recv{r}"] = recv[r][0].to(torch.float32).numpy()
        out[f"sub_blocks{r}"] = np.array(blocks[r])
        out[f"sub_back{r}"] = back[r][0].to(torch.float32).numpy()
        out[f"sub_combine{r}"] = comb[r].to(torch.float32).numpy()
    c = torch.randn((5, 16), generator=g).to(torch.bfloat16)
    act, gate = c.chunk(2, dim=-1)
    out["swiglu_in"] = c.to(torch.float32).numpy()
    out["swiglu_out"] = (act.float() * torch.sigmoid(act.float()) * gate.float()).to(torch.bfloat16).to(torch.float32).numpy()

    # full pipeline through the reference's own generator
    m, k, n, top_k, e_num, ep = 8, 256, 512, 2, 4, 2
    epr = e_num // ep
    with tempfile.TemporaryDirectory() as td:
        with contextlib.redirect_stdout(io.StringIO()):
            gm.generate_dispatch_ffn_combine(m, k, n, top_k, m * top_k, m * top_k, 0, ep, epr, 1, m * top_k * ep,
                                             torch.bfloat16, data_path=td, routing_mode="random")
        def rd(name, dt):
            return np.fromfile(os.path.join(td, name), dtype=dt)
        for r in range(ep):
            out[f"e2e_x{r}"] = rd(f"in_routing_matrix_a_{r}.bin", np.uint16).reshape(m, k)
            out[f"e2e_idx{r}"] = rd(f"in_routing_expert_idx_{r}.bin", np.int32).reshape(m, top_k)
            out[f"e2e_w1q{r}"] = rd(f"in_gmm_matrix_b_{r}.bin", np.uint8).reshape(epr, n, k)
            out[f"e2e_w1s{r}"] = rd(f"in_gmm_matrix_b_scale_{r}.bin", np.uint8).reshape(epr, n, k // 32)
            out[f"e2e_w2q{r}"] = rd(f"in_gmm_matrix_b2_{r}.bin", np.uint8).reshape(epr, k, n // 2)
            out[f"e2e_w2s{r}"] = rd(f"in_gmm_matrix_b2_scale_{r}.bin", np.uint8).reshape(epr, k, n // 2 // 32)
            out[f"e2e_gmm2{r}"] = rd(f"in_alltoallv2_permuted_{r}.bin", np.uint16).reshape(-1, k)
            out[f"e2e_back{r}"] = rd(f"out_alltoallv2_routed_back_{r}.bin", np.uint16).reshape(-1, k)
            out[f"e2e_probs{r}"] = rd(f"in_gather_gate_weight_{r}.bin", np.float32).reshape(m, top_k)
            out[f"e2e_rowidx{r}"] = rd(f"in_gather_expanded_row_idx_{r}.bin", np.int32)
            out[f"e2e_out{r}"] = rd(f"out_gather_combine_{r}.bin", np.uint16).reshape(m, k)
    out["e2e_shape"] = np.array([m, k, n, top_k, e_num, ep])
    np.savez_compressed(os.path.join(HERE, "moe.npz"), **out)



def _scales_from_pairs(raw, rows, kblocks_padded):
    """[rows, kb/2, 2] scale bytes -> [rows, kb]."""
    return raw.reshape(rows, kblocks_padded)


def mx_mmrs_fixture(ref_root):
    """MXFP8 (e5m2) Matmul-ReduceScatter: the example's own generator, 2 ranks, transB = 1."""
    sdir = os.path.join(ref_root, "examples", "ascend950_mxfp8_matmul_reduce_scatter", "scripts")
    sys.path.insert(0, sdir)
    mod = importlib.import_module("gen_data_mxfp8_mmrs")
    m, k, n, world = 32, 64, 48, 2
    out = {"shape": np.array([m, k, n, world])}
    torch.manual_seed(77)
    # the quantiser on its own: same draw as gen_data_fp8_e5m2 makes first
    x = torch.randn((8, 96), dtype=torch.float32) * 3.0
    qz = mod.MXFP8MatrixQuantizer(data_format="E5M2", axis=1, block_size=32)
    with contextlib.redirect_stdout(io.StringIO()):
        qx, sx = qz.quantize_matrix(x)
    out["q_x"] = x.numpy()
    out["q_codes"] = qx.to(torch.float8_e5m2).view(torch.uint8).numpy()
    out["q_scale"] = sx.to(torch.float8_e8m0fnu).view(torch.uint8).numpy()
    with tempfile.TemporaryDirectory() as td:
        hi, lo = [], []
        for r in range(world):
            with contextlib.redirect_stdout(io.StringIO()):
                c32, c16 = mod.gen_data(r, m, k, n, 0, 1, td)
            hi.append(c32)
            lo.append(c16)
            out[f"a{r}"] = np.fromfile(os.path.join(td, f"rank_{r}_a.bin"), dtype=np.uint8).reshape(m, k)
            out[f"b{r}"] = np.fromfile(os.path.join(td, f"rank_{r}_b.bin"), dtype=np.uint8).reshape(n, k)       # transB = 1
            out[f"a_scale{r}"] = np.fromfile(os.path.join(td, f"rank_{r}_a_scale.bin"), dtype=np.uint8).reshape(m, k // 64, 2)
            out[f"b_scale{r}"] = np.fromfile(os.path.join(td, f"rank_{r}_b_scale.bin"), dtype=np.uint8).reshape(n, k // 64, 2)
        total = hi[0] + hi[1]
        out["golden"] = torch.cat(list(torch.chunk(total, world, dim=0)), dim=0).numpy()
        out["golden_low"] = (lo[0] + lo[1]).view(torch.uint16).numpy()
    np.savez_compressed(os.path.join(HERE, "mx_mmrs.npz"), **out)


def alltoallv_gmm_fixture(ref_root):
    """Standalone MXFP8 AllToAllV-GroupedMatmul and GroupedMatmul-AllToAllV: the reference's
    generators run as scripts (2 ranks, 4 experts), files read back."""
    utils_dir = os.path.join(ref_root, "examples", "utils")
    env = dict(os.environ, PYTHONPATH=utils_dir)
    out = {}
    world, m, n, k, experts = 2, 16, 32, 64, 4
    out["shape"] = np.array([world, m, n, k, experts])
    with tempfile.TemporaryDirectory() as td:
        subprocess.check_call([sys.executable, os.path.join(utils_dir, "gen_data_fp8_mx_alltoallv_gmm.py"), "a2av_gmm",
                               "bf16", str(world), str(m), str(n), str(k), "0", "0", "--expert", str(experts), "--ep",
                               str(world), td], stdout=subprocess.DEVNULL, env=env)
        for r in range(world):
            out[f"d_a{r}"] = np.fromfile(os.path.join(td, f"input_a_{r}.bin"), dtype=np.uint8).reshape(m, k)
            out[f"d_a_scale{r}"] = np.fromfile(os.path.join(td, f"input_a_scale_{r}.bin"), dtype=np.uint8).reshape(m, k // 64, 2)
            out[f"d_b{r}"] = np.fromfile(os.path.join(td, f"input_b_{r}.bin"), dtype=np.uint8).reshape(experts // world, k, n)
            out[f"d_b_scale{r}"] = np.fromfile(os.path.join(td, f"input_b_scale_{r}.bin"), dtype=np.uint8).reshape(
                experts // world, k // 64, n, 2)
            out[f"d_local_tokens{r}"] = np.fromfile(os.path.join(td, f"local_tokens_per_expert_{r}.bin"), dtype=np.int32)
            out[f"d_global_tokens{r}"] = np.fromfile(os.path.join(td, f"global_tokens_per_local_expert_{r}.bin"),
                                                     dtype=np.int32).reshape(world, experts // world)
            out[f"d_golden{r}"] = np.fromfile(os.path.join(td, f"golden_{r}.bin"), dtype=np.float32).reshape(world * m, n)
    with tempfile.TemporaryDirectory() as td:
        os.makedirs(os.path.join(td, "output"))
        m2 = 32          # rows of A per owner; the generator draws m2 / world rows per (source, owner)
        out["c_m"] = np.array([m2])
        subprocess.check_call([sys.executable, os.path.join(utils_dir, "gen_data_gmm_alltoallv_fp8_mx.py"), "gmm_a2av",
                               "bf16", str(world), str(m2), str(n), str(k), "0", "0", "--expert", str(experts), "--ep",
                               str(world)], stdout=subprocess.DEVNULL, env=env, cwd=td)
        o = os.path.join(td, "output")
        for r in range(world):
            out[f"c_a{r}"] = np.fromfile(os.path.join(o, f"a_gm_{r}.bin"), dtype=np.uint8).reshape(m2, k)
            out[f"c_a_scale{r}"] = np.fromfile(os.path.join(o, f"a_scale_{r}.bin"), dtype=np.uint8).reshape(m2, k // 64, 2)
            out[f"c_b{r}"] = np.fromfile(os.path.join(o, f"b_gm_{r}.bin"), dtype=np.uint8).reshape(experts // world, k, n)
            out[f"c_b_scale{r}"] = np.fromfile(os.path.join(o, f"b_scale_{r}.bin"), dtype=np.uint8).reshape(
                experts // world, k // 64, n, 2)
            out[f"c_local_tokens{r}"] = np.fromfile(os.path.join(o, f"local_tokens_per_expert_{r}.bin"), dtype=np.int32)
            out[f"c_golden{r}"] = np.fromfile(os.path.join(o, f"golden_{r}.bin"), dtype=np.float32).reshape(world * m2, n)
    np.savez_compressed(os.path.join(HERE, "alltoallv_gmm.npz"), **out)



def fp4_agmm_fixture(ref_root):
    """MXFP4 (e2m1, E8M0 per 32) AllGather-Matmul: the reference's generator as a script, 2 ranks, transB = 1."""
    utils_dir = os.path.join(ref_root, "examples", "utils")
    env = dict(os.environ, PYTHONPATH=utils_dir)
    world, m, n, k = 2, 16, 32, 64
    out = {"shape": np.array([world, m, n, k])}
    with tempfile.TemporaryDirectory() as td:
        subprocess.check_call([sys.executable, os.path.join(utils_dir, "gen_data_fp4_mx_allgather_matmul.py"), "fp4agmm",
                               "bf16", str(world), str(m), str(n), str(k), "0", "1", td], stdout=subprocess.DEVNULL, env=env)
        for r in range(world):
            out[f"a{r}"] = np.fromfile(os.path.join(td, f"input_a_{r}.bin"), dtype=np.uint8).reshape(m, k // 2)
            out[f"a_scale{r}"] = np.fromfile(os.path.join(td, f"input_a_scale_{r}.bin"), dtype=np.uint8).reshape(m, -1)
            out[f"b{r}"] = np.fromfile(os.path.join(td, f"input_b_{r}.bin"), dtype=np.uint8).reshape(n, k // 2)    # B^T
            out[f"b_scale{r}"] = np.fromfile(os.path.join(td, f"input_b_scale_{r}.bin"), dtype=np.uint8).reshape(n, -1)
            out[f"golden{r}"] = np.fromfile(os.path.join(td, f"golden_{r}.bin"), dtype=np.float32).reshape(world * m, n)
    np.savez_compressed(os.path.join(HERE, "fp4_agmm.npz"), **out)


def main():
    if len(sys.argv) < 2:
        sys.exit("usage: make_golden.py /path/to/reference")
    ref_root = sys.argv[1]
    sys.path.insert(0, os.path.join(ref_root, "examples", "utils"))
    torch.manual_seed(0)
    mx_quant_fixture()
    verify_fixture()
    dense_fixture(ref_root)
    swizzle_fixture(ref_root)
    moe_fixture()
    mx_mmrs_fixture(ref_root)
    alltoallv_gmm_fixture(ref_root)
    fp4_agmm_fixture(ref_root)
    for f in sorted(os.listdir(HERE)):
        if f.endswith(".npz"):
            print(f, os.path.getsize(os.path.join(HERE, f)))


if __name__ == "__main__":
    main()
