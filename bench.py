#!/usr/bin/env python3
"""Benchmark of the fused compute-communication hot path on B200.

    python bench.py --gpus N --steps K --warmup W [--op agmm|mmrs|mmar] [--impl reference]

One process per GPU (torchrun sets RANK / LOCAL_RANK / WORLD_SIZE / MASTER_*).  A "step" is one
launch of the fused operator through the C-ABI.  Rank 0 prints ONE JSON line.

Workload (default, `--op agmm`): AllGather-Matmul bf16 with the gathered A fixed at [8192, 8192]
and a per-rank weight B [8192, 4096]: at N GPUs every rank holds 8192/N rows of A and computes the
whole [8192, 4096] product with its own B, so the work per GPU is the same at every N (weak
scaling) and N = 8 is the benchmark's 8-rank configuration (A_local [1024, 8192]).  At N = 1 the
all-gather degenerates and the step is the plain tcgen05 GEMM.  Inputs are synthetic (seeded
normal(0,1) activations, normal(0,0.02) weights); A + B + C = 268 MB per rank, larger than the
126 MB L2, so consecutive steps do not find their operands in cache.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

M_TOTAL, K_DIM, N_DIM = 8192, 8192, 4096           # allgather_matmul bf16 (benchmark configuration 2)
RS_M, RS_KLOCAL, RS_N = 8192, 2048, 8192           # matmul_reduce_scatter bf16 (configuration 3)
AR_M, AR_K, AR_N = 512, 1024, 2048                 # matmul_allreduce fp16 (configuration 1)
MX_M_TOTAL, MX_K, MX_N = 16384, 7168, 4096         # MXFP8 allgather_matmul (configuration 4)
MOE_M, MOE_K, MOE_N, MOE_TOPK = 4096, 7168, 4096, 8  # MoE (configuration 5), 32 experts per rank
SPEC_BF16_TFLOPS, SPEC_NVLINK_GBS = 2250.0, 900.0  # datasheet: dense bf16 tensor peak, NVLink 5 per direction
NVLINK_GBS = 770.0                                 # measured peer-copy bandwidth per direction (900 nominal)


def measured_peaks(sustained):
    """Measured cuBLAS bf16 peak of this GPU type: the sustained figure when the timed steps sit inside
    a long load bracket, the burst figure when they are timed cold."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        key = "bf16_tflops_sustained" if sustained else "bf16_tflops"
        return float(d[key]), float(d["hbm_gbs"]), f"measured ({'sustained' if sustained else 'burst'} cuBLAS bf16)"
    return (1400.0 if sustained else 1590.0), 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.samples = []
        self.proc = None
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 6:
                self.samples.append(parts)

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        self.proc.terminate()           # the exact process started above
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        clocks, maxes, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in self.samples:
            try:
                clocks.append(float(s[0]))
                maxes.append(float(s[1]))
            except ValueError:
                continue
            for name, val in zip(names, s[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(clocks) if clocks else None,
                "sm_max_mhz": max(maxes) if maxes else None, "reasons": sorted(reasons),
                "samples": len(clocks)}


CPU_BASELINE_SECONDS = 10.0        # timed CPU work of the cpu_baseline leg


def workload(op, world):
    if op == "agmm":
        m_local = M_TOTAL // world
        return dict(name="allgather_matmul_bf16", m=m_local, k=K_DIM, n=N_DIM, a_shape=(m_local, K_DIM),
                    b_shape=(K_DIM, N_DIM), c_shape=(M_TOTAL, N_DIM), flops=2.0 * M_TOTAL * K_DIM * N_DIM,
                    comm_bytes=(world - 1) * m_local * K_DIM * 2, dtype="bf16",
                    desc=f"allgather_matmul bf16: gathered A[8192,8192] (A_local[{m_local},8192] per rank) x "
                         f"B[8192,4096] per rank -> C[8192,4096]")
    if op == "mmrs":
        return dict(name="matmul_reduce_scatter_bf16", m=RS_M, k=RS_KLOCAL, n=RS_N, a_shape=(RS_M, RS_KLOCAL),
                    b_shape=(RS_KLOCAL, RS_N), c_shape=(RS_M // world, RS_N), flops=2.0 * RS_M * RS_KLOCAL * RS_N,
                    comm_bytes=(world - 1) * (RS_M // world) * RS_N * 2, dtype="bf16",
                    desc=f"matmul_reduce_scatter bf16: A[8192,2048] x B[2048,8192] per rank, summed over ranks, "
                         f"rows scattered -> D[{RS_M // world},8192]")
    if op == "mmar":
        return dict(name="matmul_allreduce_fp16", m=AR_M, k=AR_K, n=AR_N, a_shape=(AR_M, AR_K), b_shape=(AR_K, AR_N),
                    c_shape=(AR_M, AR_N), flops=2.0 * AR_M * AR_K * AR_N,
                    comm_bytes=2 * (world - 1) * AR_M * AR_N * 2 // max(world, 1), dtype="fp16",
                    desc="matmul_allreduce fp16: A[512,1024] x B[1024,2048] per rank, summed over ranks")
    if op == "mxag":
        m_local = MX_M_TOTAL // world
        return dict(name="mxfp8_allgather_matmul", m=m_local, k=MX_K, n=MX_N, c_shape=(MX_M_TOTAL, MX_N),
                    flops=2.0 * MX_M_TOTAL * MX_K * MX_N, comm_bytes=(world - 1) * m_local * (MX_K + MX_K // 32),
                    dtype="mxfp8", peak_scale=2.0,
                    desc=f"MXFP8 allgather_matmul: activations [{m_local},7168] per rank in e4m3 + E8M0/32 (quantised from "
                         f"bf16 normal(0,1) at set-up), gathered [16384,7168] x W[7168,4096] e4m3 -> bf16 [16384,4096]")
    if op == "mxrs":
        return dict(name="mxfp8_matmul_reduce_scatter", m=RS_M, k=RS_KLOCAL, n=RS_N, c_shape=(RS_M // world, RS_N),
                    flops=2.0 * RS_M * RS_KLOCAL * RS_N, comm_bytes=(world - 1) * (RS_M // world) * RS_N * 2,
                    dtype="mxfp8", peak_scale=2.0,
                    desc=f"MXFP8 matmul_reduce_scatter: A[8192,2048] x B[2048,8192] per rank in e4m3 + E8M0/32 (quantised from "
                         f"bf16 at set-up), summed over ranks, rows scattered -> bf16 D[{RS_M // world},8192]")
    if op == "moe":
        experts = 32 * world
        return dict(name="moe_dispatch_ffn_combine", m=MOE_M, k=MOE_K, n=MOE_N, top_k=MOE_TOPK, experts=experts,
                    flops=float(MOE_M * MOE_TOPK) * (2.0 * MOE_K * MOE_N + 2.0 * (MOE_N // 2) * MOE_K),
                    comm_bytes=int((world - 1) / max(world, 1) * MOE_M * MOE_TOPK * (MOE_K + MOE_K // 32 + 2 * MOE_K)),
                    dtype="mxfp8", peak_scale=2.0, c_shape=(MOE_M, MOE_K),
                    desc=f"MoE dispatch->GMM->SwiGLU->GMM->combine: 4096 tokens/rank, hidden 7168, {experts} experts "
                         f"(32/rank), FFN 2048, top-8 Zipf(1.1) routing, MXFP8 weights")
    if op == "fp4":
        return dict(name="nvfp4_gemm", m=M_TOTAL, k=K_DIM, n=N_DIM, c_shape=(M_TOTAL, N_DIM), flops=2.0 * M_TOTAL * K_DIM * N_DIM,
                    comm_bytes=0, dtype="nvfp4", peak_scale=4.0,
                    desc="NVFP4 GEMM (one rank; the contraction under the FP4 operators): A[8192,8192] x B[4096,8192]^T, e2m1 "
                         "codes with one UE4M3 scale per 16 along K (seeded random codes and scales), bf16 output [8192,4096]")
    if op == "quant":
        return dict(name="mx_quant_e4m3", m=MX_M_TOTAL, k=MX_K, n=0, c_shape=(MX_M_TOTAL, MX_K), flops=0.0, comm_bytes=0,
                    dtype="u8", hbm_bytes=MX_M_TOTAL * MX_K * (2 + 1 + 1.0 / 32),
                    desc="MX quantisation bf16 [16384,7168] -> e4m3 + E8M0 per 32 (HBM-bound)")
    raise ValueError(op)


def host_inputs(wl, rank, torch):
    dt = torch.float16 if wl["dtype"] == "fp16" else torch.bfloat16
    g = torch.Generator().manual_seed(1234 + rank)
    if wl["dtype"] == "fp16":
        a = (torch.rand(wl["a_shape"], generator=g) * 2 - 1).to(dt)
        b = (torch.rand(wl["b_shape"], generator=g) * 2 - 1).to(dt)
    else:
        a = torch.randn(wl["a_shape"], generator=g).to(dt)
        b = (torch.randn(wl["b_shape"], generator=g) * 0.02).to(dt)
    return a, b, dt



def bind_to_gpu_numa_node(local_rank, torch):
    """Runs this process on the CPUs of the NUMA node its GPU hangs off, so that pinned host buffers
    allocated afterwards are node-local (first touch) and host<->device copies do not cross the
    socket interconnect.  Best effort: returns the node or None."""
    try:
        pr = torch.cuda.get_device_properties(local_rank)
        dev = f"{pr.pci_domain_id:04x}:{pr.pci_bus_id:02x}:{pr.pci_device_id:02x}.0"
        with open(f"/sys/bus/pci/devices/{dev}/numa_node") as f:
            node = int(f.read().strip())
        if node < 0:
            return None
        with open(f"/sys/devices/system/node/node{node}/cpulist") as f:
            cpus = set()
            for part in f.read().strip().split(","):
                lo, _, hi = part.partition("-")
                cpus.update(range(int(lo), int(hi or lo) + 1))
        allowed = cpus & os.sched_getaffinity(0)
        if allowed:
            os.sched_setaffinity(0, allowed)
            return node
    except (OSError, ValueError, AttributeError):
        pass
    return None


TOL = {"bf16": 1e-2, "fp16": 1e-2, "mxfp8": 2e-2, "nvfp4": 5e-2}


def _sample_rows(n_rows, count, seed, torch):
    """Seeded row sample that always holds the first and the last row."""
    count = min(count, n_rows)
    g = torch.Generator().manual_seed(seed)
    idx = torch.randperm(n_rows, generator=g)[:count]
    idx[0] = 0
    idx[-1] = n_rows - 1
    return torch.unique(idx)


def _rel_err(actual, golden, torch):
    from oracle import verify                      # checker only
    return verify.max_rel_err(actual, golden)


def parity_dense(op, wl, rank, world, a_h, b_h, c_dev, torch):
    """Compares a seeded sample of this rank's output rows with the fp32 CPU golden of the operator
    (the oracle port of the reference's host golden) on the same seeded inputs.  Runs after the timed
    region.  Returns (max relative error, rows checked)."""
    from oracle import dense                       # checker only
    if op == "agmm":
        m = wl["m"]
        sources = sorted({rank, (rank + 1) % world, (rank + world - 1) % world, (rank + world // 2) % world})
        per_src = max(64, 512 // len(sources))
        worst, rows = 0.0, 0
        bf = b_h.to(torch.float32)
        for s in sources:
            a_s = a_h if s == rank else host_inputs(wl, s, torch)[0]
            idx = _sample_rows(m, per_src, 777 + s, torch)
            gold = torch.matmul(a_s[idx].to(torch.float32), bf)
            got = c_dev[(s * m + idx).cuda()].cpu()
            worst = max(worst, _rel_err(got, gold, torch))
            rows += idx.numel()
        return worst, rows
    # reduce family: this rank's output rows are sums over all ranks' products
    m_total = wl["m"]
    if op == "mmrs":
        mr = m_total // world
        idx_out = _sample_rows(mr, 256, 555 + rank, torch)
        idx_in = idx_out + rank * mr
    else:
        idx_out = _sample_rows(m_total, 256, 555, torch)
        idx_in = idx_out
    gold = None
    for r in range(world):
        a_r, b_r = (a_h, b_h) if r == rank else host_inputs(wl, r, torch)[:2]
        part = dense.matmul_fp32(a_r[idx_in], b_r)
        gold = part if gold is None else gold + part
    got = c_dev[idx_out.cuda()].cpu()
    return _rel_err(got, gold, torch), idx_out.numel()


def _dequant_e4m3_fast(codes, scales, torch):
    """dequant of MXFP8 rows on the host: uint8 codes [r, k], E8M0 bytes [r, >= k/32] -> fp32 [r, k]
    (table lookup of the oracle's e4m3 decoding; oracle.mxquant.dequant_mx_e4m3 is the slow form)."""
    import numpy as np
    from oracle import mxquant                     # checker only
    lut = torch.from_numpy(mxquant.e4m3_to_f32(np.arange(256, dtype=np.uint8)))
    r, k = codes.shape
    v = lut[codes.to(torch.int64)].view(r, k // 32, 32)
    sc = torch.exp2(scales[:, :k // 32].to(torch.float32) - 127.0)
    return (v * sc[:, :, None]).view(r, k)


def parity_mxag(wl, rank, world, act, a_codes, a_scale, wq_t, ws_t, c_dev, torch, dist):
    """MXFP8 AllGather-Matmul: the step's own quantisation must be bit-exact (codes and scales of a
    row sample against the oracle), and sampled rows of the gathered product (own rows, nearest
    and farthest peers) must match dequant(A) x dequant(B) in fp32."""
    import numpy as np
    from oracle import mxquant                     # checker only
    m, k = wl["m"], wl["k"]
    idx = _sample_rows(m, 96, 4242, torch)         # the same local rows on every rank
    mine = act[idx.cuda()].contiguous()
    if world > 1:
        allrows = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(allrows, mine)
    else:
        allrows = [mine]
    q, sc, _ = mxquant.quantize_mx_e4m3(mine.cpu().to(torch.float32).numpy(), "rne")
    bit_exact = bool(np.array_equal(q, a_codes[idx.cuda()].cpu().numpy()) and
                     np.array_equal(sc[:, :k // 32], a_scale[idx.cuda()].cpu().numpy()[:, :k // 32]))
    b_deq_t = _dequant_e4m3_fast(wq_t.cpu(), ws_t.cpu(), torch)             # [n, k]
    worst, rows = 0.0, 0
    for s in sorted({rank, (rank + 1) % world, (rank + world - 1) % world, (rank + world // 2) % world}):
        qs, ss, a_deq = mxquant.quantize_mx_e4m3(allrows[s].cpu().to(torch.float32).numpy(), "rne")
        gold = torch.matmul(torch.from_numpy(a_deq), b_deq_t.t())
        got = c_dev[(s * m + idx).cuda()].cpu()
        worst = max(worst, _rel_err(got, gold, torch))
        rows += idx.numel()
    return worst, rows, bit_exact


def parity_moe(wl, rank, world, x, idx_dev, probs, expert_weights, c_dev, torch):
    """MoE: the full dispatch -> GEMM1 -> SwiGLU -> quant -> GEMM2 -> combine -> un-permute golden
    (oracle.moe stages) for a few of this rank's tokens, using the weights of whichever experts,
    local or remote, those tokens were routed to."""
    import numpy as np
    from oracle import moe, mxquant                # checker only
    k, n, top_k = wl["k"], wl["n"], wl["top_k"]
    toks = _sample_rows(wl["m"], 3, 31 + rank, torch)
    xs = x[toks.cuda()].cpu().to(torch.float32).numpy()
    ids = idx_dev[toks.cuda()].cpu().numpy()
    pr = probs[toks.cuda()].cpu().numpy()
    _, _, x_deq = mxquant.quantize_mx_e4m3(xs, "rne")
    cols = _sample_rows(k, 512, 99, torch)          # output columns checked (GEMM2 rows of W2)
    rows_back = np.zeros((len(toks), top_k, cols.numel()), dtype=np.float32)
    for e in np.unique(ids):
        q1, s1, q2, s2 = expert_weights(int(e))
        w1 = _dequant_e4m3_fast(q1.cpu(), s1.cpu(), torch)                   # [n, k]
        w2 = _dequant_e4m3_fast(q2[cols.cuda()].cpu(), s2[cols.cuda()].cpu(), torch)   # [cols, n/2]
        t_sel, k_sel = np.nonzero(ids == e)
        c1 = torch.matmul(torch.from_numpy(x_deq[t_sel]), w1.t()).to(torch.bfloat16).to(torch.float32).numpy()
        glu = moe.swiglu_bf16(c1)
        _, _, g_deq = mxquant.quantize_mx_e4m3(glu, "rne")
        c2 = torch.matmul(torch.from_numpy(g_deq), w2.t()).to(torch.bfloat16).to(torch.float32).numpy()
        rows_back[t_sel, k_sel] = c2
    acc = np.zeros((len(toks), cols.numel()), dtype=np.float32)
    for j in range(top_k):                          # fp32 multiply then add in slot order, as moe.unpermute_fp32
        acc = (acc + rows_back[:, j] * pr[:, j:j + 1].astype(np.float32)).astype(np.float32)
    gold = torch.from_numpy(mxquant.bf16_bits_to_f32(mxquant.f32_to_bf16_bits(acc)).reshape(acc.shape))
    got = c_dev[toks.cuda()][:, cols.cuda()].cpu()
    return _rel_err(got, gold, torch), int(toks.numel())


def repeat_for(seconds, fn):
    """Runs fn() (which returns (rate, cores, secs, ...)) until `seconds` of timed CPU work have accumulated;
    returns the median rate, the cores, the total timed seconds and the number of runs."""
    rates, total, cores, last = [], 0.0, 1, None
    while total < seconds and len(rates) < 200:
        last = fn()
        rates.append(last[0])
        cores = last[1]
        total += last[2]
    return statistics.median(rates), cores, total, len(rates), last


def cpu_golden_rate(wl, sample_rows, torch):
    """Times the CPU golden (oracle port of the reference's torch fp32 matmul) on a bounded sample:
    `sample_rows` rows of the (gathered / full) A against one rank's B."""
    from oracle import dense                      # checker, used here only as the timed CPU baseline
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    g = torch.Generator().manual_seed(99)
    dt = torch.float16 if wl["dtype"] == "fp16" else torch.bfloat16
    k, n = wl["b_shape"]
    a = torch.randn((sample_rows, k), generator=g).to(dt)
    b = (torch.randn((k, n), generator=g) * 0.02).to(dt)
    dense.matmul_fp32(a[:64], b)                  # warm the thread pool
    t0 = time.perf_counter()
    dense.matmul_fp32(a, b)
    dt_s = time.perf_counter() - t0
    flops = 2.0 * sample_rows * k * n
    return flops / dt_s / 1e12, cores, dt_s


_MX_SAMPLE = {}


def cpu_golden_rate_mx(wl, op, torch):
    """CPU golden of the block-scaled operators on a bounded sample: MX-dequantise the operands, fp32 matmul
    (the reference's host golden does exactly that: gen_data_fp8_mx_allgather_matmul.py, gen_data_moe.py:546-588);
    for the MoE one expert's up projection, SwiGLU, re-quantisation and down projection on 1024 rows."""
    import numpy as np
    from oracle import dense, moe, mxquant          # checker, used here only as the timed CPU baseline
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    rows, k, n = 1024, wl["k"], wl["n"]
    key = (op, k, n)
    if key not in _MX_SAMPLE:                      # seeded operands, quantised once (set-up, not timed)
        rng = np.random.default_rng(5)
        x = rng.standard_normal((rows, k)).astype(np.float32)
        xq, xs, _ = mxquant.quantize_mx_e4m3(x, "rne")
        w1 = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
        w1q, w1s, _ = mxquant.quantize_mx_e4m3(w1, "rne")
        w2q = w2s = None
        if op == "moe":
            w2 = (rng.standard_normal((k, n // 2)) * 0.02).astype(np.float32)
            w2q, w2s, _ = mxquant.quantize_mx_e4m3(w2, "rne")
        _MX_SAMPLE[key] = (x, w1, xq, xs, w1q, w1s, w2q, w2s)
    x, w1, xq, xs, w1q, w1s, w2q, w2s = _MX_SAMPLE[key]
    dense.matmul_fp32(torch.from_numpy(x[:64]), torch.from_numpy(w1.T.copy()))       # warm the thread pool
    t0 = time.perf_counter()
    tn = torch.from_numpy
    a = _dequant_e4m3_fast(tn(xq), tn(xs), torch)
    b = _dequant_e4m3_fast(tn(w1q), tn(w1s), torch)
    c1 = torch.matmul(a, b.t())
    flops = 2.0 * rows * k * n
    what = f"{rows} of {wl['c_shape'][0]} rows: MX dequantise + fp32 matmul against the full weight"
    if op == "moe":
        c1 = c1.to(torch.bfloat16).to(torch.float32).numpy()
        glu = moe.swiglu_bf16(c1)
        _, _, g_deq = mxquant.quantize_mx_e4m3(glu, "rne")
        b2 = _dequant_e4m3_fast(tn(w2q), tn(w2s), torch)
        torch.matmul(torch.from_numpy(g_deq), b2.t()).to(torch.bfloat16)
        flops += 2.0 * rows * (n // 2) * k
        what = f"{rows} of {wl['m'] * wl['top_k']} routed rows through one expert: dequantise, up projection, SwiGLU, MX quantise, down projection (fp32 matmuls)"
    dt_s = time.perf_counter() - t0
    return flops / dt_s / 1e12, cores, dt_s, what


def run_reference(args, rank, world):
    """`--impl reference`: the reference's own implementation of the path is its CPU host golden
    (its device code targets Ascend NPUs and cannot be built here); rank 0 times the oracle port of
    that golden on the host cores, the other ranks exit."""
    if rank != 0:
        return
    import torch
    wl = workload(args.op, max(world, 1))
    if args.op in ("quant", "fp4"):
        print(json.dumps({"impl": "reference", "unavailable": f"no reference-arm leg for --op {args.op}: the reference has "
                          "no host golden timed for it (use --op agmm|mmrs|mmar|mxag|moe)"}), flush=True)
        return
    rows = 1024 if args.op != "mmar" else AR_M
    vals = []
    cores = os.cpu_count() or 1
    if args.op in ("mxag", "moe"):
        for _ in range(min(args.warmup, 1)):
            cpu_golden_rate_mx(wl, args.op, torch)
        for _ in range(args.steps):
            v, cores, secs, sample = cpu_golden_rate_mx(wl, args.op, torch)
            vals.append(v)
        value = statistics.median(vals)
        ms = secs * 1e3
        sample += f", {args.steps} runs, median"
    else:
        for _ in range(args.warmup):
            cpu_golden_rate(wl, min(rows, 256), torch)
        for _ in range(args.steps):
            v, cores, _ = cpu_golden_rate(wl, rows, torch)
            vals.append(v)
        value = statistics.median(vals)
        sample = f"{rows} of {wl['c_shape'][0] if args.op == 'agmm' else wl['m']} rows of A x full B, fp32 matmul, {args.steps} runs, median"
        ms = (2.0 * rows * wl["b_shape"][0] * wl["b_shape"][1]) / (value * 1e12) * 1e3
    line = {
        "impl": "reference", "metric": "fused-op TFLOP/s (whole job)", "value": value, "unit": "TFLOP/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": wl["desc"], "op": wl["name"]},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--op", default="agmm", choices=["agmm", "mmrs", "mmar", "mxag", "mxrs", "moe", "quant", "fp4"])
    ap.add_argument("--variant", default="push", choices=["push", "remote_read", "gather_result"],
                    help="--op agmm only: data flow of the all-gather (push = AllGatherMatmul, the headline)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-parity", action="store_true")
    ap.add_argument("--mx-quant-in-step", action="store_true",
                    help="mxag: quantise the bf16 activations inside every timed step (the reference operator takes "
                         "operands that are already MXFP8, so by default the quantisation is set-up, timed on its own)")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world != args.gpus and world == 1 and args.gpus > 1:
        raise SystemExit("launch with torchrun for --gpus > 1 (one process per GPU)")

    if args.impl == "reference":
        run_reference(args, rank, world)
        return

    import ctypes
    import torch
    import torch.distributed as dist
    from catccos_b200 import runtime as rt
    from catccos_b200 import lib, check

    assert args.warmup >= 3, "at least 3 warm-up steps"
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    wl = workload(args.op, world)
    port = os.environ.get("MASTER_PORT", "29500")
    addr = os.environ.get("MASTER_ADDR", "127.0.0.1")
    stream = torch.cuda.current_stream()
    sptr = ctypes.c_void_p(stream.cuda_stream)
    dense_op = args.op in ("agmm", "mmrs", "mmar")
    a_h = b_h = None
    if dense_op:
        comm = {"agmm": rt.ALLGATHER_MATMUL, "mmrs": rt.MATMUL_REDUCE_SCATTER, "mmar": rt.MATMUL_ALLREDUCE}[args.op]
        if args.op == "agmm" and args.variant != "push":
            comm = rt.ALLGATHER_MATMUL_REMOTE_READ if args.variant == "remote_read" else rt.ALLGATHER_MATMUL_WITH_GATHER_RESULT
        a_h, b_h, dt = host_inputs(wl, rank, torch)
        til = rt.tiling(wl["m"], wl["k"], wl["n"], world)
        dtype_code = rt.FP16 if wl["dtype"] == "fp16" else rt.BF16
        need = rt.symmetric_bytes(comm, dtype_code, til)
        rt.shmem_init(rank, world, 2 * max(need, 1 << 20) + (8 << 20), f"tcp://{addr}:{port}")
        symm = rt.shmem_malloc(max(need, 1024))
        a_d, b_d = a_h.cuda(), b_h.cuda()
        c_d = torch.empty(wl["c_shape"], dtype=dt, device="cuda")

        gathered = None
        if comm == rt.ALLGATHER_MATMUL_WITH_GATHER_RESULT:
            gathered = torch.empty((world * wl["m"], wl["k"]), dtype=dt, device="cuda")

        def step():
            rt.launch(comm, a_d, b_d, c_d, symm, til, stream=stream, custom=[gathered] if gathered is not None else None)
        launches_per_step = 1
    else:
        gen = torch.Generator(device="cuda").manual_seed(4321 + rank)

        def quant_rows(x_bf16):
            rows, kk = x_bf16.shape
            codes = torch.empty((rows, kk), dtype=torch.uint8, device="cuda")
            scales = torch.empty((rows, (kk // 32 + 1) // 2 * 2), dtype=torch.uint8, device="cuda")
            check(lib().catccos_mx_quant(sptr, ctypes.c_void_p(x_bf16.data_ptr()), ctypes.c_void_p(codes.data_ptr()),
                                         ctypes.c_void_p(scales.data_ptr()), None, rows, kk))
            return codes, scales
        if args.op == "quant":
            rt.shmem_init(rank, world, 1 << 20, f"tcp://{addr}:{port}")
            x = torch.randn((wl["m"], wl["k"]), generator=gen, device="cuda", dtype=torch.float32).to(torch.bfloat16)
            q_codes = torch.empty((wl["m"], wl["k"]), dtype=torch.uint8, device="cuda")
            q_scales = torch.empty((wl["m"], wl["k"] // 32), dtype=torch.uint8, device="cuda")

            def step():
                check(lib().catccos_mx_quant(sptr, ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(q_codes.data_ptr()),
                                             ctypes.c_void_p(q_scales.data_ptr()), None, wl["m"], wl["k"]))
            launches_per_step = 1
        elif args.op == "fp4":
            rt.shmem_init(rank, world, 1 << 20, f"tcp://{addr}:{port}")
            m, k, n = wl["m"], wl["k"], wl["n"]
            # any byte is a pair of e2m1 codes; scales: UE4M3 bytes 0x28..0x47 (2^-2 .. 1.875 x 2^1)
            fa = torch.randint(0, 256, (m, k // 2), generator=gen, device="cuda", dtype=torch.uint8)
            fb = torch.randint(0, 256, (n, k // 2), generator=gen, device="cuda", dtype=torch.uint8)
            fsa = torch.randint(0x28, 0x48, (m, k // 16), generator=gen, device="cuda", dtype=torch.uint8)
            fsb = torch.randint(0x28, 0x48, (n, k // 16), generator=gen, device="cuda", dtype=torch.uint8)
            f_alpha = 2.0 ** -6
            c_d = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
            wsp = torch.zeros(lib().catccos_fp4_gemm_workspace_bytes(1, m, n, k), dtype=torch.uint8, device="cuda")

            def step():
                check(lib().catccos_fp4_gemm(sptr, 1, rt.BF16, ctypes.c_void_p(fa.data_ptr()), ctypes.c_void_p(fb.data_ptr()),
                                             ctypes.c_void_p(c_d.data_ptr()), ctypes.c_void_p(fsa.data_ptr()),
                                             ctypes.c_void_p(fsb.data_ptr()), ctypes.c_float(f_alpha), m, n, k,
                                             ctypes.c_void_p(wsp.data_ptr()), 0))
            launches_per_step = 3
        elif args.op == "mxag":
            comm = rt.FP8_MX_ALLGATHER_MATMUL
            til = rt.tiling(wl["m"], wl["k"], wl["n"], world)
            need = rt.symmetric_bytes(comm, rt.BF16, til)
            rt.shmem_init(rank, world, 2 * max(need, 1 << 20) + (8 << 20), f"tcp://{addr}:{port}")
            symm = rt.shmem_malloc(max(need, 1024))
            act = torch.randn((wl["m"], wl["k"]), generator=gen, device="cuda", dtype=torch.float32).to(torch.bfloat16)
            w = (torch.randn((wl["k"], wl["n"]), generator=gen, device="cuda", dtype=torch.float32) * 0.02).to(torch.bfloat16)
            wq_t, ws_t = quant_rows(w.t().contiguous())                      # quantised along K, [n, k]
            b_codes = wq_t.t().contiguous()                                  # [k, n]
            kb = wl["k"] // 32
            b_scale = ws_t[:, :kb].t().contiguous().reshape(kb // 2, 2, wl["n"]).permute(0, 2, 1).contiguous()
            a_codes = torch.empty((wl["m"], wl["k"]), dtype=torch.uint8, device="cuda")
            a_scale = torch.empty((wl["m"], kb), dtype=torch.uint8, device="cuda")
            c_d = torch.empty(wl["c_shape"], dtype=torch.bfloat16, device="cuda")
            wsp = torch.zeros(lib().catccos_workspace_bytes(comm, rt.BF16, ctypes.byref(til)), dtype=torch.uint8, device="cuda")

            def quant_act():
                check(lib().catccos_mx_quant(sptr, ctypes.c_void_p(act.data_ptr()), ctypes.c_void_p(a_codes.data_ptr()),
                                             ctypes.c_void_p(a_scale.data_ptr()), None, wl["m"], wl["k"]))
            quant_act()

            def step():
                if args.mx_quant_in_step:
                    quant_act()
                rt.launch(comm, a_codes, b_codes, c_d, symm, til, stream=stream, dtype=rt.BF16,
                          custom=[a_scale, b_scale], workspace=wsp)
            launches_per_step = 4 if args.mx_quant_in_step else 3
        elif args.op == "mxrs":
            comm = rt.MXFP8_MATMUL_REDUCE_SCATTER
            til = rt.tiling(wl["m"], wl["k"], wl["n"], world)
            need = rt.symmetric_bytes(comm, rt.BF16, til)
            rt.shmem_init(rank, world, max(need, 1 << 20) + (8 << 20), f"tcp://{addr}:{port}")
            symm = rt.shmem_malloc(max(need, 1024))

            def mxrs_operands(r):
                """MXFP8 operands of rank r, seeded by r so that every rank can rebuild its peers' for the parity check."""
                gr = torch.Generator(device="cuda").manual_seed(8800 + r)
                a_bf = torch.randn((wl["m"], wl["k"]), generator=gr, device="cuda", dtype=torch.float32).to(torch.bfloat16)
                w_bf = (torch.randn((wl["n"], wl["k"]), generator=gr, device="cuda", dtype=torch.float32) * 0.02).to(torch.bfloat16)
                aq, asc = quant_rows(a_bf)
                wq, wsc = quant_rows(w_bf)                    # K-major weights [n, k] (transB = 1)
                return aq, asc, wq, wsc
            a_codes, a_scale, wq_t, ws_t = mxrs_operands(rank)
            c_d = torch.empty(wl["c_shape"], dtype=torch.bfloat16, device="cuda")
            wsp = torch.zeros(lib().catccos_workspace_bytes(comm, rt.BF16, ctypes.byref(til)), dtype=torch.uint8, device="cuda")
            kp_rs = rt.KernelParams()
            kp_rs.ptrA, kp_rs.ptrB, kp_rs.ptrC = a_codes.data_ptr(), wq_t.data_ptr(), c_d.data_ptr()
            cust_rs = (ctypes.c_void_p * 2)(a_scale.data_ptr(), ws_t.data_ptr())
            kp_rs.customPtrs = ctypes.cast(cust_rs, ctypes.POINTER(ctypes.c_void_p))
            kp_rs.customCount = 2

            def step():      # the e4m3 form of the operator (the reference's example feeds e5m2 codes to the same kernel)
                check(lib().LaunchAscend950MxFp8E4M3MatmulReduceScatterBF16(sptr, 0, 0, ctypes.byref(kp_rs),
                                                                             ctypes.c_void_p(wsp.data_ptr()), ctypes.c_void_p(symm),
                                                                             ctypes.byref(til), 0, 1))
            launches_per_step = 3
        else:   # moe
            comm = rt.DISPATCH_FFN_COMBINE
            m, k, n, top_k, experts = wl["m"], wl["k"], wl["n"], wl["top_k"], wl["experts"]
            el = experts // world
            til = rt.tiling(m, k, n, world, topK=top_k, expertNum=experts, epSize=world)
            need = rt.symmetric_bytes(comm, rt.BF16, til)
            rt.shmem_init(rank, world, 2 * need + (8 << 20), f"tcp://{addr}:{port}")
            symm = rt.shmem_malloc(need)
            x = torch.randn((m, k), generator=gen, device="cuda", dtype=torch.float32).to(torch.bfloat16)
            w1q = torch.empty((el, n, k), dtype=torch.uint8, device="cuda")
            w1s = torch.empty((el, n, k // 32), dtype=torch.uint8, device="cuda")
            w2q = torch.empty((el, k, n // 2), dtype=torch.uint8, device="cuda")
            w2s = torch.empty((el, k, (n // 2) // 32), dtype=torch.uint8, device="cuda")
            def expert_weights(e_global):
                """MXFP8 weights of one expert, seeded by its global index so that every rank can
                regenerate them (the parity check needs the weights of experts other ranks own)."""
                ge = torch.Generator(device="cuda").manual_seed(9000 + e_global)
                wt = (torch.randn((n, k), generator=ge, device="cuda", dtype=torch.float32) * 0.02).to(torch.bfloat16)
                q1, s1 = quant_rows(wt)
                wt = (torch.randn((k, n // 2), generator=ge, device="cuda", dtype=torch.float32) * 0.02).to(torch.bfloat16)
                q2, s2 = quant_rows(wt)
                return q1, s1[:, :k // 32], q2, s2[:, :(n // 2) // 32]
            for e in range(el):
                w1q[e], w1s[e], w2q[e], w2s[e] = expert_weights(rank * el + e)
            # top-8 routing: softmax(N(0,1) logits + log of a Zipf(1.1) weight per expert), renormalised gate weights
            logits = torch.randn((m, experts), generator=gen, device="cuda")
            zipf = torch.arange(1, experts + 1, device="cuda", dtype=torch.float32).pow(-1.1)
            zipf = zipf / zipf.sum()
            perm = torch.randperm(experts, generator=torch.Generator().manual_seed(7)).cuda()
            pr = torch.softmax(logits + torch.log(zipf * experts)[perm], dim=-1)
            top_p, top_i = torch.topk(pr, top_k, dim=-1)
            probs = (top_p / top_p.sum(dim=-1, keepdim=True)).float().contiguous()
            idx = top_i.to(torch.int32).contiguous()
            c_d = torch.empty((m, k), dtype=torch.bfloat16, device="cuda")
            wsp = torch.zeros(lib().catccos_workspace_bytes(comm, rt.BF16, ctypes.byref(til)), dtype=torch.uint8, device="cuda")
            # rows every expert owner receives (explains the max-over-ranks time under skewed routing)
            owner_rows = torch.bincount((idx.flatten() // el).to(torch.int64), minlength=world).to(torch.float64)
            if world > 1:
                dist.all_reduce(owner_rows)
            moe_imbalance = float(owner_rows.max() / owner_rows.mean())
            torch.cuda.synchronize()

            def step():
                rt.launch(comm, x, w1q, c_d, symm, til, stream=stream, dtype=rt.BF16,
                          custom=[w2q, idx, probs, w1s, w2s], workspace=wsp)
            launches_per_step = 10

    for _ in range(args.warmup):
        step()
    barrier()
    rc, words = rt.last_status()
    if rc != 0:
        raise SystemExit(f"device wait ran out during warm-up: {words}")

    def max_over_ranks(x):
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # nvidia-smi samples every 100 ms and the timed region can be much shorter, so the timed
    # steps are bracketed by identical untimed launches (about 0.6 s before, 0.2 s after): the clock
    # samples then describe the GPU under the same load, and the number is a sustained one.  Every
    # rank runs the same bracket (the launches are collective).
    load_steps = 0
    if not os.environ.get("BENCH_NO_LOAD_BRACKET"):
        t0 = time.perf_counter()
        for _ in range(10):
            step()
        torch.cuda.synchronize()
        load_steps = int(min(20000, max(args.warmup, 0.6 / max(max_over_ranks((time.perf_counter() - t0) / 10), 1e-6))))

    def timed_region(sample_clocks):
        sampler = ClockSampler(local_rank) if (rank == 0 and sample_clocks) else None
        if sampler:
            sampler.start()
        for _ in range(load_steps):
            step()
        barrier()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record(stream)
        for _ in range(args.steps):
            step()
        ev1.record(stream)
        torch.cuda.synchronize()
        ms = ev0.elapsed_time(ev1)
        for _ in range(load_steps // 3):
            step()
        barrier()
        clk = sampler.stop() if sampler else None
        if clk is not None:
            clk["load_bracket_steps"] = load_steps
        rc_, words_ = rt.last_status()
        if rc_ != 0:
            raise SystemExit(f"device wait ran out: {words_}")
        return max_over_ranks(ms) / args.steps, clk

    ms_per_step, clocks = timed_region(True)

    # compute-only twin under the same load bracket (peer data already in place, no flags, no
    # pushes): exposed communication = (fused - compute-only) / fused
    exposed = None
    compute_only_ms = None
    if world > 1 and args.op in ("agmm", "mmrs", "mmar", "mxag", "mxrs"):
        check(lib().catccos_debug_set_flags(1))
        compute_only_ms, _ = timed_region(False)
        check(lib().catccos_debug_set_flags(0))
        barrier()
        exposed = max(0.0, (ms_per_step - compute_only_ms) / ms_per_step)

    # MoE: one more step with CUDA events between its stages (outside the timed region); every stage's time as the
    # max over ranks, plus the times of the rank that receives the most rows
    moe_stage_ms = None
    if args.op == "moe":
        check(lib().catccos_debug_set_flags(2))
        step()
        barrier()
        check(lib().catccos_debug_set_flags(0))
        buf = (ctypes.c_float * 12)()
        n_st = lib().catccos_debug_moe_stage_ms(buf, 12)
        names = ["route", "quant_dispatch", "weight_scale_atoms", "wait_dispatch", "recv_scale_atoms", "gemm1_swiglu_quant",
                 "gemm2_combine", "unpermute"]
        if n_st == len(names):
            mine = torch.tensor([buf[i] for i in range(n_st)], dtype=torch.float64, device="cuda")
            worst = mine.clone()
            if world > 1:
                dist.all_reduce(worst, op=dist.ReduceOp.MAX)
            moe_stage_ms = {"max_over_ranks": {nm: round(float(v), 4) for nm, v in zip(names, worst.tolist())},
                            "rank0": {nm: round(float(v), 4) for nm, v in zip(names, mine.tolist())}}

    # end to end through the host-buffer entry point: H2D of the step's inputs, fused launch, D2H of the result,
    # every step.  Dense operators copy A and B; the block-scaled GEMM and the MoE keep their weights (and weight
    # scales) resident after the first call and copy activations / routing every step.
    e2e = None
    if not args.no_e2e and args.op in ("agmm", "mmrs", "mmar", "mxag", "moe") and args.variant == "push":
        numa_node = bind_to_gpu_numa_node(local_rank, torch)
        pin = lambda t_: t_.cpu().pin_memory()
        if dense_op:
            ins, cust, mask, e2e_dtype = [a_h.pin_memory(), b_h.pin_memory()], [], 1 << 1, dtype_code
            per_step = [0]
            c_p = torch.empty(wl["c_shape"], dtype=dt).pin_memory()
            resident_note = "B (this rank's weight shard) resident after the first call; A travels every step"
        elif args.op == "mxag":
            ins, cust, mask, e2e_dtype = [pin(a_codes), pin(b_codes)], [pin(a_scale), pin(b_scale)], (1 << 1) | (1 << 4), rt.BF16
            per_step = [0, 2]
            c_p = torch.empty(wl["c_shape"], dtype=torch.bfloat16).pin_memory()
            resident_note = "weights and weight scales resident after the first call"
        else:
            ins, cust = [pin(x), pin(w1q)], [pin(w2q), pin(idx), pin(probs), pin(w1s), pin(w2s)]
            mask, e2e_dtype = (1 << 1) | (1 << 3) | (1 << 6) | (1 << 7), rt.BF16
            per_step = [0, 3, 4]
            c_p = torch.empty(wl["c_shape"], dtype=torch.bfloat16).pin_memory()
            resident_note = "expert weights and weight scales resident after the first call"
        every = ins + cust
        h2d_bytes = sum(every[i].numel() * every[i].element_size() for i in per_step)
        cust_arr = (ctypes.c_void_p * max(len(cust), 1))(*[c_.data_ptr() for c_ in cust])

        def e2e_step():
            check(lib().catccos_run_host_resident(comm, e2e_dtype, 0, ctypes.c_void_p(ins[0].data_ptr()),
                                                  ctypes.c_void_p(ins[1].data_ptr()), ctypes.c_void_p(c_p.data_ptr()),
                                                  cust_arr if cust else None, len(cust), ctypes.byref(til), 0, 0, mask))
        for _ in range(3):
            e2e_step()
        barrier()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            e2e_step()
        barrier()
        e2e_s = max_over_ranks(time.perf_counter() - t0)
        e2e = {"value": world * wl["flops"] * args.steps / e2e_s / 1e12, "unit": "TFLOP/s",
               "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": c_p.numel() * 2,
               "ms_per_step": e2e_s / args.steps * 1e3, "host_numa_node": numa_node}
        if resident_note:
            e2e["resident"] = resident_note
        # the copy that came back must be the device result (guards against a stale host buffer)
        if not torch.equal(c_p[:64], c_d[:64].cpu()):
            raise SystemExit("end-to-end result differs from the device-resident result")

    # parity: after the timed region, one more plain step, then a seeded sample of this rank's output
    # against the CPU golden (oracle) on every rank; the worst rank is reported and a miss fails the run
    parity = None
    if not args.no_parity:
        step()
        barrier()
        rc_, words_ = rt.last_status()
        if rc_ != 0:
            raise SystemExit(f"device wait ran out: {words_}")
        bit_exact = None
        if dense_op:
            err, rows = parity_dense(args.op, wl, rank, world, a_h, b_h, c_d, torch)
        elif args.op == "mxag":
            err, rows, bit_exact = parity_mxag(wl, rank, world, act, a_codes, a_scale, wq_t, ws_t, c_d, torch, dist)
        elif args.op == "mxrs":
            # rows of this rank's output block: sum over all ranks of dequant(A_s)[row] x dequant(B_s)
            ridx = _sample_rows(wl["m"] // world, 48, 77, torch)
            gold = None
            for r_ in range(world):
                aq_, as_, wq_, ws_ = (a_codes, a_scale, wq_t, ws_t) if r_ == rank else mxrs_operands(r_)
                rows_g = (rank * (wl["m"] // world) + ridx).cuda()
                part = torch.matmul(_dequant_e4m3_fast(aq_[rows_g].cpu(), as_[rows_g].cpu(), torch),
                                    _dequant_e4m3_fast(wq_.cpu(), ws_.cpu(), torch).t())
                gold = part if gold is None else gold + part
            err, rows = _rel_err(c_d[ridx.cuda()].cpu(), gold, torch), int(ridx.numel())
        elif args.op == "moe":
            err, rows = parity_moe(wl, rank, world, x, idx, probs, expert_weights, c_d, torch)
        elif args.op == "fp4":
            from oracle import mxquant             # checker only
            ridx = _sample_rows(wl["m"], 128, 17, torch)
            a_deq = mxquant.dequant_nvfp4(fa[ridx.cuda()].cpu().numpy(), fsa[ridx.cuda()].cpu().numpy(), 1.0, wl["k"])
            b_deq = mxquant.dequant_nvfp4(fb.cpu().numpy(), fsb.cpu().numpy(), f_alpha, wl["k"])
            gold = torch.matmul(torch.from_numpy(a_deq), torch.from_numpy(b_deq).t())
            err, rows = _rel_err(c_d[ridx.cuda()].cpu(), gold, torch), int(ridx.numel())
        else:   # quant: bit-exact codes and scales on a row sample
            import numpy as np
            from oracle import mxquant             # checker only
            ridx = _sample_rows(wl["m"], 256, 11, torch)
            q, sc, _ = mxquant.quantize_mx_e4m3(x[ridx.cuda()].cpu().to(torch.float32).numpy(), "rne")
            bit_exact = bool(np.array_equal(q, q_codes[ridx.cuda()].cpu().numpy()) and
                             np.array_equal(sc[:, :wl["k"] // 32], q_scales[ridx.cuda()].cpu().numpy()))
            err, rows = 0.0, int(ridx.numel())
        tol = TOL.get(wl["dtype"], 0.0)
        if err != err:                              # NaN
            err = float("inf")
        err = max_over_ranks(err)
        if bit_exact is not None:
            bit_exact = max_over_ranks(0.0 if bit_exact else 1.0) == 0.0
        parity = {"max_rel_err": err, "rows": rows, "tol": tol, "ranks_checked": world,
                  "golden": "fp32 CPU golden (oracle) on the same seeded inputs, sampled rows of every rank's output",
                  "ok": bool(err <= tol and bit_exact is not False)}
        if bit_exact is not None:
            parity["quant_bit_exact"] = bit_exact

    if rank == 0:
        peak_tf, peak_hbm, peak_kind = measured_peaks(load_steps > 0)
        if args.op == "quant":
            gbs = wl["hbm_bytes"] / (ms_per_step * 1e-3) / 1e9
            line = {
                "metric": "MX quantisation GB/s (whole job)", "value": world * gbs, "unit": "GB/s", "n_gpus": world,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "u8", "data": "synthetic",
                "config": {"workload": wl["desc"], "op": wl["name"], "l2": "operands (235 MB) larger than L2"},
                "roofline": {"bound": "hbm", "achieved": gbs, "peak": peak_hbm, "unit": "GB/s", "frac": gbs / peak_hbm,
                             "traffic": None, "peak_kind": "of measured (STREAM-style copy)"},
                "e2e": None, "gpu_launches": args.steps * launches_per_step, "clocks": clocks, "parity": parity,
            }
            print(json.dumps(line), flush=True)
        else:
            peak_tf *= wl.get("peak_scale", 1.0)      # fp8 tensor peak taken as twice the measured bf16 figure
            if wl.get("peak_scale"):
                peak_kind = f"{wl['peak_scale']:g} x " + peak_kind
            per_gpu_tflops = wl["flops"] / (ms_per_step * 1e-3) / 1e12
            t_gemm_us = wl["flops"] / (peak_tf * 1e12) * 1e6
            t_comm_us = wl["comm_bytes"] / (NVLINK_GBS * 1e9) * 1e6
            traffic = None
            tpath = os.path.join(ROOT, "profiles", "dram_traffic.json")
            if os.path.exists(tpath):
                with open(tpath) as f:
                    traffic = json.load(f).get(f"{wl['name']}_n{world}")
            line = {
                "metric": "fused-op TFLOP/s (whole job)", "value": world * per_gpu_tflops, "unit": "TFLOP/s",
                "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
                "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": wl["dtype"],
                "data": "synthetic",
                "config": {"workload": wl["desc"], "op": wl["name"], "l2": "operands larger than L2 (126 MB)",
                           "parallelism": (f"ep{world}" if args.op == "moe" else "replicas" if args.op == "fp4" else f"tp{world}")},
                "tflops_per_gpu": per_gpu_tflops,
                "roofline": {"bound": "tensor", "achieved": per_gpu_tflops, "peak": peak_tf, "unit": "TFLOP/s",
                             "frac": per_gpu_tflops / peak_tf, "traffic": traffic, "peak_kind": f"of {peak_kind}",
                             "t_gemm_peak_us": t_gemm_us, "t_comm_peak_us": t_comm_us,
                             "frac_of_max_gemm_comm": max(t_gemm_us, t_comm_us) / (ms_per_step * 1e3),
                             # the same against the datasheet: dense tensor peak (2250 TFLOP/s bf16, x2 fp8, x4 fp4) and
                             # 900 GB/s NVLink per direction
                             "spec_peak": SPEC_BF16_TFLOPS * wl.get("peak_scale", 1.0),
                             "frac_of_spec_peak": per_gpu_tflops / (SPEC_BF16_TFLOPS * wl.get("peak_scale", 1.0)),
                             "frac_of_spec_max_gemm_comm":
                                 max(wl["flops"] / (SPEC_BF16_TFLOPS * wl.get("peak_scale", 1.0) * 1e12),
                                     wl["comm_bytes"] / (SPEC_NVLINK_GBS * 1e9)) / (ms_per_step * 1e-3)},
                "exposed_comm_frac": exposed, "compute_only_ms_per_step": compute_only_ms,
                "e2e": e2e, "gpu_launches": args.steps * launches_per_step, "clocks": clocks, "parity": parity,
            }
            if args.op == "agmm" and args.variant != "push":
                line["config"]["variant"] = args.variant
            if args.op == "moe":
                line["config"]["hottest_rank_rows_over_mean"] = moe_imbalance
                line["stage_ms"] = moe_stage_ms
            if args.op == "mxag":
                line["config"]["activation_quantisation"] = "inside every step" if args.mx_quant_in_step else \
                    "at set-up (operands reach the operator as MXFP8, as in the reference)"
            if world == 1 and not args.no_cpu_baseline and dense_op:
                rows_s = min(2048, wl["a_shape"][0])
                v, cores, secs, runs, _ = repeat_for(CPU_BASELINE_SECONDS, lambda: cpu_golden_rate(wl, rows_s, torch))
                line["cpu_baseline"] = {"value": v, "unit": "TFLOP/s", "cores": cores, "kind": "port",
                                        "sample": f"{rows_s} rows of A x full B fp32 matmul, {runs} runs, median ({secs:.1f} s of CPU work)"}
            elif world == 1 and not args.no_cpu_baseline and args.op in ("mxag", "moe"):
                v, cores, secs, runs, last = repeat_for(CPU_BASELINE_SECONDS, lambda: cpu_golden_rate_mx(wl, args.op, torch))
                line["cpu_baseline"] = {"value": v, "unit": "TFLOP/s", "cores": cores, "kind": "port",
                                        "sample": f"{last[3]}, {runs} runs, median ({secs:.1f} s of CPU work)"}
            print(json.dumps(line), flush=True)

    rt.shmem_finalize()
    if world > 1:
        dist.destroy_process_group()
    if parity is not None and not parity["ok"]:
        raise SystemExit(f"parity check failed: {parity}")


if __name__ == "__main__":
    main()
