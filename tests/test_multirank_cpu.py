"""World-size-2 checks that need no GPU: the benchmark's reference arm under torchrun, and the
oracle's multi-rank goldens against real gloo collectives over the same per-rank partial products."""
import json
import os
import socket
import subprocess
import sys

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import dense, inputs

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _json_lines(text):
    return [json.loads(l) for l in text.splitlines() if l.startswith("{")]


def test_reference_arm_prints_one_contract_line():
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1",
                        "--warmup", "0"], capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert r.returncode == 0, r.stderr
    lines = _json_lines(r.stdout)
    assert len(lines) == 1
    d = lines[0]
    assert d["impl"] == "reference" and d["n_gpus"] == 1 and d["steps"] == 1 and d["higher_is_better"] is True
    assert d["unit"] == "TFLOP/s" and d["value"] > 0 and d["data"] == "synthetic" and d["vs_baseline"] is None
    assert d["cpu_baseline"]["kind"] == "port" and d["cpu_baseline"]["cores"] >= 1 and d["cpu_baseline"]["sample"]
    assert d["cpu_baseline"]["value"] == d["value"]
    assert d["e2e"] == {"value": d["value"], "unit": d["unit"], "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}


def test_reference_arm_under_torchrun_only_rank0_reports():
    port = _free_port()
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                        "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, "bench.py"),
                        "--impl", "reference", "--gpus", "2", "--steps", "1", "--warmup", "0"],
                       capture_output=True, text=True, timeout=900, cwd=ROOT)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = _json_lines(r.stdout)
    assert len(lines) == 1, r.stdout
    assert lines[0]["impl"] == "reference" and lines[0]["n_gpus"] == 2


def _gloo_worker(rank, world, port, m, k, n, out_dir):
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        # AllGather-Matmul: gather the row blocks with a real all_gather, multiply with this rank's B
        a, b = inputs.allgather_matmul_inputs(world, m, k, n, torch.bfloat16)
        mine = a[rank].float()
        parts = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(parts, mine)
        ag = torch.cat(parts, dim=0) @ b[rank].float()
        # Matmul-ReduceScatter / AllReduce: reduce the fp32 partial products with real collectives
        a2, b2 = inputs.matmul_reduce_scatter_inputs(world, m * world, k, n, torch.bfloat16)
        partial = a2[rank].float() @ b2[rank].float()
        rs = torch.empty((m, n))
        dist.reduce_scatter(rs, list(torch.chunk(partial.clone(), world, dim=0)))
        ar = partial.clone()
        dist.all_reduce(ar)
        np.savez(os.path.join(out_dir, f"r{rank}.npz"), ag=ag.numpy(), rs=rs.numpy(), ar=ar.numpy())
    finally:
        dist.destroy_process_group()


def test_oracle_goldens_equal_gloo_collectives(tmp_path):
    """The goldens restate the reference's single-process generators; here two real ranks exchange
    the same data through gloo and must arrive at the same numbers (fp32 sums of two terms commute,
    so the match is exact up to the matmul's own blocking)."""
    world, m, k, n = 2, 24, 64, 40
    port = _free_port()
    mp.spawn(_gloo_worker, args=(world, port, m, k, n, str(tmp_path)), nprocs=world, join=True)
    a, b = inputs.allgather_matmul_inputs(world, m, k, n, torch.bfloat16)
    g_ag = dense.golden_allgather_matmul(a, b)
    a2, b2 = inputs.matmul_reduce_scatter_inputs(world, m * world, k, n, torch.bfloat16)
    g_rs = dense.golden_matmul_reduce_scatter(a2, b2)
    g_ar = dense.golden_matmul_allreduce(a2, b2)
    for r in range(world):
        f = np.load(os.path.join(tmp_path, f"r{r}.npz"))
        assert np.allclose(f["ag"], g_ag[r].numpy(), rtol=1e-6, atol=1e-6)
        assert np.allclose(f["rs"], g_rs[r].numpy(), rtol=1e-6, atol=1e-6)
        assert np.allclose(f["ar"], g_ar.numpy(), rtol=1e-6, atol=1e-6)
