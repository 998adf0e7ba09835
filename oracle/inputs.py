"""Seeded synthetic inputs for the five benchmark configurations and their
scaled-down twins.  Test infrastructure only (see package docstring).

The reference draws `randn` with an unseeded generator and reuses one A/B for
all ranks (examples/utils/gen_data.py:42-51); the distributions below are the
ones the benchmark configurations name, fed to the same golden functions.
"""
import numpy as np
import torch


def _gen(seed):
    g = torch.Generator()
    g.manual_seed(int(seed))
    return g


def uniform(shape, dtype, seed, lo=-1.0, hi=1.0):
    return (torch.rand(shape, generator=_gen(seed), dtype=torch.float32) * (hi - lo) + lo).to(dtype)


def normal(shape, dtype, seed, std=1.0):
    return (torch.randn(shape, generator=_gen(seed), dtype=torch.float32) * std).to(dtype)


def matmul_allreduce_inputs(world, m, k, n, dtype=torch.float16):
    """C1: per-rank A[m,k], B[k,n], uniform(-1,1), seed = rank (A) / 100+rank (B)."""
    return ([uniform((m, k), dtype, r) for r in range(world)],
            [uniform((k, n), dtype, 100 + r) for r in range(world)])


def allgather_matmul_inputs(world, m_local, k, n, dtype=torch.bfloat16):
    """C2: A_r[m_local,k] ~ N(0,1) seed r; B_r[k,n] ~ N(0,0.02) seed 1000+r."""
    return ([normal((m_local, k), dtype, r) for r in range(world)],
            [normal((k, n), dtype, 1000 + r, 0.02) for r in range(world)])


def matmul_reduce_scatter_inputs(world, m, k_local, n, dtype=torch.bfloat16):
    """C3: A_r[m,k_local] ~ N(0,1); B_r[k_local,n] ~ N(0,0.02)."""
    return ([normal((m, k_local), dtype, 2000 + r) for r in range(world)],
            [normal((k_local, n), dtype, 3000 + r, 0.02) for r in range(world)])


def zipf_topk_routing(m, expert_num, top_k, seed, s=1.1, bias_scale=1.0):
    """C5 routing: softmax(N(0,1) logits + per-expert bias proportional to the
    Zipf(s) rank weight) -> top-k ids (int32) and renormalised fp32 gate weights."""
    g = _gen(seed)
    logits = torch.randn((m, expert_num), generator=g, dtype=torch.float32)
    ranks = torch.arange(1, expert_num + 1, dtype=torch.float32)
    w = ranks.pow(-s)
    w = w / w.sum()
    perm = torch.randperm(expert_num, generator=_gen(seed + 7919))
    bias = torch.log(w * expert_num)[perm] * bias_scale
    p = torch.softmax(logits + bias, dim=-1)
    top_p, top_i = torch.topk(p, top_k, dim=-1)
    probs = (top_p / top_p.sum(dim=-1, keepdim=True)).to(torch.float32)
    return top_i.to(torch.int32).numpy(), probs.numpy()


def bf16_as_f32(t: torch.Tensor) -> np.ndarray:
    return t.to(torch.bfloat16).to(torch.float32).numpy()
