"""One rank of a multi-process parity run: `python -m tests.mp_worker RANK WORLD PORT`.

Real one-process-per-GPU path: cuMem heap exchanged over unix sockets, peers mapped over NVLink,
operators launched through the C-ABI; every rank checks its own output against the CPU oracle."""
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
os.environ.setdefault("CATCCOS_WAIT_TIMEOUT_MS", "20000")


def main():
    rank, world, port = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3]
    import torch
    from catccos_b200 import runtime as rt
    from oracle import dense, inputs, verify
    torch.cuda.set_device(rank)
    rt.shmem_init(rank, world, 256 << 20, f"tcp://127.0.0.1:{port}")
    symm = rt.shmem_malloc(200 << 20)
    failures = []

    def check(name, out, gold, tol=1e-2):
        err = verify.max_rel_err(out.cpu(), gold)
        print(f"[rank {rank}] {name}: max rel err {err:.4g}", flush=True)
        if not err <= tol:
            failures.append((name, err))

    for rep in range(2):
        # AllGather-Matmul bf16
        m, k, n = 384, 512, 768
        a, b = inputs.allgather_matmul_inputs(world, m, k, n, torch.bfloat16)
        gold = dense.golden_allgather_matmul(a, b)[rank]
        c = torch.full((world * m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
        rt.launch(rt.ALLGATHER_MATMUL, a[rank].cuda(), b[rank].cuda(), c, symm, rt.tiling(m, k, n, world))
        rc, words = rt.last_status()
        assert rc == 0, words
        check(f"agmm#{rep}", c, gold)
        # Matmul-ReduceScatter bf16
        m, k, n = 1024, 256, 520
        a, b = inputs.matmul_reduce_scatter_inputs(world, m, k, n, torch.bfloat16)
        gold = dense.golden_matmul_reduce_scatter(a, b)[rank]
        d = torch.full((m // world, n), float("nan"), dtype=torch.bfloat16, device="cuda")
        rt.launch(rt.MATMUL_REDUCE_SCATTER, a[rank].cuda(), b[rank].cuda(), d, symm, rt.tiling(m, k, n, world))
        rc, words = rt.last_status()
        assert rc == 0, words
        check(f"mmrs#{rep}", d, gold)
        # Matmul-AllReduce fp16 (benchmark configuration 1 when world == 2)
        m, k, n = 512, 1024, 2048
        a, b = inputs.matmul_allreduce_inputs(world, m, k, n, torch.float16)
        gold = dense.golden_matmul_allreduce(a, b)
        e = torch.full((m, n), float("nan"), dtype=torch.float16, device="cuda")
        rt.launch(rt.MATMUL_ALLREDUCE, a[rank].cuda(), b[rank].cuda(), e, symm, rt.tiling(m, k, n, world))
        rc, words = rt.last_status()
        assert rc == 0, words
        check(f"mmar#{rep}", e, gold)
    rt.shmem_finalize()
    if failures:
        print(f"[rank {rank}] FAILED {failures}", flush=True)
        sys.exit(1)
    print(f"[rank {rank}] ok", flush=True)


if __name__ == "__main__":
    main()
