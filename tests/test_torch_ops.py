"""`torch.ops.catccos.*`: registration, schemas, shape inference and argument checks (CPU);
the CUDA path at world size 1 (GPU).  Reference: examples/torch_binding/src/torch_bindings.cpp."""
import pytest
import torch

import catccos_b200.torch_ops as tops  # noqa: F401  (registers the operators)


def test_operators_are_registered_with_the_reference_schemas():
    ops = torch.ops.catccos
    assert str(ops.init.default._schema) == \
        "catccos::init(int rank_id, int rank_size, int local_mem_size, str ip_port) -> int"
    assert str(ops.allgather_matmul.default._schema) == \
        "catccos::allgather_matmul(Tensor a, Tensor b, int rank_size) -> Tensor"
    assert str(ops.finalize.default._schema) == "catccos::finalize() -> int"
    assert hasattr(ops, "matmul_reduce_scatter") and hasattr(ops, "matmul_allreduce")


def test_meta_kernels_infer_shapes():
    a = torch.empty((96, 64), dtype=torch.float16, device="meta")
    b = torch.empty((64, 40), dtype=torch.float16, device="meta")
    assert torch.ops.catccos.allgather_matmul(a, b, 4).shape == (384, 40)
    assert torch.ops.catccos.matmul_reduce_scatter(a, b, 4).shape == (24, 40)
    assert torch.ops.catccos.matmul_allreduce(a, b, 4).shape == (96, 40)
    assert torch.ops.catccos.allgather_matmul(a, b, 4).dtype == torch.float16
    assert torch.ops.catccos.allgather_matmul_remote_read(a, b, 4).shape == (384, 40)
    c, g = torch.ops.catccos.allgather_matmul_with_gather_result(a, b, 4)
    assert c.shape == (384, 40) and g.shape == (384, 64)
    assert torch.ops.catccos.alltoall_matmul(a, b, 4).shape == (96, 40)
    assert torch.ops.catccos.matmul_alltoall(a, b, 4).shape == (96, 40)


def test_init_argument_checks_and_idle_finalize():
    with pytest.raises(RuntimeError, match="ip_port is empty"):
        torch.ops.catccos.init(0, 2, 1 << 20, "")
    with pytest.raises(RuntimeError, match="invalid rank_size"):
        torch.ops.catccos.init(0, 0, 1 << 20, "tcp://127.0.0.1:8788")
    with pytest.raises(RuntimeError, match="invalid rank_id"):
        torch.ops.catccos.init(-1, 2, 1 << 20, "tcp://127.0.0.1:8788")
    with pytest.raises(RuntimeError, match="invalid local_mem_size"):
        torch.ops.catccos.init(0, 2, 0, "tcp://127.0.0.1:8788")
    assert torch.ops.catccos.finalize() == 0          # nothing initialised: a no-op, as in the reference


def test_operand_checks_before_any_launch():
    a = torch.zeros((8, 8), dtype=torch.float16)
    with pytest.raises(RuntimeError, match="not initialized"):
        tops._check_operands(a, a, 1)
    tops._STATE.initialized, tops._STATE.rank_size = True, 2
    try:
        with pytest.raises(RuntimeError, match="rank_size mismatch"):
            tops._check_operands(a, a, 4)
        with pytest.raises(RuntimeError, match="Only float16 / bfloat16"):
            tops._check_operands(a.float(), a.float(), 2)
        with pytest.raises(RuntimeError, match="Only CUDA supported"):
            tops._check_operands(a, a, 2)
    finally:
        tops._STATE.initialized, tops._STATE.rank_size = False, 0


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_single_rank_operators_on_cuda(dtype):
    """World size 1: every operator degenerates to the plain GEMM; max relative error 1e-2
    against the fp32 product, normalised by max(1, |golden|) as the reference's checker does."""
    torch.manual_seed(5)
    m, k, n = 384, 256, 520
    a = torch.randn((m, k), device="cuda").to(dtype)
    b = (torch.randn((k, n), device="cuda") * 0.05).to(dtype)
    gold = a.float() @ b.float()
    assert torch.ops.catccos.init(0, 1, 64 << 20, "tcp://127.0.0.1:8799") == 0
    try:
        c, g = torch.ops.catccos.allgather_matmul_with_gather_result(a, b, 1)
        torch.cuda.synchronize()
        assert torch.equal(g, a) and ((c.float() - gold).abs() / gold.abs().clamp(min=1.0)).max().item() <= 1e-2
        for op in (torch.ops.catccos.allgather_matmul, torch.ops.catccos.matmul_reduce_scatter,
                   torch.ops.catccos.matmul_allreduce, torch.ops.catccos.allgather_matmul_remote_read,
                   torch.ops.catccos.alltoall_matmul, torch.ops.catccos.matmul_alltoall):
            c = op(a, b, 1)
            torch.cuda.synchronize()
            assert c.shape == (m, n) and c.dtype == dtype
            err = ((c.float() - gold).abs() / gold.abs().clamp(min=1.0)).max().item()
            assert err <= 1e-2, (op, err)
    finally:
        assert torch.ops.catccos.finalize() == 0
