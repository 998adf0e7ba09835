"""B200 implementation of the fused compute-communication operators (AllGather-Matmul,
Matmul-ReduceScatter, Matmul-AllReduce, MX quantisation, MoE dispatch/combine).

The product is the CUDA shared library `libcatccos_b200.so` (sources in `csrc/`, C-ABI in
`include/catccos_b200.h`); this package is its loader plus thin helpers that pass torch CUDA
tensors by pointer.
"""
from ._lib import CatccosError, CocTilingParams, KernelParams, lib, check  # noqa: F401
from . import runtime  # noqa: F401
