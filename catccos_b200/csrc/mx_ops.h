// Host entry points of the MXFP8 operators.
#pragma once
#include "common.h"
#include "symm_heap.h"

namespace cb {

struct MxAgArgs {
    const uint8_t *A;        // e4m3 [m, k]
    const uint8_t *B;        // e4m3: transB=0 [k, n]; transB=1 [n, k]
    void *C;                 // 16-bit [R*m, n]
    const uint8_t *a_scale;  // E8M0 [m, even(k/32)]  (reference layout [m, k/64, 2])
    const uint8_t *b_scale;  // transB=0: [k/64, n, 2];  transB=1: [n, even(k/32)]
    uint8_t *workspace;      // mx_ag_workspace_bytes() bytes of device memory
};

// fmt: 0 = MXFP8 (e4m3 codes, k bytes per row), 1 = MXFP4 (e2m1 codes, two per byte, K-major operands only)
size_t mx_ag_symmetric_bytes(int world, int m, int n, int k, int fmt = 0);
size_t mx_ag_workspace_bytes(int m, int n, int k);

// AllGather-Matmul on MXFP8 operands; out_dtype 1 = fp16, 27 = bf16.  m = rows held by one rank.
int launch_mx_allgather_matmul(int out_dtype, cudaStream_t stream, uint32_t block_num, const MxAgArgs *args,
                               void *symmetric, int m, int n, int k, int trans_b, int fmt = 0);

// Matmul-ReduceScatter on MXFP8 operands (codes `code_format` 0 = e4m3, 1 = e5m2; E8M0 scales per 32 along k):
// D_r = rows r*m/R .. of sum_s A_s B_s.  m = rows of the full product, k = this rank's share of the
// contraction; m/R must be a multiple of 128.  MxAgArgs as above with C = [m/R, n]; the symmetric region is that
// of the f16/bf16 Matmul-ReduceScatter (dense_symmetric_bytes), the workspace mx_ag_workspace_bytes(m, n, k).
// alltoall = 1: Matmul-AllToAll -- the same movement of row blocks without the sum, C = [m, n] with block s from rank s.
int launch_mx_matmul_reduce_scatter(int out_dtype, int code_format, cudaStream_t stream, uint32_t block_num,
                                    const MxAgArgs *args, void *symmetric, int m, int n, int k, int trans_b,
                                    int alltoall = 0);

}  // namespace cb
