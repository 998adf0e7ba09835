// Host entry points of the block-scaled FP4 GEMM (single rank).
#pragma once
#include "symm_heap.h"

namespace cb {

// format 0: MXFP4 (e2m1, UE8M0 scale per 32 along k, scale rows padded to an even count);
// format 1: NVFP4 (e2m1, UE4M3 scale per 16 along k; the fp32 tensor scales go into alpha).
size_t fp4_gemm_workspace_bytes(int format, int m, int n, int k);

// C[m, n] (16-bit, out_dtype 1 = fp16 / 27 = bf16) = alpha * A[m, k] x B[n, k]^T; A and B packed two e2m1 per byte
// (low nibble = even k), scales row-major [rows, scales per row].  k % 64 == 0, n % 8 == 0.  Asynchronous on `stream`.
int launch_fp4_gemm(cudaStream_t stream, int format, int out_dtype, const uint8_t *A, const uint8_t *B, void *C,
                    const uint8_t *a_scale, const uint8_t *b_scale, float alpha, int m, int n, int k, uint8_t *workspace,
                    uint32_t block_num);

}  // namespace cb
