// MX quantisation + AllGather host entry point.
#pragma once
#include "common.h"
#include "symm_heap.h"

namespace cb {

struct MxqAgArgs {
    const void *input;   // bf16 [m, n]
    uint8_t *codes;      // e4m3 [R*m, n]
    uint8_t *scales;     // E8M0 [R*m, even(n/32)]
};

size_t mxq_allgather_symmetric_bytes(int world, int m, int n);
int launch_mx_quant_allgather(cudaStream_t stream, uint32_t block_num, const MxqAgArgs *args, void *symmetric, int m,
                              int n);

}  // namespace cb
