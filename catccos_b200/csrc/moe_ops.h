// Host entry points of the MoE dispatch -> FFN -> combine operator.
#pragma once
#include "moe_common.h"
#include "symm_heap.h"

namespace cb {

struct MoeArgs {
    const void *x;              // bf16 [m, K]
    const uint8_t *w1;          // e4m3 [E_local, N, K]   (gate/act rows first, up rows second)
    void *out;                  // bf16 [m, K]
    const uint8_t *w2;          // e4m3 [E_local, K, N/2]
    const int *expert_idx;      // int32 [m, topK]
    const float *probs;         // fp32 [m, topK]
    const uint8_t *w1_scale;    // E8M0 [E_local, N, K/32]
    const uint8_t *w2_scale;    // E8M0 [E_local, K, (N/2)/32]
    uint8_t *workspace;         // moe_workspace_bytes()
};

int moe_rows_cap(int world, int m, int top_k, int experts_per_rank);
size_t moe_symmetric_bytes(int world, int m, int k, int n, int top_k, int experts);
size_t moe_workspace_bytes(int world, int m, int k, int n, int top_k, int experts);

int launch_moe_dispatch_ffn_combine(cudaStream_t stream, uint32_t block_num, const MoeArgs *args, void *symmetric,
                                    int m, int k, int n, int top_k, int experts);

// kernels in moe_aux.cu
int moe_launch_route(const MoeParams &p, cudaStream_t stream);
int moe_launch_dispatch(const MoeParams &p, cudaStream_t stream);
int moe_launch_unpermute(const MoeParams &p, cudaStream_t stream);
int moe_launch_wait_dispatch(const MoeParams &p, cudaStream_t stream);

}  // namespace cb
