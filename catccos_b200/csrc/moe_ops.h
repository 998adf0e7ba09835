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

// Standalone MXFP8 AllToAllV-GroupedMatmul (op 0) and GroupedMatmul-AllToAllV (op 1): rows already quantised and
// sorted by expert, weights [E_local, k, n] with scales [E_local, k/64, n, 2], 16-bit output.
struct A2avArgs {
    const uint8_t *a;            // e4m3 [m, k]: op 0 rows in global-expert order, op 1 rows in owner order
    const uint8_t *b;            // e4m3 [E_local, k, n]
    void *c;                     // [world*m, n]: op 0 received rows (owner order), op 1 returned rows (expert order); rest zero
    const uint8_t *a_scale;      // E8M0 [m, k/64, 2]
    const uint8_t *b_scale;      // E8M0 [E_local, k/64, n, 2]
    const int *local_tokens;     // int32 [experts]
    uint8_t *workspace;          // a2av_workspace_bytes()
};
// fmt: 0 = MXFP8 (weights [E_local, k, n]), 1 = MXFP4 (two e2m1 codes per byte, weights K-major [E_local, n, k/2], k % 256 == 0)
size_t a2av_symmetric_bytes(int op, int world, int m, int n, int k, int experts, int fmt = 0);
size_t a2av_workspace_bytes(int op, int world, int m, int n, int k, int experts);
int launch_a2av(int op, int out_dtype, cudaStream_t stream, uint32_t block_num, const A2avArgs *args, void *symmetric,
                int m, int n, int k, int experts, int fmt = 0);

// kernels in moe_aux.cu
int a2av_launch_expert_idx(const MoeParams &p, const A2avPtrs &ptrs, cudaStream_t stream);
int a2av_launch_move_rows(const MoeParams &p, const A2avPtrs &ptrs, int mode, cudaStream_t stream);
int a2av_launch_copy_out(const MoeParams &p, int n_cols, cudaStream_t stream);
int moe_launch_route(const MoeParams &p, cudaStream_t stream);
int moe_launch_dispatch(const MoeParams &p, cudaStream_t stream);
int moe_launch_unpermute(const MoeParams &p, cudaStream_t stream);
// stage times of the last dispatch-FFN-combine launch made with debug flag 2 set; returns the number of stages
int moe_stage_ms(float *ms, int capacity);
int moe_launch_wait_dispatch(const MoeParams &p, cudaStream_t stream);

}  // namespace cb
