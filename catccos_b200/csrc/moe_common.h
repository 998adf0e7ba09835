// MoE dispatch -> grouped GEMM -> SwiGLU -> grouped GEMM -> combine: shared definitions.
//
// Pipeline per rank (stream order): route -> quant+dispatch -> GEMM1(+SwiGLU+quant) -> GEMM2(+combine)
// -> unpermute.  Tokens are quantised once (MX e4m3 / E8M0 per 32) and written straight into the
// expert owner's receive buffer; GEMM2's epilogue writes every output row straight back into its
// source rank's combine buffer at the row's position in that rank's expert-sorted order.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdint>

#include "common.h"

namespace cb {

constexpr int kMoeMaxExperts = 512;        // global experts (routing kernel keeps [32 warps][E] counters in smem)
constexpr int kMoeMaxLocalExperts = 64;

// Flag words (from kFlagOpBase) used by the MoE pipeline; each has one writer per source rank.
constexpr uint32_t kMoeFlagCounts = kFlagOpBase;                    // [R] counts of rank s have arrived
constexpr uint32_t kMoeFlagDispatch = kFlagOpBase + kMaxRanks;      // [R] rank s finished writing my receive rows
constexpr uint32_t kMoeFlagCombine = kFlagOpBase + 2 * kMaxRanks;   // [R] owner o finished writing my combine rows

// Device-side bookkeeping of one rank (lives in the caller's workspace).
struct MoeMeta {
    int counts_all[kMaxRanks][kMoeMaxExperts];      // copy of the symmetric counts (tokens[r][e])
    int prefix_all[kMaxRanks][kMoeMaxExperts];      // exclusive prefix over e: first permuted row of expert e on rank r
    int dest_base[kMoeMaxExperts];                  // for my tokens of expert e: first row in the owner's receive buffer
    int seg_base[kMoeMaxLocalExperts + 1];          // my local experts: first receive row (multiple of 128); [E_local] = end
    int seg_rows[kMoeMaxLocalExperts];              // my local experts: rows received
    int cum_src[kMaxRanks + 1][kMoeMaxLocalExperts];// [r][le] rows of local expert le coming from ranks < r
    int tile_prefix[kMoeMaxLocalExperts + 1];       // exclusive prefix of row tiles (128 rows) over local experts
    int total_rows;                                 // rows received (unpadded)
    unsigned int done_counter[4];                   // last-CTA-out counters of the pipeline's kernels
    int tile_queue[2][2];                           // next-tile counters of the two pair GEMMs (zeroed by the routing kernel)
    int overflow;                                   // receive buffer too small for the routing
};

struct MoeRankArgs {
    const void *x;             // bf16 [m, K]
    const int *expert_idx;     // int32 [m, topK]
    const float *probs;        // fp32 [m, topK]
    void *out;                 // bf16 [m, K]
    int *expanded_row_idx;     // int32 [m*topK]: src (token*topK+k) -> row in my expert-sorted order
    MoeMeta *meta;
};

struct MoeLayout {
    // byte offsets inside the symmetric heap (identical on every PE)
    uint64_t counts_off;       // int32 [R][E]
    uint64_t recv_codes_off;   // u8 [rows_cap, K]
    uint64_t recv_scale_off;   // u8 [rows_cap, scale_ld]
    uint64_t combine_off;      // bf16 [m*topK, K]
    int rows_cap;              // receive rows available per rank (multiple of 128)
    int scale_ld;              // even(K/32)
};

// Inputs of the standalone all-to-all-v operators, per local rank: rows that are already MXFP8.
struct A2avPtrs {
    const uint8_t *codes[kMaxRanks];      // e4m3 [m, K]
    const uint8_t *scales[kMaxRanks];     // E8M0 [m, scale_ld]
    const int *local_tokens[kMaxRanks];   // int32 [experts]: rows this rank holds per global expert
    int scale_ld;
};

struct MoeParams {
    MoeRankArgs ranks[kMaxRanks];
    uint8_t *heap_base[kMaxRanks];
    MoeLayout lay;
    int world, rank_base, n_local, ctas_per_rank;
    int m, K, N, top_k, experts, experts_per_rank;
    int route_ballot;           // routing kernel: equal keys by ballots (1) or by the match instruction (0)
    uint32_t epoch;
    uint64_t timeout_ns;
    int *status;
};

}  // namespace cb
