// Shared host/device definitions of the fused GEMM + collective kernels.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdint>

namespace cb {

constexpr int kMaxRanks = 8;

// Flag region: the first kFlagBytes of every PE's symmetric heap.  32-bit words,
// zeroed once at heap creation; every flag has a single writer that stores the
// launch epoch (monotonic across all operators), readers wait for >= epoch.
constexpr size_t kFlagBytes = 4u << 20;
constexpr uint32_t kFlagWords = kFlagBytes / 4;
constexpr uint32_t kFlagEntered = 0;      // entered[src PE]            (kMaxRanks words)
constexpr uint32_t kFlagBarrier = 16;     // host-visible barrier words (kMaxRanks words)
constexpr uint32_t kFlagOpBase = 64;      // per-operator flags start here

enum FusedOp : int { OP_AGMM = 0, OP_MMRS = 1, OP_MMAR = 2, OP_MMA2A = 3 /* Matmul-AllToAll: MM-RS's data flow without the sum */ };

// GEMM tile of the dense (f16/bf16) kernel.
constexpr int BM = 128, BN = 256, BK = 64;
constexpr int kStages = 4;
constexpr int kAStageBytes = BM * BK * 2;   // 16 KiB
constexpr int kBStageBytes = BN * BK * 2;   // 32 KiB
constexpr int kGemmThreads = 256;           // warp 0 TMA, 1 MMA, 2-5 epilogue, 6-7 comm
constexpr int kPairAgThreads = 352;         // pair AllGather-Matmul kernels: warps 6-9 are one push lane each (a
                                            // blocking bulk-copy wait stalls its whole warp, so lanes do not share one);
                                            // warp 10 polls the arrival flags of the CTA's coming tiles
constexpr int kPushPieceBytes = 8 * 1024;  // all-gather push: one staging piece per pusher lane
constexpr int kPushLanes = 24;             // lanes (threads with a piece in flight) of a dedicated pusher CTA
constexpr int kSideSmemBytes = 32 * 1024;  // next to the GEMM stages: push staging (AG-MM) or epilogue row staging
constexpr int kPushLanesShared = kSideSmemBytes / kPushPieceBytes;   // lanes of a CTA that also runs the GEMM
constexpr int kGemmSmemBytes =
    kStages * (kAStageBytes + kBStageBytes) + kSideSmemBytes + 1024 /*align*/ + 512 /*barriers*/;
constexpr int kAgSubChunks = 32;            // an all-gather chunk (BM rows) is pushed as 32 units of 4 rows: many more
                                            // units than pusher lanes, so the slab of the rank that needs it first goes first

struct alignas(64) RankArgs {
    CUtensorMap tmA;    // A as passed by the caller: [rows, K], K innermost, box {BK, BM}
    CUtensorMap tmAg;   // AG-MM: gathered A [R*m, K] in this PE's symmetric region
    CUtensorMap tmB;    // transB=1: [N, K] box {BK, BN};  transB=0: [K, N] box {64 (n), BK (k)}
    const void *A;      // raw pointers of the same operands
    void *C;
    void *gather_out;   // AG-MM with gather result: [R*m, K] copy of the gathered A for the caller (nullptr: none)
};

struct FusedParams {
    RankArgs ranks[kMaxRanks];        // indexed by LOCAL rank (1 entry per process; R entries when emulating)
    uint8_t *heap_base[kMaxRanks];    // VA (in this process) of every PE's symmetric heap
    uint64_t symm_off;                // byte offset of the operator's data region inside the heap
    uint8_t *mc_base;                 // multicast view of all heaps (a store lands in every heap), or nullptr
    int world, rank_base, n_local, ctas_per_rank;
    int push_ctas;                    // AG-MM: > 0: the last push_ctas CTAs of a rank only move all-gather traffic;
                                      // 0: every CTA pushes from its comm warp next to its GEMM tiles
    int M, N, K;                      // AG-MM: M = rows held by one rank; MM-RS / MM-AR: M = total rows
    uint32_t epoch;
    uint32_t entered_need;            // a peer's data region may be written once it has entered this epoch
    int compute_only;                 // measurement mode: no peer traffic, no flag waits (data left by an earlier launch)
    uint64_t timeout_ns;
    int *status;                      // cb::StatusWord[ST_WORDS], device memory
    int *sched;                       // tile queue of the pair AllGather-Matmul: per local rank {next tile, pairs finished},
                                      // zero between launches (the last pair to finish clears them)
    int rs_fp16;                      // reduce family: partial tiles cross the link as fp16 (11-bit mantissa) whatever
                                      // the output type; 0: in the output type
    int ag_group;                     // 256-row tiles per L2 group of the AllGather-Matmul tile order (sched.h)
    int ag_a2a;                       // AllToAll-Matmul: A holds world * M rows; block d goes to rank d (block `rank` stays)
    int ag_pull;                      // AG-MM data flow: 0 = every rank pushes its rows into the peers' gathered regions;
                                      // 1 = remote read: every rank stages its rows in its own region and the peers fetch them
    unsigned long long *trace;        // optional: kTraceSlots %globaltimer stamps per CTA (nullptr = off)
};

// Output tensor maps of the pair reduce-scatter kernel, per local rank: box {64 columns, 32 rows},
// 128-byte swizzle.  out[d]: d == this rank -> its rows of the operator's output; d != rank -> this
// rank's slot of rank d's staging rows.  fin[d] (Matmul-AllReduce): this rank's rows of rank d's
// "final" region.  Every map covers exactly the rows that exist, so ragged tiles are clipped by TMA.
struct alignas(64) RsMaps {
    CUtensorMap out[kMaxRanks];
    CUtensorMap fin[kMaxRanks];
};
struct RsMapsAll {
    RsMaps r[kMaxRanks];      // indexed by LOCAL rank like FusedParams::ranks
};

// Per-CTA trace slots (nanoseconds of %globaltimer).
enum TraceSlot : int {
    TR_START = 0, TR_END = 1,
    TR_PROD_WAIT_FIRST = 2,   // producer: when the first wait for pushed rows began
    TR_PROD_WAIT_NS = 3,      // producer: total time spent waiting for pushed rows
    TR_PUSH_BEGIN = 4, TR_PUSH_END = 5,
    TR_EPI_WAIT_NS = 6,       // epilogue: total time waiting for peers (entered / partial tiles)
    TR_EPI_STORE_NS = 7,      // epilogue: total time draining accumulators (TMEM -> memory)
    TR_MMA_WAIT_TMEM_NS = 8,  // MMA warp: total time waiting for a free accumulator
    TR_MMA_WAIT_SMEM_NS = 9,  // MMA warp: total time waiting for operands in shared memory
    TR_TILES = 10,
    kTraceSlots = 16
};

struct Team;   // symmetric heap + peers (symm_heap.cu)

}  // namespace cb
