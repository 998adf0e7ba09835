// Host entry points of the f16/bf16 fused operators.
#pragma once
#include "common.h"
#include "symm_heap.h"

namespace cb {

struct DenseArgs {
    const void *A;   // [m, k] row-major
    const void *B;   // transB=0: [k, n] row-major;  transB=1: [n, k] row-major
    void *C;         // AG-MM: [R*m, n];  MM-RS: [m/R, n];  MM-AR: [m, n]
    void *gather_out = nullptr;   // AG-MM with gather result: receives the gathered A [R*m, k]
};

// Data-flow variants of AllGather-Matmul (launch_dense's `variant`): same product, different movement of A.
enum AgVariant : int {
    AG_PUSH = 0,          // every rank writes its rows into the peers' gathered regions (default)
    AG_REMOTE_READ = 1,   // every rank stages its rows in its own symmetric region; the peers read them from there
    AG_ALLTOALL = 2,      // AllToAll-Matmul: A is [R*m, k]; block d is pushed to rank d, which multiplies the R blocks it
                          // holds afterwards (block s from rank s) by its B -> C [R*m, n]
};

// Bytes of the caller's symmetric buffer the operator uses (0 for a single rank).
size_t dense_symmetric_bytes(int op, int world, int m, int n, int k);

// args: one entry per LOCAL rank (1 normally; the world size when all ranks are emulated on one GPU).
// m, n, k carry the reference's meaning per operator (AG-MM: m = rows held by one rank; MM-RS and
// MM-AR: m = rows of the full product).  Asynchronous on `stream`.
int launch_dense(int op, int dtype, cudaStream_t stream, uint32_t block_num, const DenseArgs *args, void *symmetric,
                 int m, int n, int k, int trans_a, int trans_b, int variant = AG_PUSH);

// 1: the reduce family exchanges its partial tiles as fp16 (default), 0: in the output type (CATCCOS_RS_EXCHANGE=native)
int rs_exchange_fp16();

// Output tensor maps of a pair reduce-scatter kernel for every local rank (see RsMaps): `outputs[l]` is local
// rank l's output (reduce-scatter: [m/R, n]; all-reduce and all-to-all: [m, n]), 16-bit elements of type `dt`; `symm_off` the
// offset of the launch's half of the staging region.
int encode_rs_maps(const DriverApi *api, Team *t, RsMapsAll *maps, int op, CUtensorMapDataType dt,
                   void *const *outputs, int n_local, int m, int n, uint64_t symm_off, bool compute_only);

}  // namespace cb
