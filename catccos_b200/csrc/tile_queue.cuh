// Dynamic tile queue of the CTA-pair kernels.
//
// A pair (cluster of two CTAs) does not own a fixed list of tiles: it starts on a tile that follows
// from its index and afterwards takes the next unclaimed tile of its rank from a counter in global
// memory, so a pair that was held up (rows of a peer not in yet, an expert with more rows than the
// others) simply takes fewer tiles instead of finishing late.  One thread of the leader CTA claims
// tiles, never more than kTileAhead beyond what the epilogues of both CTAs have finished, and
// publishes every claim into a small ring in the shared memory of both CTAs; producer, MMA issuer
// and epilogue warps read claim number `seq` from the ring.  kTileEnd ends every role's loop.
#pragma once
#include "ptx.cuh"

namespace cb {

constexpr int kTileRing = 8;                   // ring slots; a slot is rewritten kTileRing claims later
constexpr uint32_t kTileAhead = 3;             // claims beyond the last tile both epilogues have finished
constexpr uint32_t kTileEnd = 0xFFFFFFFFu;     // ring entry: no tiles left
static_assert(kTileAhead + 2 < kTileRing, "a slot must not be rewritten while a role can still read it");

struct TileQueue {                  // one copy in each CTA of the pair
    uint32_t ring[kTileRing];       // tile index of claim number seq at [seq % kTileRing]
    uint32_t claimed;               // number of valid ring entries so far
    uint32_t done_self;             // tiles this CTA's epilogue has finished (leader's copy is read by the claimer)
    uint32_t done_peer;             // leader only: the same count of the other CTA
};

__device__ __forceinline__ void tq_init(TileQueue *q) {
    q->claimed = 0;
    q->done_self = 0;
    q->done_peer = 0;
}

// any role: tile of claim number seq (blocks, bounded, until the claim has been published)
__device__ __forceinline__ bool tq_get(const TileQueue *q, uint32_t seq, uint32_t &tile, const WaitCtl &ctl) {
    if (!wait_cluster_counter_gt(&q->claimed, seq, ctl, W_TILE_QUEUE)) return false;
    tile = q->ring[seq % kTileRing];
    return true;
}

// leader's claiming thread: entry `seq` becomes `tile` in both CTAs
__device__ __forceinline__ void tq_publish(TileQueue *q, uint32_t seq, uint32_t tile) {
    q->ring[seq % kTileRing] = tile;
    st_cluster_smem(mapa_cluster(smem_u32(&q->ring[seq % kTileRing]), 1), tile);
    st_release_cta_smem(&q->claimed, seq + 1);
    st_release_cluster_smem(mapa_cluster(smem_u32(&q->claimed), 1), seq + 1);
}

// leader's claiming thread: waits for room, claims and publishes.  Claim 0 is `first_tile`; later claims
// are `base + (value of the rank's counter)`.  Returns false when a wait ran out.
__device__ __forceinline__ bool tq_claim(TileQueue *q, uint32_t seq, int first_tile, int base, int num_tiles,
                                         int *counter, const WaitCtl &ctl, uint32_t &tile) {
    if (seq >= kTileAhead) {
        if (!wait_smem_counter_gt(&q->done_self, seq - kTileAhead, ctl, W_TILE_QUEUE) ||
            !wait_cluster_counter_gt(&q->done_peer, seq - kTileAhead, ctl, W_TILE_QUEUE))
            return false;
    }
    const int t = seq == 0 ? first_tile : base + atomicAdd(counter, 1);
    tile = t < num_tiles ? static_cast<uint32_t>(t) : kTileEnd;
    tq_publish(q, seq, tile);
    return true;
}

// leader's claiming thread, after a failed wait: the other roles must not wait for claims that will not come
__device__ __forceinline__ void tq_publish_end(TileQueue *q) { tq_publish(q, q->claimed, kTileEnd); }

// one epilogue thread per CTA, after its CTA has finished `count` tiles
__device__ __forceinline__ void tq_done(TileQueue *q, uint32_t cta_rank, uint32_t count) {
    if (cta_rank == 0)
        st_release_cta_smem(&q->done_self, count);
    else
        st_release_cluster_smem(mapa_cluster(smem_u32(&q->done_peer), 0), count);
}

// leader's claiming thread, once its pair has seen kTileEnd: `counters` = {next tile, pairs finished};
// the last pair of the rank leaves both at zero for the next launch
__device__ __forceinline__ void tq_retire(int *counters, int pairs) {
    __threadfence();
    if (atomicAdd(counters + 1, 1) == pairs - 1) {
        counters[0] = 0;
        counters[1] = 0;
        __threadfence();
    }
}

}  // namespace cb
