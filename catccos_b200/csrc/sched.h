// Tile and push orders of the fused kernels as plain integer functions, shared by the kernels and
// by the host (catccos_debug_*_order in the C-ABI), so that the orders' properties — every tile
// exactly once, partials ahead of the own tile that needs them, the first consumer served first —
// are checked on the CPU against the very code the GPU runs.
// (Re-derived scheduler; the reference's counterparts are CommSwizzle / BlockCommSwizzle,
// include/catccos/catccos.hpp:140-193, and the block schedulers under include/catccos/comm/block/.)
#pragma once

#if defined(__CUDACC__)
#define CB_HD __host__ __device__ __forceinline__
#else
#define CB_HD inline
#endif

namespace cb {

// ---- Matmul-ReduceScatter / AllReduce on CTA pairs -------------------------------------------
// The owner's rows are cut into stripes of 256 rows (nt pair tiles each).  "Super-round" q sends
// stripe q of every peer (owners rank+1, rank+2, ...) and then reduces the OWN stripe q - lag,
// whose partials the peers sent `lag` super-rounds earlier.  Peer traffic is thus spread over the
// whole kernel instead of its first (R-1)/R, and only `lag` own stripes remain for the end.  A
// partial is at least (lag + 1) * nt tiles ahead of the own tile that needs it (lag * nt when the
// lag spans all stripes and the own rows simply come last); lag is sized so that this is 1.5 tiles
// per CTA pair (compute, drain, store and the flag that follows one tile
// later take about one).
struct RsOrder {
    int R, nt, stripes, lag, head, body;
};

CB_HD RsOrder rs_order_make(int R, int nt, int stripes, int pairs) {
    RsOrder o;
    o.R = R;
    o.nt = nt;
    o.stripes = stripes;
    int lag = (3 * pairs / 2 + nt - 1) / nt - 1;
    if (lag > stripes) lag = stripes;
    if (lag < 1) lag = 1;
    o.lag = lag;
    o.head = lag * (R - 1) * nt;                 // super-rounds 0 .. lag-1: peers only
    o.body = (stripes - lag) * R * nt;           // super-rounds lag .. stripes-1: peers, then own
    return o;
}

CB_HD int rs_order_tiles(const RsOrder &o) { return o.R * o.stripes * o.nt; }

// pair tile t of `rank` -> owner d, 256-row stripe mi2 of the owner's rows, column tile ni
CB_HD void rs_order_decode(const RsOrder &o, int rank, int t, int &d, int &mi2, int &ni) {
    const int R = o.R, nt = o.nt;
    int j;      // 0 .. R-2: peer rank+1+j;  R-1: own rows
    if (t < o.head) {
        const int q = t / ((R - 1) * nt);
        const int u = t - q * (R - 1) * nt;
        j = u / nt;
        ni = u - j * nt;
        mi2 = q;
    } else if (t < o.head + o.body) {
        const int v = t - o.head;
        const int q = o.lag + v / (R * nt);
        const int u = v - (q - o.lag) * R * nt;
        j = u / nt;
        ni = u - j * nt;
        mi2 = (j == R - 1) ? q - o.lag : q;
    } else {
        const int v = t - o.head - o.body;
        j = R - 1;
        mi2 = o.stripes - o.lag + v / nt;
        ni = v - (v / nt) * nt;
    }
    d = (rank + 1 + j) % R;
}

// ---- AllGather-Matmul on CTA pairs -----------------------------------------------------------
// Tiles: own rows first, then source ranks rank+1, rank+2, ...; inside a source 256-row tile major.
CB_HD void ag_order_decode(int R, int per_src, int nt, int rank, int t, int &s, int &mi2, int &ni) {
    const int j = t / per_src;
    const int u = t - j * per_src;
    s = (rank + j) % R;
    mi2 = u / nt;
    ni = u - mi2 * nt;
}

// The same tiles in an order that keeps operands in L2 (the counterpart of the reference's MatrixSwizzle,
// include/catccos/catccos.hpp:140-163).  The 256-row tiles are listed in arrival order (own rows, then
// the rows of rank+1, rank+2, ...) and cut into groups of G rows -- the own rows and the gathered rows
// separately, so that no own tile queues behind a tile that waits for a peer.  Inside a group the walk
// is column-tile major: the CTAs that run side by side share a few column tiles of B and the group's
// G row tiles of A, instead of one row tile and every column tile of B.  Odd groups walk the column
// tiles backwards, so that a group starts on the columns the previous one just used.
CB_HD void ag_order_grouped(int R, int mt2, int nt, int G, int rank, int t, int &s, int &mi2, int &ni) {
    const int own_tiles = mt2 * nt;
    int row0 = 0, region_rows = mt2, tt = t;
    if (t >= own_tiles) {
        row0 = mt2;
        region_rows = (R - 1) * mt2;
        tt = t - own_tiles;
    }
    const int g = tt / (G * nt);
    const int r0 = g * G;
    const int rows = (region_rows - r0 < G) ? region_rows - r0 : G;
    const int u = tt - g * G * nt;
    const int c = u / rows;
    ni = (g & 1) ? nt - 1 - c : c;
    const int row = row0 + r0 + (u - c * rows);
    const int j = row / mt2;
    s = (rank + j) % R;
    mi2 = row - j * mt2;
}

// Rows per group for ag_order_grouped.  A window of `pairs` consecutive tiles touches g row tiles of A and
// pairs / g column tiles of B: the footprint g + pairs / g is smallest near sqrt(pairs), which is the
// choice unless even that exceeds the L2 budget (then still the smallest footprint).  Measured on
// 8192 x 8192 x 4096 bf16 with 74 pairs: 8 rows per group is the fastest, 16 and 32 are slower than
// none.  tile_bytes = 256 * K * element size.
CB_HD int ag_order_group_rows(long long tile_bytes, int pairs, long long l2_budget_bytes) {
    int g = 1;
    while ((g + 1) * (g + 1) <= pairs && g < 16) ++g;               // floor(sqrt(pairs)), at most 16
    while (g > 1 && (g + (pairs + g - 1) / g) * tile_bytes > l2_budget_bytes &&
           (g - 1 + (pairs + g - 2) / (g - 1)) < (g + (pairs + g - 1) / g))
        --g;
    return g;
}

// Push unit u of `rank` (units_per_dest units per destination): destination rank-1 first (it
// consumes this rank's rows first), then rank-2, ...; `cu` is the unit inside the destination.
CB_HD void ag_push_decode(int R, int units_per_dest, int rank, int u, int &dest, int &cu) {
    const int jj = u / units_per_dest;
    dest = (rank + R - 1 - jj) % R;
    cu = u - jj * units_per_dest;
}

}  // namespace cb
