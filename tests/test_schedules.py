"""Properties of the kernels' work orders, computed on the host by the functions the kernels themselves
use (catccos_b200/csrc/sched.h through catccos_debug_*_order).  No device needed."""
import ctypes

import numpy as np
import pytest

from catccos_b200 import lib

BM, BN, SUB = 128, 256, 32          # rows of a push chunk, columns of a tile, push units per chunk


def _rs(world, rank, rows_per_rank, n, pairs):
    cap = 1 << 16
    out = (ctypes.c_int32 * (3 * cap))()
    lag = ctypes.c_int32()
    cnt = lib().catccos_debug_rs_tile_order(world, rank, rows_per_rank, n, pairs, out, cap, ctypes.byref(lag))
    assert 0 <= cnt <= cap
    return np.frombuffer(out, dtype=np.int32, count=3 * cnt).reshape(cnt, 3).copy(), lag.value


def _ag(world, rank, m, n, group=4):
    cap = 1 << 16
    out = (ctypes.c_int32 * (3 * cap))()
    cnt = lib().catccos_debug_ag_tile_order(world, rank, m, n, group, out, cap)
    assert 0 <= cnt <= cap
    return np.frombuffer(out, dtype=np.int32, count=3 * cnt).reshape(cnt, 3).copy()


def _push(world, rank, m):
    cap = 1 << 16
    out = (ctypes.c_int32 * (3 * cap))()
    cnt = lib().catccos_debug_ag_push_order(world, rank, m, out, cap)
    assert 0 <= cnt <= cap
    return np.frombuffer(out, dtype=np.int32, count=3 * cnt).reshape(cnt, 3).copy()


RS_SHAPES = [(8, 1024, 8192, 74), (4, 2048, 8192, 74), (2, 4096, 8192, 74), (1, 8192, 8192, 74), (2, 256, 2048, 74),
             (8, 128, 512, 9), (4, 75, 264, 18), (3, 700, 520, 24), (8, 1024, 8192, 9)]


@pytest.mark.parametrize("world,rows,n,pairs", RS_SHAPES)
def test_reduce_scatter_order_visits_every_tile_once(world, rows, n, pairs):
    nt, stripes = -(-n // BN), -(-rows // (2 * BM))
    want = {(d, s, c) for d in range(world) for s in range(stripes) for c in range(nt)}
    for rank in range(world):
        order, lag = _rs(world, rank, rows, n, pairs)
        assert len(order) == len(want) and {tuple(x) for x in order} == want
        assert 1 <= lag <= stripes


@pytest.mark.parametrize("world,rows,n,pairs", [s for s in RS_SHAPES if s[0] > 1])
def test_partials_are_sent_before_the_own_tile_that_sums_them(world, rows, n, pairs):
    """For every own tile of a rank, every peer's partial of it sits at least (lag + 1) * nt positions
    earlier in that peer's order (lag * nt when the lag spans all stripes, i.e. own rows simply come
    last): all ranks walk their orders at the same pace, so the partial is computed, stored and
    flagged before the own tile's epilogue asks for it."""
    nt, stripes = -(-n // BN), -(-rows // (2 * BM))
    orders = [_rs(world, r, rows, n, pairs) for r in range(world)]
    for me in range(world):
        mine, lag = orders[me]
        own_pos = {(s, c): i for i, (d, s, c) in enumerate(mine) if d == me}
        for peer in range(world):
            if peer == me:
                continue
            sent = {(s, c): i for i, (d, s, c) in enumerate(orders[peer][0]) if d == me}
            assert sent.keys() == own_pos.keys()
            head_start = min(own_pos[k] - sent[k] for k in own_pos)
            assert head_start >= (lag + 1 if lag < stripes else lag) * nt


def test_reduce_scatter_lag_gives_one_and_a_half_tiles_per_pair_when_the_shape_allows():
    # benchmark shape at 4 ranks: 8 stripes, 32 column tiles, 74 pairs -> lag 3: (3 + 1) * 32 = 128 >= 1.5 * 74
    _, lag = _rs(4, 0, 2048, 8192, 74)
    assert lag == 3
    # at 8 ranks there are only 4 stripes: lag 3 as well; peer traffic still covers all but 3 of 32 stripe slots
    _, lag8 = _rs(8, 0, 1024, 8192, 74)
    assert lag8 == 3
    # a single stripe: own rows necessarily last
    order, lag1 = _rs(2, 1, 256, 2048, 74)
    assert lag1 == 1 and [d for d, _, _ in order] == [0] * 8 + [1] * 8


@pytest.mark.parametrize("group", [1, 3, 4, 8, 16])
@pytest.mark.parametrize("world,m,n", [(8, 1024, 4096), (4, 2048, 4096), (2, 320, 520), (1, 200, 264), (8, 100, 256),
                                       (1, 8192, 4096)])
def test_allgather_order_own_rows_first_then_sources_in_ring_order(world, m, n, group):
    nt, mt2 = -(-n // BN), -(-m // (2 * BM))
    for rank in range(world):
        order = _ag(world, rank, m, n, group)
        assert len(order) == world * mt2 * nt
        assert {tuple(x) for x in order} == {(s, a, b) for s in range(world) for a in range(mt2) for b in range(nt)}
        # every own tile comes before any tile that needs a peer's rows
        assert (order[:mt2 * nt, 0] == rank).all()
        # gathered sources are first needed in ring order rank+1, rank+2, ... (the order the peers push in)
        seen = []
        for s in order[mt2 * nt:, 0]:
            if int(s) not in seen:
                seen.append(int(s))
        assert seen == [(rank + j) % world for j in range(1, world)]


@pytest.mark.parametrize("group", [4, 8, 16])
def test_allgather_order_groups_share_operands(group):
    """Inside an L2 group the walk is column-tile major: `group` consecutive tiles share one column tile
    of B, a window of `pairs` consecutive tiles touches about group + pairs/group operand tiles
    instead of pairs/nt + nt, and a group starts on the column tile the previous one ended on."""
    world, m, n, pairs = 1, 8192, 4096, 74
    nt, mt2 = n // BN, m // (2 * BM)
    order = _ag(world, 0, m, n, group)
    for g0 in range(0, len(order), group):
        run = order[g0:g0 + group]
        assert len({int(x) for x in run[:, 2]}) == 1 and len({int(x) for x in run[:, 1]}) == group
    worst = max(len({int(x) for x in order[w:w + pairs, 1]}) + len({int(x) for x in order[w:w + pairs, 2]})
                for w in range(0, len(order) - pairs))
    assert worst <= group + -(-pairs // group) + 2 + (group if group < mt2 else 0)
    step = group * nt
    for g in range(1, mt2 // group):
        assert order[g * step, 2] == order[g * step - 1, 2]


def test_allgather_group_rows_are_about_the_square_root_of_the_pairs():
    # K = 8192 bf16: a 256-row operand tile is 4 MiB; 74 pairs -> 8 rows of A and 10 columns of B in flight
    assert lib().catccos_debug_ag_group_rows(4 << 20, 74, 88 << 20) == 8
    assert lib().catccos_debug_ag_group_rows(4 << 20, 9, 88 << 20) == 3
    assert lib().catccos_debug_ag_group_rows(64 << 20, 74, 88 << 20) == 8      # nothing fits: smallest footprint
    assert lib().catccos_debug_ag_group_rows(4 << 20, 1, 88 << 20) == 1


@pytest.mark.parametrize("world,m", [(8, 1024), (4, 2048), (2, 4096), (3, 200)])
def test_push_order_serves_the_first_consumer_first_and_every_unit_once(world, m):
    chunks = -(-m // BM)
    per_dest = chunks * SUB
    for rank in range(world):
        push = _push(world, rank, m)
        assert len(push) == (world - 1) * per_dest
        dests = [int(d) for d in push[::per_dest, 0]]
        assert dests == [(rank - 1 - j) % world for j in range(world - 1)]          # rank-1 consumes my rows first
        for j, d in enumerate(dests):
            block = push[j * per_dest:(j + 1) * per_dest]
            assert (block[:, 0] == d).all()
            assert [tuple(x[1:]) for x in block] == [(c, u) for c in range(chunks) for u in range(SUB)]   # row order
    # consumer side: rank r multiplies source r+1 right after its own rows, and r+1 pushes to r first
    for r in range(world):
        src_after_own = (r + 1) % world
        assert int(_push(world, src_after_own, m)[0, 0]) == r


def test_order_functions_reject_bad_arguments():
    out = (ctypes.c_int32 * 3)()
    assert lib().catccos_debug_rs_tile_order(0, 0, 128, 256, 4, out, 1, None) < 0
    assert lib().catccos_debug_rs_tile_order(2, 2, 128, 256, 4, out, 1, None) < 0
    assert lib().catccos_debug_ag_tile_order(9, 0, 128, 256, 4, out, 1) < 0
    assert lib().catccos_debug_ag_push_order(2, 0, 0, out, 1) < 0
    # a short buffer is filled up to its capacity and the full count is still reported
    assert lib().catccos_debug_ag_tile_order(2, 0, 256, 512, 4, out, 1) == 4


def _slots(sigs, foreign=None):
    n = len(sigs)
    a = (ctypes.c_uint64 * n)(*sigs)
    f = (ctypes.c_uint8 * n)(*(foreign or [0] * n))
    half, back = (ctypes.c_int32 * n)(), (ctypes.c_int32 * n)()
    assert lib().catccos_debug_slot_sequence(a, f, n, half, back) == 0
    return list(half), list(back)


def test_double_buffered_regions_alternate_only_for_back_to_back_identical_launches():
    """Same operator, shape and buffer launched back to back: the halves alternate and a peer needs only to
    have entered the previous launch.  Anything else in between (another shape, another operator family)
    makes the next launch strict again: half 0, peers must have entered this very launch."""
    A, B = 0x1111, 0x2222
    half, back = _slots([A, A, A, A])
    assert half == [0, 1, 0, 1] and back == [0, 1, 1, 1]
    half, back = _slots([A, B, A, A, B, B])
    assert half == [0, 0, 0, 1, 0, 1] and back == [0, 0, 0, 1, 0, 1]
    # a MoE / quantise-all-gather launch between two identical launches consumes an epoch: strict again
    half, back = _slots([A, A, A, A], foreign=[0, 0, 1, 0])
    assert half == [0, 1, 0, 1] and back == [0, 1, 0, 1]
    # safety argument in numbers: whenever a launch may write to a peer that is one launch behind, the launch
    # that peer may still be running uses the OTHER half
    for seq in ([A] * 7, [A, A, B, B, B, A, A, A]):
        half, back = _slots(seq)
        for i in range(1, len(seq)):
            if back[i] == 1:
                assert seq[i - 1] == seq[i] and half[i - 1] != half[i]
