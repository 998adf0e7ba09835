"""A discrete-event model of the reduce-scatter epilogue's flag protocol, driven by the tile orders the
kernels really use (sched.h through the C-ABI): partial tiles flagged one tile late, a non-blocking look
at the flags before an own tile, the pending flag raised before any blocking wait.  Under random
per-tile durations and per-rank start skews every rank must finish (no rank ever waits for a flag whose
writer waits for it) and no own tile may be reduced before all its partials were flagged.  No device."""
import ctypes
import heapq
import random

import numpy as np
import pytest

from catccos_b200 import lib


def _order(world, rank, rows, n, pairs):
    cap = 1 << 14
    out = (ctypes.c_int32 * (3 * cap))()
    cnt = lib().catccos_debug_rs_tile_order(world, rank, rows, n, pairs, out, cap, None)
    return [tuple(int(v) for v in out[3 * i:3 * i + 3]) for i in range(cnt)]


def simulate(world, rows, n, pairs, seed, skew=50.0):
    """Returns (finish time per rank, total time own tiles spent blocked).  Units are CTA pairs."""
    rng = random.Random(seed)
    orders = [_order(world, r, rows, n, pairs) for r in range(world)]
    flags = set()                                   # (src, owner, stripe, col) raised
    waiting = {}                                    # flag -> list of (rank, unit) blocked on it
    finish = [0.0] * world
    blocked_time = 0.0
    # per unit: index of the next tile, the pending (unraised) flag, what it still waits for
    state = {(r, u): dict(i=0, pend=None, need=None, since=0.0) for r in range(world) for u in range(pairs)}
    events = []                                     # (time, seq, rank, unit): the unit's accumulator for tile i is full
    seq = 0
    for r in range(world):
        start = rng.uniform(0, skew)
        for u in range(pairs):
            if u < len(orders[r]):
                heapq.heappush(events, (start + rng.uniform(8, 12), seq, r, u))
                seq += 1
    done_units = 0
    total_units = sum(1 for r in range(world) for u in range(pairs) if u < len(orders[r]))

    def raise_flag(f, now):
        nonlocal seq
        flags.add(f)
        for (r, u) in waiting.pop(f, []):
            heapq.heappush(events, (now, seq, r, u))   # re-run the blocked unit's check
            seq += 1

    while events:
        now, _, r, u = heapq.heappop(events)
        st = state[(r, u)]
        mine = orders[r][u::pairs]
        d, stripe, col = mine[st["i"]]
        own = d == r
        if own:
            missing = [(s, r, stripe, col) for s in range(world) if s != r and (s, r, stripe, col) not in flags]
            if missing:
                if st["pend"] is not None:          # slow path: raise the pending flag first, then block
                    raise_flag(st["pend"], now)
                    st["pend"] = None
                if st["need"] is None:
                    st["since"] = now
                st["need"] = missing[0]
                waiting.setdefault(missing[0], []).append((r, u))
                continue
            if st["need"] is not None:
                blocked_time += now - st["since"]
                st["need"] = None
        drain = rng.uniform(2, 4)
        t_done = now + drain
        if st["pend"] is not None:                  # the tile before this one: its stores had a whole drain to land
            raise_flag(st["pend"], t_done)
            st["pend"] = None
        if not own:
            st["pend"] = (r, d, stripe, col)
        st["i"] += 1
        if st["i"] == len(mine):
            if st["pend"] is not None:
                raise_flag(st["pend"], t_done)
                st["pend"] = None
            finish[r] = max(finish[r], t_done)
            done_units += 1
        else:
            heapq.heappush(events, (max(t_done, now + rng.uniform(8, 12)), seq, r, u))   # next accumulator full
            seq += 1
    assert done_units == total_units, f"deadlock: {total_units - done_units} units never finished, waiting on {list(waiting)[:4]}"
    every = {(s, o, a, b) for o in range(world) for s in range(world) if s != o
             for (dd, a, b) in orders[o] if dd == o}
    assert flags == every                           # every partial flagged exactly where an owner looks for it
    return finish, blocked_time


@pytest.mark.parametrize("world,rows,n,pairs", [(2, 512, 1024, 6), (4, 1024, 1024, 6), (8, 512, 512, 5), (4, 256, 2048, 9),
                                                 (3, 1536, 768, 4), (8, 1024, 2048, 12)])
def test_no_deadlock_under_random_timing(world, rows, n, pairs):
    for seed in range(6):
        finish, _ = simulate(world, rows, n, pairs, seed)
        assert all(f > 0 for f in finish)


def test_large_start_skew_only_delays_it_does_not_wedge():
    finish, blocked = simulate(4, 1024, 1024, 6, seed=3, skew=2000.0)
    assert blocked > 0.0 and max(finish) - min(finish) < 200.0   # ranks wait for the late one, then complete together
