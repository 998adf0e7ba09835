"""Worked examples of the EP x TP all-to-all-v schedulers restated in oracle/moe.py
(include/catccos/comm/block/comm_block_scheduler_alltoallv_allgather.hpp and
comm_block_scheduler_reducescatter_alltoallv.hpp).  The reference ships no test vectors for these
two classes; the expected numbers below were worked out by hand from their source, and the
property tests tie the bookkeeping to the dispatch layout the other goldens use."""
import numpy as np
import pytest

from oracle import moe

LOCAL = [5, 3, 7, 2]                       # tokens this rank sends to global experts 0..3
GLOBAL = [4, 1, 2, 2, 0, 6, 3, 3]          # tokens of ranks 0..3 for this rank's 2 local experts


def test_alltoallv_allgather_worked_example():
    s = moe.AllToAllVAllGatherSchedule(k=256, rank_size=4, rank_idx=1, ep_size=2, expert_num=4,
                                       local_tokens_per_expert=LOCAL, global_tokens_per_local_expert=GLOBAL,
                                       comm_rows=4, block_shape=(2, 128))
    assert s.block_grid == (2, 2) and s.core_loops == 16
    assert s.input_split.tolist() == [8, 9] and s.input_offset.tolist() == [0, 8]
    assert s.output_split.tolist() == [5, 4, 6, 6]
    assert s.comm_loops == 3                                     # ceil(9 / 4): EP 1 gets 9 rows
    assert [s.actual_receive_accum(i) for i in range(3)] == [16, 6, 0]
    # destination rank fastest, then block column, then block row
    assert s.block_offset(3) == ((0, 0), 3) and s.block_offset(6) == ((0, 128), 2) and s.block_offset(9) == ((2, 0), 1)
    # rank 3 belongs to EP 1 (tp rank 1): its rows start at 8; round 1 starts 4 rows further
    assert s.source_offset(1, (2, 128), 3) == (14, 128)
    assert s.actual_block_shape(1, (2, 128), 3) == (2, 128)
    assert s.actual_block_shape(2, (0, 0), 1) == (1, 128)        # one row of EP 1 is left for round 2
    assert s.actual_block_shape(2, (0, 0), 0) == (0, 128)        # EP 0 (8 rows) is finished after two rounds


def test_reducescatter_alltoallv_worked_example():
    r = moe.ReduceScatterAllToAllVSchedule(n=512, rank_size=4, ep_size=2, expert_num=4, local_tokens_per_expert=LOCAL,
                                           global_tokens_per_local_expert=GLOBAL, blocks_per_comm=3, src_ep=1,
                                           mmad_block=(4, 256), comm_block=(2, 128), core_split=(2, 2))
    assert r.block_grid == (6, 2) and r.core_loops == 12
    assert r.split_in_expert.tolist() == [[4, 2], [4, 2]] and r.input_split.tolist() == [6, 6]
    assert r.input_offset.tolist() == [[0, 5], [8, 15]]
    assert r.output_split.tolist() == [4, 4, 4, 4] and r.comm_loops == 2
    assert r.mmad_grid == [(2, 2), (1, 2)]
    r.update_comm_context(1)
    assert r.comm_offset == 3 and r.actual_comm_shape == (12, 256) and r.actual_receive_accum() == 4
    want = {0: ((0, 0), 3, 0, ((12, 256), (3, 256))),            # GEMM block 3 of expert 0: rows 4..6 of its 7, columns 256..
            5: ((4, 128), 4, 1, ((15, 128), (2, 128))),           # first block of expert 1 (2 rows)
            11: ((10, 128), 5, 1, ((17, 384), (0, 128)))}         # past the expert's last row: nothing left
    for task, (off, mmad_idx, expert, dst) in want.items():
        o = r.block_offset(task)
        r.update_local_expert_context(o)
        assert o == off and r.mmad_idx == mmad_idx and r.start_expert == expert
        assert r.destination(o) == dst
        assert r.actual_block_shape(o) == (2, 128)
    # deterministic mode folds the core split and rounds the task count up to it
    d = moe.ReduceScatterAllToAllVSchedule(n=512, rank_size=4, ep_size=2, expert_num=4, local_tokens_per_expert=LOCAL,
                                           global_tokens_per_local_expert=GLOBAL, blocks_per_comm=3, src_ep=1,
                                           mmad_block=(4, 256), comm_block=(2, 128), core_split=(5, 1), deterministic=True)
    assert d.core_split == (5, 1) and d.core_loops == 15


@pytest.mark.parametrize("seed", range(4))
def test_rounds_cover_every_row_exactly_once(seed):
    """Over all rounds and tasks, the source rows of AllToAllV-AllGather addressed to one EP are the
    rows [input_offset, input_offset + input_split) of that EP, each exactly once per TP peer."""
    rng = np.random.default_rng(seed)
    ep, tp, L, k = 2, 2, 3, 192
    local = rng.integers(0, 9, ep * L)
    glob = rng.integers(0, 9, ep * tp * L)
    s = moe.AllToAllVAllGatherSchedule(k, ep * tp, 0, ep, ep * L, local, glob, comm_rows=5, block_shape=(2, 64))
    seen = {}
    for c in range(s.comm_loops):
        for t in range(s.core_loops):
            off, dst = s.block_offset(t)
            rows, cols = s.actual_block_shape(c, off, dst)
            r0, c0 = s.source_offset(c, off, dst)
            for rr in range(rows):
                for cc in range(c0, c0 + cols):
                    key = (dst, r0 + rr, cc)
                    seen[key] = seen.get(key, 0) + 1
    assert all(v == 1 for v in seen.values())
    for dst in range(ep * tp):
        e = dst % ep
        rows = {r for (d, r, _) in seen if d == dst}
        assert rows == set(range(int(s.input_offset[e]), int(s.input_offset[e] + s.input_split[e])))
