"""Tile-order maps of the reference's block schedulers (integer arithmetic).

Test infrastructure only (see package docstring).
"""


def matrix_swizzle_coord(grid_rows: int, grid_cols: int, loop_idx: int, swizzle_offset: int = 1,
                         direction: int = 0):
    """`MatrixSwizzle<OFFSET, DIRECTION>::GetCoord` (include/catccos/catccos.hpp:140-163):
    serpentine order over groups of `swizzle_offset` rows (direction 0) or columns."""
    shape = [grid_rows, grid_cols]
    row_dim, col_dim = direction, 1 - direction
    group_size = swizzle_offset * shape[col_dim]
    group_idx = loop_idx // group_size
    group_off = loop_idx - group_idx * group_size
    in_rows = min(swizzle_offset, shape[row_dim] - group_idx * swizzle_offset)
    coord = [0, 0]
    coord[col_dim] = group_off // in_rows
    coord[row_dim] = group_idx * swizzle_offset + (group_off - coord[col_dim] * in_rows)
    if group_idx & 1:
        coord[col_dim] = shape[col_dim] - coord[col_dim] - 1
    return coord[0], coord[1]


def comm_swizzle_coord(grid_row: int, grid_col: int, grid_rank: int, split_row: int, split_col: int,
                       loop_idx: int, direction: int = 0, deterministic: bool = False):
    """`CommSwizzle<DIRECTION, IS_DETERMINISTIC>::GetCoord` (include/catccos/catccos.hpp:165-193).
    Returns (row, col, rank)."""
    row_dim, col_dim = direction, 1 - direction
    split = [split_row, split_col]
    swz = split[row_dim]
    flat = [grid_row * grid_col, grid_rank]
    group_size = swz * flat[col_dim]
    group_idx = loop_idx // group_size
    group_off = loop_idx - group_idx * group_size
    in_rows = swz if deterministic else min(swz, flat[row_dim] - group_idx * swz)
    coord = [0, 0]
    coord[col_dim] = group_off // in_rows
    coord[row_dim] = group_idx * swz + (group_off - coord[col_dim] * in_rows)
    n_stride = grid_rank // split_col
    off = coord[1] * n_stride
    coord[1] = (off + off // grid_rank + coord[0]) % grid_rank
    return coord[0] // grid_col, coord[0] % grid_col, coord[1]


def block_comm_swizzle_coord(grid_row, grid_col, grid_rank, split_row, split_col, loop_idx,
                             direction: int = 0, deterministic: bool = False):
    """`BlockCommSwizzle` view of the same map: in deterministic mode the core split is
    folded to (row*col, 1) before `CommSwizzle::GetCoord` is called
    (include/catccos/comm/block/comm_block_swizzle.hpp:84-86)."""
    if deterministic:
        split_row, split_col = split_row * split_col, 1
    return comm_swizzle_coord(grid_row, grid_col, grid_rank, split_row, split_col, loop_idx, direction,
                              deterministic)
