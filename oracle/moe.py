"""MoE dispatch -> grouped GEMM -> SwiGLU -> grouped GEMM -> combine golden.

Test infrastructure only (see package docstring).  Follows
examples/utils/gen_data_moe.py; vectorised where the reference loops in Python.
"""
import numpy as np
import torch

from . import mxquant


# --------------------------------------------------------------------------- #
# routing
# --------------------------------------------------------------------------- #
def moe_init_routing(expert_idx: np.ndarray, expert_num: int):
    """Stable sort of the flattened [m, topK] expert ids.

    gen_data_moe.py:48-57 (`moe_init_routing_cpu`): returns
      sorted_src  int32 [m*topK]  dst -> src: sorted_src[d] = flat (token*topK+k) index
                                   feeding permuted row d (stable argsort),
      tokens_per_expert int32 [E] (bincount).
    The NPU kernel stores the inverse direction (src -> dst,
    examples/aux_ops/moe_init_routing_v2/moe_init_routing_v2.h:54-241,
    consumed at include/catccos/comm/block/comm_block_mx_quant.hpp:361);
    `expanded_row_idx_src_to_dst` converts."""
    flat = np.asarray(expert_idx, dtype=np.int64).reshape(-1)
    sorted_src = np.argsort(flat, kind="stable").astype(np.int32)
    counts = np.bincount(flat, minlength=expert_num).astype(np.int32)
    return sorted_src, counts


def expanded_row_idx_src_to_dst(sorted_src: np.ndarray) -> np.ndarray:
    """Inverse permutation: out[token*topK+k] = destination row."""
    inv = np.empty_like(sorted_src)
    inv[sorted_src] = np.arange(sorted_src.size, dtype=sorted_src.dtype)
    return inv


def permute_rows(x: np.ndarray, sorted_src: np.ndarray, top_k: int) -> np.ndarray:
    """routed = x[sorted_src // topK]  (gen_data_moe.py:54-55)."""
    return x[sorted_src.astype(np.int64) // top_k]


# --------------------------------------------------------------------------- #
# all-to-all-v (dispatch and combine directions)
# --------------------------------------------------------------------------- #
def dispatch_layout(tokens_per_expert_all: np.ndarray, ep: int, experts_per_rank: int):
    """Row bookkeeping of `alltoallv1` (gen_data_moe.py:139-198).

    tokens_per_expert_all: int [EP, E] (row = token-owning rank).
    For expert-owning rank `o`, receive order is: for each local expert, for each
    source rank in rank order.  Returns per owner a list of
    (src_rank, src_row_offset, length) segments and the per-local-expert row counts."""
    t = np.asarray(tokens_per_expert_all, dtype=np.int64)
    src_prefix = np.concatenate([np.zeros((ep, 1), np.int64), np.cumsum(t, axis=1)], axis=1)
    segs, blocks = [], []
    for o in range(ep):
        s, b = [], []
        for le in range(experts_per_rank):
            e = o * experts_per_rank + le
            n = 0
            for src in range(ep):
                ln = int(t[src, e])
                s.append((src, int(src_prefix[src, e]), ln))
                n += ln
            b.append(n)
        segs.append(s)
        blocks.append(b)
    return segs, blocks


def alltoallv_dispatch(routed_list, tokens_per_expert_all, ep, experts_per_rank):
    """gen_data_moe.py:139-198: gather permuted rows to the expert owners."""
    segs, blocks = dispatch_layout(tokens_per_expert_all, ep, experts_per_rank)
    out = []
    for o in range(ep):
        parts = [routed_list[src][off:off + ln] for (src, off, ln) in segs[o]]
        out.append(np.concatenate(parts, axis=0) if parts else routed_list[0][:0])
    return out, blocks


def alltoallv_combine(expert_out_list, tokens_per_expert_all, ep, experts_per_rank):
    """gen_data_moe.py:239-283: send every row back to the permuted position it
    came from on its source rank."""
    segs, _ = dispatch_layout(tokens_per_expert_all, ep, experts_per_rank)
    t = np.asarray(tokens_per_expert_all, dtype=np.int64)
    width = expert_out_list[0].shape[1]
    back = [np.zeros((int(t[r].sum()), width), dtype=expert_out_list[0].dtype) for r in range(ep)]
    for o in range(ep):
        pos = 0
        for (src, off, ln) in segs[o]:
            back[src][off:off + ln] = expert_out_list[o][pos:pos + ln]
            pos += ln
    return back


# --------------------------------------------------------------------------- #
# AllToAllV-GMM scheduler bookkeeping (device side of the same layout)
# --------------------------------------------------------------------------- #
def cumsum_mm(tokens_per_expert_all: np.ndarray, rank: int, ep: int, experts_per_rank: int) -> np.ndarray:
    """cumsumMM[EP][E_local]: running sum over source ranks of the tokens headed
    for this rank's experts
    (include/catccos/comm/block/comm_block_scheduler_alltoallv_gmm.hpp:131-159)."""
    t = np.asarray(tokens_per_expert_all, dtype=np.int32).reshape(ep, ep * experts_per_rank)
    mine = t[:, rank * experts_per_rank:(rank + 1) * experts_per_rank]
    return np.cumsum(mine, axis=0, dtype=np.int32)


def set_comm_core(tokens_per_expert_flat, rank, ep, experts_per_rank, core_idx, core_num):
    """`SetCommCore` + accessors of BlockCommSchedulerAllToAllVGmm
    (comm_block_scheduler_alltoallv_gmm.hpp:87-127): returns
    (prevSum, commLoops, [blockOffset(i).row for i in 0,1])."""
    t = np.asarray(tokens_per_expert_flat, dtype=np.int64)
    prev = 0
    if core_idx < ep:
        prev = int(t[core_idx * ep * experts_per_rank: core_idx * ep * experts_per_rank + rank * experts_per_rank].sum())
    if core_num == 0:
        loops = 1
    else:
        loops = ep // core_num + (1 if core_idx < ep % core_num else 0)
    return prev, loops, [core_idx + i * core_num for i in range(2)]


# --------------------------------------------------------------------------- #
# math stages
# --------------------------------------------------------------------------- #
def _bf16_round(x: np.ndarray) -> np.ndarray:
    return mxquant.bf16_bits_to_f32(mxquant.f32_to_bf16_bits(x)).reshape(x.shape)


def grouped_gemm_bf16(a_deq: np.ndarray, w_deq_list, blocks) -> np.ndarray:
    """Per-expert fp32 matmul on dequantised operands, result rounded to bf16
    (gen_data_moe.py:553-559, 583-588)."""
    outs, pos = [], 0
    for w, n in zip(w_deq_list, blocks):
        a = torch.from_numpy(np.ascontiguousarray(a_deq[pos:pos + n]))
        outs.append(torch.matmul(a, torch.from_numpy(w)).to(torch.bfloat16).to(torch.float32).numpy())
        pos += n
    width = w_deq_list[0].shape[1]
    return np.concatenate(outs, axis=0) if outs else np.zeros((0, width), np.float32)


def swiglu_bf16(c: np.ndarray) -> np.ndarray:
    """y = bf16( act * sigmoid(act) * gate ), act = first half of the columns,
    gate = second half, fp32 math on bf16-valued inputs (gen_data_moe.py:562-564;
    include/catccos/epilogue/block/block_epilogue_regbase_swiglu.hpp:39-81)."""
    t = torch.from_numpy(np.ascontiguousarray(c, dtype=np.float32))
    act, gate = t.chunk(2, dim=-1)
    glu = (act * torch.sigmoid(act) * gate).to(torch.bfloat16).to(torch.float32)
    return glu.numpy()


def unpermute_fp32(rows_back: np.ndarray, expanded_src_to_dst: np.ndarray, probs: np.ndarray) -> np.ndarray:
    """out[t] = bf16_rne( sum_{k in order} fp32(row[idx[t*topK+k]]) * prob[t,k] ), fp32
    multiply then fp32 add — the device kernel's definition
    (examples/aux_ops/moe_token_unpermute/moe_token_unpermute.h:234-278)."""
    m, top_k = probs.shape
    idx = expanded_src_to_dst.reshape(m, top_k).astype(np.int64)
    acc = np.zeros((m, rows_back.shape[1]), dtype=np.float32)
    for k in range(top_k):
        acc = (acc + rows_back[idx[:, k]].astype(np.float32) * probs[:, k:k + 1].astype(np.float32)).astype(np.float32)
    return _bf16_round(acc)


def unpermute_reference_cpu(rows_back: np.ndarray, sorted_src: np.ndarray, probs: np.ndarray) -> np.ndarray:
    """The reference's CPU fallback (gen_data_moe.py:60-70): weights and products in
    bf16, index_add_ into a bf16 output.  Kept to show the two definitions agree
    within bf16 tolerance."""
    tok = torch.from_numpy(np.ascontiguousarray(rows_back)).to(torch.bfloat16)
    pr = torch.from_numpy(np.ascontiguousarray(probs))
    ind = torch.from_numpy(sorted_src.astype(np.int64))
    top_k = pr.shape[1]
    out = torch.zeros((pr.shape[0], tok.shape[-1]), dtype=tok.dtype)
    w = pr[ind // top_k, ind % top_k].to(tok.dtype).unsqueeze(-1)
    out.index_add_(0, ind // top_k, tok * w)
    return out.to(torch.float32).numpy()


# --------------------------------------------------------------------------- #
# full pipeline — gen_data_moe.py:460-615 (`generate_dispatch_ffn_combine`)
# --------------------------------------------------------------------------- #
def dispatch_ffn_combine(x_list, expert_idx_list, probs_list, w1_q_list, w1_s_list, w2_q_list, w2_s_list,
                         ep, experts_per_rank, return_intermediates=False):
    """x_list[r]: fp32 [m,K] holding bf16 values.  expert_idx_list[r]: int32 [m,topK].
    probs_list[r]: fp32 [m,topK].  w1_q_list[r]: uint8 [E_local, N, K] e4m3 codes
    (weights stored transposed, :546-552) with w1_s_list[r]: uint8 [E_local, N, K/32];
    w2_q_list[r]: [E_local, K, N/2], w2_s_list[r]: [E_local, K, N/2/32].
    Returns per-rank fp32 [m,K] arrays holding bf16 values."""
    expert_num = ep * experts_per_rank
    top_k = expert_idx_list[0].shape[1]
    sorted_src, counts, routed = [], [], []
    for r in range(ep):
        s, c = moe_init_routing(expert_idx_list[r], expert_num)
        sorted_src.append(s)
        counts.append(c)
        routed.append(permute_rows(x_list[r], s, top_k))
    counts_all = np.stack(counts)
    recv, blocks = alltoallv_dispatch(routed, counts_all, ep, experts_per_rank)

    out_back_in = []
    inter = {"sorted_src": sorted_src, "counts": counts_all, "recv": recv, "blocks": blocks,
             "gmm1": [], "glu": [], "act_q": [], "act_s": [], "gmm2": []}
    for r in range(ep):
        w1 = [mxquant.dequant_mx_e4m3(w1_q_list[r][e], w1_s_list[r][e]).T.copy() for e in range(experts_per_rank)]
        w2 = [mxquant.dequant_mx_e4m3(w2_q_list[r][e], w2_s_list[r][e]).T.copy() for e in range(experts_per_rank)]
        _, _, a_deq = mxquant.quantize_mx_e4m3(recv[r], "rne")          # :556 dynamic_quant_rne per block == whole
        c1 = grouped_gemm_bf16(a_deq, w1, blocks[r])                    # :553-559
        glu = swiglu_bf16(c1)                                           # :562-564
        gq, gs, g_deq = mxquant.quantize_mx_e4m3(glu, "rne")            # :565
        c2 = grouped_gemm_bf16(g_deq, w2, blocks[r])                    # :583-588
        out_back_in.append(c2)
        if return_intermediates:
            inter["gmm1"].append(c1); inter["glu"].append(glu)
            inter["act_q"].append(gq); inter["act_s"].append(gs); inter["gmm2"].append(c2)
    back = alltoallv_combine(out_back_in, counts_all, ep, experts_per_rank)
    outs = []
    for r in range(ep):
        inv = expanded_row_idx_src_to_dst(sorted_src[r])
        outs.append(unpermute_fp32(back[r], inv, probs_list[r]))
    if return_intermediates:
        inter["back"] = back
        return outs, inter
    return outs


# --------------------------------------------------------------------------- #
# Standalone AllToAllV-GroupedMatmul and GroupedMatmul-AllToAllV (MXFP8 operands)
# --------------------------------------------------------------------------- #
def alltoallv_grouped_matmul(a_deq_list, w_deq_lists, tokens_per_expert_all, ep, experts_per_rank):
    """Dispatch then grouped GEMM, fp32 result per expert-owning rank.

    examples/utils/gen_data_fp8_mx_alltoallv_gmm.py:575-605, 634-640: every rank's rows are
    already grouped by global expert (`local_tokens_per_expert`); owner `o` receives, local
    expert major and source rank minor, the rows of its experts and multiplies every local
    expert's rows with that expert's [k, n] weight.  a_deq_list[r]: fp32 [m, k] dequantised
    rows of rank r; w_deq_lists[o][le]: fp32 [k, n]."""
    recv, blocks = alltoallv_dispatch(a_deq_list, tokens_per_expert_all, ep, experts_per_rank)
    outs = []
    for o in range(ep):
        pos, parts = 0, []
        for le, n in enumerate(blocks[o]):
            a = torch.from_numpy(np.ascontiguousarray(recv[o][pos:pos + n]))
            parts.append(torch.matmul(a, torch.from_numpy(np.ascontiguousarray(w_deq_lists[o][le]))).numpy())
            pos += n
        width = w_deq_lists[o][0].shape[1]
        outs.append(np.concatenate(parts, axis=0) if parts else np.zeros((0, width), np.float32))
    return outs, blocks


def grouped_matmul_alltoallv(a_deq_list, w_deq_lists, tokens_per_expert_all, ep, experts_per_rank):
    """Grouped GEMM on the expert owners, then every result row goes back to its source rank.

    examples/utils/gen_data_gmm_alltoallv_fp8_mx.py:720-751, 796-806: owner `o` holds rows grouped
    local expert major / source rank minor (counts `tokens_per_expert_all[src, o*E_local + le]`),
    multiplies each local expert's rows with its weight, and rank `src` ends up with its rows in
    global-expert order.  Only the first sum(counts) rows of a_deq_list[o] are used."""
    t = np.asarray(tokens_per_expert_all, dtype=np.int64)
    outs = []
    for o in range(ep):
        pos, parts = 0, []
        for le in range(experts_per_rank):
            n = int(t[:, o * experts_per_rank + le].sum())
            a = torch.from_numpy(np.ascontiguousarray(a_deq_list[o][pos:pos + n]))
            parts.append(torch.matmul(a, torch.from_numpy(np.ascontiguousarray(w_deq_lists[o][le]))).numpy())
            pos += n
        outs.append(np.concatenate(parts, axis=0))
    return alltoallv_combine(outs, tokens_per_expert_all, ep, experts_per_rank)


# --------------------------------------------------------------------------- #
# AllToAllV-AllGather and ReduceScatter-AllToAllV block schedulers (EP x TP layouts)
# --------------------------------------------------------------------------- #
def _cdiv(a, b):
    return -(-int(a) // int(b))


def _clip_sub(a, b):
    return max(int(a) - int(b), 0)


class AllToAllVAllGatherSchedule:
    """Bookkeeping of `BlockCommSchedulerAllToAllVAllGather`
    (include/catccos/comm/block/comm_block_scheduler_alltoallv_allgather.hpp:27-178) over an
    `AllToAllVAllGatherProblemShape` (include/catccos/dgemm/alltoallv_allgather_problem_shape.hpp:
    20-133): rank_size = ep_size * tp_size ranks, `local_tokens_per_expert[e]` = tokens this rank
    sends for global expert e, `global_tokens_per_local_expert[r * L + le]` = tokens rank r sends
    to this rank's local expert le.  One communication round moves at most `comm_rows` rows per
    peer, cut into blocks of `block_shape` (rows, columns)."""

    def __init__(self, k, rank_size, rank_idx, ep_size, expert_num, local_tokens_per_expert,
                 global_tokens_per_local_expert, comm_rows, block_shape):
        self.k, self.rank_size, self.rank_idx, self.ep_size = k, rank_size, rank_idx, ep_size
        self.local_experts = expert_num // ep_size
        self.comm_rows = comm_rows
        self.block_shape = tuple(block_shape)
        self.block_grid = (_cdiv(comm_rows, block_shape[0]), _cdiv(k, block_shape[1]))       # :52-53
        self.core_loops = self.block_grid[0] * self.block_grid[1] * rank_size                # :54
        loc = np.asarray(local_tokens_per_expert, dtype=np.int64).reshape(ep_size, self.local_experts)
        glo = np.asarray(global_tokens_per_local_expert, dtype=np.int64).reshape(rank_size, self.local_experts)
        self.input_split = loc.sum(axis=1)                                                   # :58-61
        self.input_offset = np.concatenate([[0], np.cumsum(self.input_split)[:-1]])          # :62-63
        self.output_split = glo.sum(axis=1)                                                  # :68-71
        loops = [_cdiv(v, comm_rows) for v in self.input_split] + [_cdiv(v, comm_rows) for v in self.output_split]
        self.comm_loops = max([0] + loops)                                                   # :64-65, :72-73

    def actual_receive_accum(self, comm_idx):
        """Blocks this rank receives in round `comm_idx` (:83-94)."""
        total = 0
        for r in range(self.rank_size):
            rows = min(self.comm_rows, _clip_sub(self.output_split[r], comm_idx * self.comm_rows))
            total += _cdiv(rows, self.block_shape[0]) * _cdiv(self.k, self.block_shape[1])
        return total

    def block_offset(self, task_idx):
        """Task -> ((row, column) offset inside the round, destination rank): destination rank
        fastest, then block column, then block row (:128-135)."""
        dst = task_idx % self.rank_size
        blk = task_idx // self.rank_size
        return ((blk // self.block_grid[1]) * self.block_shape[0], (blk % self.block_grid[1]) * self.block_shape[1]), dst

    def source_offset(self, comm_idx, offset, dst_rank):
        """`RemapperSrc::operator()` (:143-151): row of this rank's expert-sorted tokens."""
        ep = dst_rank % self.ep_size
        return int(self.input_offset[ep]) + comm_idx * self.comm_rows + offset[0], offset[1]

    def actual_block_shape(self, comm_idx, offset, dst_rank):
        """`RemapActualBlockShape` (:153-176): the block clipped to what is left for that peer."""
        ep = dst_rank % self.ep_size
        rows_left = min(self.comm_rows, _clip_sub(self.input_split[ep], comm_idx * self.comm_rows))
        return (min(self.block_shape[0], _clip_sub(rows_left, offset[0])),
                min(self.block_shape[1], _clip_sub(self.k, offset[1])))


class ReduceScatterAllToAllVSchedule:
    """Bookkeeping of `BlockCommSchedulerReduceScatterAllToAllV`
    (include/catccos/comm/block/comm_block_scheduler_reducescatter_alltoallv.hpp:27-302), the way
    back of GroupedMatmul-AllToAllV: results leave in rounds of `blocks_per_comm` GEMM blocks
    (`mmad_block` = rows x columns of one GEMM block) and every communication block of
    `comm_block` finds its destination row through the expert it belongs to."""

    def __init__(self, n, rank_size, ep_size, expert_num, local_tokens_per_expert, global_tokens_per_local_expert,
                 blocks_per_comm, src_ep, mmad_block, comm_block, core_split, deterministic=False):
        self.n, self.rank_size, self.ep_size, self.src_ep = n, rank_size, ep_size, src_ep
        self.local_experts = L = expert_num // ep_size
        self.blocks_per_comm = blocks_per_comm
        self.mmad_block, self.comm_block = tuple(mmad_block), tuple(comm_block)
        comm_shape = (blocks_per_comm * mmad_block[0], mmad_block[1])                        # :143
        self.block_grid = (_cdiv(comm_shape[0], comm_block[0]), _cdiv(comm_shape[1], comm_block[1]))
        tiles = self.block_grid[0] * self.block_grid[1]
        if deterministic:                                                                    # :146-151
            self.core_split = (core_split[0] * core_split[1], 1)
            self.core_loops = _cdiv(tiles, self.core_split[0]) * self.core_split[0]
        else:
            self.core_split = tuple(core_split)
            self.core_loops = tiles
        n_loops = _cdiv(n, mmad_block[1])                                                    # :154
        loc = np.asarray(local_tokens_per_expert, dtype=np.int64).reshape(ep_size, L)
        glo = np.asarray(global_tokens_per_local_expert, dtype=np.int64).reshape(rank_size, L)
        self.split_in_expert = np.array([[_cdiv(t, mmad_block[0]) * n_loops for t in row] for row in loc])   # :160
        self.input_split = self.split_in_expert.sum(axis=1)
        flat = loc.reshape(-1)
        self.input_offset = np.concatenate([[0], np.cumsum(flat)[:-1]]).reshape(ep_size, L)  # :162-163
        self.actual_mmad_shape = [(int(loc[src_ep, le]), n) for le in range(L)]              # :169-173
        self.mmad_grid = [(_cdiv(r, mmad_block[0]), _cdiv(c, mmad_block[1])) for r, c in self.actual_mmad_shape]
        self.output_split = np.array([sum(_cdiv(t, mmad_block[0]) for t in row) * n_loops for row in glo])   # :175-180
        loops = [_cdiv(v, blocks_per_comm) for v in self.input_split] + [_cdiv(v, blocks_per_comm) for v in self.output_split]
        self.comm_loops = max([0] + loops)
        self.start_expert, self.accum_blocks, self.mmad_idx = 0, 0, 0
        self.comm_offset, self.actual_comm_shape = 0, (0, 0)

    def update_comm_context(self, comm_idx):                                                 # :194-202
        self.comm_offset = comm_idx * self.blocks_per_comm
        blocks = min(self.blocks_per_comm, _clip_sub(self.input_split[self.src_ep], self.comm_offset))
        self.actual_comm_shape = (blocks * self.mmad_block[0], self.mmad_block[1])

    def update_local_expert_context(self, offset):                                           # :204-217
        self.mmad_idx = self.comm_offset + offset[0] // self.mmad_block[0]
        while self.start_expert < self.local_experts:
            step = int(self.split_in_expert[self.src_ep][self.start_expert])
            if self.accum_blocks + step > self.mmad_idx:
                break
            self.accum_blocks += step
            self.start_expert += 1

    def actual_receive_accum(self):                                                          # :219-229
        return int(sum(1 for r in range(self.rank_size) if self.comm_offset < self.output_split[r]))

    def block_offset(self, task_idx):                                                        # :253-260
        m = task_idx // self.block_grid[1]
        return m * self.comm_block[0], (task_idx - m * self.block_grid[1]) * self.comm_block[1]

    def destination(self, offset):
        """`RemapperDst::operator()` (:262-287): ((row, column) in the source rank's expert-sorted
        output, rows and columns left inside the GEMM block)."""
        from . import swizzle
        le = self.start_expert
        idx = self.mmad_idx - self.accum_blocks
        br, bc = swizzle.matrix_swizzle_coord(self.mmad_grid[le][0], self.mmad_grid[le][1], idx, 7, 1)
        off = (br * self.mmad_block[0], bc * self.mmad_block[1])
        shape = self.actual_mmad_shape[le]
        actual = (min(self.mmad_block[0], _clip_sub(shape[0], off[0])), min(self.mmad_block[1], _clip_sub(shape[1], off[1])))
        inside = (offset[0] % self.mmad_block[0], offset[1] % self.mmad_block[1])
        residue = (actual[0] - min(actual[0], inside[0]), actual[1] - min(actual[1], inside[1]))
        dst = (int(self.input_offset[self.src_ep][le]) + off[0] + inside[0], off[1] + inside[1])
        return dst, residue

    def actual_block_shape(self, offset):                                                    # :289-300
        return (min(self.comm_block[0], _clip_sub(self.actual_comm_shape[0], offset[0])),
                min(self.comm_block[1], _clip_sub(self.actual_comm_shape[1], offset[1])))
