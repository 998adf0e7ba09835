"""Size-independent properties of the quantisation oracle (hypothesis): idempotence on its own grid (the
reference's bit-exact MX test feeds dequantised values for exactly this reason:
examples/utils/gen_mx_quant_allgather_data.py:529-534), error bounds, scale choice."""
import numpy as np
from hypothesis import given, settings, strategies as st
from hypothesis.extra import numpy as hnp

from oracle import mxquant

# values near the golden's 1e-12 "zero block" threshold are excluded: a block just above it dequantises to values
# just below it, so idempotence does not hold across that threshold (by the golden's own rule)
finite32 = st.floats(min_value=-3.0e4, max_value=3.0e4, allow_nan=False, allow_infinity=False, width=32).filter(
    lambda v: v == 0 or abs(v) > 1e-6)
rows = hnp.arrays(np.float32, st.tuples(st.integers(1, 4), st.sampled_from([32, 64, 96, 160])), elements=finite32)
SET = dict(max_examples=60, deadline=None, derandomize=True, database=None)


def _bf16(x):
    return mxquant.bf16_bits_to_f32(mxquant.f32_to_bf16_bits(x)).reshape(x.shape)


@settings(**SET)
@given(rows)
def test_mx_e4m3_is_idempotent_and_bounded(x):
    x = _bf16(x)
    c, s, d = mxquant.quantize_mx_e4m3(x, "rne")
    c2, s2, d2 = mxquant.quantize_mx_e4m3(d, "rne")
    assert np.array_equal(d2, d)                                   # dequantised values are a fixed point
    nb = x.shape[1] // 32
    scale = np.repeat(np.exp2(s[:, :nb].astype(np.float32) - 127), 32, axis=1)
    # e4m3 has 3 mantissa bits: relative error <= 2^-4 for normal codes, absolute <= half the smallest step below;
    # values above 448 * scale saturate
    sat = np.abs(x) > 448 * scale
    err = np.abs(d - x)
    bound = np.maximum(np.abs(x) * 2.0 ** -4, scale * 2.0 ** -10)
    assert (err[~sat] <= bound[~sat] * (1 + 1e-6)).all()
    assert (np.abs(d[sat]) == 448 * scale[sat]).all()
    # the block maximum lands in the top binade of e4m3: 256 <= |amax / scale| < 512 unless the block is ~zero
    amax = np.abs(x.reshape(x.shape[0], nb, 32)).max(axis=-1)
    live = amax >= 1e-12
    ratio = amax[live] / np.exp2(s[:, :nb].astype(np.float32) - 127)[live]
    assert ((ratio >= 256) & (ratio < 512)).all()
    assert (s[:, :nb][~live] == 127).all() and (s[:, nb:] == 127).all()


@settings(**SET)
@given(rows)
def test_mx_e5m2_and_e2m1_are_idempotent(x):
    c, s, d = mxquant.quantize_mx_e5m2(x)
    c2, s2, d2 = mxquant.quantize_mx_e5m2(d)
    assert np.array_equal(d2, d) and np.array_equal(mxquant.dequant_mx(c, s, "e5m2"), d)
    idx, packed, sb, deq = mxquant.quantize_mx_e2m1(x)
    idx2, packed2, sb2, deq2 = mxquant.quantize_mx_e2m1(deq)
    assert np.array_equal(deq2, deq)
    assert np.array_equal(mxquant.dequant_mxfp4(packed, sb, x.shape[1]), deq)


@settings(**SET)
@given(hnp.arrays(np.float32, st.tuples(st.integers(1, 4), st.sampled_from([16, 64, 128])), elements=finite32))
def test_nvfp4_round_trip_and_bound(x):
    idx, packed, sb, ts, deq = mxquant.quantize_nvfp4(x)
    assert np.array_equal(mxquant.dequant_nvfp4(packed, sb, ts, x.shape[1]), deq)
    sval = np.repeat(mxquant.e4m3_to_f32(sb) * ts, 16, axis=1)
    live = sval > 0
    # |x| <= 6 * (block amax / 6 rounded to e4m3, relative error <= 2^-4) -> at most one e2m1 step (<= 2 * scale) off
    assert (np.abs(deq - x)[live] <= (1.0 * sval + np.abs(x) * 2.0 ** -3)[live]).all()
    # a block whose scale underflows e4m3 (amax below half the smallest subnormal, 2^-10, of 6 x tensor scale)
    # is flushed to zero: the dynamic-range limit of the format
    assert (deq[~live] == 0).all() and (np.abs(x[~live]) <= 6.0 * ts * 2.0 ** -10 * (1 + 1e-6)).all()


@settings(**SET)
@given(hnp.arrays(np.float32, 64, elements=st.floats(min_value=-500, max_value=500, allow_nan=False, width=32)))
def test_e4m3_rne_agrees_with_the_lut_rounding_away_from_ties(v):
    """Both roundings of the reference (round-to-nearest-even and the LUT's ties-toward-zero) pick a nearest
    code; they may differ only on exact ties."""
    a, b = mxquant.f32_to_e4m3_rne(v), mxquant.f32_to_e4m3_lut(v)
    fa, fb = mxquant.e4m3_to_f32(a), mxquant.e4m3_to_f32(b)
    c = np.clip(v, -448, 448)
    assert np.allclose(np.abs(fa - c), np.abs(fb - c), rtol=0, atol=0)


# ----------------------------------------------------------------------------------------- MoE routing ----
from oracle import moe   # noqa: E402

routing = st.integers(1, 4).flatmap(lambda ep: st.tuples(
    st.just(ep), st.integers(1, 3), st.integers(1, 24), st.integers(1, 3), st.integers(0, 2 ** 31 - 1)))


@settings(**SET)
@given(routing)
def test_dispatch_then_combine_is_the_identity_and_tables_agree(cfg):
    """For any routing: the stable sort keeps equal experts in token order, every row reaches its expert's owner
    in (local expert, source rank) order, the way back restores the permuted rows exactly, and the device-side
    tables (cumsumMM) describe the same layout as the golden's all-to-all-v."""
    ep, epr, m, top_k, seed = cfg
    experts = ep * epr
    rng = np.random.default_rng(seed)
    idx = [rng.integers(0, experts, size=(m, top_k)).astype(np.int32) for _ in range(ep)]
    xs = [rng.integers(0, 1000, size=(m, 4)).astype(np.float32) + 10000 * r for r in range(ep)]   # rows tagged by rank
    srcs, counts, routed = [], [], []
    for r in range(ep):
        s, c = moe.moe_init_routing(idx[r], experts)
        flat = idx[r].reshape(-1)
        assert (np.diff(flat[s]) >= 0).all()                                  # sorted by expert
        same = np.diff(flat[s]) == 0
        assert (np.diff(s)[same] > 0).all()                                   # stable inside an expert
        assert c.sum() == m * top_k and np.array_equal(c, np.bincount(flat, minlength=experts))
        inv = moe.expanded_row_idx_src_to_dst(s)
        assert np.array_equal(inv[s], np.arange(m * top_k))
        srcs.append(s); counts.append(c); routed.append(moe.permute_rows(xs[r], s, top_k))
    table = np.stack(counts)
    recv, blocks = moe.alltoallv_dispatch(routed, table, ep, epr)
    for o in range(ep):
        assert blocks[o] == table[:, o * epr:(o + 1) * epr].sum(axis=0).tolist()
        # rows of local expert le coming from ranks < r, as the device schedulers count them
        cum = moe.cumsum_mm(table, o, ep, epr)
        pos = 0
        for le in range(epr):
            for src in range(ep):
                n = int(table[src, o * epr + le])
                assert int(cum[src, le]) - n == (int(cum[src - 1, le]) if src else 0)
                seg = recv[o][pos:pos + n]
                assert (seg[:, 0] // 10000 == src).all() or n == 0            # rows really come from `src`
                pos += n
        assert pos == recv[o].shape[0]
    back = moe.alltoallv_combine(recv, table, ep, epr)
    for r in range(ep):
        assert np.array_equal(back[r], routed[r])
