"""MX block quantisation golden (e4m3 / e2m1 codes, E8M0 scale per 32 along K).

Test infrastructure only (see package docstring).  numpy + torch-CPU.
"""
import numpy as np
import torch

BLOCK = 32
EPS = 1e-12
E4M3_EMAX = 8
E4M3_MAX = 448.0
E2M1_EMAX = 2
E2M1_MAX = 6.0


# --------------------------------------------------------------------------- #
# bf16 helpers (bit patterns travel as uint16, as the reference stores them:
# examples/utils/utils.py:47-58)
# --------------------------------------------------------------------------- #
def bf16_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    return (np.asarray(bits, dtype=np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even fp32 -> bf16 bits
    (examples/utils/gen_mx_quant_allgather_data.py:494-500)."""
    b = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    rb = ((b >> np.uint32(16)) & np.uint32(1)) + np.uint32(0x7FFF)
    return ((b + rb) >> np.uint32(16)).astype(np.uint16)


# --------------------------------------------------------------------------- #
# E8M0 exponent — examples/utils/gen_mx_quant_allgather_data.py:168-189
# --------------------------------------------------------------------------- #
def e8m0_exp(max_abs: np.ndarray, emax: int) -> np.ndarray:
    """exp = 0 if amax < 1e-12 else clamp(floor(log2(amax)) - emax, -128, 127),
    floor(log2) taken from the fp32 exponent field (:185-187)."""
    max_abs = np.ascontiguousarray(max_abs, dtype=np.float32)
    zero = max_abs < np.float32(EPS)
    safe = np.where(zero, np.float32(1.0), max_abs).astype(np.float32)
    e = ((safe.view(np.int32) >> 23) & 0xFF) - 127 - emax
    e = np.clip(e, -128, 127)
    return np.where(zero, 0, e).astype(np.int32)


def exp_to_e8m0_byte(exp: np.ndarray) -> np.ndarray:
    """2^exp stored as float8_e8m0fnu (:341): biased exponent, bias 127."""
    return np.clip(exp + 127, 0, 254).astype(np.uint8)


# --------------------------------------------------------------------------- #
# fp32 -> e4m3fn codes
# --------------------------------------------------------------------------- #
def f32_to_e4m3_rne(x: np.ndarray) -> np.ndarray:
    """Bit-level round-to-nearest-even, saturating to +-448, NaN -> 0x7F|sign.

    Independent restatement of the cast the goldens use
    (`.to(torch.float8_e4m3fn)` after clamp: gen_mx_quant_allgather_data.py:
    287-288, gen_data_moe.py:491) and that the device performs
    (include/catccos/comm/block/comm_block_mx_quant.hpp:594-642)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    bits = x.view(np.uint32)
    sign = ((bits >> np.uint32(24)) & np.uint32(0x80)).astype(np.uint8)
    a = np.abs(x)
    nan = np.isnan(x)
    a = np.where(nan, np.float32(0), np.minimum(a, np.float32(E4M3_MAX)))
    # Normal e4m3 range starts at 2^-6; below it the grid is uniform with step 2^-9.
    ab = a.view(np.uint32)
    e = ((ab >> np.uint32(23)) & np.uint32(0xFF)).astype(np.int32) - 127
    e = np.maximum(e, -6)
    step = np.exp2((e - 3).astype(np.float32)).astype(np.float32)      # ulp at this binade
    q = a / step                                                        # exact (power of two)
    r = np.rint(q)                                                      # numpy rint = RNE
    v = (r * step).astype(np.float32)                                   # on the e4m3 grid
    vb = v.view(np.uint32)
    ve = ((vb >> np.uint32(23)) & np.uint32(0xFF)).astype(np.int32) - 127
    man = ((vb >> np.uint32(20)) & np.uint32(0x7)).astype(np.int32)
    normal = v >= np.float32(2.0 ** -6)
    code_n = ((ve + 7) << 3) | man
    code_s = np.rint(v * np.float32(2.0 ** 9)).astype(np.int32)         # subnormal: m * 2^-9
    code = np.where(normal, code_n, code_s).astype(np.uint8)
    code = np.where(nan, np.uint8(0x7F), code)
    return (code | sign).astype(np.uint8)


_E4M3_POS = None


def _e4m3_pos_lut() -> np.ndarray:
    global _E4M3_POS
    if _E4M3_POS is None:
        v = []
        for i in range(128):
            if i == 0:
                v.append(0.0)
            elif i == 127:
                v.append(E4M3_MAX)          # the reference LUT maps the NaN code to max (:83-84)
            else:
                ex, m = (i >> 3) & 0xF, i & 7
                v.append((m / 8.0) * 2.0 ** -6 if ex == 0 else (1 + m / 8.0) * 2.0 ** (ex - 7))
        _E4M3_POS = np.array(v, dtype=np.float32)
    return _E4M3_POS


def f32_to_e4m3_lut(x: np.ndarray) -> np.ndarray:
    """Nearest grid point, ties toward the smaller magnitude — the reference's
    default `lut` backend (gen_mx_quant_allgather_data.py:198-252).  Input must
    already be clamped to +-448.  Zero keeps a positive sign (:240-247)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    lut = _e4m3_pos_lut()
    mag = np.abs(x)
    up = np.clip(np.searchsorted(lut, mag, side="left"), 0, 127)
    lo = np.clip(up - 1, 0, 127)
    pick_lo = (mag - lut[lo]) <= (lut[up] - mag)
    idx = np.where(pick_lo, lo, up)
    chosen = lut[idx]
    # code 127 and 126 share the value 448 in the LUT; the cast back through
    # float8 gives 0x7E for 448.
    code = np.where(idx == 127, 126, idx).astype(np.uint8)
    neg = (x < 0) & (chosen != 0)
    return np.where(neg, code | np.uint8(0x80), code).astype(np.uint8)


def e4m3_to_f32(code: np.ndarray) -> np.ndarray:
    code = np.asarray(code, dtype=np.uint8)
    s = np.where(code & 0x80, np.float32(-1), np.float32(1))
    ex = ((code >> 3) & 0xF).astype(np.int32)
    m = (code & 7).astype(np.float32)
    v = np.where(ex == 0, m / 8 * np.float32(2.0 ** -6), (1 + m / 8) * np.exp2((ex - 7).astype(np.float32)))
    v = np.where((code & 0x7F) == 0x7F, np.float32(np.nan), v)
    return (s * v).astype(np.float32)


# --------------------------------------------------------------------------- #
# MXFP8 quantisation along the last axis —
# examples/utils/gen_mx_quant_allgather_data.py:255-313 (`_quantize_axis_last_fp8`)
# --------------------------------------------------------------------------- #
def quantize_mx_e4m3(x: np.ndarray, rounding: str = "rne"):
    """x: fp32 [M, K] (bf16 inputs are passed as their exact fp32 values).

    Returns (codes uint8 [M,K], scale bytes uint8 [M, even(ceil(K/32))],
    dequant fp32 [M,K]).  Scale count per row is padded to an even number with
    1.0 = byte 127 (:306-311).  `rounding`: "rne" (device behaviour, MoE golden
    gen_data_moe.py:482-493, `native` backend) or "lut" (ties toward zero, the
    reference default backend)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    m, k = x.shape
    nb = (k + BLOCK - 1) // BLOCK
    pad_k = nb * BLOCK
    xp = np.zeros((m, pad_k), dtype=np.float32)
    xp[:, :k] = x
    blocks = xp.reshape(m, nb, BLOCK)
    with np.errstate(invalid="ignore"):
        amax = np.abs(blocks).max(axis=-1)
    exp = e8m0_exp(amax, E4M3_EMAX)
    scale = np.exp2(exp.astype(np.float32)).astype(np.float32)
    with np.errstate(invalid="ignore", over="ignore", divide="ignore"):
        scaled = np.clip(blocks / scale[..., None], -E4M3_MAX, E4M3_MAX).astype(np.float32)
    codes = f32_to_e4m3_rne(scaled) if rounding == "rne" else f32_to_e4m3_lut(scaled)
    deq = e4m3_to_f32(codes) * scale[..., None]
    codes = codes.reshape(m, pad_k)[:, :k].copy()
    deq = deq.reshape(m, pad_k)[:, :k].astype(np.float32).copy()
    nbp = (nb + 1) // 2 * 2
    sb = np.full((m, nbp), 127, dtype=np.uint8)
    sb[:, :nb] = exp_to_e8m0_byte(exp)
    return codes, sb, deq


def quantize_mx_e4m3_axis0(w: np.ndarray, rounding: str = "rne"):
    """Blocks of 32 along axis 0 (K of a [K,N] weight):
    gen_mx_quant_allgather_data.py:316-323 (transpose, quantise, transpose)."""
    c, s, d = quantize_mx_e4m3(np.ascontiguousarray(w.T), rounding)
    return np.ascontiguousarray(c.T), np.ascontiguousarray(s.T), np.ascontiguousarray(d.T)


def dequant_mx_e4m3(codes: np.ndarray, scale_bytes: np.ndarray) -> np.ndarray:
    """codes [M,K] uint8, scale bytes [M, >=ceil(K/32)] -> fp32 [M,K]."""
    m, k = codes.shape
    nb = (k + BLOCK - 1) // BLOCK
    sc = np.exp2(scale_bytes[:, :nb].astype(np.float32) - 127.0).astype(np.float32)
    return (e4m3_to_f32(codes) * np.repeat(sc, BLOCK, axis=1)[:, :k]).astype(np.float32)


def pack_dispatch_rows(codes: np.ndarray, scale_bytes: np.ndarray) -> np.ndarray:
    """MoE dispatch row = [K e4m3 bytes][even(ceil(K/32)) E8M0 bytes]
    (include/catccos/comm/block/comm_block_mx_quant.hpp:313-330)."""
    return np.concatenate([codes, scale_bytes], axis=1)


# --------------------------------------------------------------------------- #
# MXFP4 (e2m1, E8M0 per 32) — gen_mx_quant_allgather_data.py:353-449
# --------------------------------------------------------------------------- #
_E2M1_LUT = np.array([0, 0.5, 1, 1.5, 2, 3, 4, 6, -0.0, -0.5, -1, -1.5, -2, -3, -4, -6], dtype=np.float32)


def quantize_mx_e2m1(x: np.ndarray):
    """Returns (nibble indices uint8 [M,K], packed bytes [M,ceil(K/2)], scale
    bytes, dequant).  argmin over the 16-entry LUT, lowest index wins ties
    (:397-402); low nibble = even column (:410-412)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    m, k = x.shape
    nb = (k + BLOCK - 1) // BLOCK
    pad_k = nb * BLOCK
    xp = np.zeros((m, pad_k), dtype=np.float32)
    xp[:, :k] = x
    blocks = xp.reshape(m, nb, BLOCK)
    amax = np.abs(blocks).max(axis=-1)
    exp = np.floor(np.log2(np.maximum(amax, np.float32(EPS)))).astype(np.int32) - E2M1_EMAX
    exp = np.where(amax < np.float32(EPS), 0, exp)
    exp = np.clip(exp, -128, 127).astype(np.int32)
    scale = np.exp2(exp.astype(np.float32)).astype(np.float32)
    scaled = np.clip(blocks / scale[..., None], -E2M1_MAX, E2M1_MAX)
    idx = np.abs(scaled[..., None] - _E2M1_LUT).argmin(axis=-1).astype(np.uint8)
    deq = (_E2M1_LUT[idx] * scale[..., None]).reshape(m, pad_k)[:, :k]
    idx = idx.reshape(m, pad_k)[:, :k]
    ip = idx if k % 2 == 0 else np.concatenate([idx, np.zeros((m, 1), np.uint8)], axis=1)
    packed = (ip[:, 0::2] | (ip[:, 1::2] << 4)).astype(np.uint8)
    nbp = (nb + 1) // 2 * 2
    sb = np.full((m, nbp), 127, dtype=np.uint8)
    sb[:, :nb] = exp_to_e8m0_byte(exp)
    return idx, packed, sb, deq.astype(np.float32)


# --------------------------------------------------------------------------- #
# torch conveniences
# --------------------------------------------------------------------------- #
def quantize_bf16_tensor(x: torch.Tensor, rounding: str = "rne"):
    """bf16 [M,K] tensor -> (codes uint8 tensor, scale-bytes uint8 tensor, dequant fp32 tensor)."""
    c, s, d = quantize_mx_e4m3(x.to(torch.float32).numpy(), rounding)
    return torch.from_numpy(c), torch.from_numpy(s), torch.from_numpy(d)


# --------------------------------------------------------------------------- #
# MXFP8 with e5m2 codes — the MXFP8 Matmul-ReduceScatter example quantises its
# inputs this way (examples/ascend950_mxfp8_matmul_reduce_scatter/scripts/
# gen_data_mxfp8_mmrs.py:26-243; emax = 15, :46-53)
# --------------------------------------------------------------------------- #
E5M2_EMAX = 15
E5M2_MAX = 57344.0


def e5m2_to_f32(code: np.ndarray) -> np.ndarray:
    """float8_e5m2 bits -> fp32 (IEEE-like: exponent 31 is Inf/NaN)."""
    code = np.asarray(code, dtype=np.uint8)
    # e5m2 is the top byte of an IEEE half
    return (code.astype(np.uint16) << np.uint16(8)).view(np.float16).astype(np.float32)


def _e5m2_pos_lut() -> np.ndarray:
    """The generator's table of non-negative e5m2 values, indexed by code 0..127
    (gen_data_mxfp8_mmrs.py:124-154): codes 124..127 are stored as the maximum."""
    v = e5m2_to_f32(np.arange(124, dtype=np.uint8)).astype(np.float64)
    v = np.concatenate([v, np.full(4, E5M2_MAX)])
    return v


def f32_to_e5m2_nearest(x: np.ndarray) -> np.ndarray:
    """Nearest table value after clamping to +-57344, as `_quantize_to_fp8` does
    with `argmin(|lut - v|)` (gen_data_mxfp8_mmrs.py:172-184): the first table
    index wins a tie, i.e. the value of smaller magnitude; the result is then
    cast with `.to(torch.float8_e5m2)` (:283), exact for table values."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    lut = _e5m2_pos_lut()[:125]                      # 0 .. 57344, strictly increasing
    a = np.minimum(np.abs(x.astype(np.float64)), E5M2_MAX)
    hi = np.searchsorted(lut, a, side="left")        # first table value >= a
    hi = np.clip(hi, 0, len(lut) - 1)
    lo = np.clip(hi - 1, 0, len(lut) - 1)
    pick_lo = (a - lut[lo]) <= (lut[hi] - a)         # tie -> lower index
    idx = np.where(pick_lo, lo, hi).astype(np.uint8)
    idx = np.where(idx == 124, np.uint8(123), idx)   # 57344 is code 123 (0x7B); 124 was only the table's alias
    neg = (x < 0) & (idx != 0)
    return np.where(neg, idx | np.uint8(0x80), idx).astype(np.uint8)


def quantize_mx_e5m2(x: np.ndarray):
    """Blocks of 32 along the last axis, scale 2^(floor(log2 amax) - 15), codes by
    nearest table value (gen_data_mxfp8_mmrs.py:156-234).  Returns (codes uint8,
    scale bytes padded to an even count with 127, dequant fp32)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    m, k = x.shape
    nb = (k + BLOCK - 1) // BLOCK
    xp = np.zeros((m, nb * BLOCK), dtype=np.float32)
    xp[:, :k] = x
    blocks = xp.reshape(m, nb, BLOCK)
    amax = np.abs(blocks).max(axis=-1)
    exp = e8m0_exp(amax, E5M2_EMAX)
    scale = np.exp2(exp.astype(np.float32)).astype(np.float32)
    codes = f32_to_e5m2_nearest(blocks / scale[..., None])
    deq = (e5m2_to_f32(codes) * scale[..., None]).reshape(m, nb * BLOCK)[:, :k].astype(np.float32).copy()
    codes = codes.reshape(m, nb * BLOCK)[:, :k].copy()
    sb = np.full((m, (nb + 1) // 2 * 2), 127, dtype=np.uint8)
    sb[:, :nb] = exp_to_e8m0_byte(exp)
    return codes, sb, deq


def dequant_mx(codes: np.ndarray, scale_bytes: np.ndarray, fmt: str = "e4m3") -> np.ndarray:
    """codes [M,K] uint8 (`fmt` "e4m3" or "e5m2"), scale bytes [M, >=ceil(K/32)] -> fp32 [M,K]."""
    m, k = codes.shape
    nb = (k + BLOCK - 1) // BLOCK
    sc = np.exp2(scale_bytes[:, :nb].astype(np.float32) - 127.0).astype(np.float32)
    val = e4m3_to_f32(codes) if fmt == "e4m3" else e5m2_to_f32(codes)
    return (val * np.repeat(sc, BLOCK, axis=1)[:, :k]).astype(np.float32)


# --------------------------------------------------------------------------- #
# FP4 operands of the GEMM goldens
# --------------------------------------------------------------------------- #
def unpack_e2m1(packed: np.ndarray, k: int) -> np.ndarray:
    """[M, ceil(k/2)] bytes -> fp32 [M, k]; low nibble = even column
    (examples/utils/gen_data_fp4_mx_allgather_matmul.py:521-543)."""
    packed = np.asarray(packed, dtype=np.uint8)
    idx = np.empty((packed.shape[0], packed.shape[1] * 2), dtype=np.uint8)
    idx[:, 0::2] = packed & 0x0F
    idx[:, 1::2] = packed >> 4
    return _E2M1_LUT[idx[:, :k]]


def dequant_mxfp4(packed: np.ndarray, scale_bytes: np.ndarray, k: int) -> np.ndarray:
    """MXFP4: e2m1 nibbles [M, ceil(k/2)] and E8M0 bytes per 32 along k -> fp32 [M, k]."""
    nb = (k + BLOCK - 1) // BLOCK
    sc = np.exp2(scale_bytes[:, :nb].astype(np.float32) - 127.0).astype(np.float32)
    return (unpack_e2m1(packed, k) * np.repeat(sc, BLOCK, axis=1)[:, :k]).astype(np.float32)


# NVFP4 has no counterpart in the reference (its FP4 is MXFP4): PARITY UNPINNED.  The definition
# below is the published one: e2m1 codes, one e4m3 scale per 16 elements along k, one fp32 scale per
# tensor; tensor scale = amax / (448 * 6), block scale = e4m3_rne(block amax / (6 * tensor scale)),
# codes = e2m1 nearest (ties to the even code) of x / (block scale * tensor scale).
NVFP4_BLOCK = 16


def _e2m1_rne_index(v: np.ndarray) -> np.ndarray:
    """Nearest e2m1 magnitude index 0..7 with ties to the even mantissa code."""
    grid = np.array([0, 0.5, 1, 1.5, 2, 3, 4, 6], dtype=np.float64)
    a = np.minimum(np.abs(v.astype(np.float64)), 6.0)
    hi = np.clip(np.searchsorted(grid, a, side="left"), 0, 7)
    lo = np.clip(hi - 1, 0, 7)
    dl, dh = a - grid[lo], grid[hi] - a
    pick_lo = (dl < dh) | ((dl == dh) & (lo % 2 == 0))
    return np.where(pick_lo, lo, hi).astype(np.uint8)


def quantize_nvfp4(x: np.ndarray):
    """x fp32 [M, K] (K % 16 == 0) -> (nibble indices [M,K], packed bytes [M,K/2], e4m3 scale bytes
    [M, K/16], tensor scale fp32, dequant fp32 [M,K])."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    m, k = x.shape
    assert k % NVFP4_BLOCK == 0
    amax = float(np.abs(x).max())
    tscale = np.float32(amax / (E4M3_MAX * E2M1_MAX)) if amax > 0 else np.float32(1.0)
    blocks = x.reshape(m, k // NVFP4_BLOCK, NVFP4_BLOCK)
    bmax = np.abs(blocks).max(axis=-1)
    sbyte = f32_to_e4m3_rne((bmax / (np.float32(E2M1_MAX) * tscale)).astype(np.float32))
    sval = e4m3_to_f32(sbyte) * tscale
    safe = np.where(sval > 0, sval, np.float32(1.0))
    mag = _e2m1_rne_index(blocks / safe[..., None])
    idx = np.where(blocks < 0, mag | np.uint8(8), mag).astype(np.uint8)
    idx = np.where(mag == 0, np.uint8(0), idx)                      # no negative zero
    deq = (_E2M1_LUT[idx] * sval[..., None]).reshape(m, k).astype(np.float32)
    idx = idx.reshape(m, k)
    packed = (idx[:, 0::2] | (idx[:, 1::2] << 4)).astype(np.uint8)
    return idx, packed, sbyte, tscale, deq


def dequant_nvfp4(packed: np.ndarray, scale_bytes: np.ndarray, tscale, k: int) -> np.ndarray:
    sc = e4m3_to_f32(scale_bytes) * np.float32(tscale)
    return (unpack_e2m1(packed, k) * np.repeat(sc, NVFP4_BLOCK, axis=1)[:, :k]).astype(np.float32)
