"""Result verification: the reference's own gate and the stricter max-rel-err gate.

Test infrastructure only (see package docstring).
"""
import torch


def get_rtol(dtype: torch.dtype, compute_times: int) -> float:
    """examples/utils/utils.py:97-105."""
    if dtype == torch.float16:
        return 2 ** (-8) if compute_times < 2048 else 2 ** (-7)
    if dtype == torch.bfloat16:
        return 2 ** (-7) if compute_times < 2048 else 2 ** (-6)
    if dtype == torch.float32:
        return 2 ** (-11) if compute_times < 2048 else 2 ** (-10)
    raise ValueError(f"Invalid dtype: {dtype}.")


_EB = {torch.float16: 2 ** (-10), torch.bfloat16: 2 ** (-7), torch.float32: 2 ** (-14)}


def _sanitize(x: torch.Tensor) -> torch.Tensor:
    x = x.to(torch.float32)
    return torch.where(torch.isfinite(x), x, torch.zeros_like(x))


def reference_check(actual: torch.Tensor, golden: torch.Tensor, k: int):
    """The reference's COMPUTE_FLOAT gate.

    examples/utils/verify_result.py:154-196: NaN/Inf zeroed on both sides;
    every element must satisfy |diff| <= rtol * max(1, |golden|); and the mean
    of diff / max(1,|golden|) must not exceed the dtype's bias bound in
    magnitude (:56-64, :99).  Returns (ok, precision_percent, eb_percent)."""
    rtol = get_rtol(actual.dtype, k)
    eb_thr = _EB[actual.dtype]
    a = _sanitize(actual).flatten()
    g = _sanitize(golden).flatten()
    diff = a - g
    tmax = torch.maximum(torch.ones_like(g), g.abs())
    tol = diff.abs() - rtol * tmax
    precision = float((tol <= 0).sum()) / tol.numel() * 100
    eb = float((diff / tmax).mean().abs())
    eb_percent = 0.0 if eb == 0 else eb / eb_thr * 100
    return (precision == 100 and eb_percent <= 100), precision, eb_percent


def max_rel_err(actual: torch.Tensor, golden: torch.Tensor) -> float:
    """max |actual-golden| / max(1,|golden|) — the acceptance metric
    (1e-2 bf16/fp16, 2e-2 MXFP8, 5e-2 NVFP4), normalised as the reference
    normalises its own per-element tolerance (verify_result.py:166)."""
    a = _sanitize(actual).flatten()
    g = _sanitize(golden).flatten()
    return float(((a - g).abs() / torch.maximum(torch.ones_like(g), g.abs())).max())


def double_golden_ratios(actual, golden, golden_low, err_threshold):
    """verify_result.py:198-246: error of the kernel relative to the error of a
    low-precision golden, both against fp32.  Pass when max-rel ratio < 10,
    mean-rel ratio < 2 and rmse ratio < 2 (:105-117)."""
    eps = 1e-7
    a, g, gl = _sanitize(actual).flatten(), _sanitize(golden).flatten(), _sanitize(golden_low).flatten()
    da, dl = a - g, gl - g
    ra, rl = da.abs() / (g.abs() + eps), dl.abs() / (g.abs() + eps)
    rm_a, rm_l = torch.sqrt((da ** 2).mean()), torch.sqrt((dl ** 2).mean())
    return (float(ra.max() / max(float(rl.max()), err_threshold)),
            float(ra.mean() / max(float(rl.mean()), err_threshold)),
            float(rm_a / max(float(rm_l), err_threshold)))
