"""Shared helpers of the GPU parity tests (CUDA path through the C-ABI vs the CPU oracle)."""
import os

import torch

os.environ.setdefault("CATCCOS_WAIT_TIMEOUT_MS", "4000")


def dev(t):
    return t.cuda().contiguous()


def assert_close_to_golden(actual, golden, k, tol, what="", strict_reference=True):
    """Acceptance gate (max |diff| / max(1,|golden|) <= tol) plus the reference's own gate
    (examples/utils/verify_result.py:154-196).

    `strict_reference=False` is for reductions over more than two ranks with a short K: partial
    products cross the link rounded to the output type (as in the reference, which even adds them
    with 16-bit atomics), and the reference's per-element rtol (2^-7 below K=2048) has no room for
    those extra roundings.  There the mean-bias bound still has to hold and at most one element
    in a thousand may exceed the per-element bound."""
    from oracle import verify
    act = actual.detach().cpu()
    err = verify.max_rel_err(act, golden)
    assert err <= tol, f"{what}: max relative error {err:.4g} > {tol}"
    ok, precision, eb = verify.reference_check(act, golden, k)
    if strict_reference:
        assert ok, f"{what}: reference gate failed (precision {precision:.4f}%, eb {eb:.2f}%)"
    else:
        assert precision >= 99.9 and eb <= 100, f"{what}: precision {precision:.4f}%, eb {eb:.2f}%"
    return err


def assert_reduced_close(actual, partials, k, tol, what=""):
    """Gate for operators that sum per-rank partial products after exchanging them in the output
    type (as the reference does: include/catccos/dgemm/kernel/matmul_reduce_scatter.hpp:314,
    matmul_allreduce.hpp:323).  `partials` are the fp32 per-rank products restricted to the rows
    under test.  Hard gate: max |diff| / max(1,|golden|) <= tol.  Per element, the reference's
    tolerance rtol*max(1,|golden|) is widened by the unit round-off of every exchanged partial,
    u*|partial_s| (u = 2^-11 for fp16, 2^-8 for bf16) — the part of the error the reference's own
    tolerance model does not count — and must then hold for every element; the mean-bias bound is
    unchanged."""
    import torch
    from oracle import verify
    act = actual.detach().cpu()
    golden = sum(partials)
    err = verify.max_rel_err(act, golden)
    assert err <= tol, f"{what}: max relative error {err:.4g} > {tol}"
    u = 2.0 ** -11 if act.dtype == torch.float16 else 2.0 ** -8
    rtol = verify.get_rtol(act.dtype, k)
    slack = sum(p.abs() for p in partials) * u
    diff = (act.to(torch.float32) - golden).abs()
    bound = rtol * torch.maximum(torch.ones_like(golden), golden.abs()) + slack
    bad = int((diff > bound).sum())
    assert bad == 0, f"{what}: {bad} elements beyond the widened reference tolerance"
    _, _, eb = verify.reference_check(act, golden, k)
    assert eb <= 100, f"{what}: mean bias {eb:.1f}% of the reference bound"
    return err
