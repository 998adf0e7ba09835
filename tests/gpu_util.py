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
