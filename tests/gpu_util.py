"""Shared helpers of the GPU parity tests (CUDA path through the C-ABI vs the CPU oracle)."""
import os

import torch

os.environ.setdefault("CATCCOS_WAIT_TIMEOUT_MS", "4000")


def dev(t):
    return t.cuda().contiguous()


def assert_close_to_golden(actual, golden, k, tol, what=""):
    """Acceptance gate (max |diff| / max(1,|golden|) <= tol) plus the reference's own gate
    (examples/utils/verify_result.py:154-196)."""
    from oracle import verify
    act = actual.detach().cpu()
    err = verify.max_rel_err(act, golden)
    assert err <= tol, f"{what}: max relative error {err:.4g} > {tol}"
    ok, precision, eb = verify.reference_check(act, golden, k)
    assert ok, f"{what}: reference gate failed (precision {precision:.4f}%, eb {eb:.2f}%)"
    return err
