"""CPU oracle for the fused compute-communication hot path.

TEST INFRASTRUCTURE ONLY.  Nothing under this package is part of the product:
only the test-suite, the smoke check and the CPU-baseline legs of the benchmark
may import it, and only as the checker.  The product path is the CUDA library
(`catccos_b200/csrc`) reached through its C-ABI and fails loudly without it.

Each function restates, in numpy / torch-CPU, what the reference's own host
golden computes for one operator and cites the reference file:line it follows
(paths relative to the reference project root).

Pinning status (how each restatement is tied to the reference itself):
  * dense goldens, verifier .......... pinned by fixtures generated from the
    reference's Python (`tests/golden/make_golden.py`)
  * MX quantisation (e4m3/E8M0) ...... pinned, bit level, same way
  * MoE routing / all-to-all-v / SwiGLU / unpermute / full pipeline .. pinned
  * CommSwizzle / MatrixSwizzle ...... pinned by the reference's worked table
    and its own Python restatement
  * AllToAllV-GMM scheduler .......... pinned by the reference's known-answer
    unit test vector
  * NVFP4 (e2m1 + ue4m3 per 16) ...... PARITY UNPINNED: the reference has no
    such format (its FP4 is MXFP4), so the definition here is new.
"""
