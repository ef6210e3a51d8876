"""CPU oracle for the two hot paths (TEST INFRASTRUCTURE, never the product).

A torch-CPU fp32 restatement of the reference's own naive / chunked linear-cross-entropy
and materialised-attention implementations.  Only the test suite, the smoke check and the
benchmark's CPU-baseline leg may import this package; the shipped operators never do and
fail loudly when the CUDA library is missing.

Parity pin status: the reference's arithmetic lives in MLX (mlx 0.32.0, not installable
here), so the reference itself cannot be executed to produce golden vectors for the
numeric paths.  The restatement is pinned against every literal known-answer test the
reference's own suite holds for these paths (hand-computed two-row NLL, the int4 nibble
layout, the 4x4 block-diagonal-causal mask, first-row/GQA/`L[0]` attention identities)
and is otherwise "parity unpinned": kernel-vs-oracle comparisons inherit the reference's
tolerance classes instead of golden data.
"""
