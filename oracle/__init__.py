"""CPU oracle for the quantized-linear hot path.  TEST INFRASTRUCTURE ONLY.

Nothing in the product package imports this directory.  It is used by the test
suite, by the smoke check and by the CPU-baseline leg of the benchmark as the
checker that the CUDA path is compared against.

Parity status: the reference pins no golden vectors for FP8/NVFP4 codes or block
scales (its tests compare end-to-end model outputs at loose tolerances against a
third-party eager implementation that is not part of the reference tree), so
code-level parity is "parity unpinned": every rounding/ordering choice is fixed
explicitly in `quant_oracle.py` and documented there.  The pieces that ARE pinned:
the FP8/FP4/E4M3 number formats (checked against torch's own float8/float4 dtypes
and an independent numpy implementation), the call-site formulas of the reference
converters (cited per function), and the all-reduce known answer
(sum of fill(rank+1) == W(W+1)/2).
"""
from .quant_oracle import *  # noqa: F401,F403
