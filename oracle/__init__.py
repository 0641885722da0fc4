"""CPU oracle for the per-layer GPTQ / GPTQ+ quantization path.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package may import this
directory; only the test-suite, the smoke check and the benchmark's CPU
baseline leg use it, and there only as the checker / the timed CPU arm.

Every function restates, in plain torch-on-CPU fp32 arithmetic, what the
reference project (Mrluxianseng/gptq_plus_mp_quant) computes for the same
inputs; each cites the reference file:line it follows.  Parity is pinned
against the reference itself: ``tests/golden/make_golden.py`` imports the
unmodified reference classes, runs them on seeded inputs and stores their
outputs as fixtures, and ``tests/test_oracle_golden.py`` checks this oracle
against those fixtures.
"""
from . import quantizer, hadamard, hessian, gptq  # noqa: F401
