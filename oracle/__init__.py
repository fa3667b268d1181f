"""CPU oracle for the tensor-parallel epilogue (test infrastructure, not product code).

Everything under ``oracle/`` restates, on the CPU, what the reference computes for the
path ``allreduce -> + residual -> RMSNorm -> FP8 quantisation``.  It is the *checker*:
only the tests, the smoke entry and the benchmark's CPU-baseline leg may import it.  The
shipped package never does; it fails loudly when its CUDA library is missing.

Pinned against: golden vectors produced by running the reference's own Python
(``gpuk/__init__.py:147-173``) over gloo, stored in ``tests/golden``; and against the
reference's software FP8 conversion (``src/common/float8.h:17-150``) compiled from its
sources into ``oracle/_ref``.

``fp8_linear_oracle`` states, in float64, what the linear layer that consumes the operator's FP8
output must compute (the reference has no FP8 linear layer; the definition follows from the
operator's own quantisation rule) and is pinned by a known-answer test.
"""
