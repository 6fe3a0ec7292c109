"""CPU oracle for the cuTile.jl example-kernel suite.

TEST INFRASTRUCTURE ONLY.  This package restates, in numpy, the plain-Julia CPU
checks that the reference's examples run in their own ``verify``/``ref_*``
functions (each function below cites the file:line it follows).  Only the test
suite, the smoke check and the benchmark's CPU-baseline leg may import it; the
product (the CUDA library and its Python/Julia mirrors) never does.

Parity status: PARITY UNPINNED for kernel results.  The reference ships no
golden vectors, known-answer tests or fixtures for these kernels; every check
in its tree is "random inputs vs. an in-file CPU formula under a norm-wise
tolerance", and the reference itself (Julia + the closed ``tileiras``
compiler) cannot run in this environment.  The one known-answer table that
touches this path, the TF32 bit-packing cases of ``test/types.jl:203-245``, pins
``f32_to_tf32_bits`` (see ``tests/test_oracle.py``).
"""
from . import inputs, ref  # noqa: F401
