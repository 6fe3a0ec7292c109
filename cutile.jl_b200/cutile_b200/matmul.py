"""Dense GEMM: the call surface of examples/matmul.jl.

Memory order of the Julia arrays: A(M, K) is torch [K, M]; B(K, N) is torch
[N, K]; C(M, N) is torch [N, M].
"""
from . import _lib
from ._util import handles, ptr, rows, dtype_code


def matmul_kernel(A, B, C, tm, tn, tk, **hints):
    """matmul_kernel(A, B, C, tm, tn, tk), examples/matmul.jl:28-60."""
    ctx, stream = handles(A, hints)
    lda, K, M = rows(A, "A")
    ldb, N, Kb = rows(B, "B")
    ldc, Nc, Mc = rows(C, "C")
    if Kb != K or (Nc, Mc) != (N, M) or B.dtype != A.dtype or C.dtype != A.dtype:
        raise _lib.CtbError(_lib.BAD_ARG, "matmul_kernel: inconsistent shapes or element types")
    _lib.check(_lib.lib.ctb_gemm(ctx, stream, ptr(A), ptr(B), ptr(C), M, N, K, lda, ldb, ldc, dtype_code(A),
                                 int(tm), int(tn), int(tk)))
    return C
