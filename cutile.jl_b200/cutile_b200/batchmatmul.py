"""Batched GEMM: the call surface of examples/batchmatmul.jl.

Memory order of the Julia arrays (batch last): A(M, K, Batch) is torch
[Batch, K, M]; B(K, N, Batch) is torch [Batch, N, K]; C(M, N, Batch) is torch
[Batch, N, M].
"""
from . import _lib
from ._util import handles, ptr, dtype_code


def _dims(t, what):
    if t.dim() != 3 or t.stride(2) != 1:
        raise _lib.CtbError(_lib.BAD_ARG, f"{what}: expected a 3-D tensor with a contiguous last dimension")
    return t.shape[0], t.shape[1], t.shape[2], t.stride(1), t.stride(0)


def batch_matmul_kernel(A, B, C, tm, tn, tk, **hints):
    """batch_matmul_kernel(A, B, C, tm, tn, tk), examples/batchmatmul.jl:15-56."""
    ctx, stream = handles(A, hints)
    nb, K, M, lda, sA = _dims(A, "A")
    nb2, N, Kb, ldb, sB = _dims(B, "B")
    nb3, Nc, Mc, ldc, sC = _dims(C, "C")
    if (nb2, nb3) != (nb, nb) or Kb != K or (Nc, Mc) != (N, M) or B.dtype != A.dtype or C.dtype != A.dtype:
        raise _lib.CtbError(_lib.BAD_ARG, "batch_matmul_kernel: inconsistent shapes or element types")
    _lib.check(_lib.lib.ctb_gemm_batched(ctx, stream, ptr(A), ptr(B), ptr(C), M, N, K, nb, lda, ldb, ldc, sA, sB, sC,
                                         dtype_code(A), int(tm), int(tn), int(tk)))
    return C
