"""Matrix transpose: the call surface of examples/transpose.jl.

Memory order of the Julia arrays: x(M, N) is torch [N, M]; y(N, M) is torch [M, N].
"""
from . import _lib
from ._util import handles, ptr, rows, dtype_code


def transpose_kernel(x, y, tm, tn, **hints):
    """transpose_kernel(x, y, tm, tn), examples/transpose.jl:11-19: y = transpose(x)."""
    ctx, stream = handles(x, hints)
    ldx, N, M = rows(x, "x")
    ldy, My, Ny = rows(y, "y")
    if (My, Ny) != (M, N) or y.dtype != x.dtype:
        raise _lib.CtbError(_lib.BAD_ARG, "transpose_kernel: y must be (N, M) with the element type of x")
    _lib.check(_lib.lib.ctb_transpose(ctx, stream, ptr(x), ptr(y), M, N, ldx, ldy, int(tm), int(tn), dtype_code(x)))
    return y
