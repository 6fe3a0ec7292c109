"""Vector / matrix addition: the call surface of examples/vadd.jl.

Memory order of the Julia arrays: a 1-D array is a 1-D tensor; a 2-D array a(M, N) is torch [N, M] (M contiguous).
"""
from . import _lib
from ._util import handles, ptr, rows, dtype_code


def _check(a, b, c, who):
    if a.shape != b.shape or a.shape != c.shape or a.dtype != b.dtype or a.dtype != c.dtype:
        raise _lib.CtbError(_lib.BAD_ARG, f"{who}: a, b and c must agree in shape and element type")


def vec_add_kernel_1d(a, b, c, tile, **hints):
    """vec_add_kernel_1d(a, b, c, tile), examples/vadd.jl:10-17."""
    ctx, stream = handles(a, hints)
    _check(a, b, c, "vec_add_kernel_1d")
    if a.dim() != 1 or not (a.is_contiguous() and b.is_contiguous() and c.is_contiguous()):
        raise _lib.CtbError(_lib.BAD_ARG, "vec_add_kernel_1d: expected dense 1-D arrays")
    n = a.numel()
    _lib.check(_lib.lib.ctb_vadd(ctx, stream, ptr(a), ptr(b), ptr(c), n, 1, n, n, n, int(tile), 1, 0, dtype_code(a)))
    return c


def vec_add_kernel_1d_gather(a, b, c, tile, **hints):
    """vec_add_kernel_1d_gather(a, b, c, tile), examples/vadd.jl:31-45 (gather / add / scatter of a block's elements)."""
    ctx, stream = handles(a, hints)
    _check(a, b, c, "vec_add_kernel_1d_gather")
    if a.dim() != 1 or not (a.is_contiguous() and b.is_contiguous() and c.is_contiguous()):
        raise _lib.CtbError(_lib.BAD_ARG, "vec_add_kernel_1d_gather: expected dense 1-D arrays")
    n = a.numel()
    _lib.check(_lib.lib.ctb_vadd(ctx, stream, ptr(a), ptr(b), ptr(c), n, 1, n, n, n, int(tile), 1, 1, dtype_code(a)))
    return c


def vec_add_kernel_2d(a, b, c, tile_x, tile_y, **hints):
    """vec_add_kernel_2d(a, b, c, tile_x, tile_y), examples/vadd.jl:20-28."""
    ctx, stream = handles(a, hints)
    _check(a, b, c, "vec_add_kernel_2d")
    lda, N, M = rows(a, "a")
    ldb, _, _ = rows(b, "b")
    ldc, _, _ = rows(c, "c")
    _lib.check(_lib.lib.ctb_vadd(ctx, stream, ptr(a), ptr(b), ptr(c), M, N, lda, ldb, ldc, int(tile_x), int(tile_y), 0,
                                 dtype_code(a)))
    return c
