"""Row softmax: the call surface of examples/softmax.jl.

Tensors are in the memory order of the Julia arrays: Julia `input(N, M)` is a
torch tensor of shape [M, N] (each row is one softmax problem of N elements).
"""
from . import _lib
from ._util import handles, ptr, rows, dtype_code, next_power_of_2  # noqa: F401


def _run(output, input, variant, tile_size, hints):
    ctx, stream = handles(input, hints)
    ldi, M, N = rows(input, "input")
    ldo, Mo, No = rows(output, "output")
    if (Mo, No) != (M, N) or output.dtype != input.dtype:
        raise _lib.CtbError(_lib.BAD_ARG, "softmax: output must have the shape and element type of input")
    _lib.check(_lib.lib.ctb_softmax(ctx, stream, ptr(output), ptr(input), N, M, ldo, ldi, variant, int(tile_size),
                                    dtype_code(input)))
    return output


def softmax_tma_kernel(output, input, TILE_SIZE, **hints):
    """softmax_tma_kernel(output, input, TILE_SIZE), examples/softmax.jl:18-42:
    one tile holds the whole row (TILE_SIZE >= N)."""
    return _run(output, input, 0, TILE_SIZE, hints)


def softmax_chunked_kernel(output, input, n_elems, TILE_SIZE, **hints):
    """softmax_chunked_kernel(output, input, n_elems, TILE_SIZE), examples/softmax.jl:48-100."""
    if n_elems != input.shape[1]:
        raise _lib.CtbError(_lib.BAD_ARG, "softmax_chunked_kernel: n_elems must equal the row length")
    return _run(output, input, 1, TILE_SIZE, hints)
