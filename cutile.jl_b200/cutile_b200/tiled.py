"""Host-level array operations: the call surface of cuTile.jl's ``ct.Tiled`` (src/broadcast.jl, src/mapreduce.jl).

``Tiled(t)`` marks a torch CUDA tensor (torch shape = Julia shape reversed; at most three dimensions, f32 or f16).
Arithmetic on Tiled values builds an expression tree; ``assign(dest, expr)`` is ``ct.Tiled(dest) .= expr`` and runs the
whole expression as ONE kernel; ``materialize(expr)`` is the allocating form (``C = expr``).  ``tsum``, ``tprod``,
``tmaximum``, ``tminimum`` and ``tmapreduce`` are ``sum(ct.Tiled(A); dims)`` and friends, with Julia's 1-based ``dims``
and the reduced dimensions kept with extent 1.
"""
import ctypes as C

import torch

from . import _lib
from ._util import handles, ptr, dtype_code

_OPS = {"input": 0, "const": 1, "identity": 16, "neg": 17, "abs": 18, "sqrt": 19, "exp": 20, "exp2": 21, "log": 22,
        "log2": 23, "sin": 24, "cos": 25, "tanh": 26, "inv": 27, "abs2": 28, "add": 64, "sub": 65, "mul": 66, "div": 67,
        "max": 68, "min": 69, "pow": 70}
MAX_DIMS = 3


class Expr:
    """A node of a broadcast expression: ("leaf", tensor) | ("const", value) | (unary name, Expr) | (binary name, Expr, Expr)."""

    def __init__(self, *node):
        self.node = node

    @staticmethod
    def wrap(x):
        if isinstance(x, Expr):
            return x
        if isinstance(x, torch.Tensor):
            return Tiled(x)
        if isinstance(x, (int, float)):
            return Expr("const", float(x))
        raise TypeError(f"a Tiled broadcast takes Tiled arrays and numbers, not {type(x).__name__}")  # no device storage

    def _bin(self, name, other, swap=False):
        o = Expr.wrap(other)
        return Expr(name, o, self) if swap else Expr(name, self, o)

    __add__ = lambda self, o: self._bin("add", o)
    __radd__ = lambda self, o: self._bin("add", o, True)
    __sub__ = lambda self, o: self._bin("sub", o)
    __rsub__ = lambda self, o: self._bin("sub", o, True)
    __mul__ = lambda self, o: self._bin("mul", o)
    __rmul__ = lambda self, o: self._bin("mul", o, True)
    __truediv__ = lambda self, o: self._bin("div", o)
    __rtruediv__ = lambda self, o: self._bin("div", o, True)
    __pow__ = lambda self, o: self._bin("pow", o)
    __neg__ = lambda self: Expr("neg", self)
    __abs__ = lambda self: Expr("abs", self)


class Tiled(Expr):
    """``ct.Tiled(A)``: an array leaf."""

    def __init__(self, tensor):
        if not isinstance(tensor, torch.Tensor) or not tensor.is_cuda:
            raise ValueError("Tiled: the array must live in device memory")  # the reference's ArgumentError for host leaves
        if tensor.dim() > MAX_DIMS:
            raise _lib.CtbError(_lib.UNSUPPORTED, "Tiled: at most three dimensions")
        if not tensor.is_contiguous():
            raise _lib.CtbError(_lib.BAD_ARG, "Tiled: the array must be dense")
        Expr.__init__(self, "leaf", tensor)
        self.tensor = tensor


def _unary(name):
    return lambda x: Expr(name, Expr.wrap(x))


sin, cos, exp, exp2, log, log2, sqrt, tanh, inv, abs2 = (_unary(n) for n in
                                                         ("sin", "cos", "exp", "exp2", "log", "log2", "sqrt", "tanh", "inv", "abs2"))
tmax = lambda a, b: Expr.wrap(a)._bin("max", b)
tmin = lambda a, b: Expr.wrap(a)._bin("min", b)


def _jshape(t):
    """Julia shape (first dimension contiguous) of a torch tensor, padded to three dimensions."""
    s = list(reversed(t.shape))
    return s + [1] * (MAX_DIMS - len(s))


def _leaves(e, out):
    if e.node[0] == "leaf":
        out.append(e.node[1])
    elif e.node[0] != "const":
        for c in e.node[1:]:
            _leaves(c, out)
    return out


def broadcast_shape(expr):
    """Julia's broadcast shape of the expression: dimensions are aligned from the FIRST one, extents 1 expand."""
    shape = [1] * MAX_DIMS
    for t in _leaves(expr, []):
        for k, n in enumerate(_jshape(t)):
            if n != 1:
                if shape[k] != 1 and shape[k] != n:
                    raise ValueError(f"DimensionMismatch: arrays could not be broadcast to a common size ({shape[k]} and {n})")
                shape[k] = n
    return shape


def _compile(expr):
    inputs, consts, prog = [], [], []

    def walk(e):
        kind = e.node[0]
        if kind == "leaf":
            t = e.node[1]
            idx = next((i for i, u in enumerate(inputs) if u is t), None)
            if idx is None:
                inputs.append(t)
                idx = len(inputs) - 1
            prog.extend((_OPS["input"], idx))
        elif kind == "const":
            v = e.node[1]
            if v not in consts:
                consts.append(v)
            prog.extend((_OPS["const"], consts.index(v)))
        else:
            for c in e.node[1:]:
                walk(c)
            prog.extend((_OPS[kind], 0))

    walk(expr)
    return inputs, consts, prog


def assign(dest, expr, **hints):
    """``ct.Tiled(dest) .= expr``: evaluates the whole expression in one kernel; returns dest."""
    expr = Expr.wrap(expr)
    if not isinstance(dest, torch.Tensor) or not dest.is_cuda:
        raise ValueError("Tiled: the destination must live in device memory")
    d = Tiled(dest)
    shape = _jshape(dest)
    bshape = broadcast_shape(expr)
    for k in range(MAX_DIMS):
        if bshape[k] != shape[k] and not (bshape[k] == 1):
            raise ValueError(f"DimensionMismatch: destination {tuple(shape)} and expression {tuple(bshape)}")
    inputs, consts, prog = _compile(expr)
    for t in inputs:
        if t.dtype != dest.dtype:
            raise _lib.CtbError(_lib.BAD_ARG, "Tiled: operands and destination must share one element type")
        if t.device != dest.device:
            raise _lib.CtbError(_lib.BAD_ARG, "Tiled: operands and destination must live on one device")
    ctx, stream = handles(dest, hints)
    strides = []
    for t in inputs:
        js, run = _jshape(t), 1
        for k in range(MAX_DIMS):
            strides.append(0 if js[k] == 1 else run)
            run *= js[k]
    n_in = len(inputs)
    c_shape = (C.c_int64 * 3)(*shape)
    c_in = (C.c_void_p * max(1, n_in))(*[t.data_ptr() for t in inputs])
    c_str = (C.c_int64 * max(1, 3 * n_in))(*strides)
    c_prog = (C.c_int32 * len(prog))(*prog)
    c_const = (C.c_float * max(1, len(consts)))(*consts)
    _lib.check(_lib.lib.ctb_tiled_broadcast(ctx, stream, ptr(d.tensor), c_shape, c_in, c_str, n_in, c_prog, len(prog) // 2,
                                            c_const, len(consts), dtype_code(dest)))
    return dest


def materialize(expr, **hints):
    """``C = expr`` for a Tiled expression: allocates the result with the broadcast shape."""
    expr = Expr.wrap(expr)
    leaves = _leaves(expr, [])
    if not leaves:
        raise ValueError("a tiled broadcast requires at least one Tiled() argument")
    ndim = max(t.dim() for t in leaves)
    shape = broadcast_shape(expr)[:ndim]
    dest = torch.empty(tuple(reversed(shape)), dtype=leaves[0].dtype, device=leaves[0].device)
    return assign(dest, expr, **hints)


def tmapreduce(f, op, a, dims=None, out=None, **hints):
    """``mapreduce(f, op, ct.Tiled(A); dims)``: f a unary function name ("identity", "abs", "abs2", ...), op one of
    "add", "mul", "max", "min"; dims Julia's 1-based dimensions (an int or a tuple; None = all).  Returns a tensor with
    extent 1 along the reduced dimensions (a 0-dimensional tensor for dims=None, like Julia's scalar)."""
    t = a.tensor if isinstance(a, Tiled) else Tiled(a).tensor
    if dims is None:
        jd = tuple(range(1, t.dim() + 1))
    else:
        jd = (dims,) if isinstance(dims, int) else tuple(dims)
        for d in jd:
            if not isinstance(d, int):
                raise TypeError("dims must be integers")
            if d < 1:
                raise ValueError("ArgumentError: reduced dimension(s) must be >= 1")
    mask = 0
    for d in jd:
        if d <= t.dim():  # dimensions beyond ndims have extent 1: reducing them changes nothing
            mask |= 1 << (d - 1)
    shape = _jshape(t)
    oshape = [1 if (mask >> k) & 1 else shape[k] for k in range(MAX_DIMS)][:max(t.dim(), 1)]
    dshape = tuple(reversed(oshape)) if t.dim() else ()
    if out is None:
        dest = torch.empty(dshape, dtype=t.dtype, device=t.device)
    else:  # the in-place form (sum!(R, A)): R has extent 1 along the reduced dimensions
        if tuple(out.shape) != dshape or out.dtype != t.dtype or out.device != t.device or not out.is_contiguous():
            raise _lib.CtbError(_lib.BAD_ARG, f"tmapreduce: out must be a dense {dshape} tensor of the source's type")
        dest = out
    ctx, stream = handles(t, hints)
    _lib.check(_lib.lib.ctb_tiled_mapreduce(ctx, stream, ptr(dest), ptr(t), (C.c_int64 * 3)(*shape), mask, _OPS[f], _OPS[op],
                                            dtype_code(t)))
    return dest.reshape(()) if dims is None else dest


tsum = lambda a, dims=None, **h: tmapreduce("identity", "add", a, dims, **h)  # out=R for the in-place form
tprod = lambda a, dims=None, **h: tmapreduce("identity", "mul", a, dims, **h)
tmaximum = lambda a, dims=None, **h: tmapreduce("identity", "max", a, dims, **h)
tminimum = lambda a, dims=None, **h: tmapreduce("identity", "min", a, dims, **h)
