"""Helpers shared by the per-example modules: argument checks and handles."""
import ctypes as C

import torch

from . import _lib


def next_power_of_2(n):
    """`next_power_of_2` of examples/softmax.jl:107-114."""
    p = 1
    while p < n:
        p <<= 1
    return p


_HINT_KEYS = ("num_ctas", "occupancy", "opt_level", "num_worker_warps")


def check_hints(hints):
    """The launch keywords of `@cuda backend=cuTile ...` / `ct.launch` (src/launch.jl:855-869): `num_ctas`,
    `occupancy`, `opt_level`, `num_worker_warps` are validated with the reference's ranges (validate_hint,
    src/language/types.jl:864-882) and are advisory (the kernels pick their own configuration); `sm_arch`, `name`
    and `dependent` are accepted; `stream` is honoured by handles().  Anything else is an error, as in the reference."""
    vals = []
    for k in _HINT_KEYS:
        v = hints.get(k)
        if v is None:
            vals.append(-1)
        elif isinstance(v, bool) or not isinstance(v, int):
            raise _lib.CtbError(_lib.BAD_ARG, f"{k} must be an integer, got {type(v).__name__}")
        else:
            vals.append(v)
    for k in hints:
        if k not in _HINT_KEYS and k not in ("sm_arch", "name", "dependent", "stream"):
            raise _lib.CtbError(_lib.BAD_ARG, f"unknown hint key: {k}")
    if any(v != -1 for v in vals):
        _lib.check(_lib.lib.ctb_validate_hints(*vals))


def handles(t, hints=None):
    """(context, raw stream handle) for the device that holds tensor `t`; `hints` are the launch keywords of the
    call (checked; `stream`, a torch stream or a raw handle, replaces the current stream)."""
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        # the reference rejects host arrays the same way (src/language/types.jl:371-376)
        raise _lib.CtbError(_lib.BAD_ARG, "expected a CUDA tensor (device array); host arrays are not accepted")
    dev = t.device.index if t.device.index is not None else torch.cuda.current_device()
    stream = None
    if hints:
        check_hints(hints)
        stream = hints.get("stream")
    if stream is None:
        stream = torch.cuda.current_stream(dev)
    raw = stream.cuda_stream if hasattr(stream, "cuda_stream") else int(stream)
    return _lib.context(dev), C.c_void_p(raw)


def ptr(t):
    if t is None:
        return C.c_void_p(0)
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise _lib.CtbError(_lib.BAD_ARG, "expected a CUDA tensor (device array); host arrays are not accepted")
    return C.c_void_p(t.data_ptr())


def rows(t, what):
    """(ld, n_rows, n_cols) of a 2-D tensor whose rows are contiguous."""
    if t.dim() != 2 or (t.shape[1] > 1 and t.stride(1) != 1):
        raise _lib.CtbError(_lib.BAD_ARG, f"{what}: expected a 2-D tensor with contiguous rows")
    ld = t.stride(0) if t.shape[0] > 1 else max(t.shape[1], t.stride(0))
    return ld, t.shape[0], t.shape[1]


def dtype_code(t):
    if t.dtype == torch.float32:
        return _lib.F32
    if t.dtype == torch.float16:
        return _lib.F16
    if t.dtype == torch.bfloat16:
        return _lib.BF16
    raise _lib.CtbError(_lib.BAD_ARG, f"unsupported element type {t.dtype}")
