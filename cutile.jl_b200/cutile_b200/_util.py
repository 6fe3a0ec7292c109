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


def handles(t):
    """(context, raw stream handle) for the device that holds tensor `t`."""
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        # the reference rejects host arrays the same way (src/language/types.jl:371-376)
        raise _lib.CtbError(_lib.BAD_ARG, "expected a CUDA tensor (device array); host arrays are not accepted")
    dev = t.device.index if t.device.index is not None else torch.cuda.current_device()
    return _lib.context(dev), C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)


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
