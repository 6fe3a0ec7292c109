"""Python mirror of the Julia call surface kept by libcutile_b200.

Each module carries the name of the reference example whose entry points it
mirrors (examples/<name>.jl) and exposes functions with the same names and
argument order; tensors are torch CUDA tensors laid out like the Julia arrays
(so torch shapes are the Julia shapes reversed).  All arithmetic happens in the
CUDA library; nothing here computes on the host.
"""
from . import _lib  # noqa: F401  (fails loudly when the shared library is missing)
from ._lib import CtbError, version_info, check_device_status  # noqa: F401
from . import softmax, layernorm, matmul, batchmatmul, fmha, moe, multi, vadd, transpose, fft, tiled  # noqa: F401
