"""Batched FFT: the call surface of examples/fft.jl.

Memory order of the Julia arrays: x_packed(D, 2N / D, batch) is torch [batch, 2N / D, D] (per batch item N interleaved
(re, im) float32 pairs); W(2, F, F) is torch [F, F, 2]; T0(2, F1F2, F0) is torch [F0, F1F2, 2]; T1(2, F2, F1) is torch
[F1, F2, 2].  The tables are built on the host exactly as the example does and uploaded once.
"""
import math

import numpy as np
import torch

from . import _lib
from ._util import handles, ptr


def dft_matrix(size):
    """dft_matrix(size), examples/fft.jl:128-138: W[i, j] = exp(-2 pi i ij / size) as float32 [size, size, 2]."""
    i = np.arange(size)
    w = np.exp(-2j * np.pi * np.outer(i, i) / size).astype(np.complex64)
    return np.stack([w.real, w.imag], axis=-1).astype(np.float32)


def make_twiddles(factors):
    """make_twiddles(factors), examples/fft.jl:141-176: (W0, W1, W2, T0, T1) as float32 numpy arrays."""
    F0, F1, F2 = (int(f) for f in factors)
    N, F1F2 = F0 * F1 * F2, F1 * F2
    t0 = np.exp(-2j * np.pi * np.outer(np.arange(F0), np.arange(F1F2)) / N).astype(np.complex64)       # [i, j]
    t1 = np.exp(-2j * np.pi * np.outer(np.arange(F1), np.arange(F2)) / F1F2).astype(np.complex64)      # [j, k]
    T0 = np.stack([t0.real, t0.imag], axis=-1).astype(np.float32)
    T1 = np.stack([t1.real, t1.imag], axis=-1).astype(np.float32)
    return dft_matrix(F0), dft_matrix(F1), dft_matrix(F2), T0, T1


def fft_kernel(x_packed_in, y_packed_out, W0, W1, W2, T0, T1, N, F0, F1, F2, BS, D, **hints):
    """fft_kernel(x_packed_in, y_packed_out, W0, W1, W2, T0, T1, N, F0, F1, F2, BS, D), examples/fft.jl:22-126."""
    ctx, stream = handles(x_packed_in, hints)
    for name, t in (("x_packed_in", x_packed_in), ("y_packed_out", y_packed_out), ("W0", W0), ("W1", W1), ("W2", W2),
                    ("T0", T0), ("T1", T1)):
        if t.dtype != torch.float32 or not t.is_contiguous():
            raise _lib.CtbError(_lib.BAD_ARG, "fft_kernel: %s must be a contiguous float32 tensor" % name)
    N, F0, F1, F2 = int(N), int(F0), int(F1), int(F2)
    if x_packed_in.numel() % (2 * N) or y_packed_out.numel() != x_packed_in.numel():
        raise _lib.CtbError(_lib.BAD_ARG, "fft_kernel: x and y must hold batch * 2N floats")
    want = {"W0": 2 * F0 * F0, "W1": 2 * F1 * F1, "W2": 2 * F2 * F2, "T0": 2 * F0 * F1 * F2, "T1": 2 * F1 * F2}
    for name, t in (("W0", W0), ("W1", W1), ("W2", W2), ("T0", T0), ("T1", T1)):
        if t.numel() != want[name]:
            raise _lib.CtbError(_lib.BAD_ARG, "fft_kernel: %s has %d elements, expected %d" % (name, t.numel(), want[name]))
    batch = x_packed_in.numel() // (2 * N)
    _lib.check(_lib.lib.ctb_fft(ctx, stream, ptr(x_packed_in), ptr(y_packed_out), ptr(W0), ptr(W1), ptr(W2), ptr(T0),
                                ptr(T1), N, F0, F1, F2, batch, int(BS), int(D)))
    return y_packed_out


class FftPlan:
    """The device-side tables of prepare() (examples/fft.jl:182-212) for one factorisation."""

    def __init__(self, factors, device, atom_packing_dim=None):
        self.factors = tuple(int(f) for f in factors)
        self.N = math.prod(self.factors)
        self.D = int(atom_packing_dim) if atom_packing_dim is not None else min(64, 2 * self.N)
        if (2 * self.N) % self.D:
            raise ValueError("2 * N must be divisible by atom_packing_dim")
        self.tables = tuple(torch.from_numpy(t).to(device) for t in make_twiddles(self.factors))

    def __call__(self, input, out=None, **hints):
        """FFT along the last torch dimension (the first Julia dimension) of a complex64 [batch, N] tensor."""
        if input.dtype != torch.complex64 or input.dim() != 2 or input.shape[1] != self.N or not input.is_contiguous():
            raise _lib.CtbError(_lib.BAD_ARG, "FftPlan: input must be a contiguous complex64 [batch, %d] tensor" % self.N)
        if out is None:
            out = torch.empty_like(input)
        x = torch.view_as_real(input).view(input.shape[0], 2 * self.N // self.D, self.D)
        y = torch.view_as_real(out).view(input.shape[0], 2 * self.N // self.D, self.D)
        F0, F1, F2 = self.factors
        fft_kernel(x, y, *self.tables, self.N, F0, F1, F2, 1, self.D, **hints)
        return out
