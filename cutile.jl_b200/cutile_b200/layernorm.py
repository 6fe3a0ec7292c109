"""LayerNorm forward/backward: the call surface of examples/layernorm.jl.

Memory order of the Julia arrays: X, Y, DX, DY (N, M) are torch [M, N];
W, B, FINAL_DW, FINAL_DB are [N]; Mean, Rstd are [M]; the partial buffers
DW, DB (N, GROUP_SIZE_M) are torch [GROUP_SIZE_M, N].
"""
from . import _lib
from ._util import handles, ptr, rows


def layer_norm_fwd(X, W, B, Y, Mean, Rstd, eps, TILE_N, **hints):
    """layer_norm_fwd(X, W, B, Y, Mean, Rstd, eps, TILE_N), examples/layernorm.jl:27-68."""
    ctx, stream = handles(X, hints)
    ldx, M, N = rows(X, "X")
    ldy, My, Ny = rows(Y, "Y")
    if (My, Ny) != (M, N) or W.numel() != N or B.numel() != N or Mean.numel() != M or Rstd.numel() != M:
        raise _lib.CtbError(_lib.BAD_ARG, "layer_norm_fwd: inconsistent shapes")
    _lib.check(_lib.lib.ctb_layernorm_fwd(ctx, stream, ptr(X), ptr(W), ptr(B), ptr(Y), ptr(Mean), ptr(Rstd), N, M,
                                          ldx, ldy, float(eps), int(TILE_N)))


def layer_norm_bwd_dx_partial_dwdb(DX, DY, DW, DB, X, W, Mean, Rstd, Locks, GROUP_SIZE_M, TILE_N, **hints):
    """layer_norm_bwd_dx_partial_dwdb(...), examples/layernorm.jl:118-171.
    `Locks` is accepted for signature compatibility and never touched; DW/DB
    need no zero-fill."""
    ctx, stream = handles(X, hints)
    ldx, M, N = rows(X, "X")
    lddy, _, _ = rows(DY, "DY")
    lddx, _, _ = rows(DX, "DX")
    if DW.shape != (GROUP_SIZE_M, N) or DB.shape != (GROUP_SIZE_M, N) or not DW.is_contiguous() or not DB.is_contiguous():
        raise _lib.CtbError(_lib.BAD_ARG, "layer_norm_bwd_dx_partial_dwdb: DW/DB must be contiguous (N, GROUP_SIZE_M)")
    if DY.shape != X.shape or DX.shape != X.shape:
        raise _lib.CtbError(_lib.BAD_ARG, "layer_norm_bwd_dx_partial_dwdb: DX/DY must have the shape of X")
    _lib.check(_lib.lib.ctb_layernorm_bwd_dx_partial_dwdb(
        ctx, stream, ptr(DX), ptr(DY), ptr(DW), ptr(DB), ptr(X), ptr(W), ptr(Mean), ptr(Rstd),
        ptr(Locks), N, M, ldx, lddy, lddx, int(GROUP_SIZE_M), int(TILE_N)))


def layer_norm_bwd_dwdb(DW, DB, FINAL_DW, FINAL_DB, TILE_M, TILE_N, **hints):
    """layer_norm_bwd_dwdb(DW, DB, FINAL_DW, FINAL_DB, TILE_M, TILE_N), examples/layernorm.jl:186-205."""
    ctx, stream = handles(DW, hints)
    G, N = DW.shape
    _lib.check(_lib.lib.ctb_layernorm_bwd_dwdb(ctx, stream, ptr(DW), ptr(DB), ptr(FINAL_DW), ptr(FINAL_DB), N, G,
                                               int(TILE_M), int(TILE_N)))


def layer_norm_bwd_static(DX, DY, X, W, Mean, Rstd, FINAL_DW, FINAL_DB):
    """Backward pass for callers that must not allocate device memory where it runs (inside another runtime's
    memory plan, in a loop that may not block in the allocator, while a stream is being captured).  Same result
    as layer_norm_bwd_dx_partial_dwdb + layer_norm_bwd_dwdb with GROUP_SIZE_M = 64, but the partial buffers
    live in a fixed array inside the library (N <= 8192) and no context is created.  No counterpart in the
    reference.  Calls share that array: keep them on one stream."""
    import ctypes as C
    import torch
    from ._util import ptr, rows
    if not X.is_cuda:
        raise _lib.CtbError(_lib.BAD_ARG, "expected CUDA tensors")
    ldx, M, N = rows(X, "X")
    lddy, _, _ = rows(DY, "DY")
    lddx, _, _ = rows(DX, "DX")
    if DY.shape != X.shape or DX.shape != X.shape:
        raise _lib.CtbError(_lib.BAD_ARG, "layer_norm_bwd_static: DX/DY must have the shape of X")
    with torch.cuda.device(X.device):
        stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
        _lib.check(_lib.lib.ctb_layernorm_bwd_static(stream, ptr(DX), ptr(DY), ptr(X), ptr(W), ptr(Mean), ptr(Rstd),
                                                     ptr(FINAL_DW), ptr(FINAL_DB), N, M, ldx, lddy, lddx))


def layer_norm_bwd_static_status(device=None):
    """Synchronises the current stream and reads-and-clears the status word of layer_norm_bwd_static on `device`
    (default: the current one).  Raises CtbError(TIMEOUT) when one of its kernels gave up a bounded wait since the
    last check; allocates nothing."""
    import ctypes as C
    import torch
    with torch.cuda.device(device if device is not None else torch.cuda.current_device()):
        _lib.check(_lib.lib.ctb_layernorm_bwd_static_status(C.c_void_p(torch.cuda.current_stream().cuda_stream)))
