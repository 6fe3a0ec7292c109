"""Flash multi-head attention forward: the call surface of examples/fmha.jl.

Memory order of the Julia arrays: Q, Out (D, SeqLen_Q, Heads, Batch) are torch
[Batch, Heads, SeqLen_Q, D]; K, V (D, SeqLen_KV, KV_Heads, Batch) are torch
[Batch, KV_Heads, SeqLen_KV, D] (the layout of the reference's Python twin).
"""
import math

import torch

from . import _lib
from ._util import handles, ptr, dtype_code


def fmha_kernel(Q, K, V, Out, qk_scale, input_pos, TILE_D, H, TILE_M, TILE_N, QUERY_GROUP_SIZE, CAUSAL, EVEN_K, **hints):
    """fmha_kernel(...), examples/fmha.jl:20-139 (the launch inside cutile_fmha)."""
    ctx, stream = handles(Q, hints)
    for t, name in ((Q, "Q"), (K, "K"), (V, "V"), (Out, "Out")):
        if t.dim() != 4 or not t.is_contiguous():
            raise _lib.CtbError(_lib.BAD_ARG, f"fmha: {name} must be a dense 4-D tensor")
    B, Hq, Sq, D = Q.shape
    Bk, KVH, Skv, Dk = K.shape
    if Hq != H or TILE_D != D or Bk != B or Dk != D or V.shape[:3] != K.shape[:3] or Out.shape[:3] != Q.shape[:3] \
            or Out.shape[3] != V.shape[3]:
        raise _lib.CtbError(_lib.BAD_ARG, "fmha: inconsistent shapes")
    if bool(EVEN_K) != (Skv % TILE_N == 0):
        raise _lib.CtbError(_lib.BAD_ARG, "fmha: EVEN_K does not match SeqLen_KV % TILE_N")
    _lib.check(_lib.lib.ctb_fmha_fwd(ctx, stream, ptr(Q), ptr(K), ptr(V), ptr(Out), D, V.shape[3], Sq, Skv, Hq, KVH, B,
                                     float(qk_scale), int(input_pos), int(TILE_M), int(TILE_N),
                                     int(QUERY_GROUP_SIZE), int(bool(CAUSAL)), dtype_code(Q)))
    return Out


def cutile_fmha(Q, K, V, *, qk_scale=None, input_pos=0, tile_m=128, tile_n=128, query_group_size=1, causal=False,
                **hints):
    """cutile_fmha(Q, K, V; qk_scale, input_pos, tile_m, tile_n, query_group_size, causal),
    examples/fmha.jl:146-168: allocates and returns Out."""
    B, H, Sq, D = Q.shape
    Dv, Skv = V.shape[3], V.shape[2]
    if qk_scale is None:
        qk_scale = 1.0 / math.sqrt(D)
    Out = torch.empty((B, H, Sq, Dv), dtype=Q.dtype, device=Q.device)
    return fmha_kernel(Q, K, V, Out, qk_scale, input_pos, D, H, tile_m, tile_n, query_group_size, causal,
                       Skv % tile_n == 0, **hints)
