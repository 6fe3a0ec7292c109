"""Mixture-of-experts FFN: the call surface of examples/moe.jl.

Memory order of the Julia arrays: hidden_states (H, T) is torch [T, H];
w1 (H, 2I, E) is torch [E, 2I, H] (gate rows then up rows); w2 (I, H, E) is
torch [E, H, I]; topk_weights / topk_ids (T, topk) are torch [topk, T];
the result (H, T) is torch [T, H].  Expert ids and slot ids are 1-based.
"""
import ctypes as C

import torch

from . import _lib
from ._util import handles, ptr


def _ids_bits(t):
    if t.dtype == torch.int32:
        return 32
    if t.dtype == torch.int64:
        return 64
    raise _lib.CtbError(_lib.BAD_ARG, "expert ids must be int32 or int64")


def moe_router(hidden_states, W_r, topk, return_logits=False):
    """Router of the benchmark configuration: returns (topk_weights [topk, T] f16, topk_ids [topk, T] int32)."""
    ctx, stream = handles(hidden_states)
    T, H = hidden_states.shape
    E = W_r.shape[0]
    if W_r.shape[1] != H or not hidden_states.is_contiguous() or not W_r.is_contiguous():
        raise _lib.CtbError(_lib.BAD_ARG, "moe_router: W_r must be (H, E) and both arrays dense")
    ids = torch.empty((topk, T), dtype=torch.int32, device=hidden_states.device)
    w = torch.empty((topk, T), dtype=torch.float16, device=hidden_states.device)
    logits = torch.empty((T, E), dtype=torch.float32, device=hidden_states.device) if return_logits else None
    _lib.check(_lib.lib.ctb_moe_router(ctx, stream, ptr(hidden_states), ptr(W_r), ptr(ids), ptr(w), ptr(logits), T, H,
                                       E, int(topk)))
    return (w, ids, logits) if return_logits else (w, ids)


def moe_align_tile_size(topk_ids, tile_m, num_experts):
    """moe_align_tile_size(topk_ids, tile_m, num_experts), examples/moe.jl:142-183.
    Returns (sorted_token_ids, sorted_expert_ids) as int32 device tensors of the exact
    lengths blocks*tile_m and blocks (reading the block count synchronises, as the
    reference's host-side version does)."""
    ctx, stream = handles(topk_ids)
    topk, T = topk_ids.shape
    if not topk_ids.is_contiguous():
        raise _lib.CtbError(_lib.BAD_ARG, "moe_align_tile_size: topk_ids must be dense")
    cap = _lib.lib.ctb_moe_max_blocks(T, topk, num_experts, int(tile_m))
    tok = torch.empty(max(cap, 1) * tile_m, dtype=torch.int32, device=topk_ids.device)
    exp = torch.empty(max(cap, 1), dtype=torch.int32, device=topk_ids.device)
    nb = torch.zeros(1, dtype=torch.int32, device=topk_ids.device)
    _lib.check(_lib.lib.ctb_moe_align(ctx, stream, ptr(topk_ids), _ids_bits(topk_ids), T, topk, num_experts,
                                      int(tile_m), ptr(tok), ptr(exp), ptr(nb), cap))
    n = int(nb.item())
    _lib.check_device_status(topk_ids.device.index or 0, stream.value or 0)
    return tok[: n * tile_m], exp[:n]


def fused_moe_kernel(A, B, C, topk_weights, sorted_token_ids, sorted_expert_ids, num_token_replicas,
                     mul_routed_weight, TILE_M, TILE_N, TILE_K, **hints):
    """fused_moe_kernel(...), examples/moe.jl:45-105.  A [tokens, K]; B [E, N, K]; C [total, N];
    topk_weights flat [total] (slot fastest), as invoke_fused_moe_kernel passes it (:193)."""
    ctx, stream = handles(A, hints)
    a_cols, K = A.shape
    E, N, Kb = B.shape
    c_cols, Nc = C.shape
    if Kb != K or Nc != N or not (A.is_contiguous() and B.is_contiguous() and C.is_contiguous()):
        raise _lib.CtbError(_lib.BAD_ARG, "fused_moe_kernel: inconsistent or non-dense arrays")
    if sorted_token_ids.dtype != torch.int32 or sorted_expert_ids.dtype != torch.int32:
        raise _lib.CtbError(_lib.BAD_ARG, "fused_moe_kernel: sorted ids must be Int32")
    if sorted_expert_ids.numel() * TILE_M != sorted_token_ids.numel():
        raise _lib.CtbError(_lib.BAD_ARG, "fused_moe_kernel: one expert id per TILE_M slots expected")
    _lib.check(_lib.lib.ctb_moe_fused_gemm(ctx, stream, ptr(A), ptr(B), ptr(C), ptr(topk_weights),
                                           ptr(sorted_token_ids), ptr(sorted_expert_ids), sorted_token_ids.numel(),
                                           K, N, E, a_cols, c_cols, int(num_token_replicas),
                                           int(bool(mul_routed_weight)), int(TILE_M), int(TILE_N), int(TILE_K)))
    return C


def silu_and_mul_kernel(A, B, C, TILE_N, **hints):
    """silu_and_mul_kernel(A, B, C, TILE_N), examples/moe.jl:110-128.  A, B may be row
    views (halves of the gate/up buffer, :210-211): torch [cols, n] with any row stride."""
    ctx, stream = handles(A, hints)
    cols, n = C.shape
    for t in (A, B, C):
        if t.shape != (cols, n) or (n > 1 and t.stride(1) != 1):
            raise _lib.CtbError(_lib.BAD_ARG, "silu_and_mul_kernel: shapes must match and rows be contiguous")
    _lib.check(_lib.lib.ctb_moe_silu_and_mul(ctx, stream, ptr(A), ptr(B), ptr(C), n, cols, A.stride(0), B.stride(0),
                                             C.stride(0), int(TILE_N)))
    return C


def cutile_moe(hidden_states, w1, w2, topk_weights, topk_ids, tile_m, tile_n, tile_k):
    """cutile_moe(hidden_states, w1, w2, topk_weights, topk_ids, tile_m, tile_n, tile_k),
    examples/moe.jl:218-257: returns the (H, T) result as torch [T, H] f16."""
    ctx, stream = handles(hidden_states)
    T, H = hidden_states.shape
    E, H2, I = w2.shape
    topk = topk_ids.shape[0]
    if w1.shape != (E, 2 * I, H) or H2 != H or topk_ids.shape != (topk, T) or topk_weights.shape != (topk, T):
        raise _lib.CtbError(_lib.BAD_ARG, "cutile_moe: inconsistent shapes")
    for t in (hidden_states, w1, w2, topk_weights, topk_ids):
        if not t.is_contiguous():
            raise _lib.CtbError(_lib.BAD_ARG, "cutile_moe: arrays must be dense")
    if topk_weights.dtype != torch.float16 or hidden_states.dtype != torch.float16:
        raise _lib.CtbError(_lib.BAD_ARG, "cutile_moe: only Float16 is implemented")
    out = torch.empty((T, H), dtype=torch.float16, device=hidden_states.device)
    _lib.check(_lib.lib.ctb_moe_ffn(ctx, stream, ptr(hidden_states), ptr(w1), ptr(w2), ptr(topk_weights),
                                    ptr(topk_ids), _ids_bits(topk_ids), ptr(out), T, H, I, E, topk, int(tile_m),
                                    int(tile_n), int(tile_k)))
    return out


# Expert-parallel variants (several GPUs): cutile_b200.multi
