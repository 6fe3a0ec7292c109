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
                     mul_routed_weight, TILE_M, TILE_N, TILE_K):
    """fused_moe_kernel(...), examples/moe.jl:45-105.  A [tokens, K]; B [E, N, K]; C [total, N];
    topk_weights flat [total] (slot fastest), as invoke_fused_moe_kernel passes it (:193)."""
    ctx, stream = handles(A)
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


def silu_and_mul_kernel(A, B, C, TILE_N):
    """silu_and_mul_kernel(A, B, C, TILE_N), examples/moe.jl:110-128.  A, B may be row
    views (halves of the gate/up buffer, :210-211): torch [cols, n] with any row stride."""
    ctx, stream = handles(A)
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


# --------------------------------------------------------------------------- expert parallelism
def ep_plan(topk_ids, num_experts, world_size):
    """Dispatch plan of one rank for expert-parallel MoE.  `topk_ids` [topk, T_local] (1-based global expert ids).
    Experts are split in contiguous shards of num_experts/world_size per rank.  Returns
    (order, send_counts): `order` = 1-based flat slot ids (token*topk + slot + 1) sorted by expert, stable -- the
    order in which token rows are sent -- and `send_counts[r]` = slots that go to rank r.  Plain torch ops: runs
    on CPU tensors as well (used by the gloo tests)."""
    if num_experts % world_size:
        raise _lib.CtbError(_lib.BAD_ARG, "ep_plan: the number of experts must be a multiple of the world size")
    flat = topk_ids.t().reshape(-1).to(torch.int64)  # slot fastest, examples/moe.jl:146-148
    order = torch.argsort(flat, stable=True)
    dest = (flat[order] - 1) // (num_experts // world_size)
    send_counts = torch.bincount(dest, minlength=world_size)
    return (order + 1).to(torch.int32), send_counts


def cutile_moe_ep(hidden_states, w1_local, w2_local, topk_weights, topk_ids, num_experts, tile_m, tile_n, tile_k,
                  group=None):
    """Expert-parallel cutile_moe: this rank holds T_local tokens and the expert shard
    [rank*E/N, (rank+1)*E/N) (w1_local [E/N, 2I, H], w2_local [E/N, H, I]).  Token rows are packed in expert
    order, exchanged with one all-to-all (NCCL), run through the local experts with the single-GPU kernels
    (topk = 1, gate applied), sent back by the reverse all-to-all and summed over each token's slots.
    Returns [T_local, H] f16; bit-identical to cutile_moe on the gathered problem."""
    import torch.distributed as dist
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    ctx, stream = handles(hidden_states)
    T, H = hidden_states.shape
    topk = topk_ids.shape[0]
    El = num_experts // world
    total = T * topk
    order, send_counts = ep_plan(topk_ids, num_experts, world)
    recv_counts = torch.empty_like(send_counts)
    dist.all_to_all_single(recv_counts, send_counts, group=group)
    counts = torch.stack([send_counts, recv_counts]).cpu()  # one small D2H: NCCL needs the split sizes on the host
    send_l, recv_l = counts[0].tolist(), counts[1].tolist()
    R = int(sum(recv_l))
    dev = hidden_states.device
    # pack: token rows, local expert ids and gates in send order
    send_rows = torch.empty((total, H), dtype=torch.float16, device=dev)
    _lib.check(_lib.lib.ctb_moe_gather_rows(ctx, stream, ptr(send_rows), ptr(hidden_states), ptr(order), total, H,
                                            topk, T))
    o64 = order.to(torch.int64) - 1
    flat_e = topk_ids.t().reshape(-1)[o64].to(torch.int32)
    flat_w = topk_weights.t().reshape(-1)[o64].contiguous()
    recv_rows = torch.empty((max(R, 1), H), dtype=torch.float16, device=dev)
    recv_e = torch.empty(max(R, 1), dtype=torch.int32, device=dev)
    recv_w = torch.empty(max(R, 1), dtype=torch.float16, device=dev)
    dist.all_to_all_single(recv_rows[:R], send_rows, recv_l, send_l, group=group)
    dist.all_to_all_single(recv_e[:R], flat_e, recv_l, send_l, group=group)
    dist.all_to_all_single(recv_w[:R], flat_w, recv_l, send_l, group=group)
    # local experts: every received row is one token with topk = 1
    if R > 0:
        local_ids = (recv_e[:R] - rank * El).reshape(1, R).contiguous()
        y = cutile_moe(recv_rows[:R], w1_local, w2_local, recv_w[:R].reshape(1, R).contiguous(), local_ids,
                       tile_m, tile_n, tile_k)
    else:
        y = recv_rows[:0]
    back = torch.empty((total, H), dtype=torch.float16, device=dev)
    dist.all_to_all_single(back, y, send_l, recv_l, group=group)
    # unsort into flat slot order and add each token's slots
    slots = torch.empty((total, H), dtype=torch.float16, device=dev)
    _lib.check(_lib.lib.ctb_moe_scatter_rows(ctx, stream, ptr(slots), ptr(back), ptr(order), total, H, total))
    out = torch.empty((T, H), dtype=torch.float16, device=dev)
    _lib.check(_lib.lib.ctb_moe_combine(ctx, stream, ptr(slots), ptr(out), T, H, topk))
    return out


class EpPeerBuffers:
    """Receive and output buffers of the peer-memory expert-parallel path, allocated once per (T_local, H, topk) in
    symmetric memory (torch.distributed._symmetric_memory: the same allocation on every rank, each rank's copy mapped
    into every process), so that kernels on one GPU can store straight into another GPU's buffers over NVLink."""

    def __init__(self, T_local, H, topk, device, group=None):
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        if self.world > _lib.EP_MAX_RANKS:
            raise _lib.CtbError(_lib.UNSUPPORTED, f"at most {_lib.EP_MAX_RANKS} ranks")
        self.T, self.H, self.topk = T_local, H, topk
        self.cap = T_local * topk
        R = self.cap * self.world
        self.table = _lib.EpBuffers()
        self.table.world, self.table.rank = self.world, self.rank
        self._keep = []
        for field, shape, dtype in (("recv_rows", (R, H), torch.float16), ("recv_ids", (R,), torch.int32),
                                    ("recv_gates", (R,), torch.float16), ("slot_out", (self.cap, H), torch.float16),
                                    ("flags", (max(self.world, 4),), torch.int32)):
            t = symm.empty(*shape, dtype=dtype, device=device)
            hdl = symm.rendezvous(t, self.group)
            self._keep.append((t, hdl))
            arr = getattr(self.table, field)
            for q in range(self.world):
                arr[q] = int(hdl.buffer_ptrs[q])
            setattr(self, field, t)
        self.epoch = torch.zeros(1, dtype=torch.int32, device=device)
        self.table.epoch = self.epoch.data_ptr()
        self.flags.zero_()
        torch.cuda.synchronize(device)
        dist.barrier(group=self.group)  # every rank's flags are zero before anyone's first barrier kernel

    def barrier(self, ctx, stream):
        """Every rank's kernels issued so far have completed before any rank's later kernels start: one small kernel
        per rank that publishes an epoch in the peers' flag arrays and waits (bounded) for theirs."""
        import ctypes as C
        _lib.check(_lib.lib.ctb_moe_ep_barrier(ctx, stream, C.byref(self.table)))


def cutile_moe_ep_peer(bufs, hidden_states, w1_local, w2_local, topk_weights, topk_ids, num_experts, tile_m, tile_n,
                       tile_k):
    """Expert-parallel cutile_moe over peer memory.  This rank holds T_local tokens and the expert shard
    [rank*E/N, (rank+1)*E/N).  Token rows are stored straight into the owning rank's receive buffer by the dispatch
    kernel (no sort, no counts, no host synchronisation); after a barrier every rank runs align + gate/up + down on
    what it received, and the down projection's epilogue stores each weighted output row into the buffer of the
    rank that sent the slot; after a second barrier the slots of every token are summed locally.  Each row crosses
    NVLink once in each direction.  Returns [T_local, H] f16; bit-identical to cutile_moe on the gathered problem."""
    ctx, stream = handles(hidden_states)
    T, H = hidden_states.shape
    topk = topk_ids.shape[0]
    El, H2, I = w2_local.shape
    if (T, H, topk) != (bufs.T, bufs.H, bufs.topk) or H2 != H or w1_local.shape != (El, 2 * I, H):
        raise _lib.CtbError(_lib.BAD_ARG, "cutile_moe_ep_peer: shapes do not match the buffers")
    if El * bufs.world != num_experts:
        raise _lib.CtbError(_lib.BAD_ARG, "cutile_moe_ep_peer: the expert shard must hold E / world experts")
    if topk_ids.dtype != torch.int32 or topk_weights.dtype != torch.float16 or hidden_states.dtype != torch.float16:
        raise _lib.CtbError(_lib.BAD_ARG, "cutile_moe_ep_peer: ids must be Int32, gates and tokens Float16")
    for t in (hidden_states, w1_local, w2_local, topk_weights, topk_ids):
        if not t.is_contiguous():
            raise _lib.CtbError(_lib.BAD_ARG, "cutile_moe_ep_peer: arrays must be dense")
    import ctypes as C
    tab = C.byref(bufs.table)
    _lib.check(_lib.lib.ctb_moe_ep_dispatch(ctx, stream, tab, ptr(hidden_states), ptr(topk_ids), ptr(topk_weights), T,
                                            H, num_experts, topk))
    bufs.barrier(ctx, stream)   # every rank's rows have landed
    _lib.check(_lib.lib.ctb_moe_ep_experts(ctx, stream, tab, ptr(w1_local), ptr(w2_local), bufs.cap, H, I, El,
                                           int(tile_m), int(tile_n), int(tile_k)))
    bufs.barrier(ctx, stream)   # every rank's outputs have landed (and nobody reads its receive buffer any more)
    out = torch.empty((T, H), dtype=torch.float16, device=hidden_states.device)
    _lib.check(_lib.lib.ctb_moe_combine(ctx, stream, ptr(bufs.slot_out), ptr(out), T, H, topk))
    return out
