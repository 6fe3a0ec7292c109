"""Several GPUs: the multi-device half of the C ABI (csrc/multi.cu) behind the examples' call surface.

The reference is single-GPU; the partitioning is the benchmark configuration's: batched GEMM and FMHA split by batch
with no communication, MoE expert-parallel (experts [r*E/N, (r+1)*E/N) on rank r, tokens sharded by rank) with the
token exchange either as NCCL send/receive pairs (`a2a_mode="nccl"`) or as stores into peer memory
(`a2a_mode="peer"`).  All of it happens inside libcutile_b200.so, which owns the NCCL communicators; the host
language only carries two small byte strings between processes at set-up (the NCCL unique id and one CUDA IPC
handle per rank).

Two ways to drive it:
  * Group: one process, several devices (what a single-threaded host like the reference's examples would use);
  * EpRank: one process per GPU (torchrun); torch.distributed is used at set-up only, to carry the byte strings.
"""
import ctypes as C

import torch

from . import _lib
from ._util import ptr, dtype_code

_MODES = {"nccl": _lib.A2A_NCCL, "peer": _lib.A2A_PEER}


def _mode(a2a_mode):
    if a2a_mode not in _MODES:
        raise _lib.CtbError(_lib.BAD_ARG, "a2a_mode must be 'nccl' or 'peer'")
    return _MODES[a2a_mode]


def _stream(device):
    return C.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def _ptr_array(tensors):
    arr = (C.c_void_p * len(tensors))()
    for i, t in enumerate(tensors):
        arr[i] = t.data_ptr() if isinstance(t, torch.Tensor) else (t.value if isinstance(t, C.c_void_p) else t)
    return arr


def workspace_bytes(op, *dims):
    """ctb_workspace_bytes: scratch a context needs for `op` ("moe_ffn": T, H, I, E, topk, tile_m;
    "moe_ep": T_local, H, I, E_local, topk, tile_m, world)."""
    code = {"moe_ffn": _lib.OP_MOE_FFN, "moe_ep": _lib.OP_MOE_EP}.get(op, 0)
    arr = (C.c_int64 * len(dims))(*[int(d) for d in dims])
    return int(_lib.lib.ctb_workspace_bytes(code, arr, len(dims)))


def reserve_workspace(device, nbytes):
    """Sizes the scratch of this process's context on `device` up front (before a CUDA graph capture)."""
    _lib.check(_lib.lib.ctb_reserve_workspace(_lib.context(device), _stream(device), int(nbytes)))


def _check_moe_shapes(who, hidden, w1, w2, w, ids, E, world):
    T, H = hidden.shape
    El, H2, I = w2.shape
    topk = ids.shape[0]
    if w1.shape != (El, 2 * I, H) or H2 != H or ids.shape != (topk, T) or w.shape != (topk, T):
        raise _lib.CtbError(_lib.BAD_ARG, f"{who}: inconsistent shapes")
    if El * world != E:
        raise _lib.CtbError(_lib.BAD_ARG, f"{who}: the expert shard must hold E / world experts")
    if ids.dtype != torch.int32 or w.dtype != torch.float16 or hidden.dtype != torch.float16:
        raise _lib.CtbError(_lib.BAD_ARG, f"{who}: ids must be Int32, gates and tokens Float16")
    for t in (hidden, w1, w2, w, ids):
        if not t.is_contiguous():
            raise _lib.CtbError(_lib.BAD_ARG, f"{who}: arrays must be dense")
    return T, H, I, topk


class Group:
    """ctb_create_multi: per-device contexts of this process + peer access + one NCCL communicator per device."""

    def __init__(self, devices):
        self.devices = [int(d) for d in devices]
        arr = (C.c_int * len(self.devices))(*self.devices)
        h = C.c_void_p()
        _lib.check(_lib.lib.ctb_create_multi(C.byref(h), arr, len(self.devices)))
        self.handle = h
        self._eps = {}

    def __len__(self):
        return len(self.devices)

    def close(self):
        for eps in self._eps.values():
            for e in eps:
                _lib.lib.ctb_ep_destroy(e)
        self._eps = {}
        if self.handle:
            _lib.lib.ctb_destroy_multi(self.handle)
            self.handle = None

    def ctx(self, i):
        return C.c_void_p(_lib.lib.ctb_group_ctx(self.handle, i))

    def check_device_status(self):
        for i, d in enumerate(self.devices):
            with torch.cuda.device(d):
                _lib.check(_lib.lib.ctb_check_device_status(self.ctx(i), _stream(d)))

    def _streams(self):
        return _ptr_array([_stream(d) for d in self.devices])

    def batch_matmul_sharded(self, A, B, Cs, tm=128, tn=128, tk=64):
        """batch_matmul_kernel over the group: A[i] [b_i, K, M], B[i] [b_i, N, K], Cs[i] [b_i, N, M] on device i."""
        n = len(self)
        if not (len(A) == len(B) == len(Cs) == n):
            raise _lib.CtbError(_lib.BAD_ARG, "batch_matmul_sharded: one shard per device expected")
        _, K, M = A[0].shape
        N = B[0].shape[1]
        for a, b, c in zip(A, B, Cs):
            if a.shape[1:] != (K, M) or b.shape[1:] != (N, K) or c.shape[1:] != (N, M) or not (
                    a.is_contiguous() and b.is_contiguous() and c.is_contiguous()):
                raise _lib.CtbError(_lib.BAD_ARG, "batch_matmul_sharded: inconsistent or non-dense shards")
        per = (C.c_int64 * n)(*[a.shape[0] for a in A])
        _lib.check(_lib.lib.ctb_gemm_batched_sharded(self.handle, self._streams(), _ptr_array(A), _ptr_array(B),
                                                     _ptr_array(Cs), M, N, K, per, M, K, M, M * K, K * N, M * N,
                                                     dtype_code(A[0]), tm, tn, tk))
        return Cs

    def fmha_sharded(self, Q, K, V, Out, *, qk_scale, input_pos=0, tile_m=128, tile_n=128, query_group_size=1,
                     causal=False):
        """cutile_fmha over the group: Q[i], Out[i] [b_i, H, Sq, D]; K[i], V[i] [b_i, KVH, Skv, D] on device i."""
        n = len(self)
        _, H, Sq, D = Q[0].shape
        KVH, Skv = K[0].shape[1], K[0].shape[2]
        per = (C.c_int64 * n)(*[q.shape[0] for q in Q])
        _lib.check(_lib.lib.ctb_fmha_fwd_sharded(self.handle, self._streams(), _ptr_array(Q), _ptr_array(K),
                                                 _ptr_array(V), _ptr_array(Out), D, V[0].shape[3], Sq, Skv, H, KVH, per,
                                                 float(qk_scale), int(input_pos), tile_m, tile_n, query_group_size,
                                                 int(bool(causal)), dtype_code(Q[0])))
        return Out

    def ep_states(self, T_local, H, topk):
        """The ranks' exchange buffers for this shape (created and connected once)."""
        key = (T_local, H, topk)
        if key not in self._eps:
            eps = []
            for i in range(len(self)):
                e = C.c_void_p()
                _lib.check(_lib.lib.ctb_ep_create(self.ctx(i), len(self), i, T_local, H, topk, C.byref(e)))
                eps.append(e)
            _lib.check(_lib.lib.ctb_ep_connect_local(_ptr_array(eps), len(eps)))
            self._eps[key] = eps
        return self._eps[key]

    def cutile_moe_ep(self, hidden, w1, w2, topk_weights, topk_ids, num_experts, tile_m, tile_n, tile_k,
                      a2a_mode="peer", out=None):
        """Expert-parallel cutile_moe, all ranks of the group from this thread.  Every argument is a list with one
        tensor per device: hidden[i] [T_local, H], w1[i] [E/N, 2I, H], w2[i] [E/N, H, I], topk_weights[i] / topk_ids[i]
        [topk, T_local] (global 1-based expert ids).  Returns the list of [T_local, H] results."""
        n = len(self)
        T, H, I, topk = _check_moe_shapes("cutile_moe_ep", hidden[0], w1[0], w2[0], topk_weights[0], topk_ids[0],
                                          num_experts, n)
        if out is None:
            out = [torch.empty((T, H), dtype=torch.float16, device=h.device) for h in hidden]
        eps = self.ep_states(T, H, topk)
        _lib.check(_lib.lib.ctb_moe_ffn_ep_group(self.handle, _ptr_array(eps), self._streams(), _ptr_array(hidden),
                                                 _ptr_array(w1), _ptr_array(w2), _ptr_array(topk_weights),
                                                 _ptr_array(topk_ids), _ptr_array(out), T, H, I, num_experts, topk,
                                                 int(tile_m), int(tile_n), int(tile_k), _mode(a2a_mode)))
        return out


class EpRank:
    """One rank of a process-per-GPU job: exchange buffers (ctb_ep) mapped into every rank through CUDA IPC handles
    and, for the NCCL mode, a communicator attached to this process's context.  torch.distributed carries the NCCL
    unique id and the IPC handles at construction and is not used afterwards."""

    def __init__(self, T_local, H, topk, device, group=None, with_nccl=True):
        import torch.distributed as dist
        self.group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        self.device = torch.device(device)
        self.T, self.H, self.topk = T_local, H, topk
        dev = self.device.index
        self.ctx = _lib.context(dev)
        with torch.cuda.device(dev):
            if with_nccl and self.world > 1:
                world_c = C.c_int()
                _lib.check(_lib.lib.ctb_comm_info(self.ctx, None, C.byref(world_c), None))
                if world_c.value == 1:  # no communicator on the context yet
                    uid = C.create_string_buffer(_lib.UNIQUE_ID_BYTES)
                    if self.rank == 0:
                        _lib.check(_lib.lib.ctb_comm_unique_id(uid))
                    box = [bytes(uid.raw)]
                    dist.broadcast_object_list(box, src=dist.get_global_rank(self.group, 0), group=self.group)
                    _lib.check(_lib.lib.ctb_comm_init_rank(self.ctx, C.create_string_buffer(box[0], len(box[0])),
                                                           self.rank, self.world))
            h = C.c_void_p()
            _lib.check(_lib.lib.ctb_ep_create(self.ctx, self.world, self.rank, T_local, H, topk, C.byref(h)))
            self.handle = h
            mine = C.create_string_buffer(_lib.EP_HANDLE_BYTES)
            _lib.check(_lib.lib.ctb_ep_export(h, mine))
            handles = [None] * self.world
            dist.all_gather_object(handles, bytes(mine.raw), group=self.group)
            for q, raw in enumerate(handles):
                if q != self.rank:
                    _lib.check(_lib.lib.ctb_ep_import(h, q, C.create_string_buffer(raw, len(raw))))
            torch.cuda.synchronize(dev)
        dist.barrier(group=self.group)  # every rank's flags are zero and mapped before anyone's first step

    def close(self):
        if self.handle:
            _lib.lib.ctb_ep_destroy(self.handle)
            self.handle = None

    def cutile_moe_ep(self, hidden, w1_local, w2_local, topk_weights, topk_ids, num_experts, tile_m, tile_n, tile_k,
                      a2a_mode="peer", out=None):
        """This rank's call of the expert-parallel cutile_moe (every rank must make it).  Returns [T_local, H] f16,
        bit-identical to cutile_moe on the gathered problem."""
        T, H, I, topk = _check_moe_shapes("cutile_moe_ep", hidden, w1_local, w2_local, topk_weights, topk_ids,
                                          num_experts, self.world)
        if (T, H, topk) != (self.T, self.H, self.topk):
            raise _lib.CtbError(_lib.BAD_ARG, "cutile_moe_ep: shapes do not match the buffers")
        if out is None:
            out = torch.empty((T, H), dtype=torch.float16, device=hidden.device)
        _lib.check(_lib.lib.ctb_moe_ffn_ep(self.handle, _stream(self.device.index), ptr(hidden), ptr(w1_local),
                                           ptr(w2_local), ptr(topk_weights), ptr(topk_ids), ptr(out), T, H, I,
                                           num_experts, topk, int(tile_m), int(tile_n), int(tile_k), _mode(a2a_mode)))
        return out
