"""Worker of the expert-parallel MoE tests (launched with torch.distributed.run, one rank per device).

mode "plan" (CPU, gloo): checks the dispatch plan and the count/id exchange against a numpy ground truth.
mode "gpu" (NCCL): checks cutile_moe_ep bit for bit against the single-GPU cutile_moe on the gathered problem."""
import json
import os
import sys


def _emit(obj):
    """One write per line: the ranks share a pipe, and print() writes text and newline separately."""
    os.write(1, (json.dumps(obj) + "\n").encode())


ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "cutile.jl_b200")):
    if p not in sys.path:
        sys.path.insert(0, p)

import numpy as np
import torch
import torch.distributed as dist


def routing(T, E, topk, seed):
    g = np.random.default_rng(seed)
    ids = np.stack([g.permutation(E)[:topk] + 1 for _ in range(T)], axis=1).astype(np.int32)  # [topk, T]
    raw = np.exp(g.random((topk, T), dtype=np.float32))
    return ids, (raw / raw.sum(axis=0, keepdims=True)).astype(np.float16)


def main():
    mode = sys.argv[1]
    dist.init_process_group("gloo" if mode == "plan" else "nccl")
    rank, world = dist.get_rank(), dist.get_world_size()
    import cutile_b200 as ctb
    T, E, topk = 64, 8, 2
    Tl = T // world
    ids, w = routing(T, E, topk, seed=5)
    my = slice(rank * Tl, (rank + 1) * Tl)
    if mode == "plan":
        order, send_counts = ctb.moe.ep_plan(torch.from_numpy(ids[:, my].copy()), E, world)
        flat = ids[:, my].T.reshape(-1)
        want_order = np.argsort(flat, kind="stable") + 1
        assert np.array_equal(order.numpy(), want_order)
        dest = (flat[want_order - 1] - 1) // (E // world)
        assert np.array_equal(send_counts.numpy(), np.bincount(dest, minlength=world))
        recv_counts = torch.empty_like(send_counts)
        dist.all_to_all_single(recv_counts, send_counts)
        sent_e = torch.from_numpy(flat[want_order - 1].astype(np.int32))
        got_e = torch.empty(int(recv_counts.sum()), dtype=torch.int32)
        dist.all_to_all_single(got_e, sent_e, recv_counts.tolist(), send_counts.tolist())
        lo, hi = rank * (E // world) + 1, (rank + 1) * (E // world)
        assert ((got_e >= lo) & (got_e <= hi)).all()  # only this rank's experts arrive
        allflat = ids.T.reshape(-1)
        assert got_e.numel() == int(((allflat >= lo) & (allflat <= hi)).sum())  # and all of them
        _emit({"rank": rank, "ok": True, "received": got_e.numel()})
    else:
        from oracle import inputs
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
        H, I = 256, 512
        d = inputs.moe(tokens=T, hidden=H, experts=E, inter=I, topk=topk, seed=8)
        dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
        El = E // world
        out = ctb.moe.cutile_moe_ep(dev(d["X"][my]), dev(d["w1"][rank * El:(rank + 1) * El]),
                                    dev(d["w2"][rank * El:(rank + 1) * El]), dev(w[:, my]), dev(ids[:, my]), E,
                                    128, 128, 64)
        full = ctb.moe.cutile_moe(dev(d["X"]), dev(d["w1"]), dev(d["w2"]), dev(w), dev(ids), 128, 128, 64)
        torch.cuda.synchronize()
        ctb.check_device_status(torch.cuda.current_device())
        same = bool(torch.equal(out, full[my]))
        # the same problem through the peer-memory path (stores into the other rank's buffers, no all-to-all);
        # twice, to cover the reuse of the buffers from one step to the next
        bufs = ctb.moe.EpPeerBuffers(Tl, H, topk, torch.device("cuda", torch.cuda.current_device()))
        args = (dev(d["X"][my]), dev(d["w1"][rank * El:(rank + 1) * El]), dev(d["w2"][rank * El:(rank + 1) * El]),
                dev(w[:, my]), dev(ids[:, my]), E, 128, 128, 64)
        peer1 = ctb.moe.cutile_moe_ep_peer(bufs, *args)
        peer2 = ctb.moe.cutile_moe_ep_peer(bufs, *args)
        torch.cuda.synchronize()
        ctb.check_device_status(torch.cuda.current_device())
        same_peer = bool(torch.equal(peer1, full[my])) and bool(torch.equal(peer2, full[my]))
        _emit({"rank": rank, "ok": same and same_peer, "nccl": same, "peer": same_peer})
        assert same and same_peer
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
