"""Worker of the process-per-GPU expert-parallel MoE test (launched with torch.distributed.run, one rank per
device): cutile_moe_ep through the C ABI, in both exchange modes, against the single-GPU cutile_moe on the gathered
problem, bit for bit.  torch.distributed only carries the set-up byte strings (NCCL id, IPC handles)."""
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


def main():
    dist.init_process_group("nccl")
    rank, world = dist.get_rank(), dist.get_world_size()
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    import cutile_b200 as ctb
    from oracle import inputs
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    results = []
    # a small case (one slot block per expert) and the benchmark's 4096-token configuration
    for T, H, E, I, topk, seed in ((64 * world, 256, 8 * world, 512, 2, 8), (4096, 1024, 32, 2048, 2, 4)):
        if E % world or T % world:
            continue
        d = inputs.moe(tokens=T, hidden=H, experts=E, inter=I, topk=topk, seed=seed)
        Tl, El = T // world, E // world
        my = slice(rank * Tl, (rank + 1) * Tl)
        X, Wr, w1, w2 = dev(d["X"]), dev(d["Wr"]), dev(d["w1"]), dev(d["w2"])
        gates, ids = ctb.moe.moe_router(X, Wr, topk)
        full = ctb.moe.cutile_moe(X, w1, w2, gates, ids, 128, 128, 64)
        ep = ctb.multi.EpRank(Tl, H, topk, torch.device("cuda", local))
        args = (X[my].contiguous(), w1[rank * El:(rank + 1) * El].contiguous(), w2[rank * El:(rank + 1) * El].contiguous(),
                gates[:, my].contiguous(), ids[:, my].contiguous(), E, 128, 128, 64)
        ok = {}
        for mode in ("peer", "nccl"):
            a = ep.cutile_moe_ep(*args, a2a_mode=mode)
            b = ep.cutile_moe_ep(*args, a2a_mode=mode)  # twice: the buffers are reused from one step to the next
            torch.cuda.synchronize()
            ctb.check_device_status(local)
            ok[mode] = bool(torch.equal(a, full[my])) and bool(torch.equal(b, full[my]))
        ep.close()
        results.append(dict(tokens=T, **ok))
    good = all(r["peer"] and r["nccl"] for r in results)
    _emit({"rank": rank, "ok": good, "cases": results})
    dist.barrier()
    dist.destroy_process_group()
    assert good


if __name__ == "__main__":
    main()
