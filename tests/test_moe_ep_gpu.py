"""Several GPUs through the C ABI: expert-parallel MoE (NCCL send/receive and peer-memory stores) bit-identical to
the single-GPU result at 2, 4 and 8 ranks, as one process per GPU and as one process driving all devices; batched
GEMM and FMHA sharded by batch equal to the single-device call.  Skipped on a box with fewer GPUs."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

from oracle import inputs, ref

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _need(n):
    import torch
    if torch.cuda.device_count() < n:
        pytest.skip(f"needs {n} GPUs")


@pytest.mark.parametrize("world", [2, 4, 8])
def test_moe_ep_one_process_per_gpu(world):
    _need(world)
    # plain peer stores and NCCL without NVLS: no rank's memory is bound to an NVLink multicast object
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(world), "--master-addr",
           "127.0.0.1", "--master-port", str(29570 + world), os.path.join(ROOT, "tests", "ep_worker.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=900, env=env, cwd=ROOT)
    assert r.returncode == 0, r.stdout[-1500:] + r.stderr[-2500:]
    rows = [json.loads(l) for l in r.stdout.splitlines() if l.startswith("{")]
    assert sorted(x["rank"] for x in rows) == list(range(world)) and all(x["ok"] for x in rows), rows
    assert all(len(x["cases"]) == 2 for x in rows)  # the 4096-token case ran on every rank


@pytest.fixture(scope="module")
def group2(cuda):
    _need(2)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    g = cuda.multi.Group([0, 1])
    yield g
    g.check_device_status()
    g.close()


@pytest.mark.parametrize("mode", ["peer", "nccl"])
def test_moe_ep_single_process_group(cuda, group2, mode):
    """One host thread drives both devices through ctb_moe_ffn_ep_group: no torch.distributed anywhere."""
    import torch
    T, H, E, I, topk = 512, 512, 16, 1024, 2
    d = inputs.moe(tokens=T, hidden=H, experts=E, inter=I, topk=topk, seed=12)
    to = lambda a, i: torch.from_numpy(np.ascontiguousarray(a)).to(f"cuda:{i}")
    with torch.cuda.device(0):
        X, Wr, w1, w2 = (to(d[k], 0) for k in ("X", "Wr", "w1", "w2"))
        gates, ids = cuda.moe.moe_router(X, Wr, topk)
        full = cuda.moe.cutile_moe(X, w1, w2, gates, ids, 128, 128, 64)
        torch.cuda.synchronize()
    Tl, El = T // 2, E // 2
    sh = lambda t, i, lo, hi, dim=0: t.narrow(dim, lo, hi - lo).contiguous().to(f"cuda:{i}")
    hid = [sh(X, i, i * Tl, (i + 1) * Tl) for i in range(2)]
    w1s = [sh(w1, i, i * El, (i + 1) * El) for i in range(2)]
    w2s = [sh(w2, i, i * El, (i + 1) * El) for i in range(2)]
    gs = [sh(gates, i, i * Tl, (i + 1) * Tl, 1) for i in range(2)]
    idl = [sh(ids, i, i * Tl, (i + 1) * Tl, 1) for i in range(2)]
    for _ in range(2):  # twice: the buffers are reused
        outs = group2.cutile_moe_ep(hid, w1s, w2s, gs, idl, E, 128, 128, 64, a2a_mode=mode)
        for i in range(2):
            torch.cuda.synchronize(i)
        for i in range(2):
            assert torch.equal(outs[i].cpu(), full[i * Tl:(i + 1) * Tl].cpu())
    want = ref.moe_ffn(d["X"][:64], d["w1"], d["w2"], gates.cpu().numpy()[:, :64], ids.cpu().numpy()[:, :64])
    assert ref.rel_fro(outs[0][:64].cpu().numpy(), want) <= 2e-3


def test_sharded_fmha_and_batched_gemm(cuda, group2):
    import torch
    d = inputs.fmha(4, 4, 256, 256, 64, seed=9)
    with torch.cuda.device(0):
        Q, K, V = (torch.from_numpy(d[k]).cuda() for k in ("Q", "K", "V"))
        whole = cuda.fmha.cutile_fmha(Q, K, V, causal=True)
        torch.cuda.synchronize()
    parts = [[t[2 * i:2 * i + 2].contiguous().to(f"cuda:{i}") for i in range(2)] for t in (Q, K, V)]
    outs = [torch.empty_like(q) for q in parts[0]]
    group2.fmha_sharded(parts[0], parts[1], parts[2], outs, qk_scale=0.125, causal=True)
    for i in range(2):
        torch.cuda.synchronize(i)
        assert torch.equal(outs[i].cpu(), whole[2 * i:2 * i + 2].cpu())
    assert ref.rel_fro(outs[1].cpu().numpy(), ref.fmha(d["Q"][2:], d["K"][2:], d["V"][2:], causal=True)) <= 2e-3
    g = inputs.batched_gemm(256, 512, 128, 4, seed=2)
    A = [torch.from_numpy(g["A"][2 * i:2 * i + 2]).to(f"cuda:{i}") for i in range(2)]
    B = [torch.from_numpy(g["B"][2 * i:2 * i + 2]).to(f"cuda:{i}") for i in range(2)]
    Cs = [torch.empty(2, 128, 256, device=f"cuda:{i}") for i in range(2)]
    group2.batch_matmul_sharded(A, B, Cs)
    for i in range(2):
        torch.cuda.synchronize(i)
        assert ref.rel_fro(Cs[i].cpu().numpy(), ref.batched_gemm(g["A"][2 * i:2 * i + 2], g["B"][2 * i:2 * i + 2])) <= 5e-3


def test_group_rejections(cuda, group2):
    import ctypes as C
    import torch
    lib = cuda._lib
    x = torch.zeros(8, 64, device="cuda:0", dtype=torch.float16)
    with pytest.raises(cuda.CtbError) as e:  # one shard missing
        group2.batch_matmul_sharded([x.float().view(1, 8, 64)], [x.float().view(1, 64, 8)], [x.float().view(1, 8, 64)])
    assert e.value.status == lib.BAD_ARG
    eps = group2.ep_states(64, 128, 2)
    h = torch.zeros(32, 128, device="cuda:0", dtype=torch.float16)  # T_local differs from the buffers'
    st = lib.lib.ctb_moe_ffn_ep(eps[0], None, C.c_void_p(h.data_ptr()), C.c_void_p(h.data_ptr()), C.c_void_p(h.data_ptr()),
                                C.c_void_p(h.data_ptr()), C.c_void_p(h.data_ptr()), C.c_void_p(h.data_ptr()), 32, 128, 64,
                                8, 2, 128, 128, 64, lib.A2A_PEER)
    assert st == lib.BAD_ARG and "differs" in lib.last_error()
    st = lib.lib.ctb_moe_ffn_ep(eps[0], None, C.c_void_p(h.data_ptr()), C.c_void_p(h.data_ptr()), C.c_void_p(h.data_ptr()),
                                C.c_void_p(h.data_ptr()), C.c_void_p(h.data_ptr()), C.c_void_p(h.data_ptr()), 64, 128, 64,
                                8, 2, 128, 128, 64, 7)
    assert st == lib.BAD_ARG and "a2a_mode" in lib.last_error()
