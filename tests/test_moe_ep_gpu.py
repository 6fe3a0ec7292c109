"""Expert-parallel MoE on 2 GPUs, both through NCCL all-to-all dispatch/combine and through stores into peer
memory: bit-identical to the single-GPU result.
Skipped on a box with fewer than two GPUs."""
import json
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_moe_ep_matches_single_gpu():
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", "29577", os.path.join(ROOT, "tests", "ep_worker.py"), "gpu"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    assert r.returncode == 0, r.stdout[-1500:] + r.stderr[-2500:]
    rows = [json.loads(l) for l in r.stdout.splitlines() if l.startswith("{")]
    assert all(x.get("peer") for x in rows), rows
    assert sorted(x["rank"] for x in rows) == [0, 1] and all(x["ok"] for x in rows)
