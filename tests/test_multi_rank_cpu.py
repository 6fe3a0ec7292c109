"""World-size-2 checks of the multi-rank host logic on CPU (gloo): the job time is the maximum over ranks, the
job throughput aggregates every rank's shard, and the reference arm prints one line from rank 0 only."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = r"""
import os, sys, json
sys.path.insert(0, %r)
import torch, torch.distributed as dist
import bench
dist.init_process_group("gloo")
rank, world = dist.get_rank(), dist.get_world_size()
ms = bench.max_over_ranks(10.0 + 5.0 * rank, torch, dist, "cpu")   # rank 1 is the slow one
val = bench.aggregate_value(1e12, world, ms, "TFLOP/s")            # 1 TFLOP per rank per step
# batch shards of the multi-GPU FMHA (64) and batched GEMM (8) problems, and a ragged count: gathered over the ranks
shards = {}
for total in (64, 8, 7):
    mine = torch.tensor(list(bench.shard_range(total, world, rank)))
    got = [torch.zeros(2, dtype=mine.dtype) for _ in range(world)]
    dist.all_gather(got, mine)
    shards[str(total)] = [g.tolist() for g in got]
os.write(1, (json.dumps({"rank": rank, "ms": ms, "value": val, "shards": shards}) + "\n").encode())  # one write: ranks share the pipe
dist.destroy_process_group()
""" % ROOT


def _json_rows(text):
    """Every JSON object in `text`, also when two ranks' lines ran together on the shared pipe."""
    dec, rows, i = json.JSONDecoder(), [], 0
    while True:
        i = text.find("{", i)
        if i < 0:
            return rows
        try:
            obj, end = dec.raw_decode(text, i)
            rows.append(obj)
            i = end
        except json.JSONDecodeError:
            i += 1


def _torchrun(args, timeout=240):
    env = dict(os.environ, OMP_NUM_THREADS="2")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
           "--master-addr", "127.0.0.1", "--master-port", "29533"] + args
    return subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env, cwd=ROOT)


def test_time_is_max_over_ranks_and_value_aggregates(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    r = _torchrun([str(script)])
    assert r.returncode == 0, r.stderr[-2000:]
    rows = _json_rows(r.stdout)
    assert sorted(x["rank"] for x in rows) == [0, 1]
    for x in rows:
        assert x["ms"] == 15.0                      # the slowest rank's time on every rank
        assert abs(x["value"] - 2 / 15e-3) < 1e-9   # 2 TFLOP of work in 15 ms
        # the ranks' shards tile [0, total) without gaps or overlap, sizes differ by at most one
        assert x["shards"] == {"64": [[0, 32], [32, 64]], "8": [[0, 4], [4, 8]], "7": [[0, 4], [4, 7]]}


def test_reference_arm_prints_once_under_torchrun():
    r = _torchrun(["bench.py", "--impl", "reference", "--gpus", "2", "--steps", "1", "--warmup", "1",
                   "--headline", "softmax_tma"])
    assert r.returncode == 0, r.stderr[-2000:]
    lines = _json_rows(r.stdout)
    assert len(lines) == 1
    line = lines[0]
    assert line["impl"] == "reference" and line["n_gpus"] == 2 and line["gpu_launches"] == 0
    assert line["cpu_baseline"]["kind"] == "port" and line["e2e"]["h2d_bytes_per_step"] == 0
    assert line["value"] > 0 and line["unit"] == "GB/s"
