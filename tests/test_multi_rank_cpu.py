"""World-size-2 gloo check of the benchmark's rank plumbing on CPU: head sharding covers the job exactly once, the
max-over-ranks reduction and barriers work, and the reference arm prints its line on rank 0 only."""
import json
import os
import subprocess
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = r'''
import os, sys, json
sys.path.insert(0, os.environ["REPO_ROOT"])
import torch
import torch.distributed as dist
import bench
world, rank, local = bench.dist_setup(2, cpu_only=True)
assert world == 2
lo, hi = bench.shard_heads(37, world, rank)
spans = [None, None]
dist.all_gather_object(spans, (lo, hi))
bench.barrier(world)
mx = bench.max_over_ranks(float(rank + 1), world, torch.device("cpu"))
if rank == 0:
    print(json.dumps({"spans": spans, "max": mx}))
dist.destroy_process_group()
'''


def _run(args, env_extra=None):
    env = dict(os.environ, REPO_ROOT=ROOT, MASTER_ADDR="127.0.0.1", OMP_NUM_THREADS="2")
    env.update(env_extra or {})
    return subprocess.run(args, cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)


def test_shard_heads_partitions_every_job():
    sys.path.insert(0, ROOT)
    import bench
    for total in (1, 7, 32, 256, 257):
        for world in (1, 2, 4, 8):
            spans = [bench.shard_heads(total, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == total
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [b - a for a, b in spans]
            assert max(sizes) - min(sizes) <= 1


def test_two_rank_plumbing_over_gloo(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    res = _run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                "--master-addr", "127.0.0.1", "--master-port", "29541", str(script)])
    assert res.returncode == 0, res.stderr[-2000:]
    line = [l for l in res.stdout.splitlines() if l.startswith("{")][-1]
    out = json.loads(line)
    assert out["spans"] == [[0, 19], [19, 37]] and out["max"] == 2.0


def test_reference_arm_prints_one_line_from_rank0():
    res = _run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                "--master-addr", "127.0.0.1", "--master-port", "29542", "bench.py", "--impl", "reference",
                "--gpus", "2", "--steps", "1", "--warmup", "0"],
               {"LMK_BENCH_CPU_HEADS": "1", "LMK_BENCH_SKIP_CONFIG1": "1"})
    assert res.returncode == 0, res.stderr[-2000:]
    lines = [l for l in res.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["unit"] == "TFLOP/s" and d["value"] > 0
    # "reference" where oracle/_ref has been staged from a checkout (oracle/make_ref.py), else the restatement
    assert d["cpu_baseline"]["kind"] in ("reference", "port") and d["e2e"]["h2d_bytes_per_step"] == 0
