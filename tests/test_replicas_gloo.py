"""The N > 1 host logic on CPU: two gloo ranks (no GPU, no NCCL)."""
import json
import os
import subprocess
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, out_dir):
    os.environ.update(RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port))
    sys.path.insert(0, ROOT)
    from glm_asr_stack_b200 import replicas
    r, lr, w = replicas.rank_info()
    d = replicas.init_group("gloo", w)
    assert (r, lr, w) == (rank, rank, world) and d is not None
    d.barrier()
    # rank 1 is the slow one: everybody must report its time
    mine = 2.0 + rank
    slowest = replicas.max_over_ranks(mine, d)
    rate = replicas.whole_job_rate(100.0, w, slowest)
    begin, end = replicas.shard_rows(10001, r, w)
    with open(os.path.join(out_dir, f"rank{rank}.json"), "w") as f:
        json.dump({"slowest": slowest, "rate": rate, "rows": [begin, end]}, f)
    d.barrier()
    d.destroy_process_group()


def test_two_gloo_ranks_max_time_and_whole_job_rate(tmp_path):
    port = 29650 + os.getpid() % 200
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    res = [json.load(open(tmp_path / f"rank{r}.json")) for r in range(2)]
    for r in res:
        assert r["slowest"] == 3.0                       # max over ranks, on every rank
        assert r["rate"] == pytest.approx(2 * 100.0 / 3.0)
    assert res[0]["rows"] == [0, 5001] and res[1]["rows"] == [5001, 10001]


def test_single_rank_needs_no_group():
    sys.path.insert(0, ROOT)
    from glm_asr_stack_b200 import replicas
    assert replicas.init_group("gloo", 1) is None
    assert replicas.max_over_ranks(1.5, None) == 1.5
    assert replicas.shard_rows(10, 0, 1) == (0, 10)


def test_reference_arm_prints_on_rank0_only():
    """Under a multi-rank launch only rank 0 runs and prints the reference arm; the others exit 0 silently."""
    env = dict(os.environ, RANK="1", LOCAL_RANK="1", WORLD_SIZE="2")
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2",
                        "--steps", "1", "--warmup", "1"], env=env, capture_output=True, text=True, timeout=300)
    assert p.returncode == 0 and p.stdout.strip() == ""
