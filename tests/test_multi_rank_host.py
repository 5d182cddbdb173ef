"""Host side of the N > 1 launch, on CPU with the gloo backend and two ranks.

The data path has no collective (every rank is a full replica with its own 32 rows); what the ranks
share is the line-up before the timed region, the slowest rank's time and the whole-job rate."""

import json
import os
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent

WORKER = r"""
import json, os, sys
sys.path.insert(0, os.environ["QWC_ROOT"])
import numpy as np
import bench

group = bench.RankGroup("gloo")
contexts = bench.contexts_for(group.rank)
group.barrier()
slowest = group.max_over_ranks(1.0 + 0.5 * group.rank)     # rank 1 is the slow one
rate = group.whole_job_rate(bench.ROWS * 4, slowest)
group.barrier()
print(json.dumps({"rank": group.rank, "world": group.world, "slowest": slowest, "rate": rate,
                  "contexts": contexts.tolist()}))
group.close()
"""


def launch(world: int, port: int):
    processes = []
    for rank in range(world):
        env = dict(os.environ, WORLD_SIZE=str(world), RANK=str(rank), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(port), QWC_ROOT=str(ROOT))
        processes.append(subprocess.Popen([sys.executable, "-c", WORKER], env=env, stdout=subprocess.PIPE,
                                          stderr=subprocess.PIPE, text=True))
    results = []
    for process in processes:
        out, err = process.communicate(timeout=240)
        assert process.returncode == 0, err[-2000:]
        results.append(json.loads(out.strip().splitlines()[-1]))
    return sorted(results, key=lambda r: r["rank"])


def test_two_ranks_agree_on_the_slowest_time_and_sum_their_rows():
    first, second = launch(2, 29641)
    assert (first["world"], second["world"]) == (2, 2)
    # max over ranks, seen by both
    assert first["slowest"] == second["slowest"] == 1.5
    # whole-job rate: the rows of both ranks over the slowest rank's time
    import bench  # noqa: F401  (ROWS)
    assert first["rate"] == second["rate"] == 2 * bench.ROWS * 4 / 1.5
    # every rank draws its own slice of the workload: same distribution, different rows
    assert len(first["contexts"]) == len(second["contexts"]) == bench.ROWS
    assert first["contexts"] != second["contexts"]
    assert all(bench.CONTEXT_LOW <= c <= bench.CONTEXT_HIGH for c in first["contexts"] + second["contexts"])


def test_single_rank_needs_no_process_group():
    (only,) = launch(1, 29642)
    assert only["world"] == 1 and only["slowest"] == 1.0
    import bench
    assert only["rate"] == bench.ROWS * 4


def test_workload_slice_is_a_function_of_the_rank():
    import bench

    assert bench.contexts_for(3).tolist() == bench.contexts_for(3).tolist()
    assert bench.contexts_for(3).tolist() != bench.contexts_for(4).tolist()


# Latency mode's set-up: every rank contributes the handle of its exchange block and receives
# everybody's in rank order (the device part - mapping the blocks - is the engine's and needs GPUs).
EXCHANGE_WORKER = r"""
import json, os, sys
sys.path.insert(0, os.environ["QWC_ROOT"])
import torch.distributed as dist
from qwencore_b200 import engine as E

class FakeEngine:
    def __init__(self, rank):
        self.rank, self.opened = rank, None
    def exchange_handle(self):
        return bytes([self.rank]) * 64
    def open_peers(self, handles):
        self.opened = handles

dist.init_process_group("gloo")
fake = FakeEngine(dist.get_rank())
E.connect_exchange(fake)
print(json.dumps({"rank": fake.rank, "first_bytes": [h[0] for h in fake.opened], "sizes": [len(h) for h in fake.opened]}))
dist.destroy_process_group()
"""


def test_exchange_handles_arrive_in_rank_order_on_every_rank():
    processes = []
    for rank in range(2):
        env = dict(os.environ, WORLD_SIZE="2", RANK=str(rank), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                   MASTER_PORT="29643", QWC_ROOT=str(ROOT))
        processes.append(subprocess.Popen([sys.executable, "-c", EXCHANGE_WORKER], env=env, stdout=subprocess.PIPE,
                                          stderr=subprocess.PIPE, text=True))
    for process in processes:
        out, err = process.communicate(timeout=240)
        assert process.returncode == 0, err[-2000:]
        result = json.loads(out.strip().splitlines()[-1])
        assert result["first_bytes"] == [0, 1] and result["sizes"] == [64, 64]
