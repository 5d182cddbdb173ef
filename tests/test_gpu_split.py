"""Column-split (latency mode) engine on two GPUs, one process per GPU: every projection's output rows
are divided over the ranks.  Both forms: the fused one (partial sums stored into the peers' memory by
the projection's epilogue, summed by the consumers after a bounded wait for tagged words) and the
library one (an in-graph ncclAllGather after every projection).  NVLS is off in both.  Needs two
visible GPUs; skipped otherwise."""

import os
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


@pytest.mark.gpu
@pytest.mark.parametrize("fused", [1, 0], ids=["peer_stores", "nccl_all_gather"])
def test_column_split_step_matches_the_oracle_on_two_gpus(cuda, fused):
    if cuda.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    processes = []
    for rank in range(2):
        env = dict(os.environ, WORLD_SIZE="2", RANK=str(rank), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(29733 + fused), NCCL_NVLS_ENABLE="0", QWC_SPLIT_EXCHANGE=str(fused))
        processes.append(subprocess.Popen([sys.executable, str(ROOT / "tests" / "split_worker.py")], env=env,
                                          stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True))
    outputs = []
    for process in processes:
        try:
            out, err = process.communicate(timeout=300)
        except subprocess.TimeoutExpired:
            for other in processes:
                other.kill()
            raise
        outputs.append((process.returncode, out, err))
    assert all(code == 0 for code, _, _ in outputs), "\n".join(err[-1500:] + out[-500:] for _, out, err in outputs)
    assert "SPLIT-OK" in outputs[0][1], outputs[0][1][-1000:]
