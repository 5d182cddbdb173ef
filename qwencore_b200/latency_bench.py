"""Latency mode: one sequence, every projection column-split over the ranks (torchrun, one rank per GPU).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node G --master-addr 127.0.0.1 \
        --master-port 29555 -m qwencore_b200.latency_bench [--context 2048] [--steps 50]
    python -m qwencore_b200.latency_bench            # G = 1

Prints one JSON line on rank 0: milliseconds per decode step at batch 1 (graph replay, inputs resident,
CUDA events on the engine's stream, max over ranks).  Every rank holds N / G rows of each projection
and of the vocabulary head and an all-gather in the graph completes each output row; the recurrent
update and attention run replicated.  torch.distributed (gloo) only carries the NCCL id and the
max-over-ranks of the timing."""

from __future__ import annotations

import argparse
import json
import os

import numpy as np
import torch

from . import engine as engine_module


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--context", type=int, default=2048)
    parser.add_argument("--steps", type=int, default=50)
    parser.add_argument("--layers", type=int, default=64)
    options = parser.parse_args(argv)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    dist = None
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("gloo")
    page = 16
    blocks = (options.context + options.steps + 64) // page + 8
    config = engine_module.default_config(num_layers=options.layers, max_batch=1, max_context=options.context + 1024,
                                          kv_pool_blocks=blocks, state_slots=2, seed=3, split_rank=rank,
                                          split_size=world)
    engine = engine_module.Engine(config)
    if world > 1:
        unique = [engine_module.nccl_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(unique, src=0)
        engine.init_split(unique[0])
    cache = engine_module.CacheManager(2, blocks, page)
    cache.admit(1, options.context)
    engine.apply_edits(cache.drain_edits())
    token = np.array([17], dtype=np.uint32)
    slot = np.array([cache.sequence(1)["state_slot"]], dtype=np.uint32)
    for _ in range(4):  # eager, capture, replays
        cache.append_token(1)
        token = engine.decode(slot, token, cache.drain_edits())
    stream = torch.cuda.ExternalStream(engine.stream)
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    begin.record(stream)
    for _ in range(options.steps):
        engine.replay(1)
    end.record(stream)
    torch.cuda.synchronize()
    milliseconds = begin.elapsed_time(end) / options.steps
    if dist is not None:
        slowest = torch.tensor([milliseconds], dtype=torch.float64)
        dist.all_reduce(slowest, op=dist.ReduceOp.MAX)
        milliseconds = float(slowest.item())
    traffic = engine.traffic(1, float(options.context))
    if rank == 0:
        weights = traffic.weight_bytes
        print(json.dumps({"metric": "decode_step_latency", "unit": "ms", "value": milliseconds, "n_gpus": world,
                          "tokens_per_second": 1e3 / milliseconds, "higher_is_better": False,
                          "config": {"workload": f"batch 1, context {options.context}, {options.layers} layers, "
                                                 f"projections column-split {world} ways + all-gather"},
                          "weight_bytes_per_rank": weights,
                          "weights_gbs_per_rank": weights / (milliseconds * 1e-3) / 1e9}))
    engine.close()
    if dist is not None:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
