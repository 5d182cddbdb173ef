"""One rank of the column-split (latency mode) engine test: run by tests/test_gpu_split.py, one
process per GPU.  Every rank holds N / G rows of every projection and of the vocabulary head.  With
QWC_SPLIT_EXCHANGE=1 the ranks store their partial sums into one another's memory and the consumers
sum them (the fused form); with 0 an in-graph ncclAllGather completes each output row.  Rank 0
rebuilds the whole model on the host from all ranks' slices, runs the CPU oracle step on it and
compares."""

import os
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))


class MergedEngine:
    """Looks like one unsplit engine to HostModel: split tensors are the ranks' slices stacked by rows."""

    SPLIT = ("gate", "up", "down", "in_proj", "la_out", "qkv", "o")

    def __init__(self, engine, config, slices, shapes):
        self.engine, self.config, self.slices, self.shapes = engine, config, slices, shapes

    def read(self, name, layer=0, dtype=np.uint8):
        from oracle import oracle

        base = name.split(".")[0]
        if base in self.SPLIT:
            n, k = self.shapes[base]
            ranks = len(self.slices)
            local = n // ranks
            if name.endswith(".packed"):
                return np.concatenate([s[(name, layer)] for s in self.slices])
            logical = [oracle.unswizzle_block_scales(s[(name, layer)], local, k) for s in self.slices]
            return oracle.swizzle_block_scales(np.concatenate(logical), n, k)
        if name in ("lm_head", "lm_head_scales"):
            return np.concatenate([s[(name, 0)] for s in self.slices]).view(dtype)
        return self.engine.read(name, layer, dtype)


def main():
    import torch
    import torch.distributed as dist

    from qwencore_b200 import abi, engine as E
    from step_oracle import HostModel, decode_step
    from test_gpu_step import host_layout

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("gloo")
    fused = os.environ.get("QWC_SPLIT_EXCHANGE", "1") == "1"
    config = E.default_config(num_layers=4, vocab=8192, max_batch=1, max_context=512, kv_pool_blocks=64,
                              state_slots=2, seed=11, use_graph=1, split_rank=rank, split_size=world,
                              write_logits=1, exchange=1 if fused else 0)
    engine = E.Engine(config)
    if fused:
        E.connect_exchange(engine)
    else:
        unique = [E.nccl_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(unique, src=0)
        engine.init_split(unique[0])

    # every rank's slices of the split tensors, gathered on rank 0
    c = config
    v_heads = c.delta_value_heads
    mixer = 2 * 16 * 128 + 2 * v_heads * 128 + 2 * v_heads
    shapes = {"gate": (c.intermediate, c.hidden), "up": (c.intermediate, c.hidden), "down": (c.hidden, c.intermediate),
              "in_proj": (mixer, c.hidden), "la_out": (c.hidden, v_heads * 128),
              "qkv": (24 * 2 * 256 + 2 * 4 * 256, c.hidden), "o": (c.hidden, 24 * 256)}
    mine = {}
    for layer in range(c.num_layers):
        full = (layer + 1) % c.full_attention_interval == 0
        for base in ("gate", "up", "down") + (("qkv", "o") if full else ("in_proj", "la_out")):
            for part in ("packed", "scales"):
                mine[(f"{base}.{part}", layer)] = engine.read(f"{base}.{part}", layer)
    mine[("lm_head", 0)] = engine.read("lm_head")
    mine[("lm_head_scales", 0)] = engine.read("lm_head_scales", 0, np.float32).view(np.uint8)
    gathered = [None] * world if rank == 0 else None
    dist.gather_object(mine, gathered, dst=0)

    cache = E.CacheManager(2, 64, 16)
    cache.admit(100, 37)
    engine.apply_edits(cache.drain_edits())
    model = None
    if rank == 0:
        model = HostModel(MergedEngine(engine, config, gathered, shapes))
    tokens = np.array([1234], dtype=np.uint32)
    failures = []
    for step in range(3):  # eager, captured, replayed
        cache.append_token(100)
        edits = cache.drain_edits()
        layout = host_layout(cache, [100], 16, 2, (c.max_context + 15) // 16)
        dist.barrier()  # the ranks step together: a consumer waits a second for its peers, not for the oracle
        sampled = engine.decode(layout["state_slots"], tokens, edits)
        logits = engine.read("logits", 0, np.float32).reshape(c.max_batch, c.vocab)[:1]
        if fused:
            logits = logits[:, : c.vocab // world]  # this rank's columns; only the candidates travel
        everyone = [None] * world if rank == 0 else None
        dist.gather_object((sampled.tolist(), logits.tobytes()), everyone, dst=0)
        if rank == 0:
            if fused:
                # every rank picked the same token from everybody's candidates
                if any(other[0] != everyone[0][0] for other in everyone[1:]):
                    failures.append(f"step {step}: ranks disagree on the token")
                logits = np.concatenate([np.frombuffer(other[1], np.float32) for other in everyone]).reshape(1, c.vocab)
            else:
                # the gathered logits are the same bytes on every rank
                for other in everyone[1:]:
                    if other != everyone[0]:
                        failures.append(f"step {step}: ranks disagree")
            want_logits, want_tokens, _ = decode_step(model, layout, tokens)
            rms = np.sqrt(np.mean(want_logits.astype(np.float64) ** 2))
            rms_err = np.sqrt(np.mean((logits - want_logits).astype(np.float64) ** 2))
            worst = np.max(np.abs(logits - want_logits))
            if not (np.isfinite(logits).all() and rms_err <= 2e-2 * rms and worst <= 1e-1 * rms):
                failures.append(f"step {step}: logits rms err {rms_err} worst {worst} vs rms {rms}")
            if sampled[0] != int(np.argmax(logits[0])):
                failures.append(f"step {step}: sampled {sampled[0]} is not the argmax of the gathered logits")
            tokens = want_tokens.astype(np.uint32)
        broadcast = [tokens.tolist()]
        dist.broadcast_object_list(broadcast, src=0)
        tokens = np.array(broadcast[0], dtype=np.uint32)
    status = abi.lib.qwc_device_status()
    if status != 0:
        failures.append(f"device status {status}")
    everyone = [None] * world if rank == 0 else None
    dist.gather_object(failures, everyone, dst=0)
    engine.close()
    dist.destroy_process_group()
    if rank == 0:
        problems = [f for fs in everyone for f in fs]
        print("SPLIT-OK" if not problems else "SPLIT-FAIL " + "; ".join(problems))
        return 0 if not problems else 1
    return 0


if __name__ == "__main__":
    sys.exit(main())
