"""Decode-step benchmark: ragged c=32 step of the synthetic 27B-shaped hybrid NVFP4 model.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

One JSON line on stdout (rank 0).  `value` is decode tokens per second with every input
resident in HBM (CUDA-graph replays timed with CUDA events on the engine's stream); `e2e` is
the same metric through the worker loop a server runs - scheduler, host layout check, one
host-to-device copy of the step's slots / tokens / page-table edits, the captured step, and
the device-to-host read of the sampled tokens.  `roofline` is the NVFP4 projection kernel's
algorithmic bytes per launch over its event-timed duration (a CUDA graph of all projection
launches of one step, replayed on the engine's stream), against the measured HBM copy rate of this
pool.  `cpu_baseline` / `--impl reference` time the scalar CPU port of the
reference's own `reference` modules on the host cores, on a bounded sample of the same step.

With N > 1 (launched by torchrun) every rank owns a full replica and a disjoint slice of the
batch - no collective on the data path - so `value` is the sum over ranks (weak scaling).
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

ROWS = 32
CONTEXT_LOW, CONTEXT_HIGH = 128, 32768
PAGE = 16
METRIC = "decode_tokens_per_second"
NCU_TRAFFIC_RATIO = 104.83 / 100.35  # profiles/nvfp4_umma_34816x5120_m32.md


# ---- clocks ---------------------------------------------------------------------------------

class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi during the timed region."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self, index: int):
        self.index = index
        self.samples = []
        self.process = None
        self.thread = None

    def start(self):
        try:
            self.process = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.process.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 6:
                self.samples.append(parts)

    def stop(self):
        if self.process is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        self.process.terminate()
        try:
            self.process.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.process.kill()
        clocks, reasons, sm_max = [], set(), None
        for parts in self.samples:
            try:
                clocks.append(float(parts[0]))
                sm_max = float(parts[1])
            except ValueError:
                continue
            for name, flag in zip(self.NAMES, parts[2:6]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(clocks)) if clocks else None, "sm_max_mhz": sm_max,
                "reasons": sorted(reasons), "samples": len(clocks)}


# ---- workload ---------------------------------------------------------------------------------

def contexts_for(rank: int) -> np.ndarray:
    from qwencore_b200 import synth

    return synth.log_uniform_contexts(rank, ROWS, CONTEXT_LOW, CONTEXT_HIGH)


class RankGroup:
    """The ranks of one launch: data-parallel replicas that only meet to line up and compare clocks.

    One process per GPU under torchrun (backend "nccl"); the same class runs on CPU with "gloo" in the
    tests.  There is no collective on the data path: a rank's 32 rows, its scheduler and its engine
    are its own.  `value` of the whole job = rows of all ranks x steps / the slowest rank's time."""

    def __init__(self, backend: str, local_device=None):
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        self.backend = backend
        self.device = local_device
        self.dist = None
        if self.world > 1:
            import torch.distributed as dist

            kwargs = {"device_id": local_device} if (backend == "nccl" and local_device is not None) else {}
            dist.init_process_group(backend, **kwargs)
            self.dist = dist

    def barrier(self) -> None:
        if self.dist is not None:
            self.dist.barrier()

    def max_over_ranks(self, value: float) -> float:
        if self.dist is None:
            return value
        import torch

        t = torch.tensor([value], dtype=torch.float64, device=self.device if self.backend == "nccl" else "cpu")
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def whole_job_rate(self, units_per_rank: float, slowest_seconds: float) -> float:
        return self.world * units_per_rank / slowest_seconds

    def close(self) -> None:
        if self.dist is not None:
            self.dist.destroy_process_group()
            self.dist = None


def measured_peak_gbs():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            return float(json.loads(path.read_text())["hbm_gbs"]), "measured"
        except (ValueError, KeyError):
            pass
    return 6650.0, "fallback"


def step_macs(contexts, hidden=5120, intermediate=17408, vocab=151936, v_heads=32, layers=64, interval=4):
    """Multiply-accumulates of one step: what the scalar CPU path has to do."""
    rows = len(contexts)
    full = layers // interval
    linear = layers - full
    mixer = 2 * 2048 + 2 * v_heads * 128 + 2 * v_heads
    mlp = 3 * intermediate * hidden
    per_row = layers * mlp + linear * (mixer * hidden + hidden * v_heads * 128) + \
        full * (14336 * hidden + hidden * 6144) + vocab * hidden
    attention = full * 2 * 24 * 256 * float(np.sum(contexts))
    delta = linear * rows * v_heads * 128 * 128 * 4
    return rows * per_row + attention + delta, rows * mlp


def cpu_sample(threads: int, repeats: int = 1):
    """Times the oracle on one MLP block (gate/up SwiGLU + down) for the 32-row batch.

    Returns (seconds per sample, sample MACs, description)."""
    from oracle import oracle
    from qwencore_b200 import synth

    hidden, intermediate = 5120, 17408
    oracle.set_num_threads(threads)
    gate = synth.nvfp4_matrix(0, "bench.gate", intermediate, hidden)
    up = synth.nvfp4_matrix(0, "bench.up", intermediate, hidden)
    down = synth.nvfp4_matrix(0, "bench.down", hidden, intermediate)
    x = synth.normal_bf16(0, "bench.x", (ROWS, hidden))
    best = float("inf")
    for _ in range(repeats):
        start = time.perf_counter()
        g = oracle.gemv_w4a16(gate[0], gate[1], 1.0, x, intermediate, hidden, ROWS)
        u = oracle.gemv_w4a16(up[0], up[1], 1.0, x, intermediate, hidden, ROWS)
        h = oracle.bf16_from_f32(oracle.swiglu_combine(g, u))
        oracle.gemv_w4a16(down[0], down[1], 1.0, h, hidden, intermediate, ROWS)
        best = min(best, time.perf_counter() - start)
    return best, ROWS * 3 * intermediate * hidden, "one MLP block (NVFP4 gate/up SwiGLU + down) at c=32"


def cpu_tokens_per_second(threads: int, repeats: int = 1):
    seconds, sample_macs, what = cpu_sample(threads, repeats)
    total_macs, _ = step_macs(contexts_for(0))
    step_seconds = seconds * total_macs / sample_macs
    sample = (f"{what}: {seconds:.2f} s on {threads} threads; scaled by multiply-accumulate count to the whole "
              f"step (x{total_macs / sample_macs:.1f})")
    return ROWS / step_seconds, sample


def base_line(args, n_gpus):
    return {
        "metric": METRIC,
        "unit": "tok/s",
        "n_gpus": n_gpus,
        "steps": args.steps,
        "warmup": args.warmup,
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "nvfp4 weights x bf16 activations, fp32 accumulate (int8 DeltaNet state, e4m3 KV)",
        "data": "synthetic",
        "config": {
            "workload": "full decode step, 27B-shaped hybrid NVFP4 model (64 layers 3:1 DeltaNet:attention, hidden "
                        "5120, SwiGLU 17408, vocab 151936, FP8 lm_head), c=32 ragged per GPU, contexts log-uniform "
                        "[128, 32768], page 16, greedy argmax, CUDA graph",
            "rows_per_gpu": ROWS,
            "parallelism": f"dp{n_gpus} (independent replicas, disjoint batch slices, no collective)",
            "l2": "working set per step (13.6 GB of weights) exceeds the 126 MB L2; no flush needed",
        },
    }


# ---- reference arm: the CPU port on the host cores ------------------------------------------

def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    from oracle import oracle

    threads = os.cpu_count() or 1
    oracle.set_num_threads(threads)
    for _ in range(min(args.warmup, 1)):
        cpu_sample(threads)
    samples = []
    start = time.perf_counter()
    what = ""
    sample_macs = 1
    for _ in range(args.steps):
        seconds, sample_macs, what = cpu_sample(threads)
        samples.append(seconds)
        if time.perf_counter() - start > 150:  # bounded: the whole run must end within minutes
            break
    total_macs, _ = step_macs(contexts_for(0))
    seconds = float(np.mean(samples))
    step_seconds = seconds * total_macs / sample_macs
    value = ROWS / step_seconds
    line = base_line(args, args.gpus)
    line.update({
        "impl": "reference",
        "value": value,
        "steps": len(samples),
        "ms_per_step": step_seconds * 1e3,
        "config": {**line["config"], "parallelism": "host cores of rank 0"},
        "cpu_baseline": {"value": value, "unit": "tok/s", "cores": threads, "kind": "port",
                         "sample": f"{what}: mean {seconds:.2f} s over {len(samples)} runs; scaled by "
                                   f"multiply-accumulate count to the whole step (x{total_macs / sample_macs:.1f}); "
                                   "the reference's CPU path is Rust and cannot be built here, this is its C port"},
        "e2e": {"value": value, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    })
    print(json.dumps(line))
    return 0


# ---- our arm ------------------------------------------------------------------------------------

def run_ours(args):
    import torch

    from qwencore_b200 import engine as engine_module

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the decode step has no CPU path")
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    group = RankGroup("nccl", torch.device("cuda", local_rank))
    world, rank, distributed = group.world, group.rank, group.world > 1

    contexts = contexts_for(rank)
    total_steps = args.steps + args.warmup + 8
    blocks_needed = int(np.sum((contexts + total_steps + PAGE - 1) // PAGE)) + 64
    config = engine_module.default_config(max_batch=ROWS, max_context=CONTEXT_HIGH + 1024,
                                          kv_pool_blocks=blocks_needed, state_slots=ROWS + 1, seed=rank)
    engine = engine_module.Engine(config)
    stream = torch.cuda.ExternalStream(engine.stream)

    # The worker loop: submit 32 requests whose prompts are taken as already cached.
    scheduler = engine_module.Scheduler(ROWS, 1 << 22, ROWS + 1, blocks_needed, PAGE)
    for i, context in enumerate(contexts):
        scheduler.submit(i + 1, int(context), total_steps + 16)
    decoded = 0
    while decoded == 0:  # prompt accounting steps, then the first (eager) decode step
        decoded, _ = engine.worker_step(scheduler)
    for _ in range(max(args.warmup, 3)):  # captures the graph, then replays
        engine.worker_step(scheduler)

    def barrier():
        group.barrier()
        torch.cuda.synchronize()

    max_over_ranks = group.max_over_ranks

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()

    # ---- end to end: host inputs, copies inside the timed region ----
    barrier()
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    wall = time.perf_counter()
    begin.record(stream)
    for _ in range(args.steps):
        rows, _ = engine.worker_step(scheduler)
        assert rows == ROWS
    end.record(stream)
    barrier()
    e2e_seconds = max_over_ranks(time.perf_counter() - wall)

    # ---- device only: inputs resident, graph replays ----
    for _ in range(3):
        engine.replay(ROWS)
    barrier()
    begin.record(stream)
    for _ in range(args.steps):
        engine.replay(ROWS)
    end.record(stream)
    barrier()
    device_seconds = max_over_ranks(begin.elapsed_time(end) * 1e-3)

    clocks = sampler.stop() if rank == 0 else None

    # ---- dominant kernel: all NVFP4 projections of the step, replayed back to back as one graph ----
    # (after the timed regions: the filtered graphs run on stale activations and leave the recurrent
    # state and the newest KV rows garbage)
    graph_phases = {}
    for prefix in ("gemm.", "attn.decode", "attn.prepare", "delta.scan", "delta.prepare", "delta.norm", "norm",
                   "lm_head", "sample", "pack", "embed"):
        ms, launched = engine.time_phases(ROWS, prefix, replays=5)
        graph_phases[prefix.rstrip(".")] = {"ms": round(ms, 4), "launches": launched}
    gemv_ms, gemv_launches = graph_phases["gemm"]["ms"], graph_phases["gemm"]["launches"]
    phases = {}
    for label, ms, launches in engine.profile_step(ROWS):
        total = phases.setdefault(label, [0.0, 0])
        total[0] += ms
        total[1] += launches
    context_now = float(np.sum(contexts)) + ROWS * (args.steps + args.warmup + 4)
    traffic = engine.traffic(ROWS, context_now)
    peak, peak_kind = measured_peak_gbs()
    bytes_per_launch = traffic.gemv_bytes_per_step / traffic.gemv_launches_per_step
    seconds_per_launch = gemv_ms * 1e-3 / max(1, gemv_launches)
    achieved = bytes_per_launch / seconds_per_launch / 1e9
    step_bytes = traffic.weight_bytes + traffic.state_bytes + traffic.kv_bytes

    if rank != 0:
        engine.close()
        group.close()
        return 0

    cpu_value, cpu_sample_text = cpu_tokens_per_second(os.cpu_count() or 1)
    tokens = ROWS * args.steps  # per rank
    line = base_line(args, world)
    line.update({
        "value": group.whole_job_rate(tokens, device_seconds),
        "ms_per_step": device_seconds / args.steps * 1e3,
        "e2e": {"value": group.whole_job_rate(tokens, e2e_seconds), "unit": "tok/s", "ms_per_step": e2e_seconds / args.steps * 1e3,
                "h2d_bytes_per_step": int((2 * ROWS + 4 * 2 * ROWS) * 4), "d2h_bytes_per_step": int((ROWS + 1) * 4),
                "path": "qwc_worker_step: scheduler.next_batch, layout check, H2D of slots/tokens/edits, graph "
                        "replay, D2H of sampled tokens, scheduler.complete_batch"},
        "gpu_launches": int(traffic.kernel_launches_per_step * args.steps),
        "roofline": {"bound": "hbm", "kernel": "nvfp4_umma_kernel (all NVFP4 projections of the step)",
                     "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "peak_kind": f"of {peak_kind}",
                     # DRAM read + write of one captured launch (ncu, 34816 x 5120, 32 rows) is 1.04 x its
                     # algorithmic bytes; every launch streams its matrix once, so traffic scales with it
                     "traffic": bytes_per_launch * NCU_TRAFFIC_RATIO,
                     "bytes_per_launch": bytes_per_launch, "us_per_launch": seconds_per_launch * 1e6,
                     "launches_timed": gemv_launches},
        "step_roofline": {"bytes_per_step": step_bytes, "weights": traffic.weight_bytes,
                          "state": traffic.state_bytes, "kv": traffic.kv_bytes,
                          "achieved_gbs": step_bytes / (device_seconds / args.steps) / 1e9,
                          "frac_of_measured_peak": step_bytes / (device_seconds / args.steps) / 1e9 / peak,
                          "frac_of_8tbs": step_bytes / (device_seconds / args.steps) / 8e12},
        "phases_graph_ms_per_step": graph_phases,
        "phases_eager_ms_per_step": {label: round(total[0], 4) for label, total in sorted(phases.items())},
        "cpu_baseline": {"value": cpu_value, "unit": "tok/s", "cores": os.cpu_count() or 1, "kind": "port",
                         "sample": cpu_sample_text},
        "clocks": clocks,
    })
    print(json.dumps(line))
    engine.close()
    group.close()
    return 0


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=20)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    args = parser.parse_args()
    if args.impl == "reference":
        return run_reference(args)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
