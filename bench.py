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
reference's own `reference` modules on the host cores, on a bounded sample of the same step: four
layers (three DeltaNet, one full attention) at c=32 with the benchmark's contexts, times 16, plus
the vocabulary head timed on an eighth of its rows.  `c1` is the same engine at one row (context
2048), the other half of the metric; with N > 1 `latency_mode` adds the column-split step at batch 1
over all N GPUs.

With N > 1 (launched by torchrun) every rank owns a full replica and a disjoint slice of the
batch - no collective on the data path - so `value` is the sum over ranks (weak scaling).
"""

from __future__ import annotations

import argparse
import ctypes
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
C1_CONTEXT = 2048
# DRAM read + write of one captured projection launch (ncu, 34816 x 5120 at 32 rows) over its
# algorithmic bytes; every launch streams its matrix once, so the traffic scales with the matrix.
NCU_TRAFFIC_RATIO = 104.49 / 100.35


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

    def gather(self, values) -> list:
        """Every rank's list of floats, in rank order."""
        if self.dist is None:
            return [list(values)]
        import torch

        mine = torch.tensor(list(values), dtype=torch.float64,
                            device=self.device if self.backend == "nccl" else "cpu")
        everyone = [torch.zeros_like(mine) for _ in range(self.world)]
        self.dist.all_gather(everyone, mine)
        return [t.tolist() for t in everyone]

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


CPU_SAMPLE_LAYERS = 4
CPU_HEAD_FRACTION = 8


class CpuStep:
    """The CPU port on a bounded sample of the benchmark's step: `CPU_SAMPLE_LAYERS` layers (3 DeltaNet +
    1 full attention, the model's pattern) at c=32 with the benchmark's contexts, extrapolated linearly
    to 64 layers, plus the vocabulary head and argmax timed on 1/8 of the rows."""

    def __init__(self, threads: int):
        from oracle import oracle, step

        self.oracle, self.step = oracle, step
        self.threads = threads
        oracle.set_num_threads(threads)
        self.head_rows = 151936 // CPU_HEAD_FRACTION
        self.model = step.SyntheticModel(contexts_for(0), num_layers=CPU_SAMPLE_LAYERS, head_rows=self.head_rows)
        self.head_seconds = None

    def layers_seconds(self) -> float:
        start = time.perf_counter()
        _, _, self.normed = self.step.decode_step(self.model, self.model.layout, self.model.tokens, head=False)
        return time.perf_counter() - start

    def head_seconds_full(self) -> float:
        model, oracle = self.model, self.oracle
        start = time.perf_counter()
        logits = oracle.fp8_lm_head(model.lm_head, model.lm_head_scales, self.normed, ROWS, model.cfg.hidden,
                                    self.head_rows)
        oracle.argmax(logits, self.head_rows, ROWS)
        return (time.perf_counter() - start) * CPU_HEAD_FRACTION

    def step_seconds(self):
        """(seconds of one whole step, seconds of the layer sample, seconds of the head)."""
        layers = self.layers_seconds()
        if self.head_seconds is None:
            self.head_seconds = self.head_seconds_full()
        return layers * (64 / CPU_SAMPLE_LAYERS) + self.head_seconds, layers, self.head_seconds

    def describe(self, layers: float, head: float, runs: int = 1) -> str:
        return (f"{CPU_SAMPLE_LAYERS} layers (3 DeltaNet + 1 full attention) of the step at c=32, contexts log-uniform "
                f"[{CONTEXT_LOW}, {CONTEXT_HIGH}]: {layers:.2f} s on {self.threads} threads"
                f"{'' if runs == 1 else f' (mean of {runs} runs)'}, x{64 // CPU_SAMPLE_LAYERS} for 64 layers; "
                f"vocabulary head + argmax on 1/{CPU_HEAD_FRACTION} of the rows, x{CPU_HEAD_FRACTION}: {head:.2f} s")


def cpu_tokens_per_second(threads: int):
    sample = CpuStep(threads)
    seconds, layers, head = sample.step_seconds()
    return ROWS / seconds, sample.describe(layers, head)


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
    threads = os.cpu_count() or 1
    sample = CpuStep(threads)
    for _ in range(min(args.warmup, 1)):
        sample.step_seconds()
    steps, layer_samples = [], []
    head = 0.0
    start = time.perf_counter()
    for _ in range(args.steps):
        seconds, layers, head = sample.step_seconds()
        steps.append(seconds)
        layer_samples.append(layers)
        if time.perf_counter() - start > 150:  # bounded: the whole run must end within minutes
            break
    step_seconds = float(np.mean(steps))
    value = ROWS / step_seconds
    line = base_line(args, args.gpus)
    line.update({
        "impl": "reference",
        "value": value,
        "steps": len(steps),
        "ms_per_step": step_seconds * 1e3,
        "config": {**line["config"], "parallelism": "host cores of rank 0"},
        "cpu_baseline": {"value": value, "unit": "tok/s", "cores": threads, "kind": "port",
                         "sample": sample.describe(float(np.mean(layer_samples)), head, len(steps)) +
                                   "; the reference's CPU path is Rust and cannot be built here, this is its C port"},
        "e2e": {"value": value, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    })
    print(json.dumps(line))
    return 0


# ---- our arm ------------------------------------------------------------------------------------

def time_worker_steps(engine, scheduler, group, stream, steps, rows):
    """Wall-clock seconds of `steps` worker-loop steps (host inputs, copies inside), max over ranks."""
    import torch

    group.barrier()
    torch.cuda.synchronize()
    wall = time.perf_counter()
    for _ in range(steps):
        decoded, _ = engine.worker_step(scheduler)
        assert decoded == rows
    group.barrier()
    torch.cuda.synchronize()
    return time.perf_counter() - wall


def time_replays(engine, group, stream, steps, rows):
    """Device seconds of `steps` graph replays with the inputs resident (CUDA events on the engine's stream)."""
    import torch

    for _ in range(3):
        engine.replay(rows)
    group.barrier()
    torch.cuda.synchronize()
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    begin.record(stream)
    for _ in range(steps):
        engine.replay(rows)
    end.record(stream)
    group.barrier()
    torch.cuda.synchronize()
    return begin.elapsed_time(end) * 1e-3


def traffic_launches(engine):
    return engine.traffic(1, float(C1_CONTEXT)).gemv_launches_per_step


def time_latency_engine(args, group, local_rank, fused):
    """One latency-mode engine (fused peer stores, or the library all-gather): ms per step as the max
    over ranks, every rank's tokens of the warm-up steps, and the traffic model."""
    import torch

    from qwencore_b200 import engine as engine_module

    world, rank = group.world, group.rank
    steps = max(args.steps, 20)
    blocks = (C1_CONTEXT + steps + args.warmup + 64) // PAGE + 8
    config = engine_module.default_config(max_batch=1, max_context=C1_CONTEXT + 1024, kv_pool_blocks=blocks,
                                          state_slots=2, seed=3, split_rank=rank, split_size=world,
                                          exchange=1 if fused else 0)
    engine = engine_module.Engine(config)
    if fused:
        engine_module.connect_exchange(engine)
    else:
        unique = [engine_module.nccl_unique_id() if rank == 0 else None]
        group.dist.broadcast_object_list(unique, src=0, device=torch.device("cuda", local_rank))
        engine.init_split(unique[0])
    cache = engine_module.CacheManager(2, blocks, PAGE)
    cache.admit(1, C1_CONTEXT)
    engine.apply_edits(cache.drain_edits())
    token = np.array([17], dtype=np.uint32)
    slot = np.array([cache.sequence(1)["state_slot"]], dtype=np.uint32)
    produced = []
    for index in range(max(args.warmup, 3) + 1):  # eager, capture, replays
        cache.append_token(1)
        group.barrier()  # the ranks step together (a consumer waits a second for its peers' words)
        try:
            token = engine.decode(slot, token, cache.drain_edits())
        except Exception as error:
            detail = (ctypes.c_uint32 * 2)()
            engine_module.lib.qwc_device_status_detail(detail)
            engine_module.lib.qwc_device_status_reset()
            raise RuntimeError(f"{'fused' if fused else 'library'} engine, warm-up step {index}, rank {rank}: {error}; "
                               f"tag waited for {detail[0]:#x}, found {detail[1]:#x}") from error
        produced.append(float(token[0]))
    stream = torch.cuda.ExternalStream(engine.stream)
    seconds = group.max_over_ranks(time_replays(engine, group, stream, steps, 1))
    waits = None
    if fused:
        # After the timed region, three more steps with the wait bookkeeping on: per exchange of the step,
        # the longest a consumer thread of this rank waited for a peer's word.  The bookkeeping is an atomic
        # per late word and lengthens the waits it measures, so these are upper bounds and never timed.
        engine_module.profile_waits(engine, True)
        for _ in range(3):
            cache.append_token(1)
            group.barrier()
            token = engine.decode(slot, token, cache.drain_edits())
        nanoseconds = engine_module.exchange_waits(engine).astype(np.float64)
        engine_module.profile_waits(engine, False)
        count = int(traffic_launches(engine)) + 1
        waits = {"bookkeeping": "on for these three steps only; perturbs what it measures (upper bounds)",
                 "sum_of_longest_us": round(float(nanoseconds.sum()) / 1e3, 1),
                 "over_5us": int((nanoseconds > 5e3).sum()),
                 "mean_us_by_exchange_of_a_layer": [round(float(np.mean(nanoseconds[i:count - 1:4])) / 1e3, 1)
                                                    for i in range(4)]}
        sums = group.gather([waits["sum_of_longest_us"]])
        waits["sum_of_longest_us_per_rank"] = [s[0] for s in sums]
    tokens_of_ranks = group.gather(produced)
    traffic = engine.traffic(1, float(C1_CONTEXT))
    # where the step's time goes: one more step launched eagerly with an event between phases (every
    # rank takes it - the ranks step together); no overlap between kernels, so an upper bound per phase
    group.barrier()
    phases = {}
    for label, ms, launches in engine.profile_step(1):
        phases[label] = {"ms": round(ms, 4), "launches": launches}
    status = engine_module.lib.qwc_device_status()
    # ... and each phase's kernels alone, as a graph replayed back to back (no waits: the words of the
    # last whole step still carry the current tag; the values are stale, which is why this comes last)
    graph_phases = {}
    if fused:
        group.barrier()
        for prefix in ("gemm.", "norm", "delta.prepare", "delta.scan", "delta.norm", "attn.", "mlp.combine", "lm_head"):
            try:
                phase_ms, launched = engine.time_phases(1, prefix, replays=5)
            except Exception:
                continue
            graph_phases[prefix.rstrip(".")] = {"ms": round(phase_ms, 4), "launches": launched}
        group.barrier()
    engine.close()
    return (seconds / steps * 1e3, produced, tokens_of_ranks, traffic, status,
            {"eager": phases, "graph": graph_phases, "waits": waits})


def run_latency_mode(args, group, local_rank, single_gpu_ms):
    """Batch 1 with every projection column-split over all ranks of the launch (one sequence, context
    2048): milliseconds per step, max over ranks, and the ranks' sampled tokens compared.  The headline
    is the fused form (projections store their partial sums into the peers' memory, consumers sum
    them); the same split with an ncclAllGather after every projection is timed beside it."""
    world = group.world
    ms, produced, tokens_of_ranks, traffic, status, phases = time_latency_engine(args, group, local_rank, True)
    library_ms, _, library_tokens, _, _, _ = time_latency_engine(args, group, local_rank, False)
    return {"ms_per_step": ms, "tok_s": 1e3 / ms, "vs_1gpu": single_gpu_ms / ms, "gpus": world,
            "exchange": "partial sums stored into every rank's memory by the projection's epilogue (8-byte "
                        "tagged words over NVLink), summed by the consuming kernel after a bounded wait; no "
                        "library collective in the step",
            "exchanges_per_step": int(traffic.gemv_launches_per_step + 1),
            "kernel_launches_per_step": int(traffic.kernel_launches_per_step),
            "weight_bytes_per_rank": traffic.weight_bytes,
            "device_status": int(status),
            "phases_eager_ms_per_step": phases["eager"],
            "phases_graph_ms_per_step": phases["graph"],
            "waits_for_peers": phases["waits"],
            "library_collective": {"ms_per_step": library_ms, "vs_1gpu": single_gpu_ms / library_ms,
                                   "what": "same split, ncclAllGather after every projection",
                                   "ranks_agree_on_tokens": all(t == library_tokens[0] for t in library_tokens)},
            "preflight": {"ranks_agree_on_tokens": all(t == tokens_of_ranks[0] for t in tokens_of_ranks),
                          "steps_compared": len(produced)},
            "workload": f"batch 1, context {C1_CONTEXT}, 64 layers, every projection and the vocabulary head "
                        f"column-split {world} ways"}


def run_ours(args):
    import torch

    from qwencore_b200 import engine as engine_module

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the decode step has no CPU path")
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    group = RankGroup("nccl", torch.device("cuda", local_rank))
    world, rank = group.world, group.rank

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

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()

    # ---- c = 32: end to end (host inputs, copies inside the timed region), then device only ----
    e2e_mine = time_worker_steps(engine, scheduler, group, stream, args.steps, ROWS)
    e2e_seconds = group.max_over_ranks(e2e_mine)
    device_mine = time_replays(engine, group, stream, args.steps, ROWS)
    device_seconds = group.max_over_ranks(device_mine)

    clocks = sampler.stop() if rank == 0 else None

    # ---- dominant kernel: all NVFP4 projections of the step, replayed back to back as one graph ----
    # (after the timed regions: the filtered graphs run on stale activations and leave the recurrent
    # state and the newest KV rows garbage)
    graph_phases = {}
    for prefix in ("gemm.", "attn.decode", "attn.prepare", "delta.scan", "delta.prepare", "delta.norm", "norm",
                   "lm_head", "sample", "pack", "embed"):
        try:
            ms, launched = engine.time_phases(ROWS, prefix, replays=5)
        except Exception:  # a phase that this build folds into another launches nothing
            continue
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
    # per phase what it streams and how fast (stepprofile's table, crates/qwc-engine/src/bin/
    # stepprofile.rs:86-183, :259-310): weights for the projections and the head, KV pages for
    # attention, state read and written for the recurrent update
    phase_bytes = {"gemm": traffic.gemv_bytes_per_step, "attn.decode": traffic.kv_bytes,
                   "delta.scan": traffic.state_bytes, "lm_head": traffic.weight_bytes - traffic.gemv_bytes_per_step}
    phase_rooflines = {}
    for label, streamed in phase_bytes.items():
        if label in graph_phases and graph_phases[label]["ms"] > 0:
            rate = streamed / (graph_phases[label]["ms"] * 1e-3) / 1e9
            phase_rooflines[label] = {"GB": round(streamed / 1e9, 4), "GB/s": round(rate, 1),
                                      "frac_of_measured_peak": round(rate / peak, 4),
                                      "share_of_step_ms": round(graph_phases[label]["ms"] /
                                                                (device_seconds / args.steps * 1e3), 4)}

    # ---- c = 1: the same engine, one row of context 2048 (the other half of the metric) ----
    c1_steps = max(args.steps, 20)
    single = engine_module.Scheduler(ROWS, 1 << 22, ROWS + 1, blocks_needed, PAGE)
    single.submit(1, C1_CONTEXT, c1_steps + args.warmup + 24)
    decoded = 0
    while decoded == 0:
        decoded, _ = engine.worker_step(single)
    for _ in range(max(args.warmup, 3)):
        engine.worker_step(single)
    c1_e2e = group.max_over_ranks(time_worker_steps(engine, single, group, stream, c1_steps, 1))
    c1_device = group.max_over_ranks(time_replays(engine, group, stream, c1_steps, 1))
    c1_gemm_ms, c1_gemm_launches = engine.time_phases(1, "gemm.", replays=5)
    c1_traffic = engine.traffic(1, float(C1_CONTEXT))
    c1_bytes = c1_traffic.weight_bytes + c1_traffic.state_bytes + c1_traffic.kv_bytes

    per_rank = group.gather([device_mine / args.steps * 1e3, e2e_mine / args.steps * 1e3, traffic.kv_bytes,
                             float(np.sum(contexts))])
    engine.close()

    latency = None
    if world > 1:
        try:
            latency = run_latency_mode(args, group, local_rank, c1_device / c1_steps * 1e3)
        except Exception as error:  # the throughput line must still be printed
            latency = {"error": f"{type(error).__name__}: {error}"}

    if rank != 0:
        group.close()
        return 0

    cpu_value, cpu_sample_text = cpu_tokens_per_second(os.cpu_count() or 1)
    tokens = ROWS * args.steps  # per rank
    line = base_line(args, world)
    line.update({
        "value": group.whole_job_rate(tokens, device_seconds),
        "ms_per_step": device_seconds / args.steps * 1e3,
        "e2e": {"value": group.whole_job_rate(tokens, e2e_seconds), "unit": "tok/s", "ms_per_step": e2e_seconds / args.steps * 1e3,
                "h2d_bytes_per_step": int((2 * ROWS + 4 * 2 * ROWS) * 4), "d2h_bytes_per_step": int((ROWS + 2) * 4),
                "path": "qwc_worker_step: scheduler.next_batch, layout check, H2D of slots/tokens/edits, graph "
                        "replay, D2H of sampled tokens and status words, scheduler.complete_batch"},
        "gpu_launches": int(traffic.kernel_launches_per_step * args.steps),
        "roofline": {"bound": "hbm", "kernel": "NVFP4 projection kernel (all NVFP4 projections of the step)",
                     "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "peak_kind": f"of {peak_kind}",
                     "traffic": bytes_per_launch * NCU_TRAFFIC_RATIO,
                     "traffic_source": "ncu dram__bytes_read.sum + dram__bytes_write.sum of one captured launch "
                                       "(34816 x 5120 at 32 rows) over its algorithmic bytes, applied to the "
                                       "average projection launch of the step",
                     "bytes_per_launch": bytes_per_launch, "us_per_launch": seconds_per_launch * 1e6,
                     "launches_timed": gemv_launches},
        "step_roofline": {"bytes_per_step": step_bytes, "weights": traffic.weight_bytes,
                          "state": traffic.state_bytes, "kv": traffic.kv_bytes,
                          "achieved_gbs": step_bytes / (device_seconds / args.steps) / 1e9,
                          "frac_of_measured_peak": step_bytes / (device_seconds / args.steps) / 1e9 / peak,
                          "frac_of_8tbs": step_bytes / (device_seconds / args.steps) / 8e12},
        "c1": {"workload": f"one row, context {C1_CONTEXT}, same engine and graph path",
               "value": group.whole_job_rate(c1_steps, c1_device), "unit": "tok/s",
               "ms_per_step": c1_device / c1_steps * 1e3,
               "e2e": {"value": group.whole_job_rate(c1_steps, c1_e2e), "unit": "tok/s",
                       "ms_per_step": c1_e2e / c1_steps * 1e3},
               "bytes_per_step": c1_bytes,
               "frac_of_measured_peak": c1_bytes / (c1_device / c1_steps) / 1e9 / peak,
               "frac_of_8tbs": c1_bytes / (c1_device / c1_steps) / 8e12,
               "projections_ms": round(c1_gemm_ms, 4), "projection_launches": c1_gemm_launches},
        "per_rank": [{"rank": i, "ms_per_step": round(v[0], 4), "e2e_ms_per_step": round(v[1], 4), "kv_bytes": v[2],
                      "context_tokens": v[3]} for i, v in enumerate(per_rank)],
        "phases_graph_ms_per_step": graph_phases,
        "phase_rooflines": phase_rooflines,
        "phases_eager_ms_per_step": {label: round(total[0], 4) for label, total in sorted(phases.items())},
        "cpu_baseline": {"value": cpu_value, "unit": "tok/s", "cores": os.cpu_count() or 1, "kind": "port",
                         "sample": cpu_sample_text},
        "clocks": clocks,
    })
    if latency is not None:
        line["latency_mode"] = latency
    print(json.dumps(line))
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
