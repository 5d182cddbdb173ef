"""Per-kernel timings of the decode-step kernels on one GPU.

    python -m qwencore_b200.microbench gemv 34816 5120 32
    python -m qwencore_b200.microbench swiglu 17408 5120 32
    python -m qwencore_b200.microbench delta 32 48
    python -m qwencore_b200.microbench attention uniform 32 128 2048
    python -m qwencore_b200.microbench attention loguniform 32 128 32768 --partitions 16
    python -m qwencore_b200.microbench all

Each case rotates over enough copies of its inputs that consecutive launches never find their
weights, states or pages in the 126 MB L2.  Timings are taken with CUDA events around a captured
CUDA graph of the launches, so that host launch cost (about 18 us per call through ctypes) does not
hide kernels shorter than that.  `--plain N` instead issues N eager launches and exits: that is the
form to put under a profiler (one kernel, a handful of launches, a few hundred MB on the device).

The byte counts are the algorithmic ones the step accounting uses: packed weights + block scales +
activations in and out for a projection; pages read + query/output for attention; state codes and
scales read and written + the per-row vectors for the recurrent update.
"""

from __future__ import annotations

import argparse
import json
import os

import numpy as np
import torch

from . import abi, ops, synth

L2_BYTES = 126 << 20


def measured_hbm_gbs() -> tuple[float, str]:
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    try:
        with open(path) as handle:
            return float(json.load(handle)["hbm_gbs"]), "measured"
    except (OSError, KeyError, ValueError):
        return 6650.0, "fallback"


def _dev(array):
    return torch.from_numpy(np.ascontiguousarray(array)).cuda()


def time_launches(launch, launches: int, plain: int) -> float:
    """Mean device time per launch in microseconds (graph replay), or 0.0 after `plain` eager launches."""
    if plain:
        for _ in range(plain):
            launch()
        torch.cuda.synchronize()
        return 0.0
    launch()  # one-time set-up of each launcher happens outside the capture
    torch.cuda.synchronize()
    stream = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream):
        with torch.cuda.graph(graph, stream=stream):
            for _ in range(launches):
                launch()
        for _ in range(3):
            graph.replay()
        start = torch.cuda.Event(enable_timing=True)
        stop = torch.cuda.Event(enable_timing=True)
        rounds = 5
        start.record(stream)
        for _ in range(rounds):
            graph.replay()
        stop.record(stream)
    torch.cuda.synchronize()
    return start.elapsed_time(stop) * 1e3 / (rounds * launches)


def report(label: str, microseconds: float, nbytes: int) -> dict:
    peak, kind = measured_hbm_gbs()
    if microseconds == 0.0:
        print(f"{label}: plain launches done, status {abi.lib.qwc_device_status()}")
        return {}
    gbs = nbytes / microseconds / 1e3
    print(f"{label}: {microseconds:8.2f} us  {gbs:7.0f} GB/s  {100.0 * gbs / peak:5.1f}% of {kind} HBM peak")
    return {"label": label, "us": microseconds, "gbs": gbs, "frac": gbs / peak}


def projection(out_features: int, in_features: int, rows: int, swiglu: bool = False, plain: int = 0,
               hint: bool = False, staged: bool = False, split: bool = False) -> dict:
    matrix_bytes = out_features * in_features // 2 + ops.block_scale_storage_len(out_features, in_features)
    per_launch = matrix_bytes * (2 if swiglu else 1)
    copies = max(2, -(-2 * L2_BYTES // per_launch)) if not plain else 2
    generator = torch.Generator(device="cuda")
    generator.manual_seed(0)
    linears = []
    for _ in range(copies * (2 if swiglu else 1)):
        packed = torch.randint(0, 256, (out_features, in_features // 2), dtype=torch.uint8, device="cuda",
                               generator=generator)
        scales = torch.randint(0x20, 0x40, (ops.block_scale_storage_len(out_features, in_features),),
                               dtype=torch.uint8, device="cuda", generator=generator)
        linears.append(ops.Linear(packed, scales, 1.0, out_features, in_features))
    x = _dev(synth.normal_bf16(0, "x", (rows, in_features)))
    y = torch.zeros((rows, out_features), dtype=torch.uint16, device="cuda")
    counter = [0]
    if staged:  # the equal-share kernel: activations already in the tensor core's operand layout
        staged_x = ops.new_staged(rows, in_features)
        ops.stage_activations(x, staged_x, rows, in_features)
        workspace = ops.new_streamk_workspace()
    if split:  # regular K split: fp32 slices for the consumer to sum
        sums = torch.zeros((16, rows, out_features), dtype=torch.float32, device="cuda")

    def launch():
        index = counter[0] % copies
        counter[0] += 1
        if hint:
            # the launch after this one reads the next copy
            after = (index + 1) % copies
            if swiglu:
                ops.prefetch_next(linears[2 * after], linears[2 * after + 1])
            else:
                ops.prefetch_next(linears[after])
        if split:
            ops.w4a16_split(linears[index], staged_x, sums, rows)
        elif staged and swiglu:
            ops.swiglu_w4a16_staged(linears[2 * index], linears[2 * index + 1], staged_x, y, None, rows, workspace)
        elif staged:
            ops.w4a16_staged(linears[index], staged_x, y, None, rows, workspace)
        elif swiglu:
            ops.swiglu_w4a16(linears[2 * index], linears[2 * index + 1], x, y, rows)
        else:
            linears[index].forward_w4a16(x, y, rows)

    microseconds = time_launches(launch, 4 * copies, plain)
    nbytes = (out_features * in_features // 2 + out_features * in_features // 16) * (2 if swiglu else 1)
    nbytes += rows * in_features * 2 + rows * out_features * 2
    name = ("swiglu" if swiglu else "gemv") + (" split" if split else " staged" if staged else "") + \
        (" +hint" if hint else "")
    return report(f"{name} N={out_features} K={in_features} M={rows}", microseconds, nbytes)


def delta(batch: int, value_heads: int, plain: int = 0) -> dict:
    abi.configure(value_heads, abi.get_shape()[1])
    capacity = batch + 1
    state_bytes = capacity * value_heads * 128 * 128
    # (for a profiler: four layers, 140 MB at 32 x 32 heads - more than L2 holds, so that the DRAM counters count)
    layers = max(2, -(-2 * L2_BYTES // state_bytes)) if not plain else 4
    states = [torch.randint(-127, 128, (capacity, value_heads, 128, 128), dtype=torch.int8, device="cuda")
              for _ in range(layers)]
    scales = [torch.rand((capacity, value_heads, 128), device="cuda") * 0.01 for _ in range(layers)]
    case = synth.delta_case(0, batch, value_heads)
    q, k, v, alpha, beta, kq = [_dev(case[name]) for name in ("q", "k", "v", "alpha", "beta", "kq")]
    slots = _dev(case["slots"])
    out = torch.zeros((batch, value_heads, 128), device="cuda")
    counter = [0]

    def launch():
        layer = counter[0] % layers
        counter[0] += 1
        ops.delta_decode_slots_packed(states[layer], scales[layer], slots, q, k, v, alpha, beta, kq, out, capacity,
                                      batch)

    microseconds = time_launches(launch, 2 * layers, plain)
    nbytes = 2 * (batch * value_heads * 16384 + batch * value_heads * 512) + batch * (2 * 16 + 2 * value_heads) * 512
    return report(f"delta batch={batch} heads={value_heads}", microseconds, nbytes)


def attention(contexts, page: int = 16, partitions: int | None = None, label: str = "", plain: int = 0) -> dict:
    contexts = np.asarray(contexts, dtype=np.uint32)
    rows = contexts.size
    blocks = (contexts + page - 1) // page
    pool_blocks = int(blocks.sum()) + 8
    max_blocks = int(blocks.max())
    order = np.random.default_rng(0).permutation(pool_blocks).astype(np.uint32)
    tables = np.zeros((rows, max_blocks), dtype=np.uint32)
    cursor = 0
    for row in range(rows):
        tables[row, : blocks[row]] = order[cursor : cursor + blocks[row]]
        cursor += blocks[row]
    layer_bytes = 2 * pool_blocks * 4 * page * 256
    layers = max(2, -(-2 * L2_BYTES // layer_bytes)) if not plain else 2
    caches = [(torch.randint(0, 0x70, (pool_blocks, 4, page, 256), dtype=torch.uint8, device="cuda"),
               torch.randint(0, 0x70, (pool_blocks, 4, page, 256), dtype=torch.uint8, device="cuda"))
              for _ in range(layers)]
    query = _dev(synth.normal_bf16(0, "q", (rows, 24, 256)))
    out = torch.zeros((rows, 24, 256), dtype=torch.uint16, device="cuda")
    count = partitions or ops.packed_partition_count(rows, int(contexts.max()))
    workspace = torch.zeros(max(16, ops.packed_workspace_bytes(rows, count)), dtype=torch.uint8, device="cuda")
    table_dev, context_dev = _dev(tables), _dev(contexts)
    counter = [0]

    def launch():
        layer = counter[0] % layers
        counter[0] += 1
        ops.gated_packed(query, None, caches[layer][0], caches[layer][1], table_dev, context_dev, max_blocks, out,
                         rows, 0, count, workspace, page)

    microseconds = time_launches(launch, 2 * layers, plain)
    nbytes = int(contexts.sum()) * 2048 + 2 * rows * 24 * 256 * 2
    return report(f"attention {label} rows={rows} partitions={count} tokens={int(contexts.sum())}", microseconds,
                  nbytes)


def contexts_for(kind: str, rows: int, low: int, high: int):
    if kind == "uniform":
        return synth.uniform_contexts(0, rows, low, high)
    if kind == "loguniform":
        return synth.log_uniform_contexts(0, rows, low, high)
    if kind == "fixed":
        return np.full((rows,), high, dtype=np.uint32)
    raise SystemExit(f"unknown context distribution {kind}")


def lm_head(vocab: int, hidden: int, rows: int, plain: int = 0, staged: bool = False) -> dict:
    """The FP8 vocabulary head: e4m3 weight bytes, one fp32 scale per row, fp32 logits (staged: the
    equal-share kernel with greedy sampling folded in, no logits written)."""
    generator = torch.Generator(device="cuda")
    generator.manual_seed(0)
    copies = max(2, -(-2 * L2_BYTES // (vocab * hidden))) if not plain else 2
    tables = [torch.randint(0x20, 0x48, (vocab, hidden), dtype=torch.uint8, device="cuda", generator=generator)
              for _ in range(copies)]
    scales = torch.full((vocab,), 0.01, dtype=torch.float32, device="cuda")
    x = _dev(synth.normal_bf16(0, "x", (rows, hidden)))
    logits = torch.zeros((rows, vocab), dtype=torch.float32, device="cuda")
    counter = [0]
    if staged:
        staged_x = ops.new_staged(rows, hidden)
        ops.stage_activations(x, staged_x, rows, hidden)
        workspace = ops.new_streamk_workspace()
        tokens = torch.zeros(rows, dtype=torch.int32, device="cuda")

    def launch():
        index = counter[0] % copies
        counter[0] += 1
        if staged:
            ops.fp8_lm_head_staged(tables[index], scales, staged_x, None, tokens, None, rows, hidden, vocab, workspace)
        else:
            ops.fp8_lm_head(tables[index], scales, x, logits, rows, hidden, vocab)

    microseconds = time_launches(launch, 4 * copies, plain)
    nbytes = vocab * hidden + vocab * 4 + rows * hidden * 2 + (0 if staged else rows * vocab * 4)
    return report(f"lm_head{' staged+sample' if staged else ''} V={vocab} K={hidden} M={rows}", microseconds, nbytes)


def main(argv=None) -> None:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("kernel", choices=["gemv", "swiglu", "lm_head", "delta", "attention", "projections", "step-projections", "all"])
    parser.add_argument("args", nargs="*")
    parser.add_argument("--partitions", type=int, default=0)
    parser.add_argument("--page", type=int, default=16)
    parser.add_argument("--hint", action="store_true",
                        help="name the next launch's weights to each projection (qwc_nvfp4_prefetch_next)")
    parser.add_argument("--plain", type=int, default=0, help="issue this many eager launches and exit (for a profiler)")
    parser.add_argument("--staged", action="store_true",
                        help="projections and the head through the equal-share kernel on staged activations")
    parser.add_argument("--split", action="store_true",
                        help="with --staged: the regular K split whose sum is left to the consumer")
    options = parser.parse_args(argv)
    if not torch.cuda.is_available():
        raise SystemExit("a CUDA device is required")
    torch.cuda.set_device(0)
    values = options.args
    if options.kernel in ("gemv", "swiglu"):
        n, k, m = (int(v) for v in values[:3])
        projection(n, k, m, swiglu=options.kernel == "swiglu", plain=options.plain, hint=options.hint,
                   staged=options.staged, split=options.split)
    elif options.kernel == "lm_head":
        lm_head(int(values[0]), int(values[1]), int(values[2]), plain=options.plain, staged=options.staged)
    elif options.kernel == "step-projections":
        # every projection as the decode step runs it on one GPU
        for rows in (1, 32):
            projection(12352, 5120, rows, staged=True, split=True)
            projection(5120, 4096, rows, staged=True, split=True)
            projection(14336, 5120, rows, staged=True, split=True)
            projection(5120, 6144, rows, staged=True, split=True)
            projection(17408, 5120, rows, swiglu=True, staged=True)
            projection(5120, 17408, rows, staged=True, split=True)
            lm_head(151936, 5120, rows, staged=True)
    elif options.kernel == "projections":
        for rows in (1, 8, 32):
            projection(34816, 5120, rows, staged=options.staged, hint=options.hint)
            projection(17408, 5120, rows, swiglu=True, staged=options.staged, hint=options.hint)
            projection(5120, 17408, rows, staged=options.staged, hint=options.hint)
            projection(12352, 5120, rows, staged=options.staged, hint=options.hint)
            projection(5120, 4096, rows, staged=options.staged, hint=options.hint)
            projection(14336, 5120, rows, staged=options.staged, hint=options.hint)
            projection(5120, 6144, rows, staged=options.staged, hint=options.hint)
            lm_head(151936, 5120, rows, staged=options.staged)
    elif options.kernel == "delta":
        delta(int(values[0]), int(values[1]), plain=options.plain)
    elif options.kernel == "attention":
        kind, rows, low, high = values[0], int(values[1]), int(values[2]), int(values[3])
        attention(contexts_for(kind, rows, low, high), page=options.page, partitions=options.partitions or None,
                  label=kind, plain=options.plain)
    else:
        for rows in (1, 8, 16, 32):
            projection(34816, 5120, rows)
        for rows in (1, 8, 32):
            projection(17408, 5120, rows, swiglu=True)
            projection(5120, 17408, rows)
            projection(12352, 5120, rows)
            projection(14336, 5120, rows)
            projection(5120, 6144, rows)
        for rows in (1, 8, 32):
            lm_head(151936, 5120, rows)
        for heads in (48, 32):
            delta(32, heads)
            delta(1, heads)
        attention(contexts_for("uniform", 32, 128, 2048), label="uniform-128-2048")
        attention(contexts_for("loguniform", 32, 128, 32768), label="loguniform-128-32768")
        attention(contexts_for("fixed", 1, 2048, 2048), label="single-2048")
        attention(contexts_for("fixed", 1, 32768, 32768), label="single-32768")
    print("device status", abi.lib.qwc_device_status())


if __name__ == "__main__":
    main()
