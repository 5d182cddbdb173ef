"""The allocation-free attention entry point against the workspace-taking one (GPU).

Collected last on purpose: a run that stops at the first failure has then already run every
other test.  The entry point serves callers that cannot allocate device memory - a process
whose memory budget was fully handed out at start-up, or a binding without an allocator - by
keeping the split-context partials in a scratch array inside the library.  The scratch is
shared by all calls and keeps the previous call's contents, so the check is made on two calls
in a row with different shapes: the second must not be disturbed by what the first left.
"""

import numpy as np
import pytest

from oracle import oracle
from qwencore_b200 import synth

pytestmark = pytest.mark.gpu


def dev(torch, array):
    return torch.from_numpy(np.ascontiguousarray(array)).cuda()


def run_both(torch, ops, case, page_size, partitions):
    """Output of the existing entry point (caller-allocated workspace) and of the no-alloc one."""
    batch = case["contexts"].size
    tensors = {name: None if case[name] is None else dev(torch, case[name])
               for name in ("query", "gate_projection", "key_cache", "value_cache", "block_tables", "contexts",
                            "k_scale", "v_scale")}
    workspace = torch.zeros(max(16, ops.packed_workspace_bytes(batch, partitions)), dtype=torch.uint8, device="cuda")
    expected = dev(torch, np.zeros((batch, 24, 256), dtype=np.uint16))
    ops.gated_packed(tensors["query"], tensors["gate_projection"], tensors["key_cache"], tensors["value_cache"],
                     tensors["block_tables"], tensors["contexts"], case["max_blocks"], expected, batch, 0, partitions,
                     workspace, page_size, tensors["k_scale"], tensors["v_scale"])
    actual = dev(torch, np.zeros((batch, 24, 256), dtype=np.uint16))
    ops.gated_packed_noalloc(tensors["query"], tensors["gate_projection"], tensors["key_cache"],
                             tensors["value_cache"], tensors["block_tables"], tensors["contexts"], case["max_blocks"],
                             actual, batch, 0, partitions, page_size, tensors["k_scale"], tensors["v_scale"])
    torch.cuda.synchronize()
    return expected.cpu().numpy(), actual.cpu().numpy()


def test_noalloc_attention_matches_workspace_entry_on_two_calls_in_a_row(cuda, built_library):
    from qwencore_b200 import abi, ops

    torch = cuda
    limit = abi.lib.qwc_paged_attention_packed_noalloc_max_pairs()
    assert limit == 512

    # first call: many partitions over long rows fills a large part of the scratch
    first = synth.attention_case(41, [3000, 1500, 2047, 900, 5000, 64], page_size=16, with_gate=True, scaled=True)
    expected, actual = run_both(torch, ops, first, 16, 64)  # 6 rows x 64 partitions = 384 pairs
    assert np.array_equal(actual, expected)  # same kernels, same order of operations: bit-identical
    want = oracle.paged_attention_fp8(first["query"], first["gate_projection"], first["key_cache"],
                                      first["value_cache"], first["block_tables"], first["contexts"],
                                      first["max_blocks"], batch=6, page_size=16, k_scale=first["k_scale"],
                                      v_scale=first["v_scale"])
    got = synth.bf16_value(actual)
    rms = np.sqrt(np.mean(want.astype(np.float64) ** 2))
    assert np.all(np.abs(got - want) <= 1e-2 * rms + 2.0 ** -7 * np.abs(want))

    # second call, straight after: other shape, other page size, fewer partitions - it reads only
    # what it wrote, whatever the first call left behind
    second = synth.attention_case(42, [70, 129, 1, 640], page_size=64, with_gate=False)
    expected, actual = run_both(torch, ops, second, 64, 5)
    assert np.array_equal(actual, expected)

    # beyond the built-in scratch the call is refused before any launch
    code = abi.lib.qwc_paged_attention_packed_fp8_noalloc(1, 0, 1, 1, 1, 1, 0, 0, 1, 32, 0, 8, 16, 0, 17, 0.0625, 0)
    assert code == abi.CUDA_ERROR_INVALID_VALUE
    assert abi.lib.qwc_device_status() == 0
