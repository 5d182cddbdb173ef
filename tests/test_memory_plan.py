"""The memory plan around the two pools (crates/qwc-core/src/memory.rs:99-218 and its tests :220-328;
crates/qwc-runtime/src/cache.rs:360-378, :596-622 and its tests :657-690), stated for one B200 and the
engine's shapes.  Host arithmetic: no GPU."""

from qwencore_b200.engine import Budget, CacheGeometry, CacheManager, RuntimeError_, default_config, weight_bytes

GB = 1_000_000_000
GIB = 1 << 30


def reference_shape():
    """The checkpoint's own shape: 48 value heads, pages of 64 tokens."""
    return CacheGeometry.for_config(default_config(delta_value_heads=48, kv_page_size=64))


def test_geometry_of_the_benchmark_engine(built_library):
    geometry = CacheGeometry.for_config(default_config())
    # 16 layers x 4 KV heads x 256 x (K and V), one byte each (arch.rs:113-115)
    assert geometry.kv_bytes_per_token == 32768
    assert geometry.block_size == 16 and geometry.kv_bytes_per_block() == 16 * 32768
    # 48 layers x 32 heads x 128 rows x (128 codes + one fp32 scale) + the fp32 conv window of 8192 channels
    assert geometry.state_bytes_per_slot == 48 * 32 * 128 * (128 + 4) + 48 * 8192 * 3 * 4
    assert geometry.bytes_per_seq(17) == geometry.state_bytes_per_slot + 2 * geometry.kv_bytes_per_block()


def test_state_dominates_below_crossover(built_library):
    """memory.rs:251-272: an int8 state equals its KV pages at about 1.3K tokens on the checkpoint's shape."""
    reference = reference_shape()
    assert reference.state_bytes_per_slot == 37_748_736 + 37_748_736 // 128 * 4 + 48 * 10240 * 3 * 4
    crossover = reference.crossover_tokens()
    assert 1000 < crossover < 1700
    short = 512
    assert reference.state_bytes_per_slot > -(-short // 64) * reference.kv_bytes_per_block()
    # with 32 value heads the state is a third smaller and the break-even point that much nearer
    ours = CacheGeometry.for_config(default_config())
    assert 0.6 * crossover < ours.crossover_tokens() < 0.75 * crossover


def test_weight_bytes_of_the_benchmark_engine(built_library):
    config = default_config()
    resident = weight_bytes(config)
    # what a step streams (12.843 GB of projections + 0.779 GB of vocabulary head) plus the embedding table
    assert 14.3 * GB < resident < 14.5 * GB
    # under a column split a rank keeps its rows of every projection and of the head, and the whole
    # embedding table
    half = weight_bytes(default_config(split_size=2, max_batch=1))
    table = config.vocab * config.hidden + 4 * config.vocab
    assert abs((half - table) - (resident - table) / 2) < 0.01 * resident


def test_benchmark_matrix_feasibility(built_library):
    """memory.rs:283-296, on 180 GB: every cell of the benchmark matrix fits with room to spare."""
    geometry = CacheGeometry.for_config(default_config())
    budget = Budget.b200(weight_bytes(default_config()), 4 * GIB)
    assert 150 * GIB < budget.cache_available() < 170 * GIB
    for concurrency, context in [(1, 512), (1, 16 * 1024), (32, 2048), (32, 32 * 1024)]:
        assert budget.fits(geometry, concurrency, context)
    assert not budget.fits(geometry, 32, 256 * 1024)
    # 32 rows of the longest benchmark context take 1.0 + 34.4 GB
    assert abs(32 * geometry.bytes_per_seq(32768) - (32 * 30_670_848 + 32 * 32768 * 32768)) == 0


def test_long_context_concurrency_limits(built_library):
    """memory.rs:298-314: what bounds concurrency at 32K is the KV pool."""
    geometry = CacheGeometry.for_config(default_config())
    budget = Budget.b200(weight_bytes(default_config()), 4 * GIB)
    at_32k = budget.max_concurrency(geometry, 32 * 1024)
    assert 140 <= at_32k <= 170
    assert budget.max_concurrency(geometry, 2048) > 10 * at_32k
    # max_context is the inverse: that many sequences of that length fit, one page more does not
    for concurrency in (1, 8, 32, at_32k):
        context = budget.max_context(geometry, concurrency)
        assert budget.fits(geometry, concurrency, context - context % 16)
        assert not budget.fits(geometry, concurrency, context + 16)
    assert budget.max_context(geometry, 0) == 0


def test_a_spent_budget_leaves_nothing(built_library):
    geometry = CacheGeometry.for_config(default_config())
    budget = Budget.b200(200 * GIB, 4 * GIB)
    assert budget.cache_available() == 0 and budget.max_concurrency(geometry, 1024) == 0
    manager = CacheManager.from_budget(budget, geometry, 1024)
    assert manager.state_capacity() == 0 and manager.kv_capacity() == 0


def test_budget_split_matches_memory_model(built_library):
    """cache.rs:680-690: the slots of from_budget are the independent concurrency estimate, and the rest
    of the budget went to pages."""
    geometry = CacheGeometry.for_config(default_config())
    budget = Budget.b200(weight_bytes(default_config()), 4 * GIB)
    for context in (4096, 8192, 32768):
        manager = CacheManager.from_budget(budget, geometry, context)
        assert manager.state_capacity() == budget.max_concurrency(geometry, context)
        taken = (manager.state_capacity() * geometry.state_bytes_per_slot
                 + manager.kv_capacity() * geometry.kv_bytes_per_block())
        assert 0 <= budget.cache_available() - taken < geometry.kv_bytes_per_block()
        # enough pages for every slot at the target context
        assert manager.kv_capacity() >= manager.state_capacity() * (context // 16)


def test_bottleneck_flips_with_context_length(built_library):
    """cache.rs:657-678: with one pool layout short requests run out of state slots, long ones of pages."""
    short = CacheManager(64, 100, 64)
    admitted = 0
    try:
        while True:
            short.admit(admitted, 64)
            admitted += 1
    except RuntimeError_:
        pass
    pressure = short.pressure()
    assert pressure["bottleneck"] == "state slots" and pressure["states"] == 1.0 and pressure["worst"] == 1.0
    assert abs(pressure["kv"] - 0.64) < 1e-12

    long = CacheManager(64, 100, 64)
    admitted = 0
    try:
        while True:
            long.admit(admitted, 640)
            admitted += 1
    except RuntimeError_:
        pass
    pressure = long.pressure()
    assert pressure["bottleneck"] == "KV blocks" and pressure["kv"] == 1.0
    assert abs(pressure["states"] - 10 / 64) < 1e-12
