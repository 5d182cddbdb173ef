"""ctypes front-end of `include/qwc_engine.h`: cache manager, scheduler, batch layout, executor.

The classes keep the reference's names and error behaviour (crates/qwc-runtime/src/cache.rs,
scheduler.rs, layout.rs; crates/qwc-engine/src/executor.rs): a rejected operation raises the
matching exception with the reference's enum discriminant as `code`.
"""

from __future__ import annotations

import ctypes
from ctypes import POINTER, byref, c_char, c_char_p, c_double, c_float, c_int, c_longlong, c_size_t, c_uint32, c_void_p

import numpy as np

from . import abi

lib = abi.lib

REJECTED = {1: "NoStateSlot", 2: "NoKvBlocks", 3: "AlreadyAdmitted", 4: "UnknownSequence", 5: "NothingToRollback"}
SUBMIT_ERROR = {1: "Duplicate", 2: "EmptyPrompt", 3: "NoOutputTokens", 4: "NoStateCapacity", 5: "ContextTooLong"}
SCHEDULER_ERROR = {1: "BatchInFlight", 2: "NoBatchInFlight", 3: "SequenceInFlight", 4: "InvalidStopped",
                   5: "DuplicateStopped", 6: "Invariant", 7: "Cache"}
LAYOUT_ERROR = {1: "MissingSequence", 2: "DuplicateSequence", 3: "InvalidPrefillRange", 4: "MissingKvBlocks",
                5: "IntegerOverflow"}


class RuntimeError_(Exception):
    def __init__(self, kind: str, code: int, names: dict):
        super().__init__(f"{kind}::{names.get(code, code)}")
        self.kind = kind
        self.code = code
        self.name = names.get(code, str(code))


class PrefillChunk(ctypes.Structure):
    _fields_ = [("id", c_uint32), ("offset", c_uint32), ("tokens", c_uint32)]


class Completion(ctypes.Structure):
    _fields_ = [("id", c_uint32), ("generated_tokens", c_uint32), ("reason", c_uint32)]


class EngineConfig(ctypes.Structure):
    _fields_ = [("num_layers", c_int), ("full_attention_interval", c_int), ("hidden", c_int),
                ("intermediate", c_int), ("vocab", c_int), ("delta_value_heads", c_int), ("kv_page_size", c_int),
                ("max_batch", c_int), ("max_context", c_int), ("kv_pool_blocks", c_int), ("state_slots", c_int),
                ("seed", ctypes.c_ulonglong), ("split_rank", c_int), ("split_size", c_int), ("use_graph", c_int),
                ("attention_partitions", c_int), ("write_logits", c_int), ("exchange", c_int),
                ("memory_limit", ctypes.c_ulonglong)]


class StepTraffic(ctypes.Structure):
    _fields_ = [("weight_bytes", c_double), ("state_bytes", c_double), ("kv_bytes", c_double),
                ("gemv_bytes_per_step", c_double), ("gemv_launches_per_step", c_int),
                ("kernel_launches_per_step", c_int)]


class PhaseTime(ctypes.Structure):
    _fields_ = [("label", c_char * 24), ("milliseconds", c_float), ("launches", c_int)]


P = c_void_p
ENGINE_SYMBOLS = {
    "qwc_cache_new": (P, [c_size_t, c_size_t, c_size_t]),
    "qwc_cache_free": (None, [P]),
    "qwc_cache_admit": (c_int, [P, c_uint32, c_size_t]),
    "qwc_cache_append_token": (c_int, [P, c_uint32]),
    "qwc_cache_rollback_token": (c_int, [P, c_uint32]),
    "qwc_cache_release": (None, [P, c_uint32]),
    "qwc_cache_sequence": (c_int, [P, c_uint32, POINTER(c_uint32), POINTER(c_size_t), P, c_size_t, POINTER(c_size_t)]),
    "qwc_cache_enable_prefix_cache": (None, [P, c_size_t]),
    "qwc_cache_admit_prompt": (c_int, [P, c_uint32, P, c_size_t, P]),
    "qwc_cache_finish_restore": (None, [P, c_uint32]),
    "qwc_cache_reserve_snapshot": (c_longlong, [P]),
    "qwc_cache_cancel_snapshot": (None, [P, c_uint32]),
    "qwc_cache_commit_snapshot": (None, [P, c_uint32, c_uint32, P, c_size_t]),
    "qwc_cache_prefix_entries": (c_size_t, [P]),
    "qwc_cache_prefix_stats": (None, [P, P]),
    "qwc_cache_free_blocks": (c_size_t, [P]),
    "qwc_cache_states_in_use": (c_size_t, [P]),
    "qwc_cache_active": (c_size_t, [P]),
    "qwc_cache_last_shortage": (None, [P, POINTER(c_size_t), POINTER(c_size_t)]),
    "qwc_cache_drain_edits": (c_size_t, [P, P, c_size_t]),
    "qwc_cache_geometry_for": (None, [P, P]),
    "qwc_engine_weight_bytes": (ctypes.c_uint64, [P]),
    "qwc_budget_b200": (None, [ctypes.c_uint64, ctypes.c_uint64, P]),
    "qwc_budget_cache_available": (ctypes.c_uint64, [P]),
    "qwc_budget_max_concurrency": (c_size_t, [P, P, c_size_t]),
    "qwc_budget_max_context": (c_size_t, [P, P, c_size_t]),
    "qwc_budget_fits": (c_int, [P, P, c_size_t, c_size_t]),
    "qwc_cache_geometry_crossover_tokens": (c_size_t, [P]),
    "qwc_cache_from_budget": (P, [P, P, c_size_t]),
    "qwc_cache_state_capacity": (c_size_t, [P]),
    "qwc_cache_kv_capacity": (c_size_t, [P]),
    "qwc_cache_pressure": (None, [P, POINTER(c_double), POINTER(c_double)]),
    "qwc_scheduler_new": (P, [c_size_t, c_size_t, c_size_t, c_size_t, c_size_t]),
    "qwc_scheduler_free": (None, [P]),
    "qwc_scheduler_submit": (c_int, [P, c_uint32, c_size_t, c_size_t]),
    "qwc_scheduler_next_batch": (c_int, [P, P, POINTER(c_size_t), P, POINTER(c_size_t)]),
    "qwc_scheduler_complete_batch": (c_int, [P, P, c_size_t, P, c_size_t, POINTER(c_size_t)]),
    "qwc_scheduler_complete_batch_multi": (c_int, [P, P, c_size_t, P, P, c_size_t, P, c_size_t, POINTER(c_size_t)]),
    "qwc_scheduler_enable_prefix_cache": (None, [P, c_size_t]),
    "qwc_scheduler_submit_prompt": (c_int, [P, c_uint32, P, c_size_t, c_size_t, c_size_t]),
    "qwc_scheduler_batch_prefix_ops": (c_int, [P, P, POINTER(c_size_t), P, POINTER(c_size_t)]),
    "qwc_scheduler_abort_batch": (c_int, [P]),
    "qwc_scheduler_cancel": (c_int, [P, c_uint32, POINTER(c_int)]),
    "qwc_scheduler_remaining_tokens": (c_longlong, [P, c_uint32]),
    "qwc_scheduler_waiting": (c_size_t, [P]),
    "qwc_scheduler_active": (c_size_t, [P]),
    "qwc_scheduler_committed_kv_blocks": (c_size_t, [P]),
    "qwc_scheduler_cache": (P, [P]),
    "qwc_layout_build": (c_int, [P, P, c_size_t, P, c_size_t, P, P, P, P, P, P, P, c_size_t, POINTER(c_uint32)]),
    "qwc_engine_default_config": (None, [POINTER(EngineConfig)]),
    "qwc_engine_create": (c_int, [POINTER(EngineConfig), POINTER(P)]),
    "qwc_engine_destroy": (None, [P]),
    "qwc_engine_memory_usage": (None, [P, POINTER(c_size_t), POINTER(c_size_t)]),
    "qwc_engine_nccl_unique_id": (c_int, [P]),
    "qwc_engine_init_split": (c_int, [P, P]),
    "qwc_engine_exchange_handle": (c_int, [P, P]),
    "qwc_engine_open_peers": (c_int, [P, P, c_int]),
    "qwc_engine_exchange_waits": (c_int, [P, P, c_int]),
    "qwc_engine_profile_waits": (c_int, [P, c_int]),
    "qwc_engine_tensor": (c_int, [P, c_char_p, c_int, POINTER(P), POINTER(c_size_t)]),
    "qwc_engine_trace_layers": (c_int, [P, c_int]),
    "qwc_engine_set_weight_global_scale": (c_int, [P, c_char_p, c_int, c_float]),
    "qwc_engine_weight_global_scale": (c_int, [P, c_char_p, c_int, POINTER(c_float)]),
    "qwc_engine_read": (c_int, [P, c_char_p, c_int, P, c_size_t]),
    "qwc_engine_write": (c_int, [P, c_char_p, c_int, P, c_size_t]),
    "qwc_engine_traffic": (None, [P, c_int, c_double, POINTER(StepTraffic)]),
    "qwc_engine_apply_edits": (c_int, [P, P, c_size_t]),
    "qwc_engine_copy_kv_block": (c_int, [P, c_uint32, c_uint32]),
    "qwc_engine_decode": (c_int, [P, P, P, P, c_size_t, c_int, P]),
    "qwc_engine_replay": (c_int, [P, c_int]),
    "qwc_engine_stream": (P, [P]),
    "qwc_engine_profile_step": (c_int, [P, c_int, POINTER(PhaseTime), c_int]),
    "qwc_engine_time_phases": (c_int, [P, c_int, ctypes.c_char_p, c_int, POINTER(ctypes.c_float), POINTER(c_int)]),
    "qwc_worker_new": (P, [P, P, P, P, P, P, c_size_t]),
    "qwc_worker_free": (None, [P]),
    "qwc_worker_submit": (None, [P, c_uint32, P, c_size_t, c_size_t, c_size_t, c_int]),
    "qwc_worker_abandon": (None, [P, c_uint32]),
    "qwc_worker_shutdown": (None, [P]),
    "qwc_worker_iterate": (c_int, [P, POINTER(c_int)]),
    "qwc_worker_run": (c_int, [P]),
    "qwc_worker_jobs": (c_size_t, [P]),
    "qwc_worker_steps": (ctypes.c_uint64, [P]),
    "qwc_worker_aborted_steps": (ctypes.c_uint64, [P]),
    "qwc_worker_step": (c_int, [P, P, c_uint32, POINTER(c_size_t), P, c_size_t, POINTER(c_size_t)]),
}
for _name, (_restype, _argtypes) in ENGINE_SYMBOLS.items():
    _function = getattr(lib, _name)
    _function.restype = _restype
    _function.argtypes = _argtypes


def _u32(values) -> np.ndarray:
    return np.ascontiguousarray(values, dtype=np.uint32)


class Admission(ctypes.Structure):
    _fields_ = [("reused", c_size_t), ("has_restore", c_int), ("snapshot", c_uint32), ("copy", c_int),
                ("copy_from", c_uint32), ("copy_to", c_uint32)]


class CacheGeometry(ctypes.Structure):
    """What one sequence costs (crates/qwc-core/src/memory.rs:99-157)."""
    _fields_ = [("kv_bytes_per_token", ctypes.c_uint64), ("state_bytes_per_slot", ctypes.c_uint64),
                ("block_size", c_size_t)]

    @classmethod
    def for_config(cls, config: "EngineConfig") -> "CacheGeometry":
        geometry = cls()
        lib.qwc_cache_geometry_for(byref(config), byref(geometry))
        return geometry

    def kv_bytes_per_block(self) -> int:
        return self.kv_bytes_per_token * self.block_size

    def bytes_per_seq(self, context: int) -> int:
        return self.state_bytes_per_slot + -(-context // self.block_size) * self.kv_bytes_per_block()

    def crossover_tokens(self) -> int:
        return lib.qwc_cache_geometry_crossover_tokens(byref(self))


class Budget(ctypes.Structure):
    """What a GPU has left for the two pools (crates/qwc-core/src/memory.rs:163-218)."""
    _fields_ = [("total_vram", ctypes.c_uint64), ("reserved", ctypes.c_uint64), ("weights", ctypes.c_uint64),
                ("workspace", ctypes.c_uint64)]

    @classmethod
    def b200(cls, weights: int, workspace: int) -> "Budget":
        budget = cls()
        lib.qwc_budget_b200(weights, workspace, byref(budget))
        return budget

    def cache_available(self) -> int:
        return lib.qwc_budget_cache_available(byref(self))

    def max_concurrency(self, geometry: CacheGeometry, context: int) -> int:
        return lib.qwc_budget_max_concurrency(byref(self), byref(geometry), context)

    def max_context(self, geometry: CacheGeometry, concurrency: int) -> int:
        return lib.qwc_budget_max_context(byref(self), byref(geometry), concurrency)

    def fits(self, geometry: CacheGeometry, concurrency: int, context: int) -> bool:
        return bool(lib.qwc_budget_fits(byref(self), byref(geometry), concurrency, context))


def weight_bytes(config: "EngineConfig") -> int:
    """Resident weight bytes of the engine a config describes (this rank's share under a split)."""
    return lib.qwc_engine_weight_bytes(byref(config))


class PrefixRestoreOp(ctypes.Structure):
    _fields_ = [("id", c_uint32), ("state_slot", c_uint32), ("snapshot", c_uint32), ("copy", c_uint32),
                ("copy_from", c_uint32), ("copy_to", c_uint32)]


class PrefixSaveOp(ctypes.Structure):
    _fields_ = [("id", c_uint32), ("state_slot", c_uint32), ("snapshot", c_uint32)]


class CacheManager:
    """crates/qwc-runtime/src/cache.rs:300-449,571-594"""

    def __init__(self, state_slots: int, kv_blocks: int, block_size: int, _borrowed=None):
        if _borrowed is not None:
            self._handle, self._owned = _borrowed, False
            return
        if block_size <= 0:
            raise ValueError("KV block size must be positive")  # cache.rs:124
        self._handle = lib.qwc_cache_new(state_slots, kv_blocks, block_size)
        self._owned = True

    def __del__(self):
        if getattr(self, "_owned", False) and self._handle:
            lib.qwc_cache_free(self._handle)
            self._handle = None

    @classmethod
    def from_budget(cls, budget: Budget, geometry: CacheGeometry, target_context: int) -> "CacheManager":
        """cache.rs:360-378: as many slots as sequences of the target context fit, the rest as pages."""
        manager = cls(0, 0, 1, _borrowed=lib.qwc_cache_from_budget(byref(budget), byref(geometry), target_context))
        manager._owned = True
        return manager

    def state_capacity(self) -> int:
        return lib.qwc_cache_state_capacity(self._handle)

    def kv_capacity(self) -> int:
        return lib.qwc_cache_kv_capacity(self._handle)

    def pressure(self) -> dict:
        """cache.rs:596-622: utilisation of both pools and which one binds."""
        states, kv = c_double(), c_double()
        lib.qwc_cache_pressure(self._handle, byref(states), byref(kv))
        return {"states": states.value, "kv": kv.value,
                "bottleneck": "state slots" if states.value >= kv.value else "KV blocks",
                "worst": max(states.value, kv.value)}

    def _check(self, code: int) -> None:
        if code != 0:
            raise RuntimeError_("Rejected", code, REJECTED)

    def admit(self, seq_id: int, prompt_tokens: int) -> None:
        self._check(lib.qwc_cache_admit(self._handle, seq_id, prompt_tokens))

    def append_token(self, seq_id: int) -> None:
        self._check(lib.qwc_cache_append_token(self._handle, seq_id))

    def rollback_token(self, seq_id: int) -> None:
        self._check(lib.qwc_cache_rollback_token(self._handle, seq_id))

    def release(self, seq_id: int) -> None:
        lib.qwc_cache_release(self._handle, seq_id)

    def sequence(self, seq_id: int):
        slot, tokens, count = c_uint32(), c_size_t(), c_size_t()
        if lib.qwc_cache_sequence(self._handle, seq_id, byref(slot), byref(tokens), None, 0, byref(count)) != 0:
            return None
        blocks = np.zeros(max(1, count.value), dtype=np.uint32)
        lib.qwc_cache_sequence(self._handle, seq_id, byref(slot), byref(tokens), blocks.ctypes.data_as(P),
                               blocks.size, byref(count))
        return {"state_slot": slot.value, "tokens": tokens.value, "blocks": blocks[:count.value].tolist()}

    # ---- prefix cache (cache.rs:328-365, :451-569) ----
    def enable_prefix_cache(self, snapshots: int) -> None:
        lib.qwc_cache_enable_prefix_cache(self._handle, snapshots)

    def admit_prompt(self, seq_id: int, prompt) -> dict:
        """{"reused": tokens, "restore": None | {"snapshot": n, "copy_block": None | (from, to)}}"""
        tokens = _u32(list(prompt))
        admission = Admission()
        self._check(lib.qwc_cache_admit_prompt(self._handle, seq_id, tokens.ctypes.data_as(P), tokens.size,
                                               byref(admission)))
        restore = None
        if admission.has_restore:
            restore = {"snapshot": admission.snapshot,
                       "copy_block": (admission.copy_from, admission.copy_to) if admission.copy else None}
        return {"reused": admission.reused, "restore": restore}

    def finish_restore(self, snapshot: int) -> None:
        lib.qwc_cache_finish_restore(self._handle, snapshot)

    def reserve_snapshot(self):
        value = lib.qwc_cache_reserve_snapshot(self._handle)
        return None if value < 0 else int(value)

    def cancel_snapshot(self, snapshot: int) -> None:
        lib.qwc_cache_cancel_snapshot(self._handle, snapshot)

    def commit_snapshot(self, snapshot: int, seq_id: int, tokens) -> None:
        values = _u32(list(tokens))
        lib.qwc_cache_commit_snapshot(self._handle, snapshot, seq_id, values.ctypes.data_as(P), values.size)

    def prefix_entries(self) -> int:
        return lib.qwc_cache_prefix_entries(self._handle)

    def prefix_stats(self) -> dict:
        values = (ctypes.c_uint64 * 4)()
        lib.qwc_cache_prefix_stats(self._handle, values)
        return dict(zip(("lookups", "hits", "reused_tokens", "evictions"), (int(v) for v in values)))

    def free_blocks(self) -> int:
        return lib.qwc_cache_free_blocks(self._handle)

    def states_in_use(self) -> int:
        return lib.qwc_cache_states_in_use(self._handle)

    def active(self) -> int:
        return lib.qwc_cache_active(self._handle)

    def last_shortage(self):
        need, free = c_size_t(), c_size_t()
        lib.qwc_cache_last_shortage(self._handle, byref(need), byref(free))
        return need.value, free.value

    def drain_edits(self, capacity: int = 1 << 16) -> np.ndarray:
        """Pending device-table edits as u32[n, 4] = (slot, index, value, kind)."""
        buffer = np.zeros((capacity, 4), dtype=np.uint32)
        pending = lib.qwc_cache_drain_edits(self._handle, buffer.ctypes.data_as(P), capacity)
        if pending > capacity:
            raise OverflowError("edit buffer too small")
        return buffer[:pending].copy()


class Scheduler:
    """crates/qwc-runtime/src/scheduler.rs:190-668"""

    def __init__(self, max_num_seqs: int, max_num_batched_tokens: int, state_slots: int, kv_blocks: int,
                 block_size: int = 64):
        if max_num_seqs <= 0 or max_num_batched_tokens <= 0:
            raise ValueError("batch limits must be positive")  # scheduler.rs:22-30
        self._handle = lib.qwc_scheduler_new(max_num_seqs, max_num_batched_tokens, state_slots, kv_blocks, block_size)
        self.max_num_seqs = max_num_seqs
        self.cache = CacheManager(0, 0, 1, _borrowed=lib.qwc_scheduler_cache(self._handle))

    def __del__(self):
        if getattr(self, "_handle", None):
            lib.qwc_scheduler_free(self._handle)
            self._handle = None

    def submit(self, seq_id: int, prompt_tokens: int, max_new_tokens: int) -> None:
        code = lib.qwc_scheduler_submit(self._handle, seq_id, prompt_tokens, max_new_tokens)
        if code != 0:
            raise RuntimeError_("SubmitError", code, SUBMIT_ERROR)

    def next_batch(self):
        decode = np.zeros(self.max_num_seqs, dtype=np.uint32)
        prefill = (PrefillChunk * self.max_num_seqs)()
        n_decode, n_prefill = c_size_t(), c_size_t()
        code = lib.qwc_scheduler_next_batch(self._handle, decode.ctypes.data_as(P), byref(n_decode), prefill,
                                            byref(n_prefill))
        if code != 0:
            raise RuntimeError_("SchedulerError", code, SCHEDULER_ERROR)
        if n_decode.value == 0 and n_prefill.value == 0:
            return None
        restores = (PrefixRestoreOp * self.max_num_seqs)()
        saves = (PrefixSaveOp * self.max_num_seqs)()
        n_restores, n_saves = c_size_t(), c_size_t()
        code = lib.qwc_scheduler_batch_prefix_ops(self._handle, restores, byref(n_restores), saves, byref(n_saves))
        if code != 0:
            raise RuntimeError_("SchedulerError", code, SCHEDULER_ERROR)
        return {"decode": decode[:n_decode.value].tolist(),
                "prefill": [(c.id, c.offset, c.tokens) for c in prefill[:n_prefill.value]],
                "restores": [{"id": op.id, "state_slot": op.state_slot, "snapshot": op.snapshot,
                              "copy_block": (op.copy_from, op.copy_to) if op.copy else None}
                             for op in restores[:n_restores.value]],
                "saves": [{"id": op.id, "state_slot": op.state_slot, "snapshot": op.snapshot}
                          for op in saves[:n_saves.value]]}

    def enable_prefix_cache(self, snapshots: int) -> None:
        """scheduler.rs:226-228"""
        lib.qwc_scheduler_enable_prefix_cache(self._handle, snapshots)

    def submit_prompt(self, seq_id: int, prompt, max_new_tokens: int, snapshot_at: int) -> None:
        """scheduler.rs:237-261: the request with its prompt tokens; `snapshot_at` is the length of the
        prefix worth caching (the prefill chunk is cut there)."""
        prompt = _u32(list(prompt))
        if snapshot_at > prompt.size:
            raise ValueError("the snapshot point lies beyond the prompt")
        code = lib.qwc_scheduler_submit_prompt(self._handle, seq_id, prompt.ctypes.data_as(P), prompt.size,
                                               max_new_tokens, snapshot_at)
        if code != 0:
            raise RuntimeError_("SubmitError", code, SUBMIT_ERROR)

    def complete_batch(self, stopped=()):
        stopped = _u32(list(stopped))
        done = (Completion * self.max_num_seqs)()
        count = c_size_t()
        code = lib.qwc_scheduler_complete_batch(self._handle, stopped.ctypes.data_as(P), stopped.size, done,
                                                self.max_num_seqs, byref(count))
        if code != 0:
            raise RuntimeError_("SchedulerError", code, SCHEDULER_ERROR)
        return [(c.id, c.generated_tokens, "Stopped" if c.reason else "Length") for c in done[:count.value]]

    def complete_batch_multi(self, stopped=(), produced=()):
        """`produced`: (sequence, tokens) pairs for sequences that produced more than one token."""
        stopped = _u32(list(stopped))
        ids = _u32([p[0] for p in produced])
        tokens = _u32([p[1] for p in produced])
        done = (Completion * self.max_num_seqs)()
        count = c_size_t()
        code = lib.qwc_scheduler_complete_batch_multi(self._handle, stopped.ctypes.data_as(P), stopped.size,
                                                      ids.ctypes.data_as(P), tokens.ctypes.data_as(P), ids.size, done,
                                                      self.max_num_seqs, byref(count))
        if code != 0:
            raise RuntimeError_("SchedulerError", code, SCHEDULER_ERROR)
        return [(c.id, c.generated_tokens, "Stopped" if c.reason else "Length") for c in done[:count.value]]

    def abort_batch(self) -> None:
        code = lib.qwc_scheduler_abort_batch(self._handle)
        if code != 0:
            raise RuntimeError_("SchedulerError", code, SCHEDULER_ERROR)

    def cancel(self, seq_id: int) -> bool:
        removed = c_int()
        code = lib.qwc_scheduler_cancel(self._handle, seq_id, byref(removed))
        if code != 0:
            raise RuntimeError_("SchedulerError", code, SCHEDULER_ERROR)
        return bool(removed.value)

    def remaining_tokens(self, seq_id: int):
        value = lib.qwc_scheduler_remaining_tokens(self._handle, seq_id)
        return None if value < 0 else value

    def waiting(self) -> int:
        return lib.qwc_scheduler_waiting(self._handle)

    def active(self) -> int:
        return lib.qwc_scheduler_active(self._handle)

    def committed_kv_blocks(self) -> int:
        return lib.qwc_scheduler_committed_kv_blocks(self._handle)


class StepView(ctypes.Structure):
    """qwc_step_view: what a worker step hands to its executor."""
    _fields_ = [("num_sequences", c_size_t), ("num_decode", c_size_t), ("seq_ids", POINTER(c_uint32)),
                ("state_slots", POINTER(c_uint32)), ("position_starts", POINTER(c_uint32)),
                ("context_lens", POINTER(c_uint32)), ("token_offsets", POINTER(c_uint32)),
                ("block_table_offsets", POINTER(c_uint32)), ("block_ids", POINTER(c_uint32)),
                ("num_block_ids", c_size_t), ("tokens", POINTER(c_uint32)), ("num_tokens", c_size_t),
                ("edits", POINTER(c_uint32)), ("num_edits", c_size_t), ("restores", POINTER(PrefixRestoreOp)),
                ("num_restores", c_size_t), ("saves", POINTER(PrefixSaveOp)), ("num_saves", c_size_t)]

    def as_dict(self) -> dict:
        n = self.num_sequences
        take = lambda pointer, count: [pointer[i] for i in range(count)]  # noqa: E731
        offsets = take(self.token_offsets, n + 1)
        tokens = take(self.tokens, self.num_tokens)
        return {"num_decode": self.num_decode, "seq_ids": take(self.seq_ids, n),
                "state_slots": take(self.state_slots, n), "position_starts": take(self.position_starts, n),
                "context_lens": take(self.context_lens, n), "token_offsets": offsets,
                "tokens": [tokens[offsets[i]:offsets[i + 1]] for i in range(n)],
                "edits": [take(self.edits, 4 * self.num_edits)[4 * i:4 * i + 4] for i in range(self.num_edits)],
                "restores": [(op.id, op.state_slot, op.snapshot) for op in take(self.restores, self.num_restores)],
                "saves": [(op.id, op.state_slot, op.snapshot) for op in take(self.saves, self.num_saves)]}


EXECUTE_FN = ctypes.CFUNCTYPE(c_int, c_void_p, POINTER(StepView), POINTER(c_uint32))
EVENT_FN = ctypes.CFUNCTYPE(c_int, c_void_p, c_uint32, c_uint32, c_uint32, c_uint32)
WORKER_EVENT = {0: "token", 1: "done", 2: "error"}


class Worker:
    """The serving worker loop at token level (crates/qwc-engine/src/bin/serve.rs:777-1074).

    `executor`: an Engine (its decode step runs the decode rows) or a callable
    `executor(step: dict) -> list of one sampled token per sequence` (raise, or return an int error
    code, to fail the step).  `on_event(seq_id, kind, value, reason)` with kind "token" / "done" /
    "error"; for a token, a true return value stops the sequence after it."""

    def __init__(self, scheduler: Scheduler, executor, on_event, eos_ids=()):
        self._scheduler = scheduler  # the worker borrows it
        self.raised = None

        def event(_user, seq_id, kind, value, reason):
            try:
                return 1 if on_event(seq_id, WORKER_EVENT[kind], value, reason) else 0
            except BaseException as error:  # a callback must not unwind through the C loop
                self.raised = error
                return 1

        self._event = EVENT_FN(event)
        if callable(executor):
            def execute(_user, view, sampled):
                try:
                    result = executor(view.contents.as_dict())
                    if isinstance(result, int):
                        return result
                    for i, token in enumerate(result):
                        sampled[i] = token
                    return 0 if len(result) >= view.contents.num_sequences else 0x5102
                except BaseException as error:
                    self.raised = error
                    return 0x5200
            self._execute = EXECUTE_FN(execute)
            execute_pointer, user = ctypes.cast(self._execute, P), None
        else:
            self._engine = executor
            execute_pointer, user = ctypes.cast(lib.qwc_engine_execute_step, P), executor._handle
        eos = _u32(list(eos_ids))
        self._handle = lib.qwc_worker_new(scheduler._handle, execute_pointer, user, ctypes.cast(self._event, P), None,
                                          eos.ctypes.data_as(P), eos.size)
        if not self._handle:
            raise ValueError("qwc_worker_new refused its arguments")

    def __del__(self):
        if getattr(self, "_handle", None):
            lib.qwc_worker_free(self._handle)
            self._handle = None

    def submit(self, seq_id: int, prompt, max_new_tokens: int, history_tokens: int = 0, ignore_eos: bool = False):
        prompt = _u32(list(prompt))
        lib.qwc_worker_submit(self._handle, seq_id, prompt.ctypes.data_as(P), prompt.size, max_new_tokens,
                              history_tokens, int(ignore_eos))

    def abandon(self, seq_id: int) -> None:
        lib.qwc_worker_abandon(self._handle, seq_id)

    def shutdown(self) -> None:
        lib.qwc_worker_shutdown(self._handle)

    def iterate(self):
        """One pass of the loop body: (status code, whether a step ran)."""
        progressed = c_int()
        return lib.qwc_worker_iterate(self._handle, byref(progressed)), bool(progressed.value)

    def run(self) -> int:
        """The loop; returns after shutdown() once every job is finished, or with the failure code."""
        return lib.qwc_worker_run(self._handle)

    def jobs(self) -> int:
        return lib.qwc_worker_jobs(self._handle)

    def steps(self) -> int:
        return lib.qwc_worker_steps(self._handle)

    def aborted_steps(self) -> int:
        return lib.qwc_worker_aborted_steps(self._handle)


def build_layout(cache: CacheManager, decode=(), prefill=(), max_block_ids: int = 1 << 16):
    """BatchLayout::build (crates/qwc-runtime/src/layout.rs:54-86)."""
    decode = _u32(list(decode))
    chunks = (PrefillChunk * max(1, len(prefill)))(*[PrefillChunk(*c) for c in prefill])
    n = decode.size + len(prefill)
    out = {name: np.zeros(n + extra, dtype=np.uint32) for name, extra in
           [("seq_ids", 0), ("state_slots", 0), ("position_starts", 0), ("context_lens", 0), ("token_offsets", 1),
            ("block_table_offsets", 1)]}
    block_ids = np.zeros(max_block_ids, dtype=np.uint32)
    offender = c_uint32()
    code = lib.qwc_layout_build(cache._handle, decode.ctypes.data_as(P), decode.size, chunks, len(prefill),
                                *[out[k].ctypes.data_as(P) for k in ("seq_ids", "state_slots", "position_starts",
                                                                     "context_lens", "token_offsets",
                                                                     "block_table_offsets")],
                                block_ids.ctypes.data_as(P), max_block_ids, byref(offender))
    if code != 0:
        error = RuntimeError_("LayoutError", code, LAYOUT_ERROR)
        error.offender = offender.value
        raise error
    out["num_decode"] = int(decode.size)
    out["block_ids"] = block_ids[: int(out["block_table_offsets"][-1])].copy()
    return {k: (v.tolist() if isinstance(v, np.ndarray) else v) for k, v in out.items()}


def default_config(**overrides) -> EngineConfig:
    config = EngineConfig()
    lib.qwc_engine_default_config(byref(config))
    for key, value in overrides.items():
        if not hasattr(config, key):
            raise AttributeError(key)
        setattr(config, key, value)
    return config


class Engine:
    """The decode executor (crates/qwc-engine/src/executor.rs, decode path)."""

    def __init__(self, config: EngineConfig):
        self.config = config
        handle = P()
        abi.check(lib.qwc_engine_create(byref(config), byref(handle)), "qwc_engine_create")
        self._handle = handle

    def close(self) -> None:
        if getattr(self, "_handle", None):
            lib.qwc_engine_destroy(self._handle)
            self._handle = None

    def __del__(self):
        self.close()

    @property
    def stream(self) -> int:
        return lib.qwc_engine_stream(self._handle)

    def tensor_ptr(self, name: str, layer: int = 0):
        pointer, size = P(), c_size_t()
        if lib.qwc_engine_tensor(self._handle, name.encode(), layer, byref(pointer), byref(size)) != 0:
            raise KeyError(f"{name}[{layer}]")
        return pointer.value, size.value

    def read(self, name: str, layer: int = 0, dtype=np.uint8) -> np.ndarray:
        """Copies a resident tensor to the host (tests only)."""
        _, size = self.tensor_ptr(name, layer)
        out = np.empty(size // np.dtype(dtype).itemsize, dtype=dtype)
        abi.check(lib.qwc_engine_read(self._handle, name.encode(), layer, out.ctypes.data_as(P), size),
                  "qwc_engine_read")
        return out

    def write(self, name: str, layer: int, values: np.ndarray) -> None:
        values = np.ascontiguousarray(values)
        abi.check(lib.qwc_engine_write(self._handle, name.encode(), layer, values.ctypes.data_as(P), values.nbytes),
                  "qwc_engine_write")

    def set_weight_global_scale(self, name: str, layer: int, value: float) -> None:
        """The fp32 global divisor of an NVFP4 matrix ("gate", "in_proj", ...): what a weight loader sets."""
        abi.check(lib.qwc_engine_set_weight_global_scale(self._handle, name.encode(), layer, c_float(value)),
                  "qwc_engine_set_weight_global_scale")

    def weight_global_scale(self, name: str, layer: int) -> float:
        value = c_float()
        abi.check(lib.qwc_engine_weight_global_scale(self._handle, name.encode(), layer, byref(value)),
                  "qwc_engine_weight_global_scale")
        return value.value

    def trace_layers(self, enable: bool = True) -> None:
        """Per-layer copies of the mixer output and the residual stream into the tensor "trace" (tests)."""
        abi.check(lib.qwc_engine_trace_layers(self._handle, 1 if enable else 0), "qwc_engine_trace_layers")

    def traffic(self, rows: int, context_tokens: float) -> StepTraffic:
        out = StepTraffic()
        lib.qwc_engine_traffic(self._handle, rows, float(context_tokens), byref(out))
        return out

    def apply_edits(self, edits: np.ndarray) -> None:
        edits = np.ascontiguousarray(edits, dtype=np.uint32).reshape(-1, 4)
        abi.check(lib.qwc_engine_apply_edits(self._handle, edits.ctypes.data_as(P), edits.shape[0]),
                  "qwc_engine_apply_edits")

    def install_sequence(self, slot: int, tokens: int, blocks) -> None:
        """Makes `slot` hold a sequence of `tokens` tokens in the given pages (device tables only)."""
        edits = [(slot, i, int(b), 0) for i, b in enumerate(blocks)] + [(slot, 0, tokens, 1)]
        self.apply_edits(np.array(edits, dtype=np.uint32))

    def decode(self, row_slots, tokens, edits=None) -> np.ndarray:
        row_slots, tokens = _u32(row_slots), _u32(tokens)
        edits = np.zeros((0, 4), np.uint32) if edits is None else np.ascontiguousarray(edits, np.uint32).reshape(-1, 4)
        sampled = np.zeros(row_slots.size, dtype=np.uint32)
        abi.check(lib.qwc_engine_decode(self._handle, row_slots.ctypes.data_as(P), tokens.ctypes.data_as(P),
                                        edits.ctypes.data_as(P), edits.shape[0], row_slots.size,
                                        sampled.ctypes.data_as(P)), "qwc_engine_decode")
        return sampled

    def replay(self, rows: int) -> None:
        abi.check(lib.qwc_engine_replay(self._handle, rows), "qwc_engine_replay")

    def profile_step(self, rows: int):
        phases = (PhaseTime * 32)()
        count = lib.qwc_engine_profile_step(self._handle, rows, phases, 32)
        if count < 0:
            raise abi.QwcError(-count, "qwc_engine_profile_step")
        return [(p.label.decode(), p.milliseconds, p.launches) for p in phases[:count]]

    def time_phases(self, rows: int, label_prefix: str, replays: int = 5):
        """Mean milliseconds per replay of a graph holding only the phases whose label starts with
        `label_prefix`, and how many phases that is.  Leaves state and KV pages of the step garbage."""
        milliseconds, launches = ctypes.c_float(), c_int()
        code = lib.qwc_engine_time_phases(self._handle, rows, label_prefix.encode(), replays, byref(milliseconds),
                                          byref(launches))
        if code != 0:
            raise abi.QwcError(code if code > 0 else -code, "qwc_engine_time_phases")
        return milliseconds.value, launches.value

    def memory_usage(self) -> dict:
        """Device bytes the engine asked for and its ceiling (0: none); memory.rs:73-78."""
        used, limit = c_size_t(), c_size_t()
        lib.qwc_engine_memory_usage(self._handle, byref(used), byref(limit))
        return {"used": used.value, "limit": limit.value}

    def copy_kv_block(self, source: int, target: int) -> None:
        """Executor::copy_kv_block (executor.rs:825-835); asynchronous on the engine's stream."""
        code = lib.qwc_engine_copy_kv_block(self._handle, source, target)
        if code != 0:
            raise abi.QwcError(code, "qwc_engine_copy_kv_block")

    def worker_step(self, scheduler: Scheduler, eos_token: int = 0xFFFFFFFF):
        decoded, count = c_size_t(), c_size_t()
        done = (Completion * scheduler.max_num_seqs)()
        code = lib.qwc_worker_step(self._handle, scheduler._handle, eos_token, byref(decoded), done,
                                   scheduler.max_num_seqs, byref(count))
        if code != 0:
            raise abi.QwcError(code, "qwc_worker_step")
        return decoded.value, [(c.id, c.generated_tokens, "Stopped" if c.reason else "Length")
                               for c in done[:count.value]]

    def init_split(self, unique_id: bytes) -> None:
        buffer = ctypes.create_string_buffer(unique_id, 128)
        code = lib.qwc_engine_init_split(self._handle, buffer)
        if code != 0:
            raise abi.QwcError(code, "qwc_engine_init_split")


    def exchange_handle(self) -> bytes:
        """The 64-byte inter-process handle of this rank's exchange block (fused latency mode)."""
        buffer = ctypes.create_string_buffer(64)
        code = lib.qwc_engine_exchange_handle(self._handle, buffer)
        if code != 0:
            raise abi.QwcError(code, "qwc_engine_exchange_handle")
        return buffer.raw

    def open_peers(self, handles) -> None:
        """Maps the other ranks' exchange blocks; `handles`: every rank's exchange_handle(), in rank order."""
        joined = b"".join(handles)
        buffer = ctypes.create_string_buffer(joined, len(joined))
        code = lib.qwc_engine_open_peers(self._handle, buffer, len(handles))
        if code != 0:
            raise abi.QwcError(code, "qwc_engine_open_peers")


def profile_waits(engine, enable: bool) -> None:
    """Turns the per-exchange wait bookkeeping on or off (drops the captured graphs)."""
    code = lib.qwc_engine_profile_waits(engine._handle, 1 if enable else 0)
    if code != 0:
        raise abi.QwcError(code, "qwc_engine_profile_waits")


def exchange_waits(engine) -> np.ndarray:
    """Per exchange of the step: the longest wait (ns) of a consumer thread for a peer's word since the last call."""
    waits = np.zeros(1024, dtype=np.uint64)
    code = lib.qwc_engine_exchange_waits(engine._handle, waits.ctypes.data_as(P), 1024)
    if code != 0:
        raise abi.QwcError(code, "qwc_engine_exchange_waits")
    return waits


def connect_exchange(engine, group=None) -> None:
    """Fused latency mode, set-up over torch.distributed (any backend; gloo is enough): every rank
    contributes the handle of its exchange block and maps the others', in rank order."""
    import torch.distributed as dist

    world = dist.get_world_size(group)
    handles = [None] * world
    dist.all_gather_object(handles, engine.exchange_handle(), group=group)
    if any(not isinstance(h, bytes) or len(h) != 64 for h in handles):
        raise ValueError("every rank must contribute a 64-byte handle")
    engine.open_peers(handles)
    dist.barrier(group)  # nobody steps before everybody has mapped everybody


def nccl_unique_id() -> bytes:
    buffer = ctypes.create_string_buffer(128)
    code = lib.qwc_engine_nccl_unique_id(buffer)
    if code != 0:
        raise abi.QwcError(code, "qwc_engine_nccl_unique_id")
    return buffer.raw
