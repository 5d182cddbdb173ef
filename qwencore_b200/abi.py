"""ctypes binding of `include/qwc_abi.h` and `include/qwc_engine.h`.

This is the Python statement of the binding a Rust / cgo maintainer would write against the
same headers: plain pointers, ints and a stream handle.  Loading fails loudly when the
shared library has not been built.
"""

from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_size_t, c_void_p, POINTER
from pathlib import Path

LIBRARY_PATH = Path(__file__).resolve().parent / "libqwc_b200.so"

CUDA_SUCCESS = 0
CUDA_ERROR_INVALID_VALUE = 1
CUDA_ERROR_NOT_SUPPORTED = 801


class QwcError(RuntimeError):
    """A launcher returned a non-zero cudaError_t (mirrors crates/qwc-cuda/src/error.rs:31-37)."""

    def __init__(self, code: int, where: str):
        super().__init__(f"{where} failed with cudaError_t {code}")
        self.code = code


class Shape(ctypes.Structure):
    _fields_ = [("delta_value_heads", c_int), ("kv_page_size", c_int)]


class TableEdit(ctypes.Structure):
    _fields_ = [("slot", ctypes.c_uint32), ("index", ctypes.c_uint32), ("value", ctypes.c_uint32),
                ("kind", ctypes.c_uint32)]


class ExchangeRow(ctypes.Structure):
    """qwc_exchange_row (include/qwc_exchange.h): one activation row that the ranks of latency mode hand
    one another; pass ctypes.byref(row)."""

    _fields_ = [("blocks", c_void_p * 8), ("ranks", c_int), ("rank", c_int), ("epoch", c_void_p),
                ("instance", ctypes.c_uint32), ("offset", ctypes.c_uint64), ("width", c_int), ("flags", ctypes.c_uint32), ("wait_profile", c_void_p)]


# name -> (restype, argtypes); every symbol declared in include/qwc_abi.h
P = c_void_p
KERNEL_SYMBOLS = {
    "qwc_configure": (c_int, [POINTER(Shape)]),
    "qwc_get_shape": (None, [POINTER(Shape)]),
    "qwc_device_status": (c_int, []),
    "qwc_device_status_reset": (c_int, []),
    "qwc_device_status_detail": (c_int, [P]),
    "qwc_device_status_set": (c_int, [c_int]),
    "qwc_device_status_copy": (c_int, [P, P]),
    "qwc_nvfp4_w4a16": (c_int, [P, P, P, P, c_int, c_int, c_int, c_float, P]),
    "qwc_nvfp4_swiglu_w4a16": (c_int, [P, P, P, P, P, P, c_int, c_int, c_int, c_float, c_float, P]),
    "qwc_nvfp4_prefetch_next": (c_int, [P, P, P, P, c_int, c_int, c_int]),
    "qwc_streamk_workspace_bytes": (c_size_t, []),
    "qwc_streamk_workspace_init": (c_int, [P, P]),
    "qwc_staged_activation_bytes": (c_size_t, [c_int, c_int]),
    "qwc_stage_activations": (c_int, [P, P, c_int, c_int, P]),
    "qwc_nvfp4_w4a16_staged": (c_int, [P, P, P, P, P, c_int, c_int, c_int, c_float, P, P]),
    "qwc_nvfp4_swiglu_w4a16_staged": (c_int, [P, P, P, P, P, P, P, c_int, c_int, c_int, c_float, c_float, P, P]),
    "qwc_fp8_lm_head_staged": (c_int, [P, P, P, P, P, P, c_int, c_int, c_int, P, P]),
    "qwc_rmsnorm_bf16_staged": (c_int, [P, P, P, P, P, c_int, c_int, c_float, P]),
    "qwc_nvfp4_split_count": (c_int, [c_int, c_int]),
    # latency mode: rows exchanged between ranks (P: a qwc_exchange_row*)
    "qwc_fp8_quantize_rows": (c_int, [P, P, P, c_int, c_int, c_int, P]),
    "qwc_exchange_advance": (c_int, [P, P]),
    "qwc_exchange_row_bytes": (c_size_t, [c_int]),
    "qwc_exchange_candidate_bytes": (c_size_t, [c_int]),
    "qwc_nvfp4_exchange_slices": (c_int, [c_int, c_int, c_int]),
    "qwc_nvfp4_w4a16_exchange": (c_int, [P, P, P, P, c_int, c_int, P]),
    "qwc_nvfp4_swiglu_w4a16_exchange": (c_int, [P, P, P, P, P, P, c_int, c_int, P]),
    "qwc_rmsnorm_bf16_exchanged": (c_int, [P, c_int, c_float, P, P, P, P, P, c_int, c_float, P]),
    "qwc_delta_prepare_decode_exchanged": (c_int, [P, c_int, c_float, c_int, c_int] + [P] * 11 + [c_int, P]),
    "qwc_delta_gated_rmsnorm_exchanged": (c_int, [P, P, c_int, c_float, c_int, P, P, P, c_float, P]),
    "qwc_nvfp4_sum_exchanged": (c_int, [P, c_int, c_float, P, P]),
    "qwc_swiglu_combine_exchanged": (c_int, [P, c_int, c_float, c_float, P, P, c_int, P]),
    "qwc_fp8_lm_head_exchange": (c_int, [P, P, P, P, P, P, P, c_int, c_int, P, P]),
    "qwc_delta_prepare_decode_split": (c_int, [P, c_int, c_int, c_float, c_int, c_int] + [P] * 11 + [c_int, c_int, P]),
    "qwc_delta_gated_rmsnorm_split": (c_int, [P, P, c_int, c_int, c_float, c_int, P, P, P, c_int, c_float, P]),
    "qwc_nvfp4_sum_slices": (c_int, [P, c_int, c_float, P, c_int, c_int, P]),
    "qwc_delta_decode_fuses_norm": (c_int, [c_int]),
    "qwc_delta_decode_int8_step": (c_int, [P] * 10 + [c_int, c_int, P, c_int, c_float, P, c_int, c_int, P, c_float,
                                           P, P]),
    "qwc_nvfp4_w4a16_split": (c_int, [P, P, P, P, c_int, c_int, c_int, P]),
    "qwc_rmsnorm_bf16_split_staged": (c_int, [P, c_int, c_float, P, P, P, P, P, c_int, c_int, c_float, P]),
    "qwc_delta_gated_rmsnorm_staged": (c_int, [P, P, P, P, P, c_int, c_float, c_int, P]),
    "qwc_paged_attention_packed_fp8_staged": (c_int, [P, P, P, P, P, P, P, P, P, P, P, c_size_t, c_int, c_int,
                                                      c_int, c_int, c_int, c_int, c_float, P]),
    "qwc_paged_attention_packed_fp8": (c_int, [P, P, P, P, P, P, P, P, c_size_t, c_int, c_int, c_int, c_int,
                                               c_int, c_float, P]),
    "qwc_paged_attention_packed_fp8_scaled": (c_int, [P, P, P, P, P, P, P, P, P, P, c_size_t, c_int, c_int,
                                                      c_int, c_int, c_int, c_int, c_float, P]),
    "qwc_paged_attention_packed_workspace_bytes": (c_size_t, [c_int, c_int]),
    "qwc_paged_attention_packed_fp8_noalloc": (c_int, [P, P, P, P, P, P, P, P, P, c_int, c_int, c_int, c_int, c_int,
                                                       c_int, c_float, P]),
    "qwc_paged_attention_packed_noalloc_max_pairs": (c_int, []),
    "qwc_delta_decode_int8": (c_int, [P, P, P, P, P, P, P, P, P, P, c_int, c_int, P]),
    "qwc_delta_prepare_decode": (c_int, [P] * 14 + [c_int, c_int, c_int, c_int, P]),
    "qwc_delta_gated_rmsnorm": (c_int, [P, P, P, P, c_int, c_float, c_int, P]),
    "qwc_prepare_attention_decode_fp8": (c_int, [P] * 12 + [c_int, c_float, P]),
    "qwc_prepare_attention_decode_fp8_scaled": (c_int, [P] * 14 + [c_int, c_int, c_int, c_int, c_int, c_float,
                                                                   P]),
    "qwc_rmsnorm_bf16": (c_int, [P, P, P, P, c_int, c_int, c_float, P]),
    "qwc_fp8_embedding_gather": (c_int, [P, P, P, P, c_int, c_int, c_int, P]),
    "qwc_fp8_lm_head": (c_int, [P, P, P, P, c_int, c_int, c_int, P]),
    "qwc_fp8_lm_head_batched": (c_int, [P, P, P, P, c_int, c_int, c_int, P]),
    "qwc_fp8_max_logits_batch": (c_int, []),
    "qwc_fp8_max_batched_logits": (c_int, []),
    "qwc_argmax": (c_int, [P, P, P, P, c_int, c_int, c_int, P]),
    "qwc_page_table_apply": (c_int, [P, P, P, c_int, c_int, c_int, P]),
    "qwc_pack_decode_batch": (c_int, [P] * 18 + [c_int, c_int, c_int, c_int, P]),
}


def load() -> ctypes.CDLL:
    if not LIBRARY_PATH.exists():
        raise ImportError(
            f"{LIBRARY_PATH} is missing: build the CUDA extension with `python -m qwencore_b200.build` "
            "(there is no CPU or PyTorch fallback for these kernels)")
    lib = ctypes.CDLL(str(LIBRARY_PATH))
    for name, (restype, argtypes) in KERNEL_SYMBOLS.items():
        function = getattr(lib, name)  # AttributeError if the library lost a symbol
        function.restype = restype
        function.argtypes = argtypes
    return lib


lib = load()


def check(code: int, where: str) -> None:
    if code != CUDA_SUCCESS:
        raise QwcError(code, where)


def configure(delta_value_heads: int, kv_page_size: int) -> None:
    shape = Shape(delta_value_heads, kv_page_size)
    check(lib.qwc_configure(ctypes.byref(shape)), "qwc_configure")


def get_shape() -> tuple[int, int]:
    shape = Shape()
    lib.qwc_get_shape(ctypes.byref(shape))
    return shape.delta_value_heads, shape.kv_page_size
