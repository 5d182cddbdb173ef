"""The C-ABI library builds, loads and exports every symbol the headers declare (no GPU)."""

import ctypes
import re
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]


def declared_symbols():
    names = set()
    for header in sorted((ROOT / "include").glob("*.h")):
        text = re.sub(r"/\*.*?\*/", "", header.read_text(), flags=re.S)
        names.update(re.findall(r"\b(qwc_[a-z0-9_]+)\s*\(", text))
    return sorted(names)


def test_headers_declare_the_drop_in_symbols():
    names = declared_symbols()
    # the launchers the reference's FFI binds for this path (crates/qwc-cuda/src/ffi.rs)
    for required in ["qwc_nvfp4_w4a16", "qwc_nvfp4_swiglu_w4a16", "qwc_paged_attention_packed_fp8",
                     "qwc_delta_decode_int8", "qwc_delta_prepare_decode", "qwc_delta_gated_rmsnorm",
                     "qwc_prepare_attention_decode_fp8", "qwc_rmsnorm_bf16", "qwc_fp8_embedding_gather",
                     "qwc_fp8_lm_head", "qwc_fp8_lm_head_batched", "qwc_fp8_max_logits_batch",
                     "qwc_fp8_max_batched_logits", "qwc_argmax", "qwc_pack_decode_batch", "qwc_page_table_apply"]:
        assert required in names


def test_library_exports_every_declared_symbol(built_library):
    lib = ctypes.CDLL(str(built_library))
    missing = [name for name in declared_symbols() if not hasattr(lib, name)]
    assert not missing, f"declared in include/*.h but not exported: {missing}"


def test_binding_covers_every_kernel_symbol(built_library):
    from qwencore_b200 import abi

    header = (ROOT / "include" / "qwc_abi.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    declared = set(re.findall(r"\b(qwc_[a-z0-9_]+)\s*\(", text))
    assert declared == set(abi.KERNEL_SYMBOLS), declared ^ set(abi.KERNEL_SYMBOLS)


def test_launchers_reject_bad_arguments_before_touching_the_device(built_library):
    """Argument validation returns cudaErrorInvalidValue without any CUDA call
    (crates/qwc-cuda/cuda/nvfp4.cu:500-504, delta_net.cu:1226-1231, attention_prepare.cu:162-169)."""
    from qwencore_b200 import abi

    lib = abi.lib
    bad = abi.CUDA_ERROR_INVALID_VALUE
    one = 0x1000  # never dereferenced: validation fails first
    assert lib.qwc_nvfp4_w4a16(0, one, one, one, 16, 256, 1, 1.0, 0) == bad
    assert lib.qwc_nvfp4_w4a16(one, one, one, one, 16, 100, 1, 1.0, 0) == bad
    assert lib.qwc_nvfp4_w4a16(one, one, one, one, 16, 256, 0, 1.0, 0) == bad
    assert lib.qwc_nvfp4_swiglu_w4a16(one, one, one, 0, one, one, 16, 256, 1, 1.0, 1.0, 0) == bad
    assert lib.qwc_delta_decode_int8(one, one, one, one, one, one, one, one, one, one, 1, 2, 0) == bad
    assert lib.qwc_delta_decode_int8(0, one, one, one, one, one, one, one, one, one, 4, 2, 0) == bad
    assert lib.qwc_rmsnorm_bf16(one, 0, one, one, 1, 100, 1e-6, 0) == bad
    assert lib.qwc_rmsnorm_bf16(one, 0, one, one, 1, 256, 0.0, 0) == bad
    assert lib.qwc_argmax(one, one, one, one, 100, 1, 0, 0) == bad
    assert lib.qwc_argmax(one, one, one, one, 100, 1, 257, 0) == bad
    assert lib.qwc_fp8_lm_head(one, one, one, one, 33, 256, 10, 0) == bad
    assert lib.qwc_paged_attention_packed_fp8(one, 0, one, one, one, one, one, 0, 0, 1, 0, 4, 0, 1, 0.0625, 0) == bad
    assert lib.qwc_paged_attention_packed_fp8(one, 0, one, one, one, one, one, 0, 0, 1, 0, 4, 32, 1, 0.0625,
                                              0) == abi.CUDA_ERROR_NOT_SUPPORTED
    assert lib.qwc_fp8_max_logits_batch() == 32 and lib.qwc_fp8_max_batched_logits() == 32
    assert lib.qwc_paged_attention_packed_workspace_bytes(32, 4) == 32 * 24 * 4 * 520
    assert lib.qwc_paged_attention_packed_workspace_bytes(32, 1) == 0


def test_configure_accepts_only_supported_shapes(built_library):
    from qwencore_b200 import abi

    before = abi.get_shape()
    try:
        abi.configure(32, 16)
        assert abi.get_shape() == (32, 16)
        for bad in [(40, 16), (32, 32), (0, 0)]:
            try:
                abi.configure(*bad)
            except abi.QwcError as error:
                assert error.code == abi.CUDA_ERROR_INVALID_VALUE
            else:
                raise AssertionError(f"{bad} accepted")
        assert abi.get_shape() == (32, 16)
    finally:
        abi.configure(*before)
