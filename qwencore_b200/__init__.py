"""B200-native decode-step kernels behind the qwc C ABI.

The package is a thin host-side mirror of the reference's `qwc-cuda` wrapper modules
(crates/qwc-cuda/src/{nvfp4,paged_attention,delta_net,...}.rs): it owns no arithmetic.
Everything runs in `libqwc_b200.so`, built in-tree by `python -m qwencore_b200.build`;
importing `qwencore_b200.abi` raises if that library is missing - there is no fallback path.
"""

__all__ = ["abi", "ops", "engine", "synth"]
