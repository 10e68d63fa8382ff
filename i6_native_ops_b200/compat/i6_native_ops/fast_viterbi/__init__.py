"""``i6_native_ops.fast_viterbi`` (reference: i6_native_ops/fast_viterbi/__init__.py:23-47) served by
i6_native_ops_b200."""
from i6_native_ops_b200.fast_viterbi import align_viterbi, core  # noqa: F401

__all__ = ["align_viterbi", "core"]
