"""``i6_native_ops.fbw`` (reference: i6_native_ops/fbw/__init__.py:27-68) served by i6_native_ops_b200."""
from i6_native_ops_b200.fbw import FastBaumWelchLoss, core, fbw_loss  # noqa: F401

__all__ = ["FastBaumWelchLoss", "core", "fbw_loss"]
