"""B200-native full-sum forward-backward (fast Baum-Welch) loss.

Drop-in for the ``fbw`` op of i6_native_ops (``i6_native_ops/fbw/__init__.py``): import
``fbw_loss`` / ``FastBaumWelchLoss`` / ``core`` from ``i6_native_ops_b200.fbw``.
"""
__version__ = "0.1.0"
