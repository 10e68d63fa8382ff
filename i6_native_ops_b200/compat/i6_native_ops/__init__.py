"""``i6_native_ops`` import path served by i6_native_ops_b200 (fbw and fast_viterbi only)."""
