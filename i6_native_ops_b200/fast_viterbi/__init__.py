"""Best-path (Viterbi) alignment: same Python surface as the reference package
``i6_native_ops.fast_viterbi`` (``i6_native_ops/fast_viterbi/__init__.py:23-47``): ``core``
(extension module with ``fast_viterbi``) and ``align_viterbi``.

The native extension is required: importing this module fails if it is not built
(``python -m i6_native_ops_b200.build``); there is no CPU or eager fallback.
"""
from __future__ import annotations

import ctypes
import importlib.util
import os
from typing import Tuple

import torch

_PKG = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
_LIB = os.path.join(_PKG, "libfbw_b200.so")
_EXT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_build", "fast_viterbi_core.so")


def _load_core():
    if not (os.path.isfile(_LIB) and os.path.isfile(_EXT)):
        raise ImportError(
            "i6_native_ops_b200: native extension not built "
            f"(missing {_LIB if not os.path.isfile(_LIB) else _EXT}); "
            "run `python -m i6_native_ops_b200.build`"
        )
    # the extension links against libfbw_b200.so by soname; load it first so the loader finds it
    ctypes.CDLL(_LIB, mode=ctypes.RTLD_GLOBAL)
    spec = importlib.util.spec_from_file_location("fast_viterbi_core", _EXT)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


core = _load_core()


def align_viterbi(
    log_probs: torch.Tensor,
    fsa: Tuple[int, torch.Tensor, torch.Tensor, torch.Tensor],
    seq_lens: torch.Tensor,
    fold_transposes: bool = True,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """Find the best path of every sequence through its automaton.

    :param log_probs: (B, T, F) float32 log probabilities of the emission model (CUDA)
    :param fsa: ``(num_states, edges (4,E) int32, weights (E,) float32, start_end_states (2,B) int32)``;
        edge rows are origin state, target state, emission index, sequence index
    :param seq_lens: (B,) int32 number of valid frames per sequence, or a (T, B) index mask
    :param fold_transposes: read ``log_probs`` in place and write the (B, T) alignment directly
        (default); ``False`` takes the reference's route -- a (T, B, F) copy into ``core.fast_viterbi``
        and a transpose of its (T, B) result (``i6_native_ops/fast_viterbi/__init__.py:37-47``).
        Both give the same tensors.
    :return: (B, T) int32 emission index of the best path per frame (0 past ``seq_lens``) and
        (B,) float32 best-path scores
    """
    num_states, edge_tensor, weight_tensor, start_end_states = fsa
    if seq_lens.dim() == 2:  # (T, B) index mask: a length is the count of non-zero entries
        if tuple(seq_lens.shape) != (log_probs.shape[1], log_probs.shape[0]):
            raise RuntimeError("index mask must have shape (T, B)")
        seq_lens = (seq_lens != 0).sum(0).to(torch.int32).contiguous()
    if fold_transposes:
        alignment, scores = core.fast_viterbi_batch_major(
            log_probs.contiguous(), edge_tensor, weight_tensor, start_end_states, seq_lens, int(num_states)
        )
        return alignment, scores
    am_scores = log_probs.transpose(0, 1).contiguous()
    alignment, scores = core.fast_viterbi(
        am_scores, edge_tensor, weight_tensor, start_end_states, seq_lens, int(num_states)
    )
    return alignment.transpose(0, 1).contiguous(), scores
