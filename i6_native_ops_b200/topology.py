"""Device-side builders of the automaton tuple ``(num_states, edges, weights, start_end_states)``
that ``fbw_loss`` and ``align_viterbi`` take (format: ``i6_native_ops/fbw/__init__.py:49-63``).
The reference ships no builders -- its automata are exported by an external tool -- so these have
no counterpart there; they make the ops usable from label sequences alone.

Both run as CUDA kernels of the native library (``csrc/topology_b200.inc``) and return CUDA tensors.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

from .fbw import core

Fsa = Tuple[int, torch.Tensor, torch.Tensor, torch.Tensor]


def ctc_topology(labels: torch.Tensor, label_lens: torch.Tensor, blank: int = 0) -> Fsa:
    """CTC automata for a batch of label sequences.

    :param labels: (B, Lmax) int32 CUDA tensor, padded
    :param label_lens: (B,) int32 CUDA tensor of label counts
    :param blank: emission index of the blank symbol

    Per sequence: states 0..2L alternate blank / label, plus one separate final state; an edge
    emits the symbol of its target; loop, advance, and skip between different labels; all weights 0.
    With this construction ``fbw_loss`` equals ``torch.nn.functional.ctc_loss`` (sum reduction)."""
    S, edges, weights, start_end = core.ctc_topology(labels.contiguous(), label_lens.contiguous(), int(blank))
    return int(S), edges, weights, start_end


def hmm_topology(classes: torch.Tensor, lens: torch.Tensor, loop_prob: float, forward_prob: float,
                 skip_prob: Optional[float] = None, optional: Optional[torch.Tensor] = None) -> Fsa:
    """Left-to-right HMM automata for a batch of state-class sequences.

    :param classes: (B, Nmax) int32 CUDA tensor: emission class of each HMM state, padded
    :param lens: (B,) int32 CUDA tensor of state counts
    :param loop_prob, forward_prob: transition probabilities (weights are their negative logs)
    :param skip_prob: if given, every state also gets a j -> j+2 edge with this probability
    :param optional: (B, Nmax) uint8; without ``skip_prob``, a set flag lets the path bypass that
        state (a j -> j+2 edge around it, with the forward weight)

    A virtual start state precedes the first HMM state; the end state is the last HMM state."""
    f32 = lambda p: float(torch.tensor(-math.log(p), dtype=torch.float32))  # weights as fp32 values
    opt = optional.contiguous() if optional is not None else None
    S, edges, weights, start_end = core.hmm_topology(
        classes.contiguous(), lens.contiguous(), opt, f32(loop_prob), f32(forward_prob),
        None if skip_prob is None else f32(skip_prob))
    return int(S), edges, weights, start_end
