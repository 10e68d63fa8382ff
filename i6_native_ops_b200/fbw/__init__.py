"""Full-sum forward-backward loss: same Python surface as the reference package
``i6_native_ops.fbw`` (``i6_native_ops/fbw/__init__.py:27-68``): ``core`` (extension module with
``fbw`` and ``DebugOptions``), ``FastBaumWelchLoss`` and ``fbw_loss``.

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
_EXT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_build", "fbw_core.so")


def _load_core():
    if not (os.path.isfile(_LIB) and os.path.isfile(_EXT)):
        raise ImportError(
            "i6_native_ops_b200: native extension not built "
            f"(missing {_LIB if not os.path.isfile(_LIB) else _EXT}); "
            "run `python -m i6_native_ops_b200.build`"
        )
    # the extension links against libfbw_b200.so by soname; load it first so the loader finds it
    ctypes.CDLL(_LIB, mode=ctypes.RTLD_GLOBAL)
    spec = importlib.util.spec_from_file_location("fbw_core", _EXT)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


core = _load_core()


def lengths_of(seq_lens: torch.Tensor, T: int, B: int) -> torch.Tensor:
    """``seq_lens`` as the op wants it, (B,) int32.  Also accepts the older calling convention of a
    (T, B) index mask (non-zero where a frame belongs to its sequence, valid frames first): a
    sequence's length is then the number of non-zero entries of its column."""
    if seq_lens.dim() == 2:
        if tuple(seq_lens.shape) != (T, B):
            raise RuntimeError(f"index mask must have shape (T, B) = ({T}, {B}), got {tuple(seq_lens.shape)}")
        return (seq_lens != 0).sum(0).to(torch.int32).contiguous()
    return seq_lens


class FastBaumWelchLoss(torch.autograd.Function):
    """``FastBaumWelchLoss.apply(neg_log_probs (T,B,F), fsa, seq_lens) -> (T,B)`` per-frame sums.

    Forward saves the (T,B,F) negative log posteriors; backward returns ``exp(-saved)`` as the
    gradient with respect to ``neg_log_probs`` and, like the reference
    (``i6_native_ops/fbw/__init__.py:41-44``), does not scale by the incoming gradient."""

    @staticmethod
    def forward(ctx, am_scores, fsa, seq_lens):
        num_states, edge_tensor, weight_tensor, start_end_states = fsa
        seq_lens = lengths_of(seq_lens, am_scores.shape[0], am_scores.shape[1])
        grad, loss = core.fbw(
            am_scores, edge_tensor, weight_tensor, start_end_states, seq_lens, int(num_states),
            core.DebugOptions(),
        )
        ctx.save_for_backward(grad)
        return loss

    @staticmethod
    def backward(ctx, grad_loss):
        grad = ctx.saved_tensors[0].neg().exp()  # negative log posterior -> posterior
        return grad, None, None


def fbw_loss(
    log_probs: torch.Tensor,
    fsa: Tuple[int, torch.Tensor, torch.Tensor, torch.Tensor],
    seq_lens: torch.Tensor,
) -> torch.Tensor:
    """Negative log likelihood of an emission model given one automaton per sequence.

    :param log_probs: (B, T, F) float32 log probabilities (CUDA)
    :param fsa: ``(num_states, edges (4,E) int32 rows from/to/emission/sequence,
        weights (E,) float32, start_end_states (2,B) int32)``
    :param seq_lens: (B,) int32 lengths, or a (T, B) index mask (non-zero on the valid frames)
    :return: (T, B) per-frame normalisers (each valid frame of a sequence holds that sequence's
        negative log likelihood; frames past its length hold 0), as the reference returns
        (``i6_native_ops/fbw/__init__.py:66-68``).  ``loss.sum().backward()`` leaves
        ``-posterior`` in ``log_probs.grad``.
    """
    neg_log_probs = log_probs.neg().transpose(0, 1).contiguous()  # (T, B, F)
    return FastBaumWelchLoss.apply(neg_log_probs, fsa, seq_lens)


class FusedFastBaumWelchLoss(torch.autograd.Function):
    """``apply(log_probs (B,T,F), fsa, seq_lens) -> (T,B)`` per-frame sums, with the wrapper's
    elementwise passes done inside the kernels: the op reads ``log_probs`` in place (no negated,
    transposed copy) and writes ``d loss.sum() / d log_probs = -posterior`` directly in (B,T,F).
    Like the reference's backward it does not scale by the incoming gradient."""

    @staticmethod
    def forward(ctx, log_probs, fsa, seq_lens):
        num_states, edge_tensor, weight_tensor, start_end_states = fsa
        seq_lens = lengths_of(seq_lens, log_probs.shape[1], log_probs.shape[0])
        grad, loss = core.fbw_fused(log_probs, edge_tensor, weight_tensor, start_end_states,
                                    seq_lens, int(num_states))
        ctx.save_for_backward(grad)
        return loss

    @staticmethod
    def backward(ctx, grad_loss):
        return ctx.saved_tensors[0], None, None


def fbw_loss_fused(log_probs, fsa, seq_lens):
    """Same result and gradient as :func:`fbw_loss` (opt-in): four passes over the (B,T,F) tensor
    fewer per training step.  ``log_probs`` must be a contiguous float32 CUDA tensor."""
    return FusedFastBaumWelchLoss.apply(log_probs.contiguous(), fsa, seq_lens)


def fbw_host_scores(am_scores_pinned, fsa, seq_lens, out=None, staged=True):
    """The op on negative log scores ``(T, B, F)`` held in PINNED HOST memory (``tensor.pin_memory()``):
    returns ``(out (T,B,F), sum_output (T,B), loss2 (2,))``.  The scores are not copied to the device as
    a whole; the gather kernel fetches the ones the automata refer to over the bus (about a quarter of
    the tensor on the triphone workload).  ``out``: an optional pinned host tensor of the same shape
    that receives the (T,B,F) result; without it ``out`` is a new device tensor.  With
    ``staged=True`` (default) the library picks the faster way over the bus: where the rows are sparse
    only the class posteriors are sent and host threads of the library write the rows into ``out``
    while the device goes on (the call then returns when ``out`` is complete); dense rows are produced
    in a temporary device buffer and every finished part is copied to ``out`` while the rest is still
    being computed.  With ``staged=False`` the device's output pass writes straight into ``out``
    (slower over the bus).  No device copy of the result is kept in any of the three.
    ``sum_output`` and ``loss2`` are device tensors.  Results are bit-identical to ``core.fbw`` on a
    device copy.  No counterpart in the reference, whose op requires CUDA tensors."""
    num_states, edge_tensor, weight_tensor, start_end_states = fsa
    return core.fbw_host_scores(am_scores_pinned, edge_tensor, weight_tensor, start_end_states,
                                seq_lens, int(num_states), out, bool(staged))


class PlanCache:
    """Keeps the prepared (validated, sorted) form of automaton batches so that a batch that comes
    back -- the same tensors in a later epoch, or several score tensors for one batch -- skips the
    preparation kernels and their host synchronisation.  No counterpart in the reference, which
    re-reads the unsorted edge list every frame.

    A plan is keyed on the identity of the four automaton tensors and ``seq_lens`` (storage
    address, shape and in-place version counter) plus ``num_states`` and the (T, F) of the scores;
    the cache holds references to the key tensors, so an address cannot be reused while its entry
    lives.  Tensors modified in place get a new version and therefore a new plan.  Least recently
    used entries are dropped beyond ``capacity``."""

    def __init__(self, capacity: int = 8):
        self.capacity = int(capacity)
        self._entries = {}  # key -> (plan handle, key tensors); dicts keep insertion order
        self.hits = 0
        self.misses = 0

    @staticmethod
    def _key(fsa, seq_lens, T, F):
        num_states, edges, weights, start_end = fsa
        ident = tuple((t.data_ptr(), tuple(t.shape), t._version, str(t.device))
                      for t in (edges, weights, start_end, seq_lens))
        return (int(num_states), int(T), int(F)) + ident

    def plan(self, fsa, seq_lens, T: int, F: int):
        """The plan handle for ``core.fbw_run`` (built on a miss)."""
        key = self._key(fsa, seq_lens, T, F)
        hit = self._entries.pop(key, None)
        if hit is None:
            self.misses += 1
            num_states, edges, weights, start_end = fsa
            hit = (core.fbw_prepare(edges, weights, start_end, seq_lens, int(T), int(F), int(num_states)),
                   (edges, weights, start_end, seq_lens))
        else:
            self.hits += 1
        self._entries[key] = hit  # most recently used last
        while len(self._entries) > self.capacity:
            self._entries.pop(next(iter(self._entries)))
        return hit[0]

    def clear(self):
        self._entries.clear()


class CachedFastBaumWelchLoss(torch.autograd.Function):
    """:class:`FastBaumWelchLoss` with the automaton preparation taken from a :class:`PlanCache`."""

    @staticmethod
    def forward(ctx, am_scores, fsa, seq_lens, cache):
        handle = cache.plan(fsa, seq_lens, am_scores.shape[0], am_scores.shape[2])
        grad, loss, _ = core.fbw_run(handle, am_scores)
        ctx.save_for_backward(grad)
        return loss

    @staticmethod
    def backward(ctx, grad_loss):
        return ctx.saved_tensors[0].neg().exp(), None, None, None


def fbw_loss_cached(log_probs, fsa, seq_lens, cache: PlanCache):
    """Same result and gradient as :func:`fbw_loss`; automata already seen by ``cache`` are not
    prepared again."""
    neg_log_probs = log_probs.neg().transpose(0, 1).contiguous()  # (T, B, F)
    return CachedFastBaumWelchLoss.apply(neg_log_probs, fsa, seq_lens, cache)


__all__ = ["core", "FastBaumWelchLoss", "fbw_loss", "lengths_of", "FusedFastBaumWelchLoss", "fbw_loss_fused",
           "PlanCache", "CachedFastBaumWelchLoss", "fbw_loss_cached", "fbw_host_scores"]
