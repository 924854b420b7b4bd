"""Loop-boundary token retention and decode key selection (numpy oracle).

Restates flashloop/selection.py:26-88, flashloop/engine.py:78-109 and the inline
selection of flashloop/engine.py:438-481.

Tie rule.  ``torch.topk`` leaves the order of equal values unspecified, so the
reference's selected set is only well defined when the budget boundary does not
cut through a run of equal values.  The oracle (and the CUDA kernel it checks)
use: larger value first, then lower index.  :func:`boundary_is_tied` tells a test
whether an input is outside the well-defined region.
"""

from __future__ import annotations

import math

import numpy as np


def decode_budget(keys: int, fraction: float) -> int:
    """selection.py:81 / engine.py:443-452."""

    return min(int(keys), max(1, math.ceil(int(keys) * float(fraction))))


def topk_sorted_indices(values: np.ndarray, budget: int) -> np.ndarray:
    """Indices of the ``budget`` largest entries of a 1-D float32 array, ascending."""

    order = np.argsort(-values.astype(np.float32), kind="stable")
    return np.sort(order[:budget]).astype(np.int32)


def boundary_is_tied(values: np.ndarray, budget: int) -> bool:
    if budget >= values.shape[-1]:
        return False
    ordered = np.sort(values.astype(np.float32))[::-1]
    return bool(ordered[budget - 1] == ordered[budget])


def select_decode_keys(weights: np.ndarray, *, fraction: float):
    """selection.py:72-88.  weights [B,H,1,N] -> (indices int32 [B,H,1,k] ascending,
    global_mass float32 [B,H,1,1])."""

    batch, heads, _, keys = weights.shape
    budget = decode_budget(keys, fraction)
    indices = np.zeros((batch, heads, 1, budget), np.int32)
    mass = np.zeros((batch, heads, 1, 1), np.float32)
    for b in range(batch):
        for h in range(heads):
            row = weights[b, h, 0].astype(np.float32)
            chosen = topk_sorted_indices(row, budget)
            indices[b, h, 0] = chosen
            mass[b, h, 0, 0] = row[chosen].sum(dtype=np.float32)
    return indices, mass


def pad_decode_indices(indices: np.ndarray, *, block_size: int = 64):
    """engine.py:84-109: capacity (count // block + 1) * block, zero padded, with mask."""

    count = indices.shape[-1]
    capacity = (count // block_size + 1) * block_size
    padded = np.zeros((*indices.shape[:-1], capacity), indices.dtype)
    padded[..., :count] = indices
    valid = np.zeros(padded.shape, bool)
    valid[..., :count] = True
    return padded, valid


def pad_selected(mask: np.ndarray, *, block_size: int = 64):
    """A boolean key mask [B,H,1,N] with the same count in every row -> the engine's padded
    ascending index list and validity mask (engine.py:84-109), [B,H,cap] each."""

    batch, heads, _, keys = mask.shape
    count = int(mask[0, 0, 0].sum())
    indices = np.zeros((batch, heads, count), np.int32)
    for b in range(batch):
        for h in range(heads):
            chosen = np.nonzero(mask[b, h, 0])[0]
            if chosen.size != count:
                raise ValueError("every row must select the same number of keys")
            indices[b, h] = chosen
    return pad_decode_indices(indices, block_size=block_size)


def softmax_f32(logits: np.ndarray) -> np.ndarray:
    work = logits.astype(np.float32)
    shifted = work - work.max(axis=-1, keepdims=True)
    e = np.exp(shifted).astype(np.float32)
    return (e / e.sum(axis=-1, keepdims=True, dtype=np.float32)).astype(np.float32)


def select_from_logits(logits: np.ndarray, *, fraction: float):
    """engine.py:438-481: softmax of the scaled loop-2 logits, top budget, padded
    indices, validity, global mass and the renormalised selected weights.

    logits [B,H,1,N] float32.  Returns dict with indices [B,H,cap], valid [B,H,cap],
    global_mass [B,H,1,1], selected_weights [B,H,1,cap], budget."""

    weights = softmax_f32(logits)
    indices, _ = select_decode_keys(weights, fraction=fraction)
    budget = indices.shape[-1]
    gathered = np.take_along_axis(weights, indices.astype(np.int64), axis=-1)
    padded, valid = pad_decode_indices(indices[:, :, 0, :])
    glob = np.zeros((*gathered.shape[:-1], padded.shape[-1]), np.float32)
    glob[..., :budget] = gathered
    mass = glob.sum(axis=-1, keepdims=True, dtype=np.float32)
    return {
        "indices": padded, "valid": valid, "global_mass": mass,
        "selected_weights": (glob / mass).astype(np.float32), "budget": budget,
        "weights": weights,
    }


def hidden_delta_score(current: np.ndarray, previous: np.ndarray) -> np.ndarray:
    """engine.py:78-81: ||h_r - h_{r-1}|| / max(||h_r||, 1e-12) over the hidden axis."""

    cur = current.astype(np.float32)
    num = np.sqrt(np.sum((cur - previous.astype(np.float32)) ** 2, axis=-1, dtype=np.float32))
    den = np.maximum(np.sqrt(np.sum(cur ** 2, axis=-1, dtype=np.float32)), np.float32(1e-12))
    return (num / den).astype(np.float32)


def prefill_budget(tokens: int, fraction: float) -> int:
    return max(1, math.ceil(int(tokens) * float(fraction)))


def select_prefill_tokens(scores: np.ndarray, *, fraction: float,
                          eligible: np.ndarray | None = None,
                          force_last_token: bool = True) -> np.ndarray:
    """selection.py:26-69.  scores [B,T] float32 -> bool mask [B,T]."""

    batch, tokens = scores.shape
    if eligible is None:
        eligible = np.ones((batch, tokens), bool)
    budget = prefill_budget(tokens, fraction)
    result = np.zeros((batch, tokens), bool)
    for b in range(batch):
        candidates = np.nonzero(eligible[b])[0]
        forced = 0
        if force_last_token:
            if not eligible[b, tokens - 1]:
                raise ValueError("the forced final token must be eligible")
            candidates = candidates[candidates != tokens - 1]
            forced = 1
        count = min(budget, candidates.size + forced)
        remaining = count - forced
        if remaining > 0:
            local = scores[b, candidates].astype(np.float32)
            order = np.argsort(-local, kind="stable")[:remaining]
            result[b, candidates[order]] = True
        if forced:
            result[b, tokens - 1] = True
    return result


def positions_and_rank_map(mask: np.ndarray, tokens: int):
    """Sorted active positions and the logical->compact rank map with -1 for absent
    rows (engine.py:276-277, cache.py:281-289)."""

    positions = np.nonzero(mask[:tokens])[0].astype(np.int32)
    rank = np.full((tokens,), -1, np.int32)
    rank[positions] = np.arange(positions.size, dtype=np.int32)
    return positions, rank
