"""Loop-boundary token and decode-key selection.

Mirrors flashloop/selection.py.  ``select_decode_keys`` (:72-88) runs as one CUDA
launch (radix select + ordered compaction); ties are broken towards the lower
index, where ``torch.topk`` leaves the order unspecified.
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from . import _native


@dataclass(frozen=True)
class DecodeSelection:
    """Sorted selected key positions and their original global-softmax mass."""

    indices: torch.Tensor
    global_mass: torch.Tensor


@dataclass(frozen=True)
class PaddedDecodeSelection:
    """What FlashLoopEngine.decode keeps per layer after loop 2 (engine.py:470-497):
    indices padded to ``(budget // 64 + 1) * 64`` with zeros, their validity, the
    selected global mass and the selected weights divided by that mass."""

    indices: torch.Tensor           # int32 [B, H, capacity]
    valid: torch.Tensor             # bool  [B, H, capacity]
    global_mass: torch.Tensor       # float32 [B, H, 1, 1]
    selected_weights: torch.Tensor  # float32 [B, H, 1, capacity]
    counts: torch.Tensor            # int32 [B, H]


def _validate_fraction(fraction: float) -> float:
    fraction = float(fraction)
    if not 0.0 < fraction <= 1.0:
        raise ValueError("fraction must be in (0, 1]")
    return fraction


def decode_budget(keys: int, fraction: float) -> int:
    return min(int(keys), max(1, math.ceil(int(keys) * float(fraction))))


def padded_capacity(budget: int, block_size: int = 64) -> int:
    """engine.py:100."""

    return (int(budget) // block_size + 1) * block_size


def select_decode_keys_padded(values: torch.Tensor, *, fraction: float, values_are_logits: bool,
                              seq_state: torch.Tensor | None = None, max_keys: int | None = None,
                              out: PaddedDecodeSelection | None = None) -> PaddedDecodeSelection:
    """One launch of ``fl_select_decode_keys`` over [B, H, 1, N] (or [B, H, N]) values.

    With ``seq_state`` the number of keys of each sequence is read on the device
    (quant + tail + 1) and ``max_keys`` bounds it for sizing the outputs."""

    fraction = _validate_fraction(fraction)
    if values.ndim == 4:
        if values.shape[-2] != 1:
            raise ValueError("decode weights must have shape [batch, heads, 1, keys]")
        values = values.squeeze(-2)
    if values.ndim != 3 or values.shape[-1] == 0:
        raise ValueError("decode weights must have shape [batch, heads, 1, keys]")
    if values.dtype != torch.float32:
        values = values.float()
    _native.require_cuda(values)
    # the kernel indexes rows as (b*heads + h) * stride: keep views of a wider logits buffer
    if values.stride(-1) != 1 or values.stride(0) != values.shape[1] * values.stride(1):
        values = values.contiguous()
    batch, heads, width = (int(v) for v in values.shape)
    keys = int(max_keys) if max_keys is not None else width
    capacity = padded_capacity(decode_budget(keys, fraction))
    device = values.device
    if out is None:
        out = PaddedDecodeSelection(
            indices=torch.empty((batch, heads, capacity), dtype=torch.int32, device=device),
            valid=torch.empty((batch, heads, capacity), dtype=torch.bool, device=device),
            global_mass=torch.empty((batch, heads, 1, 1), dtype=torch.float32, device=device),
            selected_weights=torch.empty((batch, heads, 1, capacity), dtype=torch.float32, device=device),
            counts=torch.empty((batch, heads), dtype=torch.int32, device=device))
    capacity = int(out.indices.shape[-1])
    lib = _native.load()
    _native.check(lib.fl_select_decode_keys(
        _native.ptr(values), int(values.stride(1)), batch, heads, keys,
        _native.ptr(seq_state), fraction, 1 if values_are_logits else 0,
        _native.ptr(out.indices), _native.ptr(out.valid), capacity, _native.ptr(out.counts),
        _native.ptr(out.global_mass), _native.ptr(out.selected_weights),
        _native.current_stream(device)), "fl_select_decode_keys")
    return out


def select_decode_keys(weights: torch.Tensor, *, fraction: float) -> DecodeSelection:
    """Select top global probabilities independently for each decode head
    (flashloop/selection.py:72-88): indices int32 [B, H, 1, budget] ascending,
    global_mass float32 [B, H, 1, 1]."""

    fraction = _validate_fraction(fraction)
    if weights.ndim != 4 or weights.shape[-2] != 1 or weights.shape[-1] == 0:
        raise ValueError("decode weights must have shape [batch, heads, 1, keys]")
    if not bool(torch.isfinite(weights).all()):
        raise ValueError("decode weights must be finite")
    keys = int(weights.shape[-1])
    budget = decode_budget(keys, fraction)
    padded = select_decode_keys_padded(weights, fraction=fraction, values_are_logits=False)
    return DecodeSelection(indices=padded.indices[:, :, None, :budget].contiguous(),
                           global_mass=padded.global_mass)


def select_prefill_tokens(scores: torch.Tensor, *, fraction: float,
                          eligible: torch.Tensor | None = None,
                          force_last_token: bool = True) -> torch.Tensor:
    """Select a global ceil budget, optionally nested in a prior-loop mask
    (flashloop/selection.py:26-69).  Runs once per loop boundary of the prefill, on
    the GPU as one launch (``fl_select_prefill_tokens``) for CUDA scores; host tensors take
    the Torch path below.  Ties go to the lower index."""

    fraction = _validate_fraction(fraction)
    if scores.ndim != 2 or scores.shape[1] == 0:
        raise ValueError("scores must have shape [batch, tokens]")
    if not bool(torch.isfinite(scores).all()):
        raise ValueError("scores must be finite")
    if eligible is None:
        eligible = torch.ones_like(scores, dtype=torch.bool)
    if eligible.shape != scores.shape or eligible.dtype != torch.bool:
        raise ValueError("eligible must be a bool tensor matching scores")
    batch, tokens = scores.shape
    budget = max(1, math.ceil(tokens * fraction))
    if bool((~eligible).all(dim=1).any()):
        raise ValueError("eligible contains an empty batch row")
    if force_last_token and not bool(eligible[:, -1].all()):
        raise ValueError("the forced final token must be eligible")
    if scores.is_cuda:
        from .compaction import retain_tokens

        return retain_tokens(scores, fraction=fraction, eligible=eligible,
                             force_last_token=force_last_token).mask
    work = scores.float().masked_fill(~eligible, float("-inf"))
    forced = 0
    if force_last_token:
        if not bool(eligible[:, -1].all()):
            raise ValueError("the forced final token must be eligible")
        work = work.clone()
        work[:, -1] = float("-inf")
        forced = 1
    result = torch.zeros_like(eligible)
    candidates = eligible.sum(dim=1) - forced
    for b in range(batch):
        count = min(budget, int(candidates[b]) + forced)
        remaining = count - forced
        if remaining > 0:
            order = torch.sort(work[b], descending=True, stable=True).indices[:remaining]
            result[b, order] = True
    if forced:
        result[:, -1] = True
    return result
