"""Token-retention compaction on the GPU: hidden-delta score, retained-token selection with
positions and rank map, and row gather / scatter.

These replace the Torch ops around the sparse prefill loops of the reference:
``_hidden_delta_score`` (flashloop/engine.py:78-81), ``select_prefill_tokens``
(flashloop/selection.py:26-69), ``torch.nonzero`` + ``_rank_map`` (engine.py:276-277,
flashloop/cache.py:281-289) and the ``index_select`` / ``index_copy_`` of active rows
(flashloop/prefill.py:144-158, 237-254).
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from . import _native


@dataclass(frozen=True)
class RetainedTokens:
    """Result of one retention step for a batch of sequences."""

    mask: torch.Tensor       # bool  [B, T]
    positions: torch.Tensor  # int32 [B, T]: retained positions ascending, then -1
    rank: torch.Tensor       # int32 [B, T]: index of the token in ``positions`` or -1
    count: torch.Tensor      # int32 [B]


def hidden_delta_score(current: torch.Tensor, previous: torch.Tensor) -> torch.Tensor:
    """||h_r - h_{r-1}|| / max(||h_r||, 1e-12) over the hidden axis, float32 [B, T]."""

    if current.shape != previous.shape or current.ndim != 3:
        raise ValueError("hidden states must share the shape [batch, tokens, hidden]")
    if current.dtype != torch.bfloat16 or previous.dtype != torch.bfloat16:
        raise TypeError("hidden states must be bfloat16")
    _native.require_cuda(current, previous)
    cur, prev = current.contiguous(), previous.contiguous()
    batch, tokens, hidden = (int(v) for v in cur.shape)
    out = torch.empty((batch, tokens), dtype=torch.float32, device=cur.device)
    _native.check(_native.load().fl_hidden_delta_score(
        _native.ptr(cur), _native.ptr(prev), batch * tokens, hidden, _native.ptr(out),
        _native.current_stream(cur.device)), "fl_hidden_delta_score")
    return out


def retain_tokens(scores: torch.Tensor, *, fraction: float, eligible: torch.Tensor | None = None,
                  force_last_token: bool = True) -> RetainedTokens:
    """One launch: the retention mask of ``select_prefill_tokens`` plus the sorted positions,
    the rank map and the count of every sequence."""

    fraction = float(fraction)
    if not 0.0 < fraction <= 1.0:
        raise ValueError("fraction must be in (0, 1]")
    if scores.ndim != 2 or scores.shape[1] == 0:
        raise ValueError("scores must have shape [batch, tokens]")
    _native.require_cuda(scores)
    batch, tokens = (int(v) for v in scores.shape)
    values = scores.float().contiguous()
    elig = None
    if eligible is not None:
        if eligible.shape != scores.shape or eligible.dtype != torch.bool:
            raise ValueError("eligible must be a bool tensor matching scores")
        elig = eligible.contiguous().view(torch.uint8)
    device = scores.device
    mask = torch.empty((batch, tokens), dtype=torch.bool, device=device)
    positions = torch.empty((batch, tokens), dtype=torch.int32, device=device)
    rank = torch.empty((batch, tokens), dtype=torch.int32, device=device)
    count = torch.empty((batch,), dtype=torch.int32, device=device)
    _native.check(_native.load().fl_select_prefill_tokens(
        _native.ptr(values), _native.ptr(elig), batch, tokens, fraction, 1 if force_last_token else 0,
        _native.ptr(mask), _native.ptr(positions), _native.ptr(rank), _native.ptr(count),
        _native.current_stream(device)), "fl_select_prefill_tokens")
    return RetainedTokens(mask=mask, positions=positions, rank=rank, count=count)


def retained_from_mask(mask: torch.Tensor) -> RetainedTokens:
    """Positions, rank map and counts of an externally chosen retention mask [B, T]."""

    if mask.ndim != 2 or mask.dtype != torch.bool:
        raise ValueError("mask must be bool [batch, tokens]")
    scores = torch.zeros(mask.shape, dtype=torch.float32, device=mask.device)
    return retain_tokens(scores, fraction=1.0, eligible=mask, force_last_token=False)


def _move(gather: bool, full: torch.Tensor, compact: torch.Tensor, positions: torch.Tensor,
          count: torch.Tensor, per_sequence: int) -> None:
    if full.ndim != 3 or compact.ndim != 3 or full.shape[0] != compact.shape[0] or full.shape[2] != compact.shape[2]:
        raise ValueError("arrays must be [outer, rows, width] with equal outer and width")
    if full.dtype != compact.dtype:
        raise TypeError("arrays must share a dtype")
    if not (full.is_contiguous() and compact.is_contiguous()):
        raise ValueError("arrays must be contiguous")
    _native.require_cuda(full, compact, positions, count)
    row_bytes = int(full.shape[2]) * full.element_size()
    lib = _native.load()
    fn = lib.fl_gather_rows if gather else lib.fl_scatter_rows
    _native.check(fn(_native.ptr(full), _native.ptr(compact), _native.ptr(positions), _native.ptr(count),
                     int(positions.stride(0)), int(full.shape[0]), int(per_sequence), int(full.shape[1]),
                     int(compact.shape[1]), row_bytes, _native.current_stream(full.device)),
                  "fl_gather_rows" if gather else "fl_scatter_rows")


def gather_rows(full: torch.Tensor, positions: torch.Tensor, count: torch.Tensor, *, rows: int,
                per_sequence: int = 1) -> torch.Tensor:
    """compact[o, r] = full[o, positions[o // per_sequence, r]] for r < count.  ``full`` is
    [outer, T, width]; returns [outer, rows, width] (rows beyond count are left unset)."""

    compact = torch.empty((full.shape[0], int(rows), full.shape[2]), dtype=full.dtype, device=full.device)
    _move(True, full, compact, positions, count, per_sequence)
    return compact


def scatter_rows(full: torch.Tensor, compact: torch.Tensor, positions: torch.Tensor, count: torch.Tensor, *,
                 per_sequence: int = 1) -> None:
    """full[o, positions[o // per_sequence, r]] = compact[o, r] for r < count (in place)."""

    _move(False, full, compact, positions, count, per_sequence)
