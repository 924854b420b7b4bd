"""Dense and compact-row prefill loops for a batch of equally long prompts.

Mirrors flashloop/prefill.py:122-342 (``_execute_prefill_loop``, ``dense_prefill_loop``,
``sparse_prefill_loop``, ``PrefillReceipt``): a late loop sends only its retained rows
through Q/K/V, the output projection and the MLP, while every retained query still attends the
full causal composite K/V.  The GEMMs and SDPA are library calls; the row movement (gather of
retained rows, scatter of their results) goes through ``compaction.gather_rows`` /
``scatter_rows`` instead of ``index_select`` / ``index_copy_``.

Every sequence of the batch retains the same number of rows (the budget is a function of the
prompt length only), so compact tensors are rectangular.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Sequence

import torch
from torch import nn
from torch.nn import functional as F

from .compaction import RetainedTokens, gather_rows, scatter_rows
from .weights import fused_mlp, project_qkv


@dataclass(frozen=True)
class PrefillCompositeCache:
    """One full K/V version per physical layer, [B, H, T, D] (prefill.py:21-34)."""

    keys: list
    values: list


@dataclass(frozen=True)
class PrefillReceipt:
    """Proof that late-loop work scales with the retained rows (prefill.py:46-58)."""

    loop: int
    total_rows: int
    active_rows: int
    qkv_rows: int
    output_projection_rows: int
    mlp_rows: int
    dense_target_calls: int
    sparse_target_calls: int


@dataclass(frozen=True)
class PrefillLoopOutput:
    hidden_states: torch.Tensor
    composite_cache: PrefillCompositeCache
    receipt: PrefillReceipt
    # a late loop: per layer the (K, V) of its retained rows only, [B, H, rows, D] in position order
    updates: tuple = ()


def _rotate_half(values: torch.Tensor) -> torch.Tensor:
    first, second = values.chunk(2, dim=-1)
    return torch.cat((-second, first), dim=-1)


def apply_rope(query, key, cos, sin):
    """engine.py:64-75 / prefill.py:74-85: cos/sin are [B, rows, D]."""

    cos, sin = cos.unsqueeze(1), sin.unsqueeze(1)
    return query * cos + _rotate_half(query) * sin, key * cos + _rotate_half(key) * sin


def _heads(x: torch.Tensor, heads: int, head_dim: int) -> torch.Tensor:
    batch, rows, _ = x.shape
    return x.view(batch, rows, heads, head_dim).transpose(1, 2)


def _identity(t: torch.Tensor) -> torch.Tensor:
    return t


def _layer_tail(layer: nn.Module, residual: torch.Tensor, attention_output: torch.Tensor, reduce) -> torch.Tensor:
    hidden = residual + layer.input_layernorm_2(attention_output)
    mlp_out = reduce(fused_mlp(layer.mlp, layer.post_attention_layernorm(hidden)))
    return hidden + layer.post_attention_layernorm_2(mlp_out)


def dense_prefill_loop(layers: Sequence[nn.Module], hidden_states: torch.Tensor, *, position_embeddings,
                       final_norm: nn.Module, loop: int, reduce=_identity) -> PrefillLoopOutput:
    """One dense recurrent loop: every row is recomputed (prefill.py:275-304).  ``reduce`` completes
    the row-parallel partial sums of ``o_proj`` / ``down_proj`` under tensor parallelism."""

    batch, tokens, hidden_size = hidden_states.shape
    cos, sin = position_embeddings
    keys, values = [], []
    hidden = hidden_states
    for layer in layers:
        attention = layer.self_attn
        head_dim = int(attention.head_dim)
        q, k, v = project_qkv(attention, layer.input_layernorm(hidden))
        heads = q.shape[-1] // head_dim
        q, k, v = _heads(q, heads, head_dim), _heads(k, heads, head_dim), _heads(v, heads, head_dim)
        q, k = apply_rope(q, k, cos, sin)
        k, v = k.contiguous(), v.contiguous()
        keys.append(k)
        values.append(v)
        out = F.scaled_dot_product_attention(q, k, v, dropout_p=0.0, is_causal=True)
        out = reduce(attention.o_proj(out.transpose(1, 2).reshape(batch, tokens, -1)))
        hidden = _layer_tail(layer, hidden, out, reduce)
    hidden = final_norm(hidden)
    n = len(layers)
    receipt = PrefillReceipt(loop, batch * tokens, batch * tokens, 3 * batch * tokens * n, batch * tokens * n,
                             batch * tokens * n, n, 0)
    return PrefillLoopOutput(hidden, PrefillCompositeCache(keys, values), receipt)


def sparse_prefill_loop(layers: Sequence[nn.Module], hidden_states: torch.Tensor, *, retained: RetainedTokens,
                        composite_cache: PrefillCompositeCache, position_embeddings, final_norm: nn.Module,
                        loop: int, reduce=_identity, consume_inputs: bool = False) -> PrefillLoopOutput:
    """A late loop over the retained rows only (prefill.py:307-342).  Returns full composites with
    the retained rows replaced and, per layer, the compact K/V of those rows (``updates``).  With
    ``consume_inputs`` the rows are written into the tensors of ``composite_cache`` themselves
    (prefill.py:236-237), so no second full-size composite ever exists; the hidden states are
    always copied (they are small, and the Loop-4 score needs the previous loop's)."""

    if int(loop) not in (3, 4):
        raise ValueError("sparse prefill is defined for Loop 3 or Loop 4")
    batch, tokens, hidden_size = hidden_states.shape
    counts = retained.count.tolist()
    rows = int(counts[0])
    if any(c != rows for c in counts) or rows <= 0:
        raise ValueError("every sequence must retain the same, positive number of rows")
    positions, count = retained.positions, retained.count
    cos_full, sin_full = position_embeddings
    cos = gather_rows(cos_full.contiguous(), positions, count, rows=rows)
    sin = gather_rows(sin_full.contiguous(), positions, count, rows=rows)
    hidden = hidden_states.clone()
    active = gather_rows(hidden, positions, count, rows=rows)
    # retained queries attend the causal prefix of the full composite
    pos = positions[:, :rows].long()
    allowed = torch.arange(tokens, device=hidden.device)[None, None, :] <= pos[:, :, None]
    attn_mask = torch.zeros((batch, 1, rows, tokens), dtype=hidden.dtype, device=hidden.device)
    attn_mask.masked_fill_(~allowed[:, None], float("-inf"))
    keys, values, updates = [], [], []
    for index, layer in enumerate(layers):
        attention = layer.self_attn
        head_dim = int(attention.head_dim)
        q, k, v = project_qkv(attention, layer.input_layernorm(active))
        heads = q.shape[-1] // head_dim
        q, k, v = _heads(q, heads, head_dim), _heads(k, heads, head_dim), _heads(v, heads, head_dim)
        q, k = apply_rope(q, k, cos, sin)
        k, v = k.contiguous(), v.contiguous()
        full_k, full_v = composite_cache.keys[index], composite_cache.values[index]
        if not consume_inputs:
            full_k, full_v = full_k.clone(), full_v.clone()
        scatter_rows(full_k.view(batch * heads, tokens, head_dim), k.view(batch * heads, rows, head_dim),
                     positions, count, per_sequence=heads)
        scatter_rows(full_v.view(batch * heads, tokens, head_dim), v.view(batch * heads, rows, head_dim),
                     positions, count, per_sequence=heads)
        keys.append(full_k)
        values.append(full_v)
        updates.append((k, v))
        out = F.scaled_dot_product_attention(q, full_k, full_v, attn_mask=attn_mask, dropout_p=0.0)
        out = reduce(attention.o_proj(out.transpose(1, 2).reshape(batch, rows, -1)))
        active = _layer_tail(layer, active, out, reduce)
    active = final_norm(active)
    scatter_rows(hidden, active.contiguous(), positions, count)
    n = len(layers)
    receipt = PrefillReceipt(loop, batch * tokens, batch * rows, 3 * batch * rows * n, batch * rows * n,
                             batch * rows * n, 0, n)
    return PrefillLoopOutput(hidden, PrefillCompositeCache(keys, values), receipt, tuple(updates))
