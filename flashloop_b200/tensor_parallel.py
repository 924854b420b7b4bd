"""Head / FFN-column tensor parallelism for the end-to-end configurations.

Attention shards by head with no traffic inside it (every reader, selection and append kernel is
independent per (sequence, head)); the only exchange of a decoder layer is the sum of the
row-parallel ``o_proj`` and ``down_proj`` outputs, one NCCL all-reduce each.  The reference is
single-GPU (flashloop/engine.py:112-150), so this module has no counterpart there; the sharded
modules keep the attribute names the engine walks (flashloop/engine.py:396-437, 533-537).
"""

from __future__ import annotations

import torch
import torch.distributed as dist
from torch import nn


def shard_range(total: int, world: int, rank: int) -> tuple[int, int]:
    if total % world:
        raise ValueError(f"{total} does not divide over {world} ranks")
    per = total // world
    return rank * per, (rank + 1) * per


def _rows(linear: nn.Linear, lo: int, hi: int) -> None:
    """Keep output features [lo, hi) (column-parallel)."""

    linear.weight = nn.Parameter(linear.weight.data[lo:hi].clone(), requires_grad=False)
    linear.out_features = hi - lo


def _cols(linear: nn.Linear, lo: int, hi: int) -> None:
    """Keep input features [lo, hi) (row-parallel: the outputs are partial sums)."""

    linear.weight = nn.Parameter(linear.weight.data[:, lo:hi].clone(), requires_grad=False)
    linear.in_features = hi - lo


@torch.no_grad()
def shard_ouro_model(model: nn.Module, rank: int, world: int) -> nn.Module:
    """Slice an Ouro-style model in place to ``rank``'s heads and FFN columns.  Embeddings, norms
    and the LM head stay replicated.  Call before the engine repacks the projections."""

    if world == 1:
        return model
    for layer in model.model.layers:
        attention, mlp = layer.self_attn, layer.mlp
        if hasattr(attention, "_flashloop_qkv_weight"):
            raise RuntimeError("shard the model before its projections are repacked")
        head_dim = int(attention.head_dim)
        heads = attention.q_proj.out_features // head_dim
        kv_heads = attention.k_proj.out_features // head_dim
        h0, h1 = shard_range(heads, world, rank)
        g0, g1 = shard_range(kv_heads, world, rank)
        _rows(attention.q_proj, h0 * head_dim, h1 * head_dim)
        _rows(attention.k_proj, g0 * head_dim, g1 * head_dim)
        _rows(attention.v_proj, g0 * head_dim, g1 * head_dim)
        _cols(attention.o_proj, h0 * head_dim, h1 * head_dim)
        f0, f1 = shard_range(mlp.gate_proj.out_features, world, rank)
        _rows(mlp.gate_proj, f0, f1)
        _rows(mlp.up_proj, f0, f1)
        _cols(mlp.down_proj, f0, f1)
    return model


class PartialSum:
    """Callable that turns a row-parallel partial sum into the full sum, in place."""

    def __init__(self, group=None) -> None:
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_available() and dist.is_initialized() else 1

    def __call__(self, partial: torch.Tensor) -> torch.Tensor:
        if self.world > 1:
            dist.all_reduce(partial, group=self.group)
        return partial
