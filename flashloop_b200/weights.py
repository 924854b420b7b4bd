"""Fused projection weights (flashloop/weights.py:20-117): Q/K/V and gate/up are stored as one
buffer each so that a decode step issues one GEMM instead of three / two.  The GEMMs themselves
are library calls (cuBLAS through ``F.linear``)."""

from __future__ import annotations

from collections.abc import Sequence

import torch
from torch import nn
from torch.nn import functional as F


@torch.no_grad()
def repack_projection_weights(layers: Sequence[nn.Module]) -> None:
    """weights.py:20-71: concatenate the weights, register them as buffers, release the originals."""

    for layer in layers:
        attention, mlp = layer.self_attn, layer.mlp
        if hasattr(attention, "_flashloop_qkv_weight"):
            if not hasattr(mlp, "_flashloop_gate_up_weight"):
                raise RuntimeError("partially repacked FlashLoop layer")
            continue
        modules = {"q_proj": attention.q_proj, "k_proj": attention.k_proj, "v_proj": attention.v_proj,
                   "gate_proj": mlp.gate_proj, "up_proj": mlp.up_proj}
        for name, module in modules.items():
            if module.bias is not None:
                raise ValueError(f"FlashLoop fused projection requires biasless {name}")
            if module.weight is None:
                raise ValueError(f"{name} has already released its weight")
        attention._flashloop_qkv_splits = tuple(int(modules[n].out_features) for n in ("q_proj", "k_proj", "v_proj"))
        mlp._flashloop_gate_up_splits = (int(mlp.gate_proj.out_features), int(mlp.up_proj.out_features))
        attention.register_buffer("_flashloop_qkv_weight", torch.cat(
            [modules[n].weight for n in ("q_proj", "k_proj", "v_proj")], dim=0).detach(), persistent=False)
        mlp.register_buffer("_flashloop_gate_up_weight", torch.cat(
            [mlp.gate_proj.weight, mlp.up_proj.weight], dim=0).detach(), persistent=False)
        for module in modules.values():
            module.weight = None


def project_qkv(attention: nn.Module, values: torch.Tensor):
    """weights.py:74-88."""

    weight = getattr(attention, "_flashloop_qkv_weight", None)
    if weight is None:
        return attention.q_proj(values), attention.k_proj(values), attention.v_proj(values)
    return tuple(F.linear(values, weight).split(attention._flashloop_qkv_splits, dim=-1))


def project_value(attention: nn.Module, values: torch.Tensor) -> torch.Tensor:
    """weights.py:91-105: only V, from the packed QKV weight without copying it."""

    weight = getattr(attention, "_flashloop_qkv_weight", None)
    if weight is None:
        return attention.v_proj(values)
    q_features, k_features, v_features = attention._flashloop_qkv_splits
    return F.linear(values, weight.narrow(0, q_features + k_features, v_features))


def fused_mlp(mlp: nn.Module, values: torch.Tensor) -> torch.Tensor:
    """weights.py:108-117."""

    weight = getattr(mlp, "_flashloop_gate_up_weight", None)
    if weight is None:
        return mlp(values)
    gate, up = F.linear(values, weight).split(mlp._flashloop_gate_up_splits, dim=-1)
    return mlp.down_proj(mlp.act_fn(gate) * up)
