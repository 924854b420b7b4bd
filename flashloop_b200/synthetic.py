"""Seeded synthetic loop K/V in the shapes of the benchmark configurations.

Loop-1 K and V are N(0, 1); a few K channels are scaled up as outliers; every later
loop adds N(0, residual_std) to the previous loop's K/V.  Everything is rounded to
bfloat16, the cache's storage dtype.  There is no dataset behind these tensors:
they stand in for the K/V a four-loop Ouro-shaped decoder would produce.
"""

from __future__ import annotations

import torch


def make_loop_kv(heads: int, tokens: int, *, head_dim: int = 128, loops: int = 4,
                 seed: int = 0, outlier_channels: int = 4, outlier_scale: float = 8.0,
                 residual_std: float = 0.1, device: str | torch.device = "cpu"):
    """One sequence: lists of ``loops`` K and V tensors [1, heads, tokens, head_dim] bf16.

    A CPU generator is used when ``device`` is the CPU (bit-reproducible across
    machines for one torch version); on a CUDA device the generator lives on the
    device so that large benchmark tensors never cross PCIe."""

    device = torch.device(device)
    gen = torch.Generator(device=device).manual_seed(int(seed))
    shape = (1, heads, tokens, head_dim)

    def normal() -> torch.Tensor:
        return torch.randn(shape, generator=gen, device=device, dtype=torch.float32)

    key = normal()
    value = normal()
    if outlier_channels:
        picks = torch.randperm(head_dim, generator=gen, device=device)[:outlier_channels]
        key[..., picks] *= outlier_scale
    keys = [key.to(torch.bfloat16)]
    values = [value.to(torch.bfloat16)]
    for _ in range(1, loops):
        keys.append((keys[-1].float() + residual_std * normal()).to(torch.bfloat16))
        values.append((values[-1].float() + residual_std * normal()).to(torch.bfloat16))
    return keys, values


def make_query(heads: int, *, head_dim: int = 128, seed: int = 0,
               device: str | torch.device = "cpu"):
    """Query, current key and current value of one decode step, each [1, heads, 1, head_dim]."""

    device = torch.device(device)
    gen = torch.Generator(device=device).manual_seed(int(seed) + 7919)
    make = lambda: torch.randn((1, heads, 1, head_dim), generator=gen, device=device,
                               dtype=torch.float32).to(torch.bfloat16)
    return make(), make(), make()


def make_masks(tokens: int, *, fraction3: float = 0.25, fraction4: float = 0.10,
               seed: int = 0, all_active: bool = False):
    """Nested loop-3/loop-4 retention masks [tokens] with the last token forced on."""

    if all_active:
        ones = torch.ones(tokens, dtype=torch.bool)
        return ones, ones.clone()
    import math

    gen = torch.Generator().manual_seed(int(seed) + 104729)
    score = torch.rand(tokens, generator=gen)
    score[-1] = 2.0
    n3 = max(1, math.ceil(tokens * fraction3))
    n4 = max(1, math.ceil(tokens * fraction4))
    order = torch.argsort(score, descending=True)
    mask3 = torch.zeros(tokens, dtype=torch.bool)
    mask3[order[:n3]] = True
    mask4 = torch.zeros(tokens, dtype=torch.bool)
    mask4[order[:n4]] = True
    return mask3, mask4
