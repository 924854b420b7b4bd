"""A random-init decoder with the attributes the engine touches on an Ouro checkpoint.

There are no Ouro weights or modelling code in this build's environment, so the end-to-end
configurations run on this stand-in: same widths, same layer structure (sandwich RMSNorms,
MHA with rotate-half RoPE, SwiGLU), same attribute names as the module tree the reference's
engine walks (flashloop/config.py:95-126, flashloop/engine.py:128-129, 184-187, 396-437,
533-537).  RoPE theta is not fixed by the reference's repository; 10000 is used.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch
from torch import nn


@dataclass
class OuroShapedConfig:
    num_hidden_layers: int = 24
    hidden_size: int = 2048
    intermediate_size: int = 5632
    num_attention_heads: int = 16
    num_key_value_heads: int | None = None
    head_dim: int = 128
    vocab_size: int = 49152
    total_ut_steps: int = 4
    rope_theta: float = 10000.0
    rms_norm_eps: float = 1e-6
    model_type: str = "ouro"
    sliding_window: int | None = None
    eos_token_id: int | None = None
    layer_types: tuple = field(default=())

    def __post_init__(self) -> None:
        if self.num_key_value_heads is None:
            self.num_key_value_heads = self.num_attention_heads
        if not self.layer_types:
            self.layer_types = tuple("full_attention" for _ in range(self.num_hidden_layers))


class RMSNorm(nn.Module):
    def __init__(self, width: int, eps: float) -> None:
        super().__init__()
        self.weight = nn.Parameter(torch.ones(width))
        self.eps = eps

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        work = x.float()
        work = work * torch.rsqrt(work.pow(2).mean(-1, keepdim=True) + self.eps)
        return (self.weight * work.to(x.dtype))


class Rotary(nn.Module):
    def __init__(self, head_dim: int, theta: float) -> None:
        super().__init__()
        inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))
        self.register_buffer("inv_freq", inv, persistent=False)

    @torch.no_grad()
    def forward(self, hidden: torch.Tensor, position_ids: torch.Tensor):
        freqs = position_ids[..., None].float() * self.inv_freq.float()
        emb = torch.cat((freqs, freqs), dim=-1)
        return emb.cos().to(hidden.dtype), emb.sin().to(hidden.dtype)


class Attention(nn.Module):
    def __init__(self, cfg: OuroShapedConfig) -> None:
        super().__init__()
        self.head_dim = cfg.head_dim
        self.scaling = cfg.head_dim ** -0.5
        self.num_key_value_groups = cfg.num_attention_heads // cfg.num_key_value_heads
        self.q_proj = nn.Linear(cfg.hidden_size, cfg.num_attention_heads * cfg.head_dim, bias=False)
        self.k_proj = nn.Linear(cfg.hidden_size, cfg.num_key_value_heads * cfg.head_dim, bias=False)
        self.v_proj = nn.Linear(cfg.hidden_size, cfg.num_key_value_heads * cfg.head_dim, bias=False)
        self.o_proj = nn.Linear(cfg.num_attention_heads * cfg.head_dim, cfg.hidden_size, bias=False)


class MLP(nn.Module):
    def __init__(self, cfg: OuroShapedConfig) -> None:
        super().__init__()
        self.gate_proj = nn.Linear(cfg.hidden_size, cfg.intermediate_size, bias=False)
        self.up_proj = nn.Linear(cfg.hidden_size, cfg.intermediate_size, bias=False)
        self.down_proj = nn.Linear(cfg.intermediate_size, cfg.hidden_size, bias=False)
        self.act_fn = nn.SiLU()

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.down_proj(self.act_fn(self.gate_proj(x)) * self.up_proj(x))


class DecoderLayer(nn.Module):
    def __init__(self, cfg: OuroShapedConfig) -> None:
        super().__init__()
        self.self_attn = Attention(cfg)
        self.mlp = MLP(cfg)
        self.input_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps)
        self.input_layernorm_2 = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps)
        self.post_attention_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps)
        self.post_attention_layernorm_2 = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps)


class Backbone(nn.Module):
    def __init__(self, cfg: OuroShapedConfig) -> None:
        super().__init__()
        self.embed_tokens = nn.Embedding(cfg.vocab_size, cfg.hidden_size)
        self.layers = nn.ModuleList(DecoderLayer(cfg) for _ in range(cfg.num_hidden_layers))
        self.norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps)
        self.rotary_emb = Rotary(cfg.head_dim, cfg.rope_theta)


class OuroShapedForCausalLM(nn.Module):
    """Random-init (normal, std 0.02) four-loop decoder of the given widths.  With ``device`` the
    parameters are created and drawn there (a 1.4B-parameter model takes a second on a GPU)."""

    def __init__(self, cfg: OuroShapedConfig, *, seed: int = 0, dtype: torch.dtype = torch.bfloat16,
                 device: str | torch.device | None = None) -> None:
        super().__init__()
        self.config = cfg
        device = torch.device(device) if device is not None else torch.device("cpu")
        with torch.device(device):
            self.model = Backbone(cfg)
            self.lm_head = nn.Linear(cfg.hidden_size, cfg.vocab_size, bias=False)
        self.to(dtype)
        gen = torch.Generator(device=device).manual_seed(seed)
        with torch.no_grad():
            for name, param in self.named_parameters():
                if param.ndim >= 2:
                    param.copy_(torch.randn(param.shape, generator=gen, device=device, dtype=torch.float32) * 0.02)
