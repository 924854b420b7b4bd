"""Host-side logic of the engine row: configuration contract, model validation, fused projection
weights, and that the engine refuses to run without the CUDA path (no CPU fallback)."""

from __future__ import annotations

import pytest
import torch

from flashloop_b200 import FlashLoopConfig, FlashLoopEngine
from flashloop_b200.config import validate_ouro_model
from flashloop_b200.ouro_shape import OuroShapedConfig, OuroShapedForCausalLM
from flashloop_b200.selection import decode_budget, padded_capacity
from flashloop_b200.weights import fused_mlp, project_qkv, repack_projection_weights

from tests.helpers import tiny_ouro_model


def test_config_defaults_and_fractions():
    cfg = FlashLoopConfig()
    assert cfg.effective_prefill_fractions == (0.25, 0.10)
    assert cfg.effective_decode_key_fraction == 0.10
    assert FlashLoopConfig(enable_token_sparse_prefill=False).effective_prefill_fractions == (1.0, 1.0)
    assert FlashLoopConfig(enable_sparse_decode=False).effective_decode_key_fraction == 1.0
    assert FlashLoopConfig(kv_bits=2).kv_bits == 2
    assert FlashLoopConfig(reuse_selected_probabilities=True).reuse_selected_probabilities


@pytest.mark.parametrize("kwargs", [
    dict(prefill_fraction_loop3=0.05, prefill_fraction_loop4=0.10),
    dict(decode_key_fraction=0.0),
    dict(kv_bits=8),
    dict(group_size=32),
    dict(residual_length=128),
    dict(absolute_late_overrides=True),
    dict(kv_reader_backend="triton_row"),
    dict(quantize_cross_loop_kv=False),
])
def test_config_rejects(kwargs):
    with pytest.raises(ValueError):
        FlashLoopConfig(**kwargs)


def test_config_type_check():
    with pytest.raises(TypeError):
        FlashLoopConfig(enable_sparse_decode=1)


def test_validate_ouro_model_contract():
    full = OuroShapedConfig(num_hidden_layers=24, hidden_size=256, intermediate_size=128,
                            num_attention_heads=2, vocab_size=64)
    spec = validate_ouro_model(OuroShapedForCausalLM(full))
    assert (spec.num_layers, spec.num_heads, spec.head_dim, spec.total_loops) == (24, 2, 128, 4)
    tiny = tiny_ouro_model()
    with pytest.raises(ValueError, match="24 or 48"):
        validate_ouro_model(tiny)
    tiny.config.total_ut_steps = 3
    with pytest.raises(ValueError, match="four"):
        validate_ouro_model(tiny)
    with pytest.raises(ValueError, match="four"):
        FlashLoopEngine(tiny, validate_model=False)
    with pytest.raises(ValueError):
        validate_ouro_model(object())


def test_repacked_projections_match_separate_ones():
    model = tiny_ouro_model().float()
    layer = model.model.layers[0]
    x = torch.randn(2, 5, 256, generator=torch.Generator().manual_seed(0))
    q0, k0, v0 = project_qkv(layer.self_attn, x)
    m0 = fused_mlp(layer.mlp, x)
    repack_projection_weights(model.model.layers)
    assert layer.self_attn.q_proj.weight is None and layer.mlp.gate_proj.weight is None
    q1, k1, v1 = project_qkv(layer.self_attn, x)
    for a, b in ((q0, q1), (k0, k1), (v0, v1), (m0, fused_mlp(layer.mlp, x))):
        torch.testing.assert_close(a, b, atol=1e-5, rtol=1e-5)
    repack_projection_weights(model.model.layers)  # idempotent


def test_decode_budget_and_capacity():
    assert decode_budget(201, 0.10) == 21
    assert decode_budget(1, 0.10) == 1
    assert decode_budget(5, 1.0) == 5
    assert padded_capacity(21) == 64 and padded_capacity(64) == 128 and padded_capacity(820) == 832


def test_engine_state_errors_and_no_cpu_fallback():
    engine = FlashLoopEngine(tiny_ouro_model(), validate_model=False)
    with pytest.raises(RuntimeError, match="not initialized"):
        engine.state
    with pytest.raises(ValueError):
        engine.prefill(torch.zeros((2, 0), dtype=torch.long))
    with pytest.raises(ValueError, match="padding"):
        engine.prefill(torch.zeros((1, 4), dtype=torch.long), torch.tensor([[1, 1, 0, 1]]))
    # a CPU model reaches the first CUDA entry point and stops there
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        engine.prefill(torch.zeros((1, 8), dtype=torch.long))
    with pytest.raises(ValueError, match="positive"):
        engine.generate(torch.zeros((1, 8), dtype=torch.long), max_new_tokens=0)
    with pytest.raises(ValueError, match="preallocated"):
        engine.generate(torch.zeros((1, 8), dtype=torch.long), max_new_tokens=10_000)
