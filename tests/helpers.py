"""Conversions between golden arrays, numpy oracle arrays and torch tensors."""

from __future__ import annotations

import numpy as np

from oracle import bf16
from oracle.packing import PackedKivi, PackedRows


def bf(bits: np.ndarray) -> np.ndarray:
    """uint16 bf16 bit patterns -> float32."""
    return bf16.from_bits(bits)


def f16(bits: np.ndarray) -> np.ndarray:
    return bits.view(np.float16)


def golden_inputs(g):
    keys = [bf(g[f"in.key{r}"]) for r in range(4)]
    values = [bf(g[f"in.value{r}"]) for r in range(4)]
    return keys, values, g["in.mask3"], g["in.mask4"], bf(g["in.query"]), bf(g["in.cur_k"]), bf(g["in.cur_v"])


def golden_stream(g, prefix):
    """Reference stream as stored by make_golden.put_stream, or None."""
    if prefix + ".none" in g:
        return None
    return {
        "payload": g[prefix + ".payload"],
        "minimum": f16(g[prefix + ".minimum"]),
        "scale": f16(g[prefix + ".scale"]),
        "shape": tuple(int(v) for v in g[prefix + ".shape"]),
        "row_groups": g.get(prefix + ".row_groups"),
    }


def assert_rows_equal(packed: PackedRows | None, ref, *, what=""):
    if ref is None:
        assert packed is None, what
        return
    assert packed is not None, what
    assert packed.shape == ref["shape"], what
    np.testing.assert_array_equal(packed.payload, ref["payload"], err_msg=what + " payload")
    np.testing.assert_array_equal(packed.minimum.view(np.uint16), ref["minimum"].view(np.uint16),
                                  err_msg=what + " minimum")
    np.testing.assert_array_equal(packed.scale.view(np.uint16), ref["scale"].view(np.uint16),
                                  err_msg=what + " scale")


def assert_kivi_equal(packed: PackedKivi | None, ref, *, what=""):
    if ref is None:
        assert packed is None, what
        return
    assert packed.shape == ref["shape"], what
    np.testing.assert_array_equal(packed.payload, ref["payload"], err_msg=what + " payload")
    np.testing.assert_array_equal(packed.minimum.view(np.uint16), ref["minimum"].view(np.uint16),
                                  err_msg=what + " minimum")
    np.testing.assert_array_equal(packed.scale.view(np.uint16), ref["scale"].view(np.uint16),
                                  err_msg=what + " scale")


TINY_OURO = dict(vocab_size=256, hidden_size=256, intermediate_size=384, num_hidden_layers=2,
                 num_attention_heads=2)


def tiny_ouro_model(seed: int = 11):
    """A two-layer, two-head Ouro-shaped model whose weights come from numpy's legacy
    RandomState, so the golden script and the tests build the same bfloat16 tensors on any
    machine and any torch version."""

    import torch

    from flashloop_b200.ouro_shape import OuroShapedConfig, OuroShapedForCausalLM

    model = OuroShapedForCausalLM(OuroShapedConfig(**TINY_OURO))
    rng = np.random.RandomState(seed)
    with torch.no_grad():
        for name, param in sorted(model.named_parameters()):
            if param.ndim >= 2:
                w = rng.standard_normal(param.shape).astype(np.float32) * (0.08 if "embed" not in name else 1.0)
            else:
                w = 1.0 + 0.1 * rng.standard_normal(param.shape).astype(np.float32)
            param.copy_(torch.from_numpy(w).to(param.dtype))
    return model.eval()
