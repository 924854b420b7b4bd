"""Helpers shared by the GPU parity tests: torch <-> numpy oracle conversions."""

from __future__ import annotations

import numpy as np
import torch

from oracle import bf16
from oracle.cache import LayerOracle


def to_np(t: torch.Tensor) -> np.ndarray:
    """bf16/f16/f32 tensor -> float32 numpy (exact)."""
    return t.detach().float().cpu().numpy()


def bf16_tensor(a: np.ndarray, device="cuda") -> torch.Tensor:
    """float32 numpy holding bf16 values -> bf16 tensor (exact)."""
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(torch.bfloat16).to(device)


def bits16(t: torch.Tensor) -> np.ndarray:
    return t.detach().contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def oracle_layer(keys, values, mask3, mask4, bits=4) -> LayerOracle:
    """keys/values: four torch tensors [1,H,T,128]; masks bool [T]."""
    return LayerOracle.from_prefill([to_np(k) for k in keys], [to_np(v) for v in values],
                                    mask_loop3=mask3.cpu().numpy(), mask_loop4=mask4.cpu().numpy(),
                                    bits=bits)


def assert_stream_matches(exported: dict, s: int, ok, ov, what=""):
    """Device stream ``s`` of an exported sequence vs oracle PackedRows ``ok``/``ov``."""
    if ok is None:
        assert exported[f"k{s}.payload"].shape[1] == 0, what
        return
    np.testing.assert_array_equal(exported[f"k{s}.payload"].cpu().numpy(), ok.payload[0], err_msg=f"{what} k{s} payload")
    np.testing.assert_array_equal(bits16(exported[f"k{s}.minimum"]), ok.minimum[0].view(np.uint16), err_msg=f"{what} k{s} min")
    np.testing.assert_array_equal(bits16(exported[f"k{s}.scale"]), ok.scale[0].view(np.uint16), err_msg=f"{what} k{s} scale")
    np.testing.assert_array_equal(exported[f"v{s}.payload"].cpu().numpy(), ov.payload[0], err_msg=f"{what} v{s} payload")
    np.testing.assert_array_equal(bits16(exported[f"v{s}.minimum"]), ov.minimum[0].view(np.uint16), err_msg=f"{what} v{s} min")
    np.testing.assert_array_equal(bits16(exported[f"v{s}.scale"]), ov.scale[0].view(np.uint16), err_msg=f"{what} v{s} scale")
    if ok.row_groups is not None:
        np.testing.assert_array_equal(exported[f"k{s}.row_groups"].cpu().numpy(), ok.row_groups, err_msg=f"{what} k{s} groups")


def assert_layer_matches(layer, b: int, oracle: LayerOracle, what=""):
    ex = layer.export_sequence(b)
    assert ex["quantized_tokens"] == oracle.quantized_tokens, what
    assert ex["tail_tokens"] == oracle.tail_tokens, what
    for s in range(4):
        assert_stream_matches(ex, s, oracle.keys[s], oracle.values[s], what)
    if oracle.quantized_tokens:
        np.testing.assert_array_equal(ex["rank3"].cpu().numpy(), oracle.rank_maps[0], err_msg=what + " rank3")
        np.testing.assert_array_equal(ex["rank4"].cpu().numpy(), oracle.rank_maps[1], err_msg=what + " rank4")
        np.testing.assert_array_equal(ex["pos3"].cpu().numpy(), oracle.override_indices[0], err_msg=what + " pos3")
    for r in range(4):
        np.testing.assert_array_equal(bits16(ex[f"tail_k{r}"]), bf16.to_bits(oracle.tail_keys[r][0]), err_msg=f"{what} tail_k{r}")
        np.testing.assert_array_equal(bits16(ex[f"tail_v{r}"]), bf16.to_bits(oracle.tail_values[r][0]), err_msg=f"{what} tail_v{r}")
    np.testing.assert_array_equal(ex["tail_active3"].cpu().numpy(), oracle.tail_active[0], err_msg=what + " active3")
    np.testing.assert_array_equal(ex["tail_active4"].cpu().numpy(), oracle.tail_active[1], err_msg=what + " active4")


def max_err(a, b) -> float:
    return float(np.max(np.abs(np.asarray(a, np.float64) - np.asarray(b, np.float64))))


def assert_bf16_tolerance(actual, desired, what=""):
    """The reader tolerance: 2e-2 max-abs / 1e-2 relative."""
    np.testing.assert_allclose(actual, desired, rtol=1e-2, atol=2e-2, err_msg=what)
