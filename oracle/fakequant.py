"""Fake-quant closed-loop codec (numpy oracle) -- the tolerance target for attention.

Restates flashloop_torch/kv_quantization.py:395-486 and 531-602: a min/max
asymmetric quantise-dequantise with float32 ``min``/``scale`` (no float16 rounding
of the metadata), K per channel over 64-token groups, V per token over 64-channel
groups, applied to the anchor loop and then to each loop-to-loop residual of the
active rows, with every intermediate tensor held in the input dtype (bfloat16).
"""

from __future__ import annotations

import numpy as np

from . import bf16

PROFILE_BITS = {"kivi4_channel": 4, "kivi2_channel": 2}


def _fake_quant(values: np.ndarray, *, bits: int, reduce_axis: int) -> np.ndarray:
    """kv_quantization.py:395-414 (result cast back to bfloat16)."""

    if values.size == 0:
        return values.copy()
    work = values.astype(np.float32)
    levels = np.float32((1 << bits) - 1)
    minimum = work.min(axis=reduce_axis, keepdims=True)
    span = (work.max(axis=reduce_axis, keepdims=True) - minimum).astype(np.float32)
    scale = np.where(span > 0, span / levels, np.float32(1.0)).astype(np.float32)
    codes = np.clip(np.rint(((work - minimum).astype(np.float32) / scale).astype(np.float32)),
                    0, levels).astype(np.float32)
    return bf16.round_to_bf16((codes * scale).astype(np.float32) + minimum)


def quantize_dequantize_k_per_channel(values, *, bits, group_size=64):
    """kv_quantization.py:417-433."""

    chunks = [_fake_quant(values[:, :, s:s + group_size], bits=bits, reduce_axis=2)
              for s in range(0, values.shape[2], group_size)]
    return np.concatenate(chunks, axis=2) if chunks else values.copy()


def quantize_dequantize_v_per_token(values, *, bits, group_size=64):
    """kv_quantization.py:436-452."""

    chunks = [_fake_quant(values[..., s:s + group_size], bits=bits, reduce_axis=3)
              for s in range(0, values.shape[3], group_size)]
    return np.concatenate(chunks, axis=3) if chunks else values.copy()


def _quantize_active_delta(delta, mask, *, bits, axis, group_size):
    """kv_quantization.py:455-486: only active rows carry a residual (batch of one)."""

    out = np.zeros_like(delta)
    positions = np.nonzero(np.asarray(mask, bool).reshape(-1))[0]
    if positions.size == 0:
        return out
    selected = delta[:, :, positions]
    fn = quantize_dequantize_k_per_channel if axis == "per_channel" else quantize_dequantize_v_per_token
    out[:, :, positions] = fn(selected, bits=bits, group_size=group_size)
    return out


def encode_temporal_group(keys, values, *, active_masks=None, group_size=64,
                          codec_profile="kivi4_channel"):
    """kv_quantization.py:531-602.  keys/values: 1..4 arrays [1,H,T,D] (bf16 values in
    float32).  Returns per-loop reconstructed (keys, values)."""

    bits = PROFILE_BITS[codec_profile]
    steps = len(keys)
    tokens = keys[0].shape[2]
    if active_masks is None:
        active_masks = [np.ones(tokens, bool)] * (steps - 1)
    rk = [quantize_dequantize_k_per_channel(keys[0], bits=bits, group_size=group_size)]
    rv = [quantize_dequantize_v_per_token(values[0], bits=bits, group_size=group_size)]
    for step, mask in enumerate(active_masks, start=1):
        dk = bf16.sub(keys[step], rk[-1])
        dv = bf16.sub(values[step], rv[-1])
        rk.append(bf16.add(rk[-1], _quantize_active_delta(
            dk, mask, bits=bits, axis="per_channel", group_size=group_size)))
        rv.append(bf16.add(rv[-1], _quantize_active_delta(
            dv, mask, bits=bits, axis="per_token", group_size=group_size)))
    return rk, rv


def fake_quant_attention(keys, values, *, loop, query, current_key, current_value, scaling,
                         active_masks=None, group_size=64, residual_length=64,
                         codec_profile="kivi4_channel"):
    """The tolerance oracle for the dense reader: fake-quantise the prefix of ``loop``
    (loops 0..loop), keep the last ``T - Tq`` tokens in bf16, then
    ``softmax(q K^T scaling) V`` (same formula as flashloop/cache.py:1749-1755)."""

    tokens = keys[0].shape[2]
    packed = max(0, ((tokens - residual_length) // group_size) * group_size)
    masks = None if active_masks is None else [np.asarray(m, bool).reshape(-1)[:packed]
                                               for m in active_masks[:loop]]
    if packed:
        rk, rv = encode_temporal_group([k[:, :, :packed] for k in keys[:loop + 1]],
                                       [v[:, :, :packed] for v in values[:loop + 1]],
                                       active_masks=masks, group_size=group_size,
                                       codec_profile=codec_profile)
        k_all = np.concatenate([rk[loop], keys[loop][:, :, packed:], current_key], axis=2)
        v_all = np.concatenate([rv[loop], values[loop][:, :, packed:], current_value], axis=2)
    else:
        k_all = np.concatenate([keys[loop], current_key], axis=2)
        v_all = np.concatenate([values[loop], current_value], axis=2)
    logits = np.einsum("bhqd,bhnd->bhqn", query.astype(np.float64),
                       k_all.astype(np.float64)) * float(scaling)
    w = np.exp(logits - logits.max(axis=-1, keepdims=True))
    w /= w.sum(axis=-1, keepdims=True)
    out = np.einsum("bhqn,bhnd->bhqd", w, v_all.astype(np.float64))
    return out.astype(np.float32), logits.astype(np.float32)
