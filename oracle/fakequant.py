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


def _fake_quant_contexts(keys, values, *, loops, currents, active_masks, group_size, residual_length,
                         codec_profile):
    """K and V of every key the given loops attend: fake-quantised prefix, BF16 tail, current
    token.  The temporal group is encoded once; ``currents[loop]`` = (current_key, current_value)."""

    tokens = keys[0].shape[2]
    last = max(loops)
    packed = max(0, ((tokens - residual_length) // group_size) * group_size)
    masks = None if active_masks is None else [np.asarray(m, bool).reshape(-1)[:packed]
                                               for m in active_masks[:last]]
    if packed:
        rk, rv = encode_temporal_group([k[:, :, :packed] for k in keys[:last + 1]],
                                       [v[:, :, :packed] for v in values[:last + 1]],
                                       active_masks=masks, group_size=group_size, codec_profile=codec_profile)
    out = {}
    for loop in loops:
        current_key, current_value = currents[loop]
        if packed:
            k_all = np.concatenate([rk[loop], keys[loop][:, :, packed:], current_key], axis=2)
            v_all = np.concatenate([rv[loop], values[loop][:, :, packed:], current_value], axis=2)
        else:
            k_all = np.concatenate([keys[loop], current_key], axis=2)
            v_all = np.concatenate([values[loop], current_value], axis=2)
        out[loop] = (k_all.astype(np.float64), v_all.astype(np.float64))
    return out


def _subset_softmax(logits, mask):
    """flashloop_torch/attention_utils.py:152-168 masked_subset_softmax."""

    masked = np.where(mask, logits, -np.inf)
    w = np.exp(masked - masked.max(axis=-1, keepdims=True))
    w = np.where(mask, w, 0.0)
    return w / w.sum(axis=-1, keepdims=True)


def fake_quant_sparse_deltas(keys, values, *, loops, source_query, source_current_key, source_current_value,
                             query, current_key, current_value, scaling, fraction=0.10, active_masks=None,
                             group_size=64, residual_length=64, codec_profile="kivi4_channel"):
    """The tolerance oracle for the sparse late-loop reader: the reference's
    ``mass_scaled_sparse_output`` (flashloop_torch/attention_utils.py:216-248, both scales equal
    to the selected mass, source_output zero) over the fake-quant reconstructions.  The source is
    loop 2 (index 1) with its own query / current K,V; the keys are the top ``fraction`` of the
    source's global softmax weights (attention_utils.py:139-148, 196-213); the targets are
    ``loops`` (indices 2 and/or 3) with ``query`` / ``current_key`` / ``current_value``.

    Returns a dict: ``delta[loop]`` float32 [1,H,1,D] = mass * (target_subset - source_subset),
    ``mask`` bool [1,H,1,N+1], ``mass`` [1,H,1,1], ``source_subset`` [1,H,1,D]."""

    currents = {1: (source_current_key, source_current_value)}
    for loop in loops:
        currents[loop] = (current_key, current_value)
    ctx = _fake_quant_contexts(keys, values, loops=sorted(currents), currents=currents, active_masks=active_masks,
                               group_size=group_size, residual_length=residual_length, codec_profile=codec_profile)
    src_k, src_v = ctx[1]
    src_logits = np.einsum("bhqd,bhnd->bhqn", source_query.astype(np.float64), src_k) * float(scaling)
    weights = np.exp(src_logits - src_logits.max(axis=-1, keepdims=True))
    weights /= weights.sum(axis=-1, keepdims=True)
    n = weights.shape[-1]
    budget = min(n, max(1, int(np.ceil(n * float(fraction)))))
    order = np.argsort(-weights, axis=-1, kind="stable")[..., :budget]
    mask = np.zeros(weights.shape, bool)
    np.put_along_axis(mask, order, True, axis=-1)
    mass = (weights * mask).sum(axis=-1, keepdims=True)
    source_subset = np.einsum("bhqn,bhnd->bhqd", _subset_softmax(src_logits, mask), src_v)
    deltas = {}
    for loop in loops:
        tgt_k, tgt_v = ctx[loop]
        tgt_logits = np.einsum("bhqd,bhnd->bhqn", query.astype(np.float64), tgt_k) * float(scaling)
        target_subset = np.einsum("bhqn,bhnd->bhqd", _subset_softmax(tgt_logits, mask), tgt_v)
        deltas[loop] = (mass * (target_subset - source_subset)).astype(np.float32)
    return {"delta": deltas, "mask": mask, "mass": mass.astype(np.float32),
            "source_subset": source_subset.astype(np.float32)}
