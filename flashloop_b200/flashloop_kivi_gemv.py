"""The seven entry points of the reference's ``flashloop_kivi_gemv`` extension, served by the
B200 library.

The reference binds its CUDA extension with pybind (flashloop/csrc/kivi_outer_gemv_binding.cpp:5-34,
signatures flashloop/csrc/kivi_outer_gemv_cuda.h:6-120) and calls it from
flashloop/kivi_backend.py:534, 579, 609, 715, 767, 859, 959 with flattened ``[batch*heads, ...]``
tensors in the KIVI word layout.  This module keeps those seven names and argument lists, so
those call sites work unchanged when ``load_kivi_outer_extension()`` returns it:

    gemv_forward_cuda_outer_dim_logical, qk_selected_cuda, pv_selected_cuda,
    qk_cross_loop_cuda, pv_cross_loop_cuda, sparse_attention_delta_cuda,
    dense_source_attention_cuda

The kernels behind it read the row layout.  A set of KIVI word streams handed in here is
re-arranged on the GPU once (``fl_kivi_to_rows_*``: same codes, same metadata) into a
:class:`flashloop_b200.cache.CrossLoopKVLayer` and kept in a small cache; later calls with the
same tensors reuse it, so the per-call cost is the tail copy and the reader launch.  A cache
entry is found by the address, shape and version counter of every tensor of the call and holds
those tensors alive, so an address can never be taken over by another live tensor while the
entry exists, and an in-place update through Torch (which bumps the version counter) misses.
Writes that bypass Torch (another extension writing through a raw pointer) are not seen:
call :func:`forget` after them.  Callers that own their cache should hold a ``CrossLoopKVLayer``
and call its readers directly; nothing is converted there.

As in the reference, outputs are freshly allocated, launches go to the current stream, and
nothing synchronises.  Differences: the packed streams are read with the BF16 query (the
reference rounds it to float16 and rounds every stream's partial sum to float16,
kivi_outer_gemv_cuda.cu:803, 969, 997; these kernels keep float32 partial sums), and the
float16 ``query`` / ``inputs`` arguments are converted back to bfloat16, which is exact for the
bfloat16 queries the reference's callers start from.
"""

from __future__ import annotations

from collections import OrderedDict
from typing import Sequence

import torch

from . import _native
from .packing import Packed4Bit

_CACHE_CAPACITY = 64
_ADOPTED: "OrderedDict[tuple, tuple]" = OrderedDict()


def forget() -> None:
    """Drop every adopted layer (and the references to the tensors they were built from)."""

    _ADOPTED.clear()


def set_cache_capacity(entries: int) -> None:
    """Number of stream sets kept converted (default 64: one per physical layer and more)."""

    global _CACHE_CAPACITY
    _CACHE_CAPACITY = max(1, int(entries))
    while len(_ADOPTED) > _CACHE_CAPACITY:
        _ADOPTED.popitem(last=False)


def _ident(t: torch.Tensor | None):
    if t is None:
        return None
    return (t.data_ptr(), tuple(t.shape), t.dtype, int(t._version))


def _rows_from_words(payload: torch.Tensor, scale: torch.Tensor, minimum: torch.Tensor, tokens: int,
                     axis: str) -> Packed4Bit | None:
    """One flattened KIVI stream -> row layout with batch 1 and heads = batch*heads."""

    if tokens <= 0:
        return None
    lib = _native.load()
    bh = int(payload.shape[0])
    device = payload.device
    stream = _native.current_stream(device)
    codes = torch.empty((1, bh, tokens, 64), dtype=torch.uint8, device=device)
    if axis == "per_channel":
        if tuple(payload.shape) != (bh, (tokens + 7) // 8, 128) or tuple(scale.shape) != (bh, (tokens + 63) // 64, 128):
            raise ValueError("K stream shape differs from its logical token count")
        _native.check(lib.fl_kivi_to_rows_k(_native.ptr(payload.contiguous()), bh, tokens, _native.ptr(codes),
                                            stream), "fl_kivi_to_rows_k")
        out_min, out_scale = minimum.contiguous().view(1, bh, -1, 128), scale.contiguous().view(1, bh, -1, 128)
    else:
        if tuple(payload.shape) != (bh, 16, tokens) or tuple(scale.shape) != (bh, 2, tokens):
            raise ValueError("V stream shape differs from its logical token count")
        out_min = torch.empty((1, bh, tokens, 2), dtype=torch.float16, device=device)
        out_scale = torch.empty_like(out_min)
        _native.check(lib.fl_kivi_to_rows_v(
            _native.ptr(payload.contiguous()), _native.ptr(minimum.contiguous()), _native.ptr(scale.contiguous()),
            bh, tokens, _native.ptr(codes), _native.ptr(out_min), _native.ptr(out_scale), 2, stream),
            "fl_kivi_to_rows_v")
    return Packed4Bit(payload=codes, minimum=out_min, scale=out_scale, original_shape=(1, bh, tokens, 128),
                      original_dtype=torch.bfloat16, axis=axis, group_size=64)


def _check_stream_tensors(kernels, scales, zeros, what: str) -> None:
    for group in (kernels, scales, zeros):
        if len(group) != 4:
            raise ValueError(f"{what}: four streams are required")
    for k, s, z in zip(kernels, scales, zeros):
        if not (k.is_cuda and s.is_cuda and z.is_cuda):
            raise RuntimeError(f"{what}: CUDA tensors are required (there is no CPU fallback)")
        if k.dtype != torch.int32 or s.dtype != torch.float16 or z.dtype != torch.float16:
            raise TypeError(f"{what}: payload must be int32 and metadata float16")


def _adopt(key_words, value_words, rank3: torch.Tensor | None, rank4: torch.Tensor | None,
           logical_tokens: Sequence[int]):
    """The CrossLoopKVLayer (batch 1, heads = batch*heads) holding the given word streams.
    ``key_words`` / ``value_words``: (kernels[4], scales[4], zeros[4]) or None."""

    from .cache import CrossLoopKVLayer

    tensors = []
    for words in (key_words, value_words):
        if words is not None:
            for group in words:
                tensors.extend(group)
    tensors += [t for t in (rank3, rank4) if t is not None]
    key = (tuple(_ident(t) for t in tensors), key_words is None, value_words is None,
           tuple(int(n) for n in logical_tokens))
    hit = _ADOPTED.get(key)
    if hit is not None:
        _ADOPTED.move_to_end(key)
        return hit[0]
    tokens = [int(n) for n in logical_tokens]
    k_rows = [None] * 4
    v_rows = [None] * 4
    if key_words is not None:
        k_rows = [_rows_from_words(key_words[0][s], key_words[1][s], key_words[2][s], tokens[s], "per_channel")
                  for s in range(4)]
    if value_words is not None:
        v_rows = [_rows_from_words(value_words[0][s], value_words[1][s], value_words[2][s], tokens[s], "per_token")
                  for s in range(4)]
    first = k_rows if key_words is not None else v_rows
    if first[0] is None:
        raise ValueError("a physical anchor stream is required")
    device = first[0].payload.device
    empty = torch.empty(0, dtype=torch.int32, device=device)
    ranks = [empty if r is None else r.to(device=device, dtype=torch.int32) for r in (rank3, rank4)]
    layer = CrossLoopKVLayer.from_streams(first, v_rows, ranks)
    _ADOPTED[key] = (layer, tensors)  # the tensors stay alive with the entry: no address can be re-used
    while len(_ADOPTED) > _CACHE_CAPACITY:
        _ADOPTED.popitem(last=False)
    return layer


def _as_bf16_vectors(t: torch.Tensor, bh: int) -> torch.Tensor:
    return t.reshape(1, bh, 1, 128).to(torch.bfloat16).contiguous()


def _empty_tail(bh: int, device) -> torch.Tensor:
    return torch.zeros((1, bh, 0, 128), dtype=torch.bfloat16, device=device)


# ---------------------------------------------------------------------------------- single stream


def gemv_forward_cuda_outer_dim_logical(inputs, kernel, scaling_factors, zeros, bit, group_size, num_heads,
                                        num_kv_heads, output_channels):
    """kivi_outer_gemv_cuda.h:6-15 / kivi_outer_gemv_cuda.cu:1335-1411: ``out[bh, row, oc] = sum_ic
    inputs[bh, row, ic] * (scale * code + zero)`` over one KIVI stream.  With a K stream
    (inputs [BH, rows, 128], output_channels = tokens) these are the logits of every token; with a
    V stream (inputs [BH, rows, tokens], output_channels = 128) the weighted value sum.
    Returns float16 [BH, rows, output_channels]."""

    if int(bit) != 4 or int(group_size) != 64:
        raise ValueError("the CUDA readers specialize 4-bit codes in groups of 64")
    if int(num_heads) != int(num_kv_heads):
        raise ValueError("the CUDA readers specialize num_heads == num_kv_heads")
    if inputs.ndim != 3 or not inputs.is_cuda:
        raise RuntimeError("inputs must be a CUDA tensor [batch*heads, rows, input_channels]")
    bh, rows, width = (int(v) for v in inputs.shape)
    oc = int(output_channels)
    is_key = tuple(kernel.shape[1:]) == ((oc + 7) // 8, 128) and width == 128
    device = inputs.device
    out = torch.empty((bh, rows, oc), dtype=torch.float16, device=device)
    tokens = oc if is_key else width
    counts = (tokens, 0, 0, 0)
    words = ([kernel] * 4, [scaling_factors] * 4, [zeros] * 4)
    every = torch.arange(tokens, dtype=torch.int32, device=device)
    if is_key:
        layer = _adopt(words, None, None, None, counts)
        layer.set_tail(0, _empty_tail(bh, device), _empty_tail(bh, device))
        for row in range(rows):
            out[:, row] = layer.qk(0, _as_bf16_vectors(inputs[:, row], bh), every, validate_indices=False)[0, :, 0]
    else:
        if tuple(kernel.shape) != (bh, 16, tokens) or oc != 128:
            raise ValueError("kernel shape differs from a KIVI K or V stream of these sizes")
        layer = _adopt(None, words, None, None, counts)
        layer.set_tail(0, _empty_tail(bh, device), _empty_tail(bh, device))
        for row in range(rows):
            weights = inputs[:, row].float().reshape(1, bh, 1, tokens)
            out[:, row] = layer.pv(0, weights, every, validate_indices=False)[0, :, 0]
    return out


def qk_selected_cuda(inputs, kernel, scaling_factors, zeros, indices, group_size, num_heads, num_kv_heads,
                     logical_tokens):
    """kivi_outer_gemv_cuda.h:17-26 / .cu:1413-1474: logits of the selected rows of one K stream.
    inputs float16 [BH, 1, 128], indices int32 [BH, K]; returns float16 [BH, 1, K]."""

    bh = int(inputs.shape[0])
    words = ([kernel] * 4, [scaling_factors] * 4, [zeros] * 4)
    layer = _adopt(words, None, None, None, (int(logical_tokens), 0, 0, 0))
    layer.set_tail(0, _empty_tail(bh, inputs.device), _empty_tail(bh, inputs.device))
    out = layer.qk(0, _as_bf16_vectors(inputs, bh), indices.reshape(1, bh, -1), validate_indices=False)
    return out.reshape(bh, 1, -1).to(torch.float16)


def pv_selected_cuda(inputs, kernel, scaling_factors, zeros, indices, group_size, num_heads, num_kv_heads,
                     logical_tokens, output_channels):
    """kivi_outer_gemv_cuda.h:28-38 / .cu:1476-1539: weighted sum of the selected rows of one V
    stream.  inputs float16 [BH, 1, K]; returns float16 [BH, 1, 128]."""

    bh, selected = int(inputs.shape[0]), int(inputs.shape[-1])
    words = ([kernel] * 4, [scaling_factors] * 4, [zeros] * 4)
    layer = _adopt(None, words, None, None, (int(logical_tokens), 0, 0, 0))
    layer.set_tail(0, _empty_tail(bh, inputs.device), _empty_tail(bh, inputs.device))
    out = layer.pv(0, inputs.float().reshape(1, bh, 1, selected), indices.reshape(1, bh, selected),
                   validate_indices=False)
    return out.reshape(bh, 1, int(output_channels)).to(torch.float16)


# ---------------------------------------------------------------------------------- four streams


def qk_cross_loop_cuda(inputs, kernels, scaling_factors, zeros, indices, rank3, rank4, group_size, num_heads,
                       num_kv_heads, loop, logical_tokens):
    """kivi_outer_gemv_cuda.h:40-52 / .cu:1541-1623: selected logits summed over streams 0..loop.
    Returns float32 [BH, 1, K]."""

    _check_stream_tensors(kernels, scaling_factors, zeros, "qk_cross_loop_cuda")
    bh = int(inputs.shape[0])
    layer = _adopt((list(kernels), list(scaling_factors), list(zeros)), None, rank3, rank4, logical_tokens)
    layer.set_tail(int(loop), _empty_tail(bh, inputs.device), _empty_tail(bh, inputs.device))
    out = layer.qk(int(loop), _as_bf16_vectors(inputs, bh), indices.reshape(1, bh, -1), validate_indices=False)
    return out.reshape(bh, 1, -1)


def pv_cross_loop_cuda(inputs, kernels, scaling_factors, zeros, indices, rank3, rank4, group_size, num_heads,
                       num_kv_heads, loop, logical_tokens, output_channels):
    """kivi_outer_gemv_cuda.h:54-67 / .cu:1625-1709: weighted V sum over streams 0..loop.
    Returns float32 [BH, 1, 128]."""

    _check_stream_tensors(kernels, scaling_factors, zeros, "pv_cross_loop_cuda")
    bh, selected = int(inputs.shape[0]), int(inputs.shape[-1])
    layer = _adopt(None, (list(kernels), list(scaling_factors), list(zeros)), rank3, rank4, logical_tokens)
    layer.set_tail(int(loop), _empty_tail(bh, inputs.device), _empty_tail(bh, inputs.device))
    out = layer.pv(int(loop), inputs.float().reshape(1, bh, 1, selected), indices.reshape(1, bh, selected),
                   validate_indices=False)
    return out.reshape(bh, 1, int(output_channels))


def sparse_attention_delta_cuda(query, query_bf16, current_key, current_value, key_kernels, key_scaling_factors,
                                key_zeros, value_kernels, value_scaling_factors, value_zeros, indices, valid, rank3,
                                rank4, tail_key, tail_value, source_output, global_mass, current_position, scaling,
                                group_size, num_heads, num_kv_heads, loop, logical_tokens, output_channels,
                                return_current_logits):
    """kivi_outer_gemv_cuda.h:69-96 / .cu:1711-1912: cached-mass sparse delta of loops 3 / 4
    (``loop`` 2 or 3) as one launch.  Returns [float32 [BH, 1, 128] (, float32 [BH])]."""

    _check_stream_tensors(key_kernels, key_scaling_factors, key_zeros, "sparse_attention_delta_cuda")
    _check_stream_tensors(value_kernels, value_scaling_factors, value_zeros, "sparse_attention_delta_cuda")
    bh = int(query_bf16.shape[0])
    layer = _adopt((list(key_kernels), list(key_scaling_factors), list(key_zeros)),
                   (list(value_kernels), list(value_scaling_factors), list(value_zeros)), rank3, rank4,
                   logical_tokens)
    tail = int(current_position) - int(logical_tokens[0])
    if tail < 0 or tail > int(tail_key.shape[1]):
        raise ValueError("current_position differs from the packed prefix plus the tail")
    layer.set_tail(int(loop), tail_key[:, :tail].reshape(1, bh, tail, 128), tail_value[:, :tail].reshape(1, bh, tail, 128))
    # heads whose selection misses the current token keep NaN, as in the reference (.cu:1826-1831)
    current_logits = (torch.full((bh,), float("nan"), dtype=torch.float32, device=query_bf16.device)
                      if return_current_logits else None)
    out = layer.cached_mass_sparse_attention_delta(
        int(loop), query=query_bf16.reshape(1, bh, 1, 128), current_key=current_key.reshape(1, bh, 1, 128),
        current_value=current_value.reshape(1, bh, 1, 128), indices=indices.reshape(1, bh, -1),
        valid=valid.reshape(1, bh, -1), source_selected_output=source_output.reshape(1, bh, 1, 128),
        global_mass=global_mass.reshape(1, bh, 1, 1), scaling=float(scaling), current_logits_out=current_logits)
    out = out.reshape(bh, 1, int(output_channels))
    return [out, current_logits] if return_current_logits else [out]


def dense_source_attention_cuda(query, query_bf16, current_key, current_value, key_kernels, key_scaling_factors,
                                key_zeros, value_kernels, value_scaling_factors, value_zeros, rank3, rank4, tail_key,
                                tail_value, scaling, group_size, num_heads, num_kv_heads, loop, logical_tokens,
                                output_channels, return_logits):
    """kivi_outer_gemv_cuda.h:98-120 / .cu:1914-2076: dense attention of loop 1 / 2 (``loop`` 0 or
    1) over the packed prefix, the BF16 tail and the current token as one launch.  Returns
    [float32 [BH, 1, 128] (, float32 scaled logits [BH, 1, T0 + tail + 1])]."""

    _check_stream_tensors(key_kernels, key_scaling_factors, key_zeros, "dense_source_attention_cuda")
    _check_stream_tensors(value_kernels, value_scaling_factors, value_zeros, "dense_source_attention_cuda")
    bh = int(query_bf16.shape[0])
    if int(logical_tokens[0]) % 64:
        raise ValueError("the dense reader needs a packed prefix of whole 64-token groups")
    layer = _adopt((list(key_kernels), list(key_scaling_factors), list(key_zeros)),
                   (list(value_kernels), list(value_scaling_factors), list(value_zeros)), rank3, rank4,
                   logical_tokens)
    tail = int(tail_key.shape[1])
    layer.set_tail(int(loop), tail_key.reshape(1, bh, tail, 128), tail_value.reshape(1, bh, tail, 128))
    out, logits = layer.dense_source_attention(
        int(loop), query=query_bf16.reshape(1, bh, 1, 128), current_key=current_key.reshape(1, bh, 1, 128),
        current_value=current_value.reshape(1, bh, 1, 128), scaling=float(scaling), return_logits=bool(return_logits))
    out = out.reshape(bh, 1, int(output_channels))
    if return_logits:
        return [out, logits.reshape(bh, 1, -1).contiguous()]
    return [out]
