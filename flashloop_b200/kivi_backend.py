"""KIVI-style output-parallel physical 4-bit KV storage and its fused readers.

Mirrors the interface of the reference's flashloop/kivi_backend.py: the
``KiviPacked4Bit`` word layout (:325-401), ``pack_kivi_k_per_channel`` /
``pack_kivi_v_per_token`` (:404-475) and the fused reader entry points
``kivi_fused_dense_source_attention`` (:899-992), ``kivi_fused_sparse_attention_delta``
(:784-896), ``kivi_fused_cross_loop_qk`` / ``kivi_fused_cross_loop_pv`` (:678-781).

Packing runs in the CUDA kernels ``fl_pack_kivi_k`` / ``fl_pack_kivi_v`` (the
reference uses Triton kernels on the GPU, :162-256) and is bit-exact with the
reference's CPU codec.  Every reader here marshals its tensors as the reference does
(flattened ``[batch*heads, ...]`` views) and calls the extension object it is given; the
default extension is :mod:`flashloop_b200.flashloop_kivi_gemv`, which serves the reference
extension's seven entry points from the B200 library (the word streams are re-arranged into
the row layout once and cached there).  Also mirrored: ``kivi_outer_gemv`` (:494-548),
``kivi_selected_qk`` / ``kivi_selected_pv`` (:551-620), ``kivi_cross_loop_qk`` /
``kivi_cross_loop_pv`` (:995-1119) and ``outer_matmul_reference`` (:478-491).
Callers that own their cache should hold a ``CrossLoopKVLayer`` directly and skip the
re-arrangement.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable

import torch

from . import _native
from .packing import Packed4Bit, _validate_values

_PACK_FACTOR = 8


def load_kivi_outer_extension() -> Any:
    """The object that stands in for the reference's ``flashloop_kivi_gemv`` module
    (flashloop/kivi_backend.py:38-49): it exports the same seven functions.  Raises
    RuntimeError when the CUDA library has not been built."""

    _native.load()
    from . import flashloop_kivi_gemv

    return flashloop_kivi_gemv


@dataclass(frozen=True)
class KiviPacked4Bit:
    """One physical KIVI-layout affine 4-bit matrix (flashloop/kivi_backend.py:325-366).

    per_channel (K): payload int32 [B, H, ceil(n/8), 128], word = 8 consecutive tokens of
    one channel; metadata float16 [B, H, ceil(n/64), 128].
    per_token (V): payload int32 [B, H, 16, n], word = 8 consecutive channels of one
    token; metadata float16 [B, H, 2, n]."""

    payload: torch.Tensor
    minimum: torch.Tensor
    scale: torch.Tensor
    original_shape: tuple[int, int, int, int]
    original_dtype: torch.dtype
    axis: str
    group_size: int

    def __post_init__(self) -> None:
        if self.payload.dtype != torch.int32:
            raise TypeError("KIVI payload must be int32")
        if self.minimum.dtype != torch.float16 or self.scale.dtype != torch.float16:
            raise TypeError("KIVI affine metadata must be float16")
        if self.minimum.shape != self.scale.shape:
            raise ValueError("minimum and scale shapes differ")
        if self.axis not in {"per_channel", "per_token"}:
            raise ValueError("unknown KIVI quantization axis")
        batch, heads, tokens, channels = self.original_shape
        g = self.group_size
        if self.axis == "per_channel":
            expected_payload = (batch, heads, (tokens + 7) // 8, channels)
            expected_metadata = (batch, heads, (tokens + g - 1) // g, channels)
        else:
            expected_payload = (batch, heads, (channels + 7) // 8, tokens)
            expected_metadata = (batch, heads, (channels + g - 1) // g, tokens)
        if tuple(self.payload.shape) != expected_payload:
            raise ValueError("KIVI payload shape differs from logical KV shape")
        if tuple(self.minimum.shape) != expected_metadata:
            raise ValueError("KIVI metadata shape differs from logical KV shape")

    @property
    def storage_bytes(self) -> int:
        return sum(int(t.numel() * t.element_size()) for t in (self.payload, self.minimum, self.scale))

    @property
    def matrix_shape(self) -> tuple[int, int, int, int]:
        batch, heads, tokens, channels = self.original_shape
        return (batch, heads, tokens, channels) if self.axis == "per_channel" else (batch, heads, channels, tokens)

    def decode(self) -> torch.Tensor:
        """flashloop/kivi_backend.py:381-401, via the row layout."""

        return kivi_to_rows(self).decode()


def _pack_kivi(values: torch.Tensor, *, axis: str, group_size: int) -> KiviPacked4Bit:
    lib = _native.load()
    values = values.contiguous()
    batch, heads, tokens, channels = (int(v) for v in values.shape)
    device = values.device
    stream = _native.current_stream(device)
    if axis == "per_channel":
        payload = torch.empty((batch, heads, (tokens + 7) // 8, channels), dtype=torch.int32, device=device)
        minimum = torch.empty((batch, heads, (tokens + group_size - 1) // group_size, channels),
                              dtype=torch.float16, device=device)
        scale = torch.empty_like(minimum)
        _native.check(lib.fl_pack_kivi_k(_native.ptr(values), _native.DTYPE_CODES[values.dtype], batch * heads,
                                         tokens, _native.ptr(payload), _native.ptr(minimum), _native.ptr(scale),
                                         stream), "fl_pack_kivi_k")
    else:
        payload = torch.empty((batch, heads, channels // 8, tokens), dtype=torch.int32, device=device)
        minimum = torch.empty((batch, heads, channels // group_size, tokens), dtype=torch.float16, device=device)
        scale = torch.empty_like(minimum)
        _native.check(lib.fl_pack_kivi_v(_native.ptr(values), _native.DTYPE_CODES[values.dtype], batch * heads,
                                         tokens, _native.ptr(payload), _native.ptr(minimum), _native.ptr(scale),
                                         stream), "fl_pack_kivi_v")
    return KiviPacked4Bit(payload=payload, minimum=minimum, scale=scale,
                          original_shape=(batch, heads, tokens, channels), original_dtype=values.dtype,
                          axis=axis, group_size=group_size)


def pack_kivi_k_per_channel(values: torch.Tensor, *, group_size: int = 64) -> KiviPacked4Bit:
    """Pack K so one GEMV output feature corresponds to one token (kivi_backend.py:404-438)."""

    group_size = _validate_values(values, group_size)
    return _pack_kivi(values, axis="per_channel", group_size=group_size)


def pack_kivi_v_per_token(values: torch.Tensor, *, group_size: int = 64) -> KiviPacked4Bit:
    """Pack V so one GEMV output feature corresponds to one channel (kivi_backend.py:441-475)."""

    group_size = _validate_values(values, group_size)
    return _pack_kivi(values, axis="per_token", group_size=group_size)


def kivi_to_rows(packed: KiviPacked4Bit) -> Packed4Bit:
    """Re-arrange a KIVI word stream into the row layout on the GPU (same codes and
    metadata values; kivi_backend.py:286-322 describes the word layout)."""

    _native.require_cuda(packed.payload)
    lib = _native.load()
    batch, heads, tokens, channels = packed.original_shape
    if channels != 128 or packed.group_size != 64:
        raise ValueError("the CUDA readers specialize head_dim=128, group_size=64")
    device = packed.payload.device
    stream = _native.current_stream(device)
    codes = torch.empty((batch, heads, tokens, 64), dtype=torch.uint8, device=device)
    if packed.axis == "per_channel":
        _native.check(lib.fl_kivi_to_rows_k(_native.ptr(packed.payload.contiguous()), batch * heads, tokens,
                                            _native.ptr(codes), stream), "fl_kivi_to_rows_k")
        minimum, scale = packed.minimum, packed.scale
    else:
        minimum = torch.empty((batch, heads, tokens, 2), dtype=torch.float16, device=device)
        scale = torch.empty_like(minimum)
        _native.check(lib.fl_kivi_to_rows_v(
            _native.ptr(packed.payload.contiguous()), _native.ptr(packed.minimum.contiguous()),
            _native.ptr(packed.scale.contiguous()), batch * heads, tokens, _native.ptr(codes),
            _native.ptr(minimum), _native.ptr(scale), 2, stream), "fl_kivi_to_rows_v")
    return Packed4Bit(payload=codes, minimum=minimum, scale=scale, original_shape=packed.original_shape,
                      original_dtype=packed.original_dtype, axis=packed.axis, group_size=packed.group_size)


# ---------------------------------------------------------------------------------- readers


def _ext(extension):
    return load_kivi_outer_extension() if extension is None else extension


def _flat(t: torch.Tensor, batch_heads: int) -> torch.Tensor:
    """[B, H, a, b] -> contiguous [B*H, a, b] (a view when the tensor is contiguous already)."""

    return t.reshape(batch_heads, int(t.shape[2]), int(t.shape[3])).contiguous()


def _flat_streams(streams) -> tuple[list, list, list, tuple]:
    """Payloads, scales, minima and token counts of four streams, flattened over (batch, head)."""

    bh = int(streams[0].original_shape[0]) * int(streams[0].original_shape[1])
    return ([_flat(s.payload, bh) for s in streams], [_flat(s.scale, bh) for s in streams],
            [_flat(s.minimum, bh) for s in streams], tuple(int(s.original_shape[2]) for s in streams))


def _four_streams(streams, axis: str):
    """kivi_backend.py:657-675: the fused readers need four physical streams of one axis."""

    if len(streams) != 4 or any(s is None for s in streams):
        raise ValueError("the fused cross-loop reader requires four physical streams")
    anchor = streams[0]
    for s in streams:
        if (s.axis != axis or s.group_size != 64 or s.original_shape[:2] != anchor.original_shape[:2]
                or s.original_shape[3] != anchor.original_shape[3]):
            raise ValueError("fused cross-loop streams have incompatible storage")
    return tuple(streams)


def _logical_indices(streams, rank_maps, indices: torch.Tensor, *, loop: int, axis: str):
    """kivi_backend.py:623-654: shape checks shared by the cross-loop readers; returns the anchor
    and the indices as int64 [B, H, selected]."""

    if len(streams) != 4 or streams[0] is None:
        raise ValueError("four stream slots with a physical anchor are required")
    if len(rank_maps) != 2:
        raise ValueError("Loop-3/4 rank maps are required")
    if int(loop) not in range(4):
        raise ValueError("loop must be in [0, 3]")
    anchor = streams[0]
    if anchor.axis != axis:
        raise ValueError("cross-loop stream uses the wrong quantization axis")
    for s in streams:
        if s is not None and (s.axis != axis or s.original_shape[:2] != anchor.original_shape[:2]
                              or s.original_shape[3] != anchor.original_shape[3]):
            raise ValueError("cross-loop streams have incompatible matrix shapes")
    if indices.ndim == 1:
        indices = indices[None, None].expand(*anchor.original_shape[:2], -1)
    elif indices.ndim == 4 and indices.shape[-2] == 1:
        indices = indices.squeeze(-2)
    if indices.ndim != 3 or tuple(indices.shape[:2]) != tuple(anchor.original_shape[:2]):
        raise ValueError("indices must have shape [selected] or [batch, heads, selected]")
    return anchor, indices.to(device=anchor.payload.device, dtype=torch.int64).contiguous()


def outer_matmul_reference(inputs: torch.Tensor, packed: KiviPacked4Bit) -> torch.Tensor:
    """The GEMV on the decoded tensor (kivi_backend.py:478-491): the plain-Torch check of
    :func:`kivi_outer_gemv`."""

    if inputs.ndim != 4 or tuple(inputs.shape[:2]) != tuple(packed.original_shape[:2]):
        raise ValueError("input batch/head shape differs from packed storage")
    decoded = packed.decode().float()
    if packed.axis == "per_channel":
        if int(inputs.shape[-1]) != packed.original_shape[3]:
            raise ValueError("input width differs from K channels")
        return torch.matmul(inputs.float(), decoded.transpose(-1, -2))
    if int(inputs.shape[-1]) != packed.original_shape[2]:
        raise ValueError("input width differs from V tokens")
    return torch.matmul(inputs.float(), decoded)


def kivi_outer_gemv(inputs: torch.Tensor, packed: KiviPacked4Bit, *, extension: Any = None,
                    require_cuda: bool = True) -> torch.Tensor:
    """GEMV of ``inputs`` with one packed stream (kivi_backend.py:494-548): with K the logits of
    every token, with V the weighted sum over every token; float32 [B, H, rows, outputs]."""

    if inputs.ndim != 4 or tuple(inputs.shape[:2]) != tuple(packed.original_shape[:2]):
        raise ValueError("input batch/head shape differs from packed storage")
    if require_cuda and (not inputs.is_cuda or not packed.payload.is_cuda):
        raise RuntimeError("KIVI outer GEMV requires CUDA tensors")
    batch, heads = int(inputs.shape[0]), int(inputs.shape[1])
    outputs, width = packed.matrix_shape[2:]
    if int(inputs.shape[-1]) != width:
        raise ValueError("input width differs from packed matrix")
    bh, rows = batch * heads, int(inputs.shape[2])
    out = _ext(extension).gemv_forward_cuda_outer_dim_logical(
        inputs.to(torch.float16).reshape(bh, rows, width).contiguous(), _flat(packed.payload, bh),
        _flat(packed.scale, bh), _flat(packed.minimum, bh), 4, packed.group_size, heads, heads, outputs)
    if tuple(out.shape) != (bh, rows, outputs):
        raise RuntimeError("KIVI extension returned an unexpected output shape")
    return out.reshape(batch, heads, rows, outputs).float()


def kivi_selected_qk(query: torch.Tensor, packed: KiviPacked4Bit, indices: torch.Tensor, *,
                     extension: Any = None) -> torch.Tensor:
    """Logits of selected rows of one K stream (kivi_backend.py:551-584)."""

    if packed.axis != "per_channel":
        raise ValueError("selected QK requires per-channel K storage")
    batch, heads, tokens, channels = packed.original_shape
    if tuple(query.shape) != (batch, heads, 1, channels):
        raise ValueError("query shape differs from K storage")
    if indices.ndim == 1:
        indices = indices[None, None].expand(batch, heads, -1)
    if indices.ndim != 3 or tuple(indices.shape[:2]) != (batch, heads):
        raise ValueError("selected K indices must have shape [batch, heads, selected]")
    bh = batch * heads
    idx = indices.to(device=query.device, dtype=torch.int32).reshape(bh, -1).contiguous()
    out = _ext(extension).qk_selected_cuda(
        query.to(torch.float16).reshape(bh, 1, channels).contiguous(), _flat(packed.payload, bh),
        _flat(packed.scale, bh), _flat(packed.minimum, bh), idx, packed.group_size, heads, heads, tokens)
    return out.reshape(batch, heads, 1, idx.shape[-1]).float()


def kivi_selected_pv(weights: torch.Tensor, packed: KiviPacked4Bit, indices: torch.Tensor, *,
                     extension: Any = None) -> torch.Tensor:
    """Weighted sum of selected rows of one V stream (kivi_backend.py:587-620)."""

    if packed.axis != "per_token":
        raise ValueError("selected PV requires per-token V storage")
    batch, heads, tokens, channels = packed.original_shape
    if indices.ndim == 1:
        indices = indices[None, None].expand(batch, heads, -1)
    selected = int(indices.shape[-1])
    if tuple(weights.shape) != (batch, heads, 1, selected):
        raise ValueError("weights shape differs from selected V indices")
    bh = batch * heads
    idx = indices.to(device=weights.device, dtype=torch.int32).reshape(bh, selected).contiguous()
    out = _ext(extension).pv_selected_cuda(
        weights.to(torch.float16).reshape(bh, 1, selected).contiguous(), _flat(packed.payload, bh),
        _flat(packed.scale, bh), _flat(packed.minimum, bh), idx, packed.group_size, heads, heads, tokens, channels)
    return out.reshape(batch, heads, 1, channels).float()


def kivi_fused_cross_loop_qk(query, streams, rank_maps, indices, *, loop, extension=None, require_cuda=True):
    """Read anchor plus all active K deltas in one CUDA launch (kivi_backend.py:678-727)."""

    prepared = _four_streams(streams, "per_channel")
    anchor, logical = _logical_indices(streams, rank_maps, indices, loop=loop, axis="per_channel")
    batch, heads, _, channels = anchor.original_shape
    if tuple(query.shape) != (batch, heads, 1, channels):
        raise ValueError("query shape differs from the K anchor")
    if require_cuda and (not query.is_cuda or not anchor.payload.is_cuda):
        raise RuntimeError("fused KIVI cross-loop QK requires CUDA tensors")
    bh = batch * heads
    payloads, scales, minima, counts = _flat_streams(prepared)
    idx = logical.to(torch.int32).reshape(bh, -1).contiguous()
    out = _ext(extension).qk_cross_loop_cuda(
        query.to(torch.float16).reshape(bh, 1, channels).contiguous(), payloads, scales, minima, idx,
        rank_maps[0].to(device=query.device, dtype=torch.int32).contiguous(),
        rank_maps[1].to(device=query.device, dtype=torch.int32).contiguous(), 64, heads, heads, int(loop), counts)
    return out.reshape(batch, heads, 1, idx.shape[-1]).float()


def kivi_fused_cross_loop_pv(weights, streams, rank_maps, indices, *, loop, extension=None, require_cuda=True):
    """Accumulate anchor plus all active V deltas in one CUDA launch (kivi_backend.py:730-781)."""

    prepared = _four_streams(streams, "per_token")
    anchor, logical = _logical_indices(streams, rank_maps, indices, loop=loop, axis="per_token")
    batch, heads, _, channels = anchor.original_shape
    selected = int(logical.shape[-1])
    if tuple(weights.shape) != (batch, heads, 1, selected):
        raise ValueError("weights shape differs from selected logical rows")
    if require_cuda and (not weights.is_cuda or not anchor.payload.is_cuda):
        raise RuntimeError("fused KIVI cross-loop PV requires CUDA tensors")
    bh = batch * heads
    payloads, scales, minima, counts = _flat_streams(prepared)
    out = _ext(extension).pv_cross_loop_cuda(
        weights.to(torch.float16).reshape(bh, 1, selected).contiguous(), payloads, scales, minima,
        logical.to(torch.int32).reshape(bh, selected).contiguous(),
        rank_maps[0].to(device=weights.device, dtype=torch.int32).contiguous(),
        rank_maps[1].to(device=weights.device, dtype=torch.int32).contiguous(), 64, heads, heads, int(loop), counts,
        channels)
    return out.reshape(batch, heads, 1, channels).float()


def kivi_fused_sparse_attention_delta(*, query, current_key, current_value, key_streams, value_streams,
                                      rank_maps, tail_key, tail_value, indices, valid,
                                      source_selected_output, global_mass, current_position, scaling, loop,
                                      extension=None, require_cuda=True, return_current_logits=False):
    """Fuse KIVI QK, subset softmax, PV and cached-mass correction (kivi_backend.py:784-896)."""

    keys = _four_streams(key_streams, "per_channel")
    values = _four_streams(value_streams, "per_token")
    anchor, logical = _logical_indices(key_streams, rank_maps, indices, loop=loop, axis="per_channel")
    batch, heads, _, channels = anchor.original_shape
    vector = (batch, heads, 1, channels)
    if any(tuple(t.shape) != vector for t in (query, current_key, current_value, source_selected_output)):
        raise ValueError("fused attention vectors differ from the KIVI anchor")
    if tuple(valid.shape) != tuple(logical.shape):
        raise ValueError("valid mask must match selected indices")
    if tuple(global_mass.shape) != (batch, heads, 1, 1):
        raise ValueError("global mass must have shape [batch, heads, 1, 1]")
    if (tuple(tail_key.shape[:2]) != (batch, heads) or tuple(tail_value.shape) != tuple(tail_key.shape)
            or int(tail_key.shape[-1]) != channels):
        raise ValueError("tail K/V shape differs from the KIVI anchor")
    if any(t.dtype != torch.bfloat16 for t in (current_key, current_value, tail_key, tail_value)):
        raise ValueError("fused attention currently specializes BF16 tail/current K/V")
    if query.dtype != torch.bfloat16:
        raise ValueError("fused attention currently specializes BF16 queries")
    if require_cuda and (not query.is_cuda or not current_key.is_cuda or not anchor.payload.is_cuda):
        raise RuntimeError("fused KIVI sparse attention requires CUDA tensors")
    bh, selected = batch * heads, int(logical.shape[-1])
    kp, ks, km, counts = _flat_streams(keys)
    vp, vs, vm, _ = _flat_streams(values)
    raw = _ext(extension).sparse_attention_delta_cuda(
        query.to(torch.float16).reshape(bh, 1, channels).contiguous(), query.reshape(bh, channels).contiguous(),
        current_key.reshape(bh, channels).contiguous(), current_value.reshape(bh, channels).contiguous(),
        kp, ks, km, vp, vs, vm, logical.to(torch.int32).reshape(bh, selected).contiguous(),
        valid.to(device=query.device, dtype=torch.bool).reshape(bh, selected).contiguous(),
        rank_maps[0].to(device=query.device, dtype=torch.int32).contiguous(),
        rank_maps[1].to(device=query.device, dtype=torch.int32).contiguous(),
        _flat(tail_key, bh), _flat(tail_value, bh), source_selected_output.float().reshape(bh, channels).contiguous(),
        global_mass.float().reshape(bh).contiguous(), int(current_position), float(scaling), 64, heads, heads,
        int(loop), counts, channels, bool(return_current_logits))
    output = raw[0].reshape(batch, heads, 1, channels).float()
    if return_current_logits:
        return output, raw[1].reshape(batch, heads).float()
    return output


def kivi_fused_dense_source_attention(*, query, current_key, current_value, key_streams, value_streams,
                                      rank_maps, tail_key, tail_value, scaling, loop, extension=None,
                                      require_cuda=True, return_logits=False):
    """Fuse full Loop-1/2 KIVI QK, softmax and PV in one launch (kivi_backend.py:899-992)."""

    if int(loop) not in (0, 1):
        raise ValueError("dense source attention is only valid for Loop 1/2")
    keys = _four_streams(key_streams, "per_channel")
    values = _four_streams(value_streams, "per_token")
    anchor = keys[0]
    batch, heads, base_tokens, channels = anchor.original_shape
    vector = (batch, heads, 1, channels)
    if any(tuple(t.shape) != vector for t in (query, current_key, current_value)):
        raise ValueError("dense attention vectors differ from the KIVI anchor")
    if any(s.original_shape[:2] != (batch, heads) for s in (*keys, *values)):
        raise ValueError("dense attention streams differ from the KIVI anchor")
    if tuple(tail_key.shape[:2]) != (batch, heads) or tuple(tail_value.shape) != tuple(tail_key.shape):
        raise ValueError("tail K/V shape differs from the KIVI anchor")
    if int(tail_key.shape[-1]) != channels:
        raise ValueError("tail K/V channels differ from the KIVI anchor")
    if any(t.dtype != torch.bfloat16 for t in (query, current_key, current_value, tail_key, tail_value)):
        raise ValueError("fused dense attention currently specializes BF16 vectors")
    if require_cuda and (not query.is_cuda or not current_key.is_cuda or not anchor.payload.is_cuda):
        raise RuntimeError("fused KIVI dense source attention requires CUDA tensors")
    if any(int(s.original_shape[2]) != base_tokens for s in keys[:2]):
        raise ValueError("Loop-1/2 K streams must share the anchor token count")
    bh = batch * heads
    kp, ks, km, counts = _flat_streams(keys)
    vp, vs, vm, _ = _flat_streams(values)
    raw = _ext(extension).dense_source_attention_cuda(
        query.to(torch.float16).reshape(bh, 1, channels).contiguous(), query.reshape(bh, channels).contiguous(),
        current_key.reshape(bh, channels).contiguous(), current_value.reshape(bh, channels).contiguous(),
        kp, ks, km, vp, vs, vm, rank_maps[0].to(device=query.device, dtype=torch.int32).contiguous(),
        rank_maps[1].to(device=query.device, dtype=torch.int32).contiguous(), _flat(tail_key, bh),
        _flat(tail_value, bh), float(scaling), 64, heads, heads, int(loop), counts, channels, bool(return_logits))
    output = raw[0].reshape(batch, heads, 1, channels).float()
    logits = None
    if return_logits:
        logits = raw[1].reshape(batch, heads, 1, base_tokens + int(tail_key.shape[2]) + 1).float()
    return output, logits


def _stream_rows(logical: torch.Tensor, stream_index: int, anchor_tokens: int, rank_maps):
    """Rows of ``logical`` in stream ``stream_index`` and which of them exist
    (kivi_backend.py:1025-1038): streams 0 / 1 hold every prefix token, streams 2 / 3 the
    retained ones through their rank map."""

    inside = logical < anchor_tokens
    if stream_index < 2:
        return torch.where(inside, logical, torch.zeros_like(logical)), inside
    ranks = rank_maps[stream_index - 2].to(logical.device)[torch.where(inside, logical, torch.zeros_like(logical))]
    active = inside & (ranks >= 0)
    return torch.where(active, ranks, torch.zeros_like(ranks)).long(), active


def kivi_cross_loop_qk(query, streams, rank_maps, indices, *, loop: int,
                       gemv: Callable[[torch.Tensor, KiviPacked4Bit], torch.Tensor],
                       selected_gemv: Callable[[torch.Tensor, KiviPacked4Bit, torch.Tensor], torch.Tensor] | None = None):
    """Selected logits over an anchor and nested K deltas, one stream at a time
    (kivi_backend.py:995-1044): the un-fused fallback of :func:`kivi_fused_cross_loop_qk`."""

    anchor, logical = _logical_indices(streams, rank_maps, indices, loop=loop, axis="per_channel")
    if tuple(query.shape) != (*anchor.original_shape[:2], 1, anchor.original_shape[3]):
        raise ValueError("query shape differs from the K anchor")
    total = torch.zeros((*anchor.original_shape[:2], 1, int(logical.shape[-1])), dtype=torch.float32,
                        device=query.device)
    for index in range(int(loop) + 1):
        stream = streams[index]
        if stream is None:
            continue
        rows, active = _stream_rows(logical, index, anchor.original_shape[2], rank_maps)
        if selected_gemv is None:
            part = torch.gather(gemv(query, stream).float(), -1, rows[:, :, None, :])
        else:
            part = selected_gemv(query, stream, rows).float()
        total += part * active[:, :, None, :]
    return total


def kivi_cross_loop_pv(weights, streams, rank_maps, indices, *, loop: int,
                       gemv: Callable[[torch.Tensor, KiviPacked4Bit], torch.Tensor],
                       workspaces=None,
                       selected_gemv: Callable[[torch.Tensor, KiviPacked4Bit, torch.Tensor], torch.Tensor] | None = None):
    """Weighted V sum over an anchor and nested compact deltas, one stream at a time
    (kivi_backend.py:1047-1119): the un-fused fallback of :func:`kivi_fused_cross_loop_pv`."""

    anchor, logical = _logical_indices(streams, rank_maps, indices, loop=loop, axis="per_token")
    if tuple(weights.shape) != (*anchor.original_shape[:2], 1, int(logical.shape[-1])):
        raise ValueError("weights shape differs from selected logical rows")
    if workspaces is None:
        workspaces = (None, None, None, None)
    if len(workspaces) != 4:
        raise ValueError("four optional PV input workspaces are required")
    total = torch.zeros((*anchor.original_shape[:2], 1, anchor.original_shape[3]), dtype=torch.float32,
                        device=weights.device)
    for index in range(int(loop) + 1):
        stream = streams[index]
        if stream is None:
            continue
        rows, active = _stream_rows(logical, index, anchor.original_shape[2], rank_maps)
        masked = weights.float() * active[:, :, None, :]
        if selected_gemv is not None:
            total += selected_gemv(masked, stream, rows).float()
            continue
        shape = (*anchor.original_shape[:2], 1, stream.original_shape[2])
        spread = workspaces[index]
        if spread is None:
            spread = torch.zeros(shape, dtype=torch.float32, device=weights.device)
        elif tuple(spread.shape) != shape or spread.device != weights.device:
            raise ValueError("PV input workspace shape/device differs from its stream")
        else:
            spread.zero_()
        spread.scatter_add_(-1, rows[:, :, None, :], masked)
        total += gemv(spread, stream).float()
    return total
