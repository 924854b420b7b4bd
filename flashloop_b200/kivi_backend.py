"""KIVI-style output-parallel physical 4-bit KV storage and its fused readers.

Mirrors the interface of the reference's flashloop/kivi_backend.py: the
``KiviPacked4Bit`` word layout (:325-401), ``pack_kivi_k_per_channel`` /
``pack_kivi_v_per_token`` (:404-475) and the fused reader entry points
``kivi_fused_dense_source_attention`` (:899-992), ``kivi_fused_sparse_attention_delta``
(:784-896), ``kivi_fused_cross_loop_qk`` / ``kivi_fused_cross_loop_pv`` (:678-781).

Packing runs in the CUDA kernels ``fl_pack_kivi_k`` / ``fl_pack_kivi_v`` (the
reference uses Triton kernels on the GPU, :162-256) and is bit-exact with the
reference's CPU codec.  The readers work on the row layout: a KIVI word stream handed
to a fused entry point is re-arranged on the GPU (same codes, same metadata) into a
:class:`flashloop_b200.cache.CrossLoopKVLayer`, cached per set of payload tensors.
Callers that own their cache should hold a ``CrossLoopKVLayer`` directly and skip the
re-arrangement.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

import torch

from . import _native
from .packing import Packed4Bit, _validate_values

_PACK_FACTOR = 8


def load_kivi_outer_extension() -> Any:
    """Load the CUDA library once (flashloop/kivi_backend.py:38-49); raises RuntimeError
    when it has not been built."""

    return _native.load()


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


# ---------------------------------------------------------------------------------- fused readers

_ADOPTED: dict[tuple, Any] = {}


def _adopt(key_streams, value_streams, rank_maps, tail_key, tail_value, loop):
    """A CrossLoopKVLayer holding the given streams (cached on their storage identity)."""

    from .cache import CrossLoopKVLayer

    if len(key_streams) != 4 or len(value_streams) != 4 or key_streams[0] is None:
        raise ValueError("four stream slots with a physical anchor are required")
    if len(rank_maps) != 2:
        raise ValueError("Loop-3/4 rank maps are required")
    ident = tuple((s.payload.data_ptr(), tuple(s.payload.shape)) if s is not None else None
                  for s in (*key_streams, *value_streams))
    ident += tuple((r.data_ptr(), int(r.numel())) for r in rank_maps)
    layer = _ADOPTED.get(ident)
    if layer is None:
        if len(_ADOPTED) > 64:
            _ADOPTED.clear()
        rows_k = [kivi_to_rows(s) if isinstance(s, KiviPacked4Bit) else s for s in key_streams]
        rows_v = [kivi_to_rows(s) if isinstance(s, KiviPacked4Bit) else s for s in value_streams]
        layer = CrossLoopKVLayer.from_streams(rows_k, rows_v, rank_maps)
        _ADOPTED[ident] = layer
    layer.set_tail(int(loop), tail_key, tail_value)
    return layer


def _check_axis(streams, axis: str) -> None:
    for s in streams:
        if s is not None and s.axis != axis:
            raise ValueError("cross-loop stream uses the wrong quantization axis")


def kivi_fused_dense_source_attention(*, query, current_key, current_value, key_streams, value_streams,
                                      rank_maps, tail_key, tail_value, scaling, loop, extension=None,
                                      require_cuda=True, return_logits=False):
    """Fuse full Loop-1/2 KIVI QK, softmax and PV in one launch (kivi_backend.py:899-992)."""

    if int(loop) not in (0, 1):
        raise ValueError("dense source attention is only valid for Loop 1/2")
    _check_axis(key_streams, "per_channel")
    _check_axis(value_streams, "per_token")
    if any(t.dtype != torch.bfloat16 for t in (query, current_key, current_value, tail_key, tail_value)):
        raise ValueError("fused dense attention currently specializes BF16 vectors")
    layer = _adopt(key_streams, value_streams, rank_maps, tail_key, tail_value, loop)
    return layer.dense_source_attention(int(loop), query=query, current_key=current_key,
                                        current_value=current_value, scaling=float(scaling),
                                        return_logits=bool(return_logits))


def kivi_fused_sparse_attention_delta(*, query, current_key, current_value, key_streams, value_streams,
                                      rank_maps, tail_key, tail_value, indices, valid,
                                      source_selected_output, global_mass, current_position, scaling, loop,
                                      extension=None, require_cuda=True, return_current_logits=False):
    """Fuse KIVI QK, subset softmax, PV and cached-mass correction (kivi_backend.py:784-896)."""

    _check_axis(key_streams, "per_channel")
    _check_axis(value_streams, "per_token")
    if any(t.dtype != torch.bfloat16 for t in (current_key, current_value, tail_key, tail_value)):
        raise ValueError("fused attention currently specializes BF16 tail/current K/V")
    if query.dtype != torch.bfloat16:
        raise ValueError("fused attention currently specializes BF16 queries")
    layer = _adopt(key_streams, value_streams, rank_maps, tail_key, tail_value, loop)
    if int(current_position) != layer.token_count:
        raise ValueError("current_position differs from the packed prefix plus the tail")
    return layer.cached_mass_sparse_attention_delta(
        int(loop), query=query, current_key=current_key, current_value=current_value, indices=indices,
        valid=valid, source_selected_output=source_selected_output, global_mass=global_mass,
        scaling=float(scaling))


def kivi_fused_cross_loop_qk(query, streams, rank_maps, indices, *, loop, extension=None, require_cuda=True):
    """Read anchor plus all active K deltas in one CUDA launch (kivi_backend.py:678-727)."""

    _check_axis(streams, "per_channel")
    empty = query.new_zeros((*query.shape[:2], 0, query.shape[-1]))
    layer = _adopt(streams, streams, rank_maps, empty, empty, loop)
    return layer.qk(int(loop), query, indices, validate_indices=False)


def kivi_fused_cross_loop_pv(weights, streams, rank_maps, indices, *, loop, extension=None, require_cuda=True):
    """Accumulate anchor plus all active V deltas in one CUDA launch (kivi_backend.py:730-781)."""

    _check_axis(streams, "per_token")
    anchor = streams[0]
    empty = torch.zeros((*anchor.original_shape[:2], 0, anchor.original_shape[3]), dtype=torch.bfloat16,
                        device=anchor.payload.device)
    layer = _adopt(streams, streams, rank_maps, empty, empty, loop)
    return layer.pv(int(loop), weights, indices, validate_indices=False)
