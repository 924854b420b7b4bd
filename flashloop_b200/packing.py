"""Row-layout 4-bit (and 2-bit) KV storage, packed on the GPU.

Mirrors the interface of the reference's flashloop/packing.py: ``Packed4Bit``
(:71-143), ``pack_k_per_channel`` (:146-170) and ``pack_v_per_token`` (:173-197).
Codes are packed along the channel dimension, the even channel in the low nibble.
The reference's Torch codec is replaced by the ``fl_pack_k_rows`` /
``fl_pack_v_rows`` kernels, which produce the same bytes.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from . import _native

_FLOAT_DTYPES = (torch.float16, torch.bfloat16, torch.float32)


def _validate_values(values: torch.Tensor, group_size: int) -> int:
    """Same checks and messages as flashloop/packing.py:22-32."""

    if values.ndim != 4:
        raise ValueError("KV values must have shape [batch, heads, tokens, channels]")
    if values.dtype not in _FLOAT_DTYPES:
        raise TypeError("KV values must use a floating-point dtype")
    if values.shape[-2] <= 0 or values.shape[-1] <= 0:
        raise ValueError("KV values require non-empty token and channel dimensions")
    group_size = int(group_size)
    if group_size <= 0:
        raise ValueError("group_size must be positive")
    if int(values.shape[-1]) != 128 or group_size != 64:
        raise ValueError("the CUDA pack specializes head_dim=128, group_size=64")
    _native.require_cuda(values)
    return group_size


@dataclass(frozen=True)
class Packed4Bit:
    """Packed payload and two-byte affine metadata (flashloop/packing.py:71-99).

    payload uint8 [B, H, n, 16*bits]; K metadata float16 [B, H, ceil(n/64), 128]; V
    metadata float16 [B, H, n, 2].  ``bits`` is 4 for the reference's layout."""

    payload: torch.Tensor
    minimum: torch.Tensor
    scale: torch.Tensor
    original_shape: tuple[int, int, int, int]
    original_dtype: torch.dtype
    axis: str
    group_size: int
    row_groups: torch.Tensor | None = None
    bits: int = 4

    def __post_init__(self) -> None:
        if self.payload.dtype != torch.uint8:
            raise TypeError("packed payload must be uint8")
        if self.minimum.dtype != torch.float16 or self.scale.dtype != torch.float16:
            raise TypeError("packed metadata must be float16")
        if self.minimum.shape != self.scale.shape:
            raise ValueError("minimum and scale shapes differ")
        if self.axis not in {"per_channel", "per_token"}:
            raise ValueError("unknown packed axis")
        if self.row_groups is not None:
            if self.axis != "per_channel":
                raise ValueError("explicit row groups are only valid for per-channel K")
            if self.row_groups.dtype != torch.int32 or self.row_groups.ndim != 1:
                raise TypeError("row_groups must be one-dimensional int32")
            if self.row_groups.numel() != self.original_shape[2]:
                raise ValueError("row_groups must identify every stored token row")

    @property
    def storage_bytes(self) -> int:
        tensors = [self.payload, self.minimum, self.scale]
        if self.row_groups is not None:
            tensors.append(self.row_groups)
        return sum(int(t.numel() * t.element_size()) for t in tensors)

    def decode(self) -> torch.Tensor:
        """``code * scale + minimum`` in float32, cast to bfloat16 (packing.py:108-132).

        Streams with explicit ``row_groups`` are decoded through a gathered copy of the
        metadata so that the same kernel serves both cases."""

        batch, heads, tokens, channels = self.original_shape
        if tuple(self.payload.shape[:3]) != (batch, heads, tokens):
            raise RuntimeError("packed payload shape no longer matches metadata")
        lib = _native.load()
        out = torch.empty((batch, heads, tokens, channels), dtype=torch.bfloat16, device=self.payload.device)
        per_channel = self.axis == "per_channel"
        minimum, scale = self.minimum, self.scale
        if per_channel and self.row_groups is not None:
            first = torch.arange(0, tokens, 64, device=self.payload.device)
            groups = self.row_groups.to(self.payload.device).long().index_select(0, first)
            blocks = self.row_groups.to(self.payload.device).long()
            expected = groups.repeat_interleave(64)[:tokens]
            if not torch.equal(expected, blocks):
                raise ValueError("row_groups must be constant on 64-row blocks")
            minimum = minimum.index_select(2, groups)
            scale = scale.index_select(2, groups)
        minimum = minimum.contiguous()
        scale = scale.contiguous()
        _native.check(lib.fl_decode_rows(
            _native.ptr(self.payload.contiguous()), _native.ptr(minimum), _native.ptr(scale),
            1 if per_channel else 0, 2, batch * heads, tokens, self.bits, _native.ptr(out),
            _native.current_stream(out.device)), "fl_decode_rows")
        return out if self.original_dtype == torch.bfloat16 else out.to(self.original_dtype)

    def decode_rows(self, indices: torch.Tensor) -> torch.Tensor:
        """packing.py:134-143."""

        if indices.ndim != 1:
            raise ValueError("decode_rows expects one-dimensional indices")
        indices = indices.to(device=self.payload.device, dtype=torch.long)
        if indices.numel() and (int(indices.min().item()) < 0
                                or int(indices.max().item()) >= self.original_shape[2]):
            raise IndexError("decode row index is outside the packed token range")
        return self.decode().index_select(2, indices)


def _pack(values: torch.Tensor, *, axis: str, group_size: int, bits: int) -> Packed4Bit:
    if bits not in (4, 2):
        raise ValueError("bits must be 4 or 2")
    lib = _native.load()
    values = values.contiguous()
    batch, heads, tokens, channels = (int(v) for v in values.shape)
    device = values.device
    payload = torch.empty((batch, heads, tokens, 16 * bits), dtype=torch.uint8, device=device)
    stream = _native.current_stream(device)
    if axis == "per_channel":
        groups = (tokens + group_size - 1) // group_size
        minimum = torch.empty((batch, heads, groups, channels), dtype=torch.float16, device=device)
        scale = torch.empty_like(minimum)
        _native.check(lib.fl_pack_k_rows(
            _native.ptr(values), _native.DTYPE_CODES[values.dtype], batch * heads, tokens, bits,
            _native.ptr(payload), _native.ptr(minimum), _native.ptr(scale), stream), "fl_pack_k_rows")
    else:
        minimum = torch.empty((batch, heads, tokens, 2), dtype=torch.float16, device=device)
        scale = torch.empty_like(minimum)
        _native.check(lib.fl_pack_v_rows(
            _native.ptr(values), _native.DTYPE_CODES[values.dtype], batch * heads, tokens, bits,
            _native.ptr(payload), _native.ptr(minimum), _native.ptr(scale), 2, stream), "fl_pack_v_rows")
    return Packed4Bit(payload=payload, minimum=minimum, scale=scale,
                      original_shape=(batch, heads, tokens, channels),
                      original_dtype=values.dtype, axis=axis, group_size=group_size, bits=bits)


def pack_k_per_channel(values: torch.Tensor, *, group_size: int = 64, bits: int = 4) -> Packed4Bit:
    """Pack K with affine parameters per channel over token groups (packing.py:146-170)."""

    group_size = _validate_values(values, group_size)
    return _pack(values, axis="per_channel", group_size=group_size, bits=bits)


def pack_v_per_token(values: torch.Tensor, *, group_size: int = 64, bits: int = 4) -> Packed4Bit:
    """Pack V with affine parameters per token over channel groups (packing.py:173-197)."""

    group_size = _validate_values(values, group_size)
    return _pack(values, axis="per_token", group_size=group_size, bits=bits)
