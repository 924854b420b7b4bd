"""Asymmetric min/max group quantiser and the two physical layouts (numpy oracle).

Restates, with numpy float32 arithmetic:

* the group quantiser ``_codes_for_group`` (flashloop/packing.py:35-46 and its twin
  flashloop/kivi_backend.py:272-283): ``min``/``max`` over the group, ``span/levels``
  by IEEE division, ``(x - min) / scale`` by IEEE subtraction then division,
  round-half-to-even, clamp, metadata stored as float16 while the codes are
  computed with the float32 ``min``/``scale``;
* the row layout ``Packed4Bit`` (flashloop/packing.py:49-54, 71-132, 146-197): one
  token per row, two channels per byte, even channel in the low nibble;
* the KIVI word layout ``KiviPacked4Bit`` (flashloop/kivi_backend.py:286-322,
  325-401, 404-475): eight outputs per int32 word, output ``8w + j`` in bits
  ``4j .. 4j+3``; outputs are tokens for K and channels for V.

The 2-bit variant is an extension (the reference engine rejects ``kv_bits != 4``,
flashloop/config.py:38-39; its fake-quant profile "kivi2_channel" uses 3 levels,
flashloop_torch/kv_quantization.py:28-33, 409).  Its row layout packs four
channels per byte, channel ``4j + i`` in bits ``2i .. 2i+1`` of byte ``j``.
"""

from __future__ import annotations

from dataclasses import dataclass

import numpy as np

from . import bf16

PACK_FACTOR = 8  # outputs per int32 word in the KIVI layout (kivi_backend.py:34)


def quantize_group(work: np.ndarray, *, reduce_axis: int, bits: int = 4):
    """codes (uint8), float16 minimum, float16 scale for one group (packing.py:35-46)."""

    work = work.astype(np.float32)
    levels = np.float32((1 << int(bits)) - 1)
    minimum = work.min(axis=reduce_axis, keepdims=True)
    maximum = work.max(axis=reduce_axis, keepdims=True)
    span = (maximum - minimum).astype(np.float32)
    with np.errstate(divide="ignore", invalid="ignore"):
        scale = np.where(span > 0, span / levels, np.float32(1.0)).astype(np.float32)
        scaled = ((work - minimum).astype(np.float32) / scale).astype(np.float32)
    codes = np.clip(np.rint(scaled), 0, levels).astype(np.uint8)
    with np.errstate(over="ignore"):
        return codes, minimum.astype(np.float16), scale.astype(np.float16)


def k_codes(values: np.ndarray, *, group_size: int = 64, bits: int = 4):
    """Per-channel K quantisation over token groups (packing.py:146-161).

    values: float array [B, H, n, D].  Returns codes [B,H,n,D] uint8 and float16
    minimum/scale [B,H,ceil(n/group),D].  A trailing partial group is allowed.
    """

    tokens = values.shape[2]
    codes, minima, scales = [], [], []
    for start in range(0, tokens, group_size):
        c, m, s = quantize_group(values[:, :, start:start + group_size, :], reduce_axis=2, bits=bits)
        codes.append(c)
        minima.append(m)
        scales.append(s)
    return (np.concatenate(codes, axis=2), np.concatenate(minima, axis=2),
            np.concatenate(scales, axis=2))


def v_codes(values: np.ndarray, *, group_size: int = 64, bits: int = 4):
    """Per-token V quantisation over channel groups (packing.py:173-188).

    Returns codes [B,H,n,D] and float16 minimum/scale [B,H,n,ceil(D/group)].
    """

    channels = values.shape[3]
    codes, minima, scales = [], [], []
    for start in range(0, channels, group_size):
        c, m, s = quantize_group(values[..., start:start + group_size], reduce_axis=3, bits=bits)
        codes.append(c)
        minima.append(m)
        scales.append(s)
    return (np.concatenate(codes, axis=3), np.concatenate(minima, axis=3),
            np.concatenate(scales, axis=3))


# ----------------------------------------------------------------------------- row layout


def pack_row_codes(codes: np.ndarray, *, bits: int = 4) -> np.ndarray:
    """[.., D] codes -> [.., D*bits/8] bytes (packing.py:49-54 for 4 bits)."""

    per_byte = 8 // bits
    if codes.shape[-1] % per_byte:
        pad = per_byte - codes.shape[-1] % per_byte
        codes = np.concatenate([codes, np.zeros((*codes.shape[:-1], pad), np.uint8)], axis=-1)
    out = np.zeros((*codes.shape[:-1], codes.shape[-1] // per_byte), np.uint8)
    for i in range(per_byte):
        out |= (codes[..., i::per_byte].astype(np.uint8) << np.uint8(bits * i)).astype(np.uint8)
    return out


def unpack_row_codes(payload: np.ndarray, channels: int, *, bits: int = 4) -> np.ndarray:
    """Inverse of :func:`pack_row_codes` (packing.py:57-68)."""

    per_byte = 8 // bits
    mask = np.uint8((1 << bits) - 1)
    codes = np.zeros((*payload.shape[:-1], payload.shape[-1] * per_byte), np.uint8)
    for i in range(per_byte):
        codes[..., i::per_byte] = (payload >> np.uint8(bits * i)) & mask
    return codes[..., :channels]


@dataclass
class PackedRows:
    """Row layout: payload uint8 [B,H,n,D*bits/8]; K metadata [B,H,groups,D], V metadata
    [B,H,n,D/group] (packing.py:71-99).  ``row_groups`` (int32 [n]) names the metadata
    group of every K row when groups are not plain ``row // group_size`` blocks."""

    payload: np.ndarray
    minimum: np.ndarray
    scale: np.ndarray
    shape: tuple
    axis: str
    group_size: int = 64
    bits: int = 4
    row_groups: np.ndarray | None = None

    def codes(self) -> np.ndarray:
        return unpack_row_codes(self.payload, self.shape[3], bits=self.bits)

    def decode_f32(self) -> np.ndarray:
        """code * scale + minimum in float32, before the cast to the storage dtype
        (packing.py:108-132)."""

        tokens, channels = self.shape[2], self.shape[3]
        codes = self.codes().astype(np.float32)
        if self.axis == "per_channel":
            if self.row_groups is None:
                groups = np.arange(tokens) // self.group_size
            else:
                groups = self.row_groups.astype(np.int64)
            minimum = self.minimum[:, :, groups, :].astype(np.float32)
            scale = self.scale[:, :, groups, :].astype(np.float32)
        else:
            cg = np.arange(channels) // self.group_size
            minimum = self.minimum[..., cg].astype(np.float32)
            scale = self.scale[..., cg].astype(np.float32)
        return (codes * scale).astype(np.float32) + minimum

    def decode(self) -> np.ndarray:
        """Decoded values rounded to bfloat16 (the cache's storage dtype)."""

        return bf16.round_to_bf16(self.decode_f32())

    @property
    def storage_bytes(self) -> int:
        total = self.payload.nbytes + self.minimum.nbytes + self.scale.nbytes
        if self.row_groups is not None:
            total += self.row_groups.nbytes
        return int(total)


def pack_k_rows(values: np.ndarray, *, group_size: int = 64, bits: int = 4) -> PackedRows:
    codes, minimum, scale = k_codes(values, group_size=group_size, bits=bits)
    return PackedRows(pack_row_codes(codes, bits=bits), minimum, scale, tuple(values.shape),
                      "per_channel", group_size, bits)


def pack_v_rows(values: np.ndarray, *, group_size: int = 64, bits: int = 4) -> PackedRows:
    codes, minimum, scale = v_codes(values, group_size=group_size, bits=bits)
    return PackedRows(pack_row_codes(codes, bits=bits), minimum, scale, tuple(values.shape),
                      "per_token", group_size, bits)


def concat_rows(left: PackedRows | None, right: PackedRows | None) -> PackedRows | None:
    """Append ``right`` after ``left`` keeping every row's own metadata group
    (flashloop/cache.py:202-242, the ``Packed4Bit`` branch of ``_concat_packed``)."""

    if left is None:
        return right
    if right is None:
        return left
    row_groups = None
    if left.axis == "per_channel":
        lg = left.row_groups if left.row_groups is not None else (
            np.arange(left.shape[2]) // left.group_size).astype(np.int32)
        rg = right.row_groups if right.row_groups is not None else (
            np.arange(right.shape[2]) // right.group_size).astype(np.int32)
        row_groups = np.concatenate([lg, rg + np.int32(left.minimum.shape[2])]).astype(np.int32)
    return PackedRows(
        np.concatenate([left.payload, right.payload], axis=2),
        np.concatenate([left.minimum, right.minimum], axis=2),
        np.concatenate([left.scale, right.scale], axis=2),
        (left.shape[0], left.shape[1], left.shape[2] + right.shape[2], left.shape[3]),
        left.axis, left.group_size, left.bits, row_groups)


# ----------------------------------------------------------------------------- KIVI word layout


def pack_output_words(codes: np.ndarray) -> np.ndarray:
    """[B,H,out,in] codes -> int32 [B,H,ceil(out/8),in] (kivi_backend.py:286-311)."""

    out = codes.shape[2]
    padded = -(-out // PACK_FACTOR) * PACK_FACTOR
    if padded != out:
        codes = np.concatenate(
            [codes, np.zeros((*codes.shape[:2], padded - out, codes.shape[3]), codes.dtype)], axis=2)
    words = codes.reshape(*codes.shape[:2], padded // PACK_FACTOR, PACK_FACTOR, codes.shape[3])
    acc = np.zeros((*codes.shape[:2], padded // PACK_FACTOR, codes.shape[3]), np.uint32)
    for j in range(PACK_FACTOR):
        acc |= words[:, :, :, j, :].astype(np.uint32) << np.uint32(4 * j)
    return acc.view(np.int32)


def unpack_output_words(payload: np.ndarray, outputs: int) -> np.ndarray:
    """Inverse of :func:`pack_output_words` (kivi_backend.py:314-322)."""

    words = payload.view(np.uint32)
    codes = np.stack([(words >> np.uint32(4 * j)) & np.uint32(0xF) for j in range(PACK_FACTOR)],
                     axis=3)
    codes = codes.reshape(*payload.shape[:2], payload.shape[2] * PACK_FACTOR, payload.shape[3])
    return codes[:, :, :outputs, :].astype(np.uint8)


@dataclass
class PackedKivi:
    """KIVI layout (kivi_backend.py:325-366).  K: payload [B,H,ceil(n/8),D], metadata
    [B,H,ceil(n/group),D].  V: payload [B,H,ceil(D/8),n], metadata [B,H,ceil(D/group),n]."""

    payload: np.ndarray
    minimum: np.ndarray
    scale: np.ndarray
    shape: tuple
    axis: str
    group_size: int = 64

    def codes(self) -> np.ndarray:
        """Codes in logical [B,H,n,D] order."""

        _, _, tokens, channels = self.shape
        if self.axis == "per_channel":
            return unpack_output_words(self.payload, tokens)
        return unpack_output_words(self.payload, channels).transpose(0, 1, 3, 2)

    def decode_f32(self) -> np.ndarray:
        _, _, tokens, channels = self.shape
        codes = self.codes().astype(np.float32)
        if self.axis == "per_channel":
            groups = np.arange(tokens) // self.group_size
            minimum = self.minimum[:, :, groups, :].astype(np.float32)
            scale = self.scale[:, :, groups, :].astype(np.float32)
        else:
            cg = np.arange(channels) // self.group_size
            minimum = self.minimum[:, :, cg, :].astype(np.float32).transpose(0, 1, 3, 2)
            scale = self.scale[:, :, cg, :].astype(np.float32).transpose(0, 1, 3, 2)
        return (codes * scale).astype(np.float32) + minimum

    def decode(self) -> np.ndarray:
        return bf16.round_to_bf16(self.decode_f32())

    @property
    def storage_bytes(self) -> int:
        return int(self.payload.nbytes + self.minimum.nbytes + self.scale.nbytes)


def pack_kivi_k(values: np.ndarray, *, group_size: int = 64) -> PackedKivi:
    """kivi_backend.py:404-438 (CPU branch)."""

    codes, minimum, scale = k_codes(values, group_size=group_size)
    return PackedKivi(pack_output_words(codes), minimum, scale, tuple(values.shape),
                      "per_channel", group_size)


def pack_kivi_v(values: np.ndarray, *, group_size: int = 64) -> PackedKivi:
    """kivi_backend.py:441-475 (CPU branch): codes transposed to [channel, token]."""

    codes, minimum, scale = v_codes(values, group_size=group_size)
    matrix = np.ascontiguousarray(codes.transpose(0, 1, 3, 2))
    return PackedKivi(pack_output_words(matrix),
                      np.ascontiguousarray(minimum.transpose(0, 1, 3, 2)),
                      np.ascontiguousarray(scale.transpose(0, 1, 3, 2)),
                      tuple(values.shape), "per_token", group_size)


def kivi_to_rows(packed: PackedKivi) -> PackedRows:
    """Same codes and metadata, row layout (pure re-arrangement of bits)."""

    codes = packed.codes()
    if packed.axis == "per_channel":
        return PackedRows(pack_row_codes(codes), packed.minimum, packed.scale, packed.shape,
                          "per_channel", packed.group_size)
    return PackedRows(pack_row_codes(codes),
                      np.ascontiguousarray(packed.minimum.transpose(0, 1, 3, 2)),
                      np.ascontiguousarray(packed.scale.transpose(0, 1, 3, 2)),
                      packed.shape, "per_token", packed.group_size)
