"""bfloat16 arithmetic on numpy float32 arrays (numpy has no bfloat16 dtype).

A "bf16 array" here is a float32 array whose values are all representable in
bfloat16.  Torch's CPU bfloat16 operators convert both operands to float32,
apply the float32 operation and round the result back to bfloat16 with
round-to-nearest-even; ``sub`` and ``add`` below restate exactly that, which is
what the reference relies on when it forms loop-to-loop residuals
(flashloop/cache.py:425, 1021-1026, 1061-1074).
"""

from __future__ import annotations

import numpy as np


def round_to_bf16(values: np.ndarray) -> np.ndarray:
    """Round float32 values to the nearest bfloat16 (ties to even); keeps float32 dtype."""

    work = np.ascontiguousarray(values, dtype=np.float32)
    bits = work.view(np.uint32)
    lsb = (bits >> np.uint32(16)) & np.uint32(1)
    rounded = (bits + np.uint32(0x7FFF) + lsb) & np.uint32(0xFFFF0000)
    nan = np.isnan(work)
    if nan.any():
        rounded = np.where(nan, bits | np.uint32(0x00400000), rounded)
    return rounded.astype(np.uint32).view(np.float32).reshape(work.shape)


def to_bits(values: np.ndarray) -> np.ndarray:
    """bf16-representable float32 array -> uint16 bit patterns."""

    work = np.ascontiguousarray(values, dtype=np.float32)
    return (work.view(np.uint32) >> np.uint32(16)).astype(np.uint16).reshape(work.shape)


def from_bits(bits: np.ndarray) -> np.ndarray:
    """uint16 bfloat16 bit patterns -> float32 array."""

    wide = np.ascontiguousarray(bits, dtype=np.uint16).astype(np.uint32) << np.uint32(16)
    return wide.view(np.float32).reshape(bits.shape)


def sub(left: np.ndarray, right: np.ndarray) -> np.ndarray:
    return round_to_bf16(left.astype(np.float32) - right.astype(np.float32))


def add(left: np.ndarray, right: np.ndarray) -> np.ndarray:
    return round_to_bf16(left.astype(np.float32) + right.astype(np.float32))
