"""One-launch versions of the elementwise glue of a decode step (``csrc/fl_step.cu``): RMSNorm,
residual add + RMSNorm (+ the next RMSNorm), Q/K/V split with rotate-half RoPE, SwiGLU.

They restate what the reference's decode loop calls on the model's modules
(flashloop/engine.py:396-437, 533-537; flashloop/weights.py:108-117) for one token per row,
with the roundings of bfloat16 tensor ops.
"""

from __future__ import annotations

import torch

from . import _native


def _rows(x: torch.Tensor) -> tuple[int, int]:
    width = int(x.shape[-1])
    return x.numel() // width, width


def _bf16(*tensors) -> None:
    for t in tensors:
        if t is not None and (t.dtype != torch.bfloat16 or not t.is_contiguous()):
            raise TypeError("decode-step kernels take contiguous bfloat16 tensors")
    _native.require_cuda(*[t for t in tensors if t is not None])


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, *, residual: torch.Tensor | None = None,
            weight2: torch.Tensor | None = None, eps2: float = 0.0):
    """``out = [residual +] RMSNorm(x)``; with ``weight2`` also ``RMSNorm2(out)``.  Returns out or
    (out, out2)."""

    _bf16(x, weight, residual, weight2)
    rows, width = _rows(x)
    if weight.numel() != width or (residual is not None and residual.shape != x.shape):
        raise ValueError("weight / residual do not match the rows")
    out = torch.empty_like(x)
    out2 = torch.empty_like(x) if weight2 is not None else None
    _native.check(_native.load().fl_rmsnorm(
        _native.ptr(x), _native.ptr(residual), _native.ptr(weight), float(eps), _native.ptr(weight2), float(eps2),
        rows, width, _native.ptr(out), _native.ptr(out2), _native.current_stream(x.device)), "fl_rmsnorm")
    return out if weight2 is None else (out, out2)


def rope_split(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, *,
               heads: int):
    """q, k, v: [B, 1, heads*128] (views of one fused projection are fine: rows may be strided);
    cos, sin: [B, 1, 128].  Returns q, k (RoPE applied) and v as [B, heads, 1, 128]."""

    batch = int(q.shape[0])
    width = heads * 128
    for t in (q, k, v):
        if t.dtype != torch.bfloat16 or t.shape[-1] != width or t.stride(-1) != 1 or t.numel() != batch * width:
            raise ValueError("projections must be bfloat16 [batch, 1, heads*128] with unit inner stride")
    stride = int(q.stride(0))
    if int(k.stride(0)) != stride or int(v.stride(0)) != stride:
        raise ValueError("projections must share their row stride")
    _bf16(cos.contiguous(), sin.contiguous())
    _native.require_cuda(q, k, v)
    outs = [torch.empty((batch, heads, 1, 128), dtype=torch.bfloat16, device=q.device) for _ in range(3)]
    _native.check(_native.load().fl_rope_split(
        _native.ptr(q), _native.ptr(k), _native.ptr(v), stride, _native.ptr(cos.contiguous()),
        _native.ptr(sin.contiguous()), batch, heads, *[_native.ptr(o) for o in outs],
        _native.current_stream(q.device)), "fl_rope_split")
    return outs


def swiglu(gate_up: torch.Tensor) -> torch.Tensor:
    """``silu(gate) * up`` of [..., 2*width] (gate first)."""

    _bf16(gate_up)
    rows, double = _rows(gate_up)
    out = torch.empty((*gate_up.shape[:-1], double // 2), dtype=torch.bfloat16, device=gate_up.device)
    _native.check(_native.load().fl_swiglu(_native.ptr(gate_up), rows, double // 2, _native.ptr(out),
                                           _native.current_stream(gate_up.device)), "fl_swiglu")
    return out

