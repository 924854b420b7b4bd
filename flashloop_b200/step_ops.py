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
            weight2: torch.Tensor | None = None, eps2: float = 0.0, addend: torch.Tensor | None = None):
    """``out = [residual +] RMSNorm([addend +] x)``; with ``weight2`` also ``RMSNorm2(out)``.  Returns
    out or (out, out2)."""

    _bf16(x, weight, residual, weight2, addend)
    if addend is not None and addend.shape != x.shape:
        raise ValueError("addend does not match the rows")
    rows, width = _rows(x)
    if weight.numel() != width or (residual is not None and residual.shape != x.shape):
        raise ValueError("weight / residual do not match the rows")
    out = torch.empty_like(x)
    out2 = torch.empty_like(x) if weight2 is not None else None
    _native.check(_native.load().fl_rmsnorm(
        _native.ptr(x), _native.ptr(addend), _native.ptr(residual), _native.ptr(weight), float(eps),
        _native.ptr(weight2), float(eps2),
        rows, width, _native.ptr(out), _native.ptr(out2), _native.current_stream(x.device)), "fl_rmsnorm")
    return out if weight2 is None else (out, out2)


def rmsnorm_partial(partial: torch.Tensor, weight: torch.Tensor, eps: float, *,
                    residual: torch.Tensor | None = None, weight2: torch.Tensor | None = None, eps2: float = 0.0,
                    addend: torch.Tensor | None = None, want_sum: bool = False):
    """:func:`rmsnorm` of ``x = bfloat16(sum of the float32 slices partial[s])`` ([splits, rows, 1, width],
    as :func:`linear_partial` leaves them), the sum and its one rounding done in the same launch.
    Returns (out, out2 or None, x or None): x only with ``want_sum``."""

    if partial.dtype != torch.float32 or partial.ndim != 4 or not partial.is_contiguous():
        raise ValueError("partial sums must be contiguous float32 [splits, rows, 1, width]")
    _native.require_cuda(partial)
    splits, rows, _, width = (int(v) for v in partial.shape)
    _bf16(weight, residual, weight2, addend)
    shape = (rows, 1, width)
    for t in (residual, addend):
        if t is not None and tuple(t.shape) != shape:
            raise ValueError("addend / residual do not match the rows")
    if weight.numel() != width:
        raise ValueError("weight does not match the rows")
    out = torch.empty(shape, dtype=torch.bfloat16, device=partial.device)
    out2 = torch.empty_like(out) if weight2 is not None else None
    total = torch.empty_like(out) if want_sum else None
    _native.check(_native.load().fl_rmsnorm_partial(
        _native.ptr(partial), splits, _native.ptr(addend), _native.ptr(residual), _native.ptr(weight), float(eps),
        _native.ptr(weight2), float(eps2), rows, width, _native.ptr(total), _native.ptr(out), _native.ptr(out2),
        _native.current_stream(partial.device)), "fl_rmsnorm_partial")
    return out, out2, total


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



MAX_LINEAR_ROWS = 16


def linear_fits(x: torch.Tensor, weight: torch.Tensor) -> bool:
    """Whether :func:`linear` takes this product (a decode step's shapes); otherwise the caller uses
    the framework's GEMM."""

    return (x.is_cuda and x.dtype in (torch.bfloat16, torch.float32) and weight.dtype == torch.bfloat16
            and weight.is_contiguous() and x.is_contiguous() and x.numel() // x.shape[-1] <= MAX_LINEAR_ROWS
            and weight.shape[1] % 32 == 0 and weight.shape[0] % 32 == 0 and x.data_ptr() % 16 == 0
            and weight.data_ptr() % 16 == 0)


def linear(x: torch.Tensor, weight: torch.Tensor, *, swiglu: bool = False) -> torch.Tensor:
    """``x @ weight.T`` for at most 16 rows, one launch that streams the weight once; bfloat16 out.
    A float32 ``x`` is rounded to bfloat16 as it is read.  With ``swiglu`` the weight is gate rows then
    up rows and the result is ``silu(gate) * up`` (as :func:`swiglu` of the product)."""

    if x.dtype not in (torch.bfloat16, torch.float32) or not x.is_contiguous():
        raise TypeError("x must be contiguous bfloat16 or float32")
    _bf16(weight)
    _native.require_cuda(x)
    rows, width = _rows(x)
    out_features, in_features = (int(v) for v in weight.shape)
    if width != in_features:
        raise ValueError("x and weight do not match")
    out = torch.empty((*x.shape[:-1], out_features // 2 if swiglu else out_features), dtype=torch.bfloat16,
                      device=x.device)
    _native.check(_native.load().fl_linear_rows(
        _native.ptr(x), _native.DTYPE_CODES[x.dtype], _native.ptr(weight), rows, out_features, in_features,
        int(bool(swiglu)), _native.ptr(out), _native.current_stream(x.device)), "fl_linear_rows")
    return out


LINEAR_SPLITS = 4              # slices of in_features of a split projection
MAX_SPLIT_OUT_FEATURES = 4096  # above that the weight has tiles enough for linear()'s kernels


def linear_partial_fits(x: torch.Tensor, weight: torch.Tensor) -> bool:
    """Whether :func:`linear_partial` takes this product: what :func:`linear` takes, few output
    rows, and in_features that fall into LINEAR_SPLITS slices of at most 1536 values."""

    if not linear_fits(x, weight):
        return False
    out_features, in_features = (int(v) for v in weight.shape)
    return (out_features <= MAX_SPLIT_OUT_FEATURES and out_features % 8 == 0
            and in_features % (32 * LINEAR_SPLITS) == 0 and in_features // LINEAR_SPLITS <= 1536)


def linear_partial(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """``x @ weight.T`` left as LINEAR_SPLITS float32 partial sums [splits, rows, 1, out_features] over
    slices of in_features (``fl_linear_rows_partial``): every CTA keeps one slice of x in registers
    instead of reading all of it, which for the projections with few output rows (``o_proj``,
    ``down_proj``) is more bytes than the weight.  :func:`rmsnorm_partial` adds the slices."""

    if not linear_partial_fits(x, weight):
        raise ValueError("this product does not fit linear_partial")
    rows = x.numel() // x.shape[-1]
    out_features, in_features = (int(v) for v in weight.shape)
    partial = torch.empty((LINEAR_SPLITS, rows, 1, out_features), dtype=torch.float32, device=x.device)
    _native.check(_native.load().fl_linear_rows_partial(
        _native.ptr(x), _native.DTYPE_CODES[x.dtype],
        _native.ptr(weight), rows, out_features, in_features, LINEAR_SPLITS, _native.ptr(partial),
        _native.current_stream(x.device)), "fl_linear_rows_partial")
    return partial


def qkv_rope(x: torch.Tensor, weight: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, *, heads: int):
    """The fused Q/K/V projection with rotate-half RoPE on the way out: x [B, 1, hidden], weight
    [3 * heads * 128, hidden] (q, k, v rows), cos/sin [B, 1, 128].  Returns q, k (rotated) and v as
    [B, heads, 1, 128]: what :func:`linear` followed by :func:`rope_split` returns."""

    cos, sin = cos.contiguous(), sin.contiguous()
    _bf16(x, weight, cos, sin)
    batch, width = _rows(x)
    if tuple(weight.shape) != (3 * heads * 128, width) or cos.numel() != batch * 128 or sin.numel() != batch * 128:
        raise ValueError("weight must be [3 * heads * 128, hidden] and cos / sin [batch, 1, 128]")
    outs = [torch.empty((batch, heads, 1, 128), dtype=torch.bfloat16, device=x.device) for _ in range(3)]
    _native.check(_native.load().fl_qkv_rope_rows(
        _native.ptr(x), _native.ptr(weight), batch, heads, width, _native.ptr(cos), _native.ptr(sin),
        _native.ptr(outs[0]), _native.ptr(outs[1]), _native.ptr(outs[2]), _native.current_stream(x.device)),
        "fl_qkv_rope_rows")
    return tuple(outs)
