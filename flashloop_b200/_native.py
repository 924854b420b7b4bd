"""ctypes binding of ``csrc/libflashloop_b200.so`` (the C ABI of include/flashloop_b200.h).

There is no fallback: when the library is missing or a call fails, a RuntimeError is
raised.  Build the library with ``python -m flashloop_b200.build_kernels``.
"""

from __future__ import annotations

import ctypes as C
from pathlib import Path

import torch

LIBRARY_PATH = Path(__file__).resolve().parent / "csrc" / "libflashloop_b200.so"

FL_STREAMS = 4
FL_STATE_WORDS = 8
STATE_QUANT_TOKENS, STATE_TAIL_LEN, STATE_TAIL_START, STATE_ROWS2, STATE_ROWS3 = 0, 1, 2, 3, 4
DTYPE_CODES = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}

_vp = C.c_void_p
_i32, _i64, _f32, _f64, _sz = C.c_int32, C.c_int64, C.c_float, C.c_double, C.c_size_t


class FlLayer(C.Structure):
    """``fl_layer`` of include/flashloop_b200.h."""

    _fields_ = [
        ("batch", _i32), ("heads", _i32), ("bits", _i32), ("tail_capacity", _i32),
        ("k_codes", _vp * FL_STREAMS), ("k_min", _vp * FL_STREAMS), ("k_scale", _vp * FL_STREAMS),
        ("v_rows", _vp * FL_STREAMS),
        ("row_base", _vp * FL_STREAMS), ("group_base", _vp * FL_STREAMS),
        ("rank", _vp * 2), ("rank_base", _vp),
        ("tail_k", _vp * FL_STREAMS), ("tail_v", _vp * FL_STREAMS),
        ("tail_active", _vp * 2), ("seq_state", _vp),
    ]


# name -> (restype, argtypes); every name here is declared in include/flashloop_b200.h
SIGNATURES = {
    "fl_last_error": (C.c_char_p, []),
    "fl_version": (C.c_int, []),
    "fl_pack_k_rows": (C.c_int, [_vp, _i32, _i64, _i64, _i32, _vp, _vp, _vp, _vp]),
    "fl_pack_v_rows": (C.c_int, [_vp, _i32, _i64, _i64, _i32, _vp, _vp, _vp, _i64, _vp]),
    "fl_pack_kivi_k": (C.c_int, [_vp, _i32, _i64, _i64, _vp, _vp, _vp, _vp]),
    "fl_pack_kivi_v": (C.c_int, [_vp, _i32, _i64, _i64, _vp, _vp, _vp, _vp]),
    "fl_decode_rows": (C.c_int, [_vp, _vp, _vp, _i32, _i64, _i64, _i64, _i32, _vp, _vp]),
    "fl_kivi_to_rows_k": (C.c_int, [_vp, _i64, _i64, _vp, _vp]),
    "fl_kivi_to_rows_v": (C.c_int, [_vp, _vp, _vp, _i64, _i64, _vp, _vp, _vp, _i64, _vp]),
    "fl_reader_workspace_bytes": (_sz, [_i64, _i64]),
    "fl_workspace_init": (C.c_int, [_vp, _sz, _vp]),
    "fl_workspace_status": (C.c_int, [_vp, _i64, C.POINTER(_i32), _vp]),
    "fl_dense_source_attention": (C.c_int, [C.POINTER(FlLayer), _i32, _vp, _vp, _vp, _f32, _vp, _vp,
                                            _i64, _i64, _vp, _sz, _vp]),
    "fl_dense_source_attention_static": (C.c_int, [C.POINTER(FlLayer), _i32, _vp, _vp, _vp, _f32, _vp, _vp,
                                                   _i64, _i64, _vp]),
    "fl_static_status": (C.c_int, [C.POINTER(_i32), _vp]),
    "fl_sparse_attention_delta": (C.c_int, [C.POINTER(FlLayer), _i32, _vp, _vp, _vp, _vp, _vp, _i64,
                                            _vp, _vp, _f32, _vp, _vp, _vp, _sz, _vp]),
    "fl_selected_pv": (C.c_int, [C.POINTER(FlLayer), _i32, _vp, _vp, _vp, _i64, _vp, _vp, _vp, _sz, _vp]),
    "fl_selected_qk": (C.c_int, [C.POINTER(FlLayer), _i32, _vp, _vp, _vp, _i64, _vp, _vp, _vp]),
    "fl_append_decode_token": (C.c_int, [C.POINTER(FlLayer), C.POINTER(_vp), C.POINTER(_vp), _vp]),
    "fl_select_decode_keys": (C.c_int, [_vp, _i64, _i32, _i32, _i32, _vp, _f64, _i32, _vp, _vp, _i64,
                                        _vp, _vp, _vp, _vp]),
    "fl_hidden_delta_score": (C.c_int, [_vp, _vp, _i64, _i32, _vp, _vp]),
    "fl_select_prefill_tokens": (C.c_int, [_vp, _vp, _i32, _i32, _f64, _i32, _vp, _vp, _vp, _vp, _vp]),
    "fl_gather_rows": (C.c_int, [_vp, _vp, _vp, _vp, _i64, _i64, _i32, _i64, _i64, _i32, _vp]),
    "fl_scatter_rows": (C.c_int, [_vp, _vp, _vp, _vp, _i64, _i64, _i32, _i64, _i64, _i32, _vp]),
    "fl_encode_prefill": (C.c_int, [_vp, _i32, _i32, _i64, _vp, _vp, _vp, _vp, _i64, _vp, _vp, _vp]),
    "fl_encode_prefill_stage": (C.c_int, [_vp, _i32, _i32, _i64, _i32, _vp, _vp, _vp, _i64, _i32, _vp]),
    "fl_rmsnorm": (C.c_int, [_vp, _vp, _vp, _vp, _f32, _vp, _f32, _i64, _i32, _vp, _vp, _vp]),
    "fl_rope_split": (C.c_int, [_vp, _vp, _vp, _i64, _vp, _vp, _i64, _i32, _vp, _vp, _vp, _vp]),
    "fl_swiglu": (C.c_int, [_vp, _i64, _i32, _vp, _vp]),
    "fl_linear_rows": (C.c_int, [_vp, _i32, _vp, _i64, _i32, _i32, _i32, _vp, _vp]),
    "fl_qkv_rope_rows": (C.c_int, [_vp, _vp, _i64, _i32, _i32, _vp, _vp, _vp, _vp, _vp, _vp]),
    "fl_linear_rows_partial": (C.c_int, [_vp, _i32, _vp, _i64, _i32, _i32, _i32, _vp, _vp]),
    "fl_rmsnorm_partial": (C.c_int, [_vp, _i32, _vp, _vp, _vp, _f32, _vp, _f32, _i64, _i32, _vp, _vp, _vp, _vp]),
    "fl_comm_handle_bytes": (_sz, []),
    "fl_comm_create": (C.c_int, [_i32, _i32, _i32, _i32, C.POINTER(_vp), _vp]),
    "fl_comm_connect": (C.c_int, [_vp, _vp]),
    "fl_comm_destroy": (C.c_int, [_vp]),
    "fl_comm_status": (C.c_int, [_vp, C.POINTER(_i32), _i32, _vp]),
    "fl_allreduce_rmsnorm": (C.c_int, [_vp, _vp, _vp, _vp, _vp, _f32, _vp, _f32, _i64, _vp, _vp, _vp, _i32, _i32,
                                       _vp]),
}

# kernels launched by one call of an entry point (entry points that launch nothing are absent)
LAUNCHES_PER_CALL = {
    "fl_pack_k_rows": 1, "fl_pack_v_rows": 1, "fl_pack_kivi_k": 1, "fl_pack_kivi_v": 1, "fl_decode_rows": 1,
    "fl_kivi_to_rows_k": 1, "fl_kivi_to_rows_v": 1, "fl_dense_source_attention": 1,
    "fl_dense_source_attention_static": 1, "fl_sparse_attention_delta": 1, "fl_selected_pv": 1, "fl_selected_qk": 1,
    "fl_append_decode_token": 3, "fl_select_decode_keys": 1, "fl_hidden_delta_score": 1,
    "fl_select_prefill_tokens": 1, "fl_gather_rows": 1, "fl_scatter_rows": 1, "fl_encode_prefill": 3, "fl_encode_prefill_stage": 1,
    "fl_rmsnorm": 1, "fl_rope_split": 1, "fl_swiglu": 1, "fl_allreduce_rmsnorm": 1, "fl_linear_rows": 1, "fl_qkv_rope_rows": 1, "fl_linear_rows_partial": 1, "fl_rmsnorm_partial": 1,
}

_LIB = None
_COUNTER = None


class _CountingLibrary:
    """The library with every kernel-launching entry point wrapped so that its launches are
    counted (``count_launches``); used by the benchmark to report how many of this library's
    kernels one step launches."""

    def __init__(self, lib: C.CDLL) -> None:
        self._lib = lib
        self.counts: dict[str, int] = {}

    def __getattr__(self, name: str):
        fn = getattr(self._lib, name)
        per_call = LAUNCHES_PER_CALL.get(name, 0)
        if not per_call:
            return fn

        def counted(*args):
            self.counts[name] = self.counts.get(name, 0) + per_call
            return fn(*args)

        return counted


def count_launches(enable: bool) -> dict[str, int]:
    """Start (True) or stop (False) counting kernel launches per entry point; returns the counts
    gathered so far."""

    global _COUNTER
    counts = dict(_COUNTER.counts) if _COUNTER is not None else {}
    _COUNTER = _CountingLibrary(load()) if enable else None
    return counts


def load():
    """Load the CUDA library once; raise if it has not been built."""

    global _LIB
    if _COUNTER is not None:
        return _COUNTER
    if _LIB is None:
        if not LIBRARY_PATH.exists():
            raise RuntimeError(
                f"flashloop_b200 requires its CUDA library {LIBRARY_PATH.name}; build it with "
                "`python -m flashloop_b200.build_kernels` (there is no CPU fallback)")
        lib = C.CDLL(str(LIBRARY_PATH))
        for name, (restype, argtypes) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = restype
            fn.argtypes = argtypes
        _LIB = lib
    return _LIB


def check(status: int, what: str = "") -> None:
    if status != 0:
        message = load().fl_last_error().decode("utf-8", "replace")
        raise RuntimeError(f"flashloop_b200 {what} failed ({status}): {message}")


def ptr(tensor: torch.Tensor | None) -> int | None:
    """Device address of a tensor (None -> NULL)."""

    if tensor is None:
        return None
    return tensor.data_ptr()


def current_stream(device: torch.device | None = None) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def require_cuda(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("flashloop_b200 kernels need CUDA tensors (there is no CPU fallback)")
