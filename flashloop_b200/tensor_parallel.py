"""Head / FFN-column tensor parallelism for the end-to-end configurations.

Attention shards by head with no traffic inside it (every reader, selection and append kernel is
independent per (sequence, head)); the only exchange of a decoder layer is the sum of the
row-parallel ``o_proj`` and ``down_proj`` outputs.  Prefill sums them with NCCL (large tensors:
bandwidth); a decode step sums them inside the norm launch that consumes them
(:class:`PeerAllReduce`, ``csrc/fl_comm.cu``: one-shot peer stores over NVLink, no collective
library on the path, so the step can be recorded in a CUDA graph).  The reference is
single-GPU (flashloop/engine.py:112-150), so this module has no counterpart there; the sharded
modules keep the attribute names the engine walks (flashloop/engine.py:396-437, 533-537).
"""

from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist
from torch import nn

from . import _native


def shard_range(total: int, world: int, rank: int) -> tuple[int, int]:
    if total % world:
        raise ValueError(f"{total} does not divide over {world} ranks")
    per = total // world
    return rank * per, (rank + 1) * per


def _rows(linear: nn.Linear, lo: int, hi: int) -> None:
    """Keep output features [lo, hi) (column-parallel)."""

    linear.weight = nn.Parameter(linear.weight.data[lo:hi].clone(), requires_grad=False)
    linear.out_features = hi - lo


def _cols(linear: nn.Linear, lo: int, hi: int) -> None:
    """Keep input features [lo, hi) (row-parallel: the outputs are partial sums)."""

    linear.weight = nn.Parameter(linear.weight.data[:, lo:hi].clone(), requires_grad=False)
    linear.in_features = hi - lo


@torch.no_grad()
def shard_ouro_model(model: nn.Module, rank: int, world: int) -> nn.Module:
    """Slice an Ouro-style model in place to ``rank``'s heads and FFN columns.  Embeddings, norms
    and the LM head stay replicated.  Call before the engine repacks the projections."""

    if world == 1:
        return model
    for layer in model.model.layers:
        attention, mlp = layer.self_attn, layer.mlp
        if hasattr(attention, "_flashloop_qkv_weight"):
            raise RuntimeError("shard the model before its projections are repacked")
        head_dim = int(attention.head_dim)
        heads = attention.q_proj.out_features // head_dim
        kv_heads = attention.k_proj.out_features // head_dim
        h0, h1 = shard_range(heads, world, rank)
        g0, g1 = shard_range(kv_heads, world, rank)
        _rows(attention.q_proj, h0 * head_dim, h1 * head_dim)
        _rows(attention.k_proj, g0 * head_dim, g1 * head_dim)
        _rows(attention.v_proj, g0 * head_dim, g1 * head_dim)
        _cols(attention.o_proj, h0 * head_dim, h1 * head_dim)
        f0, f1 = shard_range(mlp.gate_proj.out_features, world, rank)
        _rows(mlp.gate_proj, f0, f1)
        _rows(mlp.up_proj, f0, f1)
        _cols(mlp.down_proj, f0, f1)
    return model


class PartialSum:
    """Callable that turns a row-parallel partial sum into the full sum, in place."""

    def __init__(self, group=None) -> None:
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_available() and dist.is_initialized() else 1

    def __call__(self, partial: torch.Tensor) -> torch.Tensor:
        if self.world > 1:
            dist.all_reduce(partial, group=self.group)
        return partial


def exchange_bytes(group, payload: bytes) -> list[bytes]:
    """Every rank's ``payload`` in rank order (the carrier of the IPC handles)."""

    gathered: list = [None] * dist.get_world_size(group)
    dist.all_gather_object(gathered, bytes(payload), group=group)
    return [bytes(item) for item in gathered]


class PeerAllReduce:
    """The decode step's sum over the tensor-parallel ranks as one launch of this library per rank
    (``fl_allreduce_rmsnorm``), fused with the residual add and the RMSNorms that follow it.

    Construction is collective over ``group`` (the handles travel through it); after that the
    group is not used: the kernels talk through peer memory.  Rows are bfloat16 ``[rows, width]``
    with ``rows <= rows_max``.  Every rank must make the same sequence of calls.  A peer that does
    not show up within ``wait_limit`` polls does not block the GPU: the call sums what arrived and
    :meth:`status` reports 1.
    """

    def __init__(self, group, *, rows_max: int, width: int, device: torch.device, wait_limit: int = 0) -> None:
        self.group = group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.rows_max, self.width, self.device = int(rows_max), int(width), torch.device(device)
        self.wait_limit = int(wait_limit)
        lib = _native.load()
        handle = ctypes.create_string_buffer(int(lib.fl_comm_handle_bytes()))
        comm = ctypes.c_void_p()
        with torch.cuda.device(self.device):
            _native.check(lib.fl_comm_create(self.rank, self.world, self.rows_max, self.width, ctypes.byref(comm),
                                             handle), "fl_comm_create")
            self._comm = comm
            handles = b"".join(exchange_bytes(group, handle.raw))
            _native.check(lib.fl_comm_connect(self._comm, handles), "fl_comm_connect")
        dist.barrier(group)  # nobody stores into a buffer that its owner has not mapped and zeroed

    def reduce_norm(self, partial: torch.Tensor, weight: torch.Tensor | None = None, eps: float = 0.0, *,
                    residual: torch.Tensor | None = None, weight2: torch.Tensor | None = None, eps2: float = 0.0,
                    addend: torch.Tensor | None = None, want_sum: bool = False, _skip_store: bool = False):
        """``s = [addend +] sum over ranks of partial``; ``out = [residual +] RMSNorm(s)``;
        ``out2 = RMSNorm2(out)``.  Returns (out, out2, s); out2 / s are None when not asked for, and
        without ``weight`` out is s."""

        if self._comm is None:
            raise RuntimeError("the communicator is closed")
        for t in (partial, addend, residual, weight, weight2):
            if t is not None and (t.dtype != torch.bfloat16 or not t.is_contiguous()):
                raise TypeError("the peer all-reduce takes contiguous bfloat16 tensors")
        _native.require_cuda(partial, addend, residual, weight, weight2)
        rows = partial.numel() // self.width
        if partial.shape[-1] != self.width or rows > self.rows_max:
            raise ValueError(f"rows of {self.width} values, at most {self.rows_max} of them")
        for t in (addend, residual):
            if t is not None and t.shape != partial.shape:
                raise ValueError("addend / residual do not match the rows")
        out = torch.empty_like(partial)
        out2 = torch.empty_like(partial) if weight2 is not None else None
        total = torch.empty_like(partial) if (want_sum and weight is not None) else None
        _native.check(_native.load().fl_allreduce_rmsnorm(
            self._comm, _native.ptr(partial), _native.ptr(addend), _native.ptr(residual), _native.ptr(weight),
            float(eps), _native.ptr(weight2), float(eps2), rows, _native.ptr(total), _native.ptr(out),
            _native.ptr(out2), int(bool(_skip_store)), self.wait_limit, _native.current_stream(partial.device)),
            "fl_allreduce_rmsnorm")
        if weight is None:
            total = out
        return out, out2, total

    def __call__(self, partial: torch.Tensor) -> torch.Tensor:
        return self.reduce_norm(partial)[0]

    def status(self, *, reset: bool = False) -> int:
        """0, or 1 if a wait for a peer ran out since the last reset.  Synchronises the stream."""

        word = ctypes.c_int32(-1)
        _native.check(_native.load().fl_comm_status(self._comm, ctypes.byref(word), int(reset),
                                                    _native.current_stream(self.device)), "fl_comm_status")
        return int(word.value)

    def close(self) -> None:
        if self._comm is not None:
            torch.cuda.synchronize(self.device)
            _native.load().fl_comm_destroy(self._comm)
            self._comm = None

    def __del__(self) -> None:  # pragma: no cover - interpreter shutdown order
        try:
            self.close()
        except Exception:
            pass
