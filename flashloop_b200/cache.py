"""Physical anchor-plus-delta Cross-Loop KV cache on the GPU (batched, ragged).

Mirrors the interface of the reference's flashloop/cache.py (``CrossLoopKVLayer``
:628-1838, ``CrossLoopKVCache`` :1841-1950) for the packed path with additive
deltas.  Differences that follow from being batched and preallocated:

* one layer object holds every sequence of the batch; per-sequence lengths live in
  a small device array (``seq_state``) that the kernels read, so sequences of
  different lengths share every launch;
* streams are preallocated to a capacity instead of being re-concatenated at every
  rollover (flashloop/cache.py:179-187 reallocates the whole context);
* the physical layout is the row layout of flashloop/packing.py, whose append rule
  (flashloop/cache.py:202-242) keeps every rollover block's metadata group apart;
  each rollover block of a compact stream starts on a 64-row boundary;
* the BF16 tail is a 128-slot ring, so a rollover moves no tail rows.

There is no Torch fallback for the readers: without the CUDA library they raise.
"""

from __future__ import annotations

import ctypes as C
from typing import Sequence

import torch

from . import _native
from .packing import Packed4Bit
from .selection import PaddedDecodeSelection, select_decode_keys_padded

GROUP = 64
HEAD_DIM = 128
TAIL_CAPACITY = 128

_WORKSPACES: dict[tuple[int, int], torch.Tensor] = {}


def reader_workspace(device: torch.device, batch_heads: int, max_context_tokens: int) -> torch.Tensor:
    """Zero-initialised reader scratch on ``device`` for ``batch_heads`` pairs (the kernels leave
    it zeroed again).  Layers of equal batch*heads on one device share one tensor, which is never
    replaced: a layer keeps a reference to the tensor it was given, so an address recorded in a
    CUDA graph stays valid for as long as that layer lives, whatever other layers or engines the
    process creates.  Calls that share a workspace must run on one stream."""

    lib = _native.load()
    need = int(lib.fl_reader_workspace_bytes(batch_heads, max_context_tokens))
    key = (device.index if device.index is not None else torch.cuda.current_device(), int(batch_heads))
    current = _WORKSPACES.get(key)
    if current is None or current.numel() < need:
        current = torch.zeros(need, dtype=torch.uint8, device=device)
        _WORKSPACES[key] = current
    return current


def _round_up(value: int, multiple: int) -> int:
    return -(-int(value) // multiple) * multiple


def _validate_loop_tensors(keys: Sequence[torch.Tensor], values: Sequence[torch.Tensor]):
    """flashloop/cache.py:263-278, without the batch-one restriction."""

    if len(keys) != 4 or len(values) != 4:
        raise ValueError("exactly four loop K/V tensors are required")
    shape = tuple(int(v) for v in keys[0].shape)
    if len(shape) != 4:
        raise ValueError("loop K/V tensors must have shape [batch, heads, tokens, channels]")
    if any(tuple(t.shape) != shape for t in (*keys, *values)):
        raise ValueError("all loop K/V tensors must have the same shape")
    if any(t.dtype != keys[0].dtype for t in (*keys, *values)):
        raise ValueError("all loop K/V tensors must have the same dtype")
    if any(t.device != keys[0].device for t in (*keys, *values)):
        raise ValueError("all loop K/V tensors must share a device")
    return shape


class CrossLoopKVLayer:
    """One physical layer's packed recurrent cache for a batch of sequences."""

    def __init__(self, *, batch: int, heads: int, token_capacities: Sequence[int],
                 compact_capacities: Sequence[tuple[int, int]] | None, bits: int = 4,
                 group_size: int = GROUP, residual_length: int = 64,
                 device: torch.device | str = "cuda", dtype: torch.dtype = torch.bfloat16) -> None:
        if group_size != GROUP or residual_length != 64:
            raise ValueError("the CUDA cache specializes group_size=64 and residual_length=64")
        if bits not in (4, 2):
            raise ValueError("bits must be 4 or 2")
        if dtype != torch.bfloat16:
            raise ValueError("the CUDA cache stores BF16 tails; loop K/V must be bfloat16")
        _native.load()
        self.group_size = group_size
        self.residual_length = residual_length
        self.bits = bits
        self.reader_backend = "kivi_outer"
        self.absolute_late_overrides = False
        self.batch, self.heads = int(batch), int(heads)
        self._device = torch.device(device)
        self._dtype = dtype
        self._shape_prefix = (self.batch, self.heads, HEAD_DIM)
        dev = self._device
        self._caps: list = [None] * 4
        self._k_codes, self._k_min, self._k_scale = [None] * 4, [None] * 4, [None] * 4
        self._v_rows, self._v_codes, self._v_meta = [None] * 4, [None] * 4, [None] * 4
        self._row_base, self._group_base, self._row_base_host = [None] * 4, [None] * 4, [None] * 4
        token_caps = [_round_up(c, GROUP) for c in token_capacities]
        self._allocate_stream(0, token_caps)
        self._allocate_stream(1, token_caps)
        if compact_capacities is not None:
            self._allocate_stream(2, [_round_up(c[0], GROUP) for c in compact_capacities])
            self._allocate_stream(3, [_round_up(c[1], GROUP) for c in compact_capacities])
        caps = self._caps
        rank_bases, off = [], 0
        for b in range(self.batch):
            rank_bases.append(off)
            off += caps[0][b]
        self._rank_base_host = rank_bases
        self._rank_base = torch.tensor(rank_bases, dtype=torch.int64, device=dev)
        self._rank = [torch.full((max(off, 1),), -1, dtype=torch.int32, device=dev) for _ in range(2)]
        bh = self.batch * self.heads
        self._tail_k = torch.zeros((4, bh, TAIL_CAPACITY, HEAD_DIM), dtype=dtype, device=dev)
        self._tail_v = torch.zeros_like(self._tail_k)
        self._tail_active = torch.zeros((2, self.batch, TAIL_CAPACITY), dtype=torch.uint8, device=dev)
        self._state_host = torch.zeros((self.batch, _native.FL_STATE_WORDS), dtype=torch.int32)
        self._seq_state = torch.zeros((self.batch, _native.FL_STATE_WORDS), dtype=torch.int32, device=dev)
        # host mirrors: rows held by the compact streams and the tail's retention flags
        self._compact_counts = [[0, 0] for _ in range(self.batch)]
        self._tail_active_host: list[list[list[bool]]] = [[[], []] for _ in range(self.batch)]
        self.context_bound: int | None = None
        self._native = self._make_native()
        # this layer's reader scratch: held here so that nothing can free it under a recorded graph
        self._ws = reader_workspace(self._device, self.batch * self.heads, max(caps[0]) + TAIL_CAPACITY)

    def _allocate_stream(self, s: int, caps: Sequence[int]) -> None:
        """Storage of stream ``s`` with ``caps[b]`` rows (multiples of 64) per head of sequence b."""

        row_bytes = 16 * self.bits
        dev = self._device
        bases, off = [], 0
        for b in range(self.batch):
            for h in range(self.heads):
                bases.append(off + h * caps[b])
            off += self.heads * caps[b]
        total = max(off, GROUP)
        self._caps[s] = list(caps)
        self._k_codes[s] = torch.zeros((total, row_bytes), dtype=torch.uint8, device=dev)
        # V records: codes, then float16 min0 min1 scale0 scale1, then 8 bytes of padding
        records = torch.zeros((total, row_bytes + 16), dtype=torch.uint8, device=dev)
        self._v_rows[s] = records
        self._v_codes[s] = records[:, :row_bytes]
        self._v_meta[s] = records[:, row_bytes:row_bytes + 8].view(torch.float16)
        self._k_min[s] = torch.zeros((total // GROUP, HEAD_DIM), dtype=torch.float16, device=dev)
        self._k_scale[s] = torch.zeros((total // GROUP, HEAD_DIM), dtype=torch.float16, device=dev)
        self._row_base_host[s] = bases
        self._row_base[s] = torch.tensor(bases, dtype=torch.int64, device=dev)
        self._group_base[s] = torch.tensor([x // GROUP for x in bases], dtype=torch.int64, device=dev)

    def _allocate_compact(self, compact_capacities: Sequence[tuple[int, int]]) -> None:
        """Streams 2 and 3, once the retained counts are known (staged construction)."""

        self._allocate_stream(2, [_round_up(c[0], GROUP) for c in compact_capacities])
        self._allocate_stream(3, [_round_up(c[1], GROUP) for c in compact_capacities])
        self._native = self._make_native()

    # ------------------------------------------------------------------ native descriptor

    def _make_native(self) -> _native.FlLayer:
        n = _native.FlLayer()
        n.batch, n.heads, n.bits, n.tail_capacity = self.batch, self.heads, self.bits, TAIL_CAPACITY
        for s in range(4):
            if self._k_codes[s] is None:  # compact streams of a layer still under construction
                n.tail_k[s] = self._tail_k[s].data_ptr()
                n.tail_v[s] = self._tail_v[s].data_ptr()
                continue
            n.k_codes[s] = self._k_codes[s].data_ptr()
            n.k_min[s] = self._k_min[s].data_ptr()
            n.k_scale[s] = self._k_scale[s].data_ptr()
            n.v_rows[s] = self._v_rows[s].data_ptr()
            n.row_base[s] = self._row_base[s].data_ptr()
            n.group_base[s] = self._group_base[s].data_ptr()
            n.tail_k[s] = self._tail_k[s].data_ptr()
            n.tail_v[s] = self._tail_v[s].data_ptr()
        for i in range(2):
            n.rank[i] = self._rank[i].data_ptr()
            n.tail_active[i] = self._tail_active[i].data_ptr()
        n.rank_base = self._rank_base.data_ptr()
        n.seq_state = self._seq_state.data_ptr()
        return n

    def _push_state(self) -> None:
        self._seq_state.copy_(self._state_host, non_blocking=False)

    # ------------------------------------------------------------------ per-sequence views

    def _rows(self, tensor_list, s: int, b: int, per_row: int = 1) -> torch.Tensor:
        """View [heads, capacity(/per_row), ...] of sequence ``b`` in stream ``s``."""

        cap = self._caps[s][b]
        start = self._row_base_host[s][b * self.heads] // per_row
        count = self.heads * cap // per_row
        t = tensor_list[s]
        return t[start:start + count].view(self.heads, cap // per_row, *t.shape[1:])

    # ------------------------------------------------------------------ construction

    @classmethod
    def from_prefill(cls, keys: Sequence[torch.Tensor], values: Sequence[torch.Tensor], *,
                     mask_loop3: torch.Tensor, mask_loop4: torch.Tensor, group_size: int = 64,
                     residual_length: int = 64, absolute_late_overrides: bool = False,
                     absolute_override_dtype: str = "int4", reader_backend: str = "kivi_outer",
                     bits: int = 4, max_new_tokens: int = 0) -> "CrossLoopKVLayer":
        """flashloop/cache.py:752-817 for a batch of equally long prompts.

        keys/values: four tensors [B, H, T, 128] bfloat16; masks bool [B, T].
        ``max_new_tokens`` sizes the preallocated room for decode appends."""

        batch, heads, tokens, channels = _validate_loop_tensors(keys, values)
        if channels != HEAD_DIM:
            raise ValueError("the CUDA cache specializes head_dim=128")
        if absolute_late_overrides:
            raise ValueError("the CUDA cache supports additive cross-loop deltas only")
        if reader_backend not in {"kivi_outer", "triton_row"}:
            raise ValueError("unknown KV reader backend")
        if mask_loop3.shape != (batch, tokens) or mask_loop4.shape != (batch, tokens):
            raise ValueError("prefill masks must have shape [batch, tokens]")
        device = keys[0].device
        mask3 = mask_loop3.to(device=device, dtype=torch.bool).contiguous()
        mask4 = mask_loop4.to(device=device, dtype=torch.bool).contiguous()
        if not bool(torch.all(~mask4 | mask3).item()):
            raise ValueError("Loop-4 overrides must be nested in Loop-3 overrides")
        packed = max(0, ((tokens - residual_length) // group_size) * group_size)
        counts3 = mask3[:, :packed].sum(1).tolist()
        counts4 = mask4[:, :packed].sum(1).tolist()
        extra = _round_up(max_new_tokens, GROUP) + 2 * GROUP
        layer = cls(batch=batch, heads=heads, token_capacities=[packed + extra] * batch,
                    compact_capacities=[(_round_up(n3, GROUP) + extra, _round_up(n4, GROUP) + extra)
                                        for n3, n4 in zip(counts3, counts4)],
                    bits=bits, group_size=group_size, residual_length=residual_length, device=device,
                    dtype=keys[0].dtype)
        layer._encode_sequences(0, keys, values, mask3, mask4, packed, counts3, counts4)
        layer._push_state()
        return layer

    @classmethod
    def from_prefill_ragged(cls, sequences, *, group_size: int = 64, residual_length: int = 64,
                            bits: int = 4, max_new_tokens: int = 0) -> "CrossLoopKVLayer":
        """Build a layer from per-sequence prompts of different lengths.

        sequences: list of (keys[4], values[4], mask3 [T_b], mask4 [T_b]) with K/V
        tensors [1, H, T_b, 128]."""

        if not sequences:
            raise ValueError("at least one sequence is required")
        heads = int(sequences[0][0][0].shape[1])
        device = sequences[0][0][0].device
        dtype = sequences[0][0][0].dtype
        token_caps, compact_caps, prepared = [], [], []
        extra = _round_up(max_new_tokens, GROUP) + 2 * GROUP
        for keys, values, mask3, mask4 in sequences:
            shape = _validate_loop_tensors(keys, values)
            if shape[0] != 1 or shape[1] != heads or shape[3] != HEAD_DIM:
                raise ValueError("ragged sequences must be [1, heads, tokens, 128] with equal heads")
            tokens = shape[2]
            mask3 = mask3.reshape(-1).to(device=device, dtype=torch.bool)
            mask4 = mask4.reshape(-1).to(device=device, dtype=torch.bool)
            if mask3.numel() != tokens or mask4.numel() != tokens:
                raise ValueError("prefill masks must cover every prompt token")
            if not bool(torch.all(~mask4 | mask3).item()):
                raise ValueError("Loop-4 overrides must be nested in Loop-3 overrides")
            packed = max(0, ((tokens - residual_length) // group_size) * group_size)
            n3 = int(mask3[:packed].sum().item())
            n4 = int(mask4[:packed].sum().item())
            token_caps.append(packed + extra)
            compact_caps.append((_round_up(n3, GROUP) + extra, _round_up(n4, GROUP) + extra))
            prepared.append((keys, values, mask3, mask4, packed))
        layer = cls(batch=len(sequences), heads=heads, token_capacities=token_caps,
                    compact_capacities=compact_caps, bits=bits, group_size=group_size,
                    residual_length=residual_length, device=device, dtype=dtype)
        for b, (keys, values, mask3, mask4, packed) in enumerate(prepared):
            layer._encode_sequences(b, keys, values, mask3[None], mask4[None], packed,
                                    [int(mask3[:packed].sum().item())], [int(mask4[:packed].sum().item())])
        layer._push_state()
        return layer

    @classmethod
    def from_prefill_updates(cls, *, loop1_key: torch.Tensor, loop1_value: torch.Tensor, loop2_key: torch.Tensor,
                             loop2_value: torch.Tensor, loop3_positions: torch.Tensor, loop3_keys: torch.Tensor,
                             loop3_values: torch.Tensor, loop4_positions: torch.Tensor, loop4_keys: torch.Tensor,
                             loop4_values: torch.Tensor, group_size: int = 64, residual_length: int = 64,
                             absolute_late_overrides: bool = False, absolute_override_dtype: str = "int4",
                             reader_backend: str = "kivi_outer", bits: int = 4,
                             max_new_tokens: int = 0) -> "CrossLoopKVLayer":
        """Build the layer from the dense Loop-1/2 K/V and the compact Loop-3/4 rows without ever
        forming full Loop-3/4 tensors (flashloop/cache.py:820-1006): the three builder stages in
        one call."""

        builder = CrossLoopKVLayerBuilder.from_loop1(
            loop1_key, loop1_value, group_size=group_size, residual_length=residual_length,
            absolute_late_overrides=absolute_late_overrides, absolute_override_dtype=absolute_override_dtype,
            reader_backend=reader_backend, bits=bits, max_new_tokens=max_new_tokens)
        builder.add_loop2(loop2_key, loop2_value)
        return builder.finalize(loop3_positions=loop3_positions, loop3_keys=loop3_keys, loop3_values=loop3_values,
                                loop4_positions=loop4_positions, loop4_keys=loop4_keys, loop4_values=loop4_values)

    @classmethod
    def from_streams(cls, key_streams, value_streams, rank_maps) -> "CrossLoopKVLayer":
        """Adopt already packed row-layout streams (``Packed4Bit``, ``None`` for an empty
        compact stream) with the reference's rank maps (int32 [Tq], -1 = absent).  Streams
        of the wrong axis are ignored, so a K-only or V-only set can be adopted for
        ``qk`` / ``pv``.  The tail starts empty; see :meth:`set_tail`."""

        anchor = key_streams[0]
        batch, heads, quant, channels = anchor.original_shape
        if channels != HEAD_DIM:
            raise ValueError("the CUDA cache specializes head_dim=128")
        counts = [0 if s is None else int(s.original_shape[2]) for s in key_streams]
        layer = cls(batch=batch, heads=heads, token_capacities=[quant + GROUP] * batch,
                    compact_capacities=[(counts[2] + GROUP, counts[3] + GROUP)] * batch, bits=anchor.bits,
                    device=anchor.payload.device)
        for b in range(batch):
            for s in range(4):
                ks, vs = key_streams[s], value_streams[s]
                if ks is None:
                    continue
                n, rb = counts[s], 16 * anchor.bits
                if ks.axis == "per_channel":
                    g = ks.minimum.shape[2]
                    layer._rows(layer._k_codes, s, b)[:, :n].copy_(ks.payload[b])
                    layer._rows(layer._k_min, s, b, GROUP)[:, :g].copy_(ks.minimum[b])
                    layer._rows(layer._k_scale, s, b, GROUP)[:, :g].copy_(ks.scale[b])
                if vs is not None and vs.axis == "per_token":
                    layer._rows(layer._v_codes, s, b)[:, :n].copy_(vs.payload[b])
                    meta = layer._rows(layer._v_meta, s, b)[:, :n]
                    meta[..., 0:2].copy_(vs.minimum[b])
                    meta[..., 2:4].copy_(vs.scale[b])
            base = layer._rank_base_host[b]
            for i in range(2):
                rank = rank_maps[i].to(device=layer._device, dtype=torch.int32)
                if rank.numel() not in (0, quant):
                    raise ValueError("rank maps must cover the packed prefix")
                if rank.numel():
                    layer._rank[i][base:base + quant] = rank
                    layer._compact_counts[b][i] = int((rank >= 0).sum().item())
            st = layer._state_host[b]
            st[_native.STATE_QUANT_TOKENS] = quant
            st[_native.STATE_ROWS2] = _round_up(counts[2], GROUP)
            st[_native.STATE_ROWS3] = _round_up(counts[3], GROUP)
        layer._push_state()
        return layer

    def set_tail(self, loop: int, tail_key: torch.Tensor, tail_value: torch.Tensor) -> None:
        """Install the BF16 tail of ``loop`` ([B, H, tail, 128], tail <= 128) for every
        sequence, in token order from ring slot 0."""

        tail = int(tail_key.shape[2])
        if tail > TAIL_CAPACITY or tuple(tail_key.shape) != (self.batch, self.heads, tail, HEAD_DIM) \
                or tail_value.shape != tail_key.shape:
            raise ValueError("tail K/V shape differs from this cache layer")
        bh = self.batch * self.heads
        if tail:
            self._tail_k[loop, :, :tail].copy_(tail_key.reshape(bh, tail, HEAD_DIM))
            self._tail_v[loop, :, :tail].copy_(tail_value.reshape(bh, tail, HEAD_DIM))
        if bool((self._state_host[:, _native.STATE_TAIL_LEN] != tail).any()) or \
                bool((self._state_host[:, _native.STATE_TAIL_START] != 0).any()):
            self._state_host[:, _native.STATE_TAIL_LEN] = tail
            self._state_host[:, _native.STATE_TAIL_START] = 0
            self._tail_active_host = [[[False] * tail, [False] * tail] for _ in range(self.batch)]
            self._push_state()

    def _encode_sequences(self, first: int, keys, values, mask3: torch.Tensor, mask4: torch.Tensor, packed: int,
                          counts3, counts4) -> None:
        """Encode sequences ``first .. first + n`` from their prompts: keys/values are four
        [n, H, T, 128] tensors, masks bool [n, T], ``packed`` the quantised prefix length of all
        of them, counts the retained tokens inside the prefix.  One ``fl_encode_prefill`` call
        (three launches) runs the residual chain of flashloop/cache.py:1008-1074 and writes the
        streams; rank maps, tails and state words are filled around it."""

        from .compaction import retained_from_mask

        n, tokens = int(keys[0].shape[0]), int(keys[0].shape[2])
        tail = tokens - packed
        if tail > TAIL_CAPACITY:
            raise RuntimeError("tail longer than the ring")
        _native.require_cuda(*keys, *values)
        if keys[0].dtype != torch.bfloat16:
            raise ValueError("prefill K/V must be bfloat16")
        for i in range(n):
            b = first + i
            if packed > self._caps[0][b] or _round_up(counts3[i], GROUP) > self._caps[2][b] \
                    or _round_up(counts4[i], GROUP) > self._caps[3][b]:
                raise RuntimeError(f"sequence {b} does not fit its preallocated streams")
            st = self._state_host[b]
            st[_native.STATE_QUANT_TOKENS] = packed
            st[_native.STATE_ROWS2] = _round_up(int(counts3[i]), GROUP)
            st[_native.STATE_ROWS3] = _round_up(int(counts4[i]), GROUP)
            st[_native.STATE_TAIL_LEN] = tail
            st[_native.STATE_TAIL_START] = 0
            self._compact_counts[b] = [int(counts3[i]), int(counts4[i])]
        self._seq_state[first:first + n].copy_(self._state_host[first:first + n])  # the kernels read the prefix length
        if packed:
            kept3, kept4 = retained_from_mask(mask3), retained_from_mask(mask4)
            for i in range(n):
                base = self._rank_base_host[first + i]
                self._rank[0][base:base + packed].copy_(kept3.rank[i, :packed])
                self._rank[1][base:base + packed].copy_(kept4.rank[i, :packed])
            ks = [k.contiguous() for k in keys]
            vs = [v.contiguous() for v in values]
            recon_k, recon_v = torch.empty_like(ks[0]), torch.empty_like(vs[0])
            key_table = (C.c_void_p * 4)(*[k.data_ptr() for k in ks])
            value_table = (C.c_void_p * 4)(*[v.data_ptr() for v in vs])
            _native.check(_native.load().fl_encode_prefill(
                C.byref(self._native), first, n, tokens, key_table, value_table, _native.ptr(kept3.positions),
                _native.ptr(kept4.positions), tokens, _native.ptr(recon_k), _native.ptr(recon_v),
                _native.current_stream(self._device)), "fl_encode_prefill")
        heads = self.heads
        sl = slice(first * heads, (first + n) * heads)
        for r in range(4):
            self._tail_k[r, sl, :tail].copy_(keys[r][:, :, packed:].reshape(n * heads, tail, HEAD_DIM))
            self._tail_v[r, sl, :tail].copy_(values[r][:, :, packed:].reshape(n * heads, tail, HEAD_DIM))
        self._tail_active[0, first:first + n, :tail].copy_(mask3[:, packed:].to(torch.uint8))
        self._tail_active[1, first:first + n, :tail].copy_(mask4[:, packed:].to(torch.uint8))
        flags3, flags4 = mask3[:, packed:].tolist(), mask4[:, packed:].tolist()
        for i in range(n):
            self._tail_active_host[first + i] = [flags3[i], flags4[i]]

    # ------------------------------------------------------------------ bookkeeping

    def quantized_tokens_of(self, b: int) -> int:
        return int(self._state_host[b, _native.STATE_QUANT_TOKENS])

    def tail_tokens_of(self, b: int) -> int:
        return int(self._state_host[b, _native.STATE_TAIL_LEN])

    @property
    def quantized_tokens(self) -> int:
        return self.quantized_tokens_of(0)

    @property
    def tail_tokens(self) -> int:
        return self.tail_tokens_of(0)

    @property
    def token_count(self) -> int:
        return self.quantized_tokens + self.tail_tokens

    def token_counts(self) -> list[int]:
        return [self.quantized_tokens_of(b) + self.tail_tokens_of(b) for b in range(self.batch)]

    @property
    def max_context_tokens(self) -> int:
        """Longest context of the batch, or ``context_bound`` when one is set.  Launch
        geometry and buffer sizes derive from this number only, so a decode step recorded
        in a CUDA graph with a bound stays valid while contexts grow up to it."""

        if self.context_bound is not None:
            return self.context_bound
        st = self._state_host
        return int((st[:, _native.STATE_QUANT_TOKENS] + st[:, _native.STATE_TAIL_LEN]).max())

    @property
    def storage_bytes(self) -> int:
        """Bytes in use (flashloop/cache.py:1084-1101), not the preallocated capacity."""

        row_bytes = 16 * self.bits
        total = 0
        for b in range(self.batch):
            q = self.quantized_tokens_of(b)
            n = [q, q, self._compact_counts[b][0], self._compact_counts[b][1]]
            for s in range(4):
                groups = -(-n[s] // GROUP)
                total += self.heads * (2 * n[s] * row_bytes + 2 * groups * HEAD_DIM * 2 + n[s] * 8)
            total += 8 * self.heads * self.tail_tokens_of(b) * HEAD_DIM * 2
            total += 2 * q * 4 + (n[2] + n[3]) * 4 + 2 * self.tail_tokens_of(b)
        return total

    @property
    def dense_bf16_bytes(self) -> int:
        return sum(4 * 2 * self.heads * t * HEAD_DIM * 2 for t in self.token_counts())

    @property
    def storage_ratio(self) -> float:
        dense = self.dense_bf16_bytes
        return self.storage_bytes / dense if dense else 0.0

    # ------------------------------------------------------------------ export (tests, audits)

    def export_sequence(self, b: int) -> dict:
        """The sequence's streams in the reference's logical order: for each stream the
        payload rows, K metadata groups and V metadata of the rows in use (compact
        streams without their padding), the rank maps and the tails in token order."""

        q = self.quantized_tokens_of(b)
        out: dict = {"quantized_tokens": q, "tail_tokens": self.tail_tokens_of(b)}
        base = self._rank_base_host[b]
        for s in range(4):
            if s < 2:
                rows = torch.arange(q, device=self._device)
            else:
                rank = self._rank[s - 2][base:base + q]
                rows = rank[rank >= 0].long()
                out[f"rank{s + 1}"] = torch.where(
                    rank >= 0, torch.cumsum((rank >= 0).to(torch.int32), 0, dtype=torch.int32) - 1,
                    torch.full_like(rank, -1))
                out[f"pos{s + 1}"] = torch.nonzero(rank >= 0, as_tuple=False).flatten().to(torch.int32)
            groups = torch.unique_consecutive(rows // GROUP) if rows.numel() else rows
            out[f"k{s}.payload"] = self._rows(self._k_codes, s, b).index_select(1, rows)
            out[f"k{s}.minimum"] = self._rows(self._k_min, s, b, GROUP).index_select(1, groups)
            out[f"k{s}.scale"] = self._rows(self._k_scale, s, b, GROUP).index_select(1, groups)
            out[f"k{s}.row_groups"] = (torch.searchsorted(groups, rows // GROUP).to(torch.int32)
                                       if rows.numel() else rows.to(torch.int32))
            out[f"v{s}.payload"] = self._rows(self._v_codes, s, b).index_select(1, rows)
            meta = self._rows(self._v_meta, s, b).index_select(1, rows)
            out[f"v{s}.minimum"] = meta[..., 0:2]
            out[f"v{s}.scale"] = meta[..., 2:4]
        tail = self.tail_tokens_of(b)
        start = int(self._state_host[b, _native.STATE_TAIL_START])
        slots = (start + torch.arange(tail, device=self._device)) % TAIL_CAPACITY
        sl = slice(b * self.heads, (b + 1) * self.heads)
        for r in range(4):
            out[f"tail_k{r}"] = self._tail_k[r, sl].index_select(1, slots)
            out[f"tail_v{r}"] = self._tail_v[r, sl].index_select(1, slots)
        out["tail_active3"] = self._tail_active[0, b].index_select(0, slots).bool()
        out["tail_active4"] = self._tail_active[1, b].index_select(0, slots).bool()
        return out

    def _decode_rows(self, s: int, b: int, rows: torch.Tensor, kind: str) -> torch.Tensor:
        """bfloat16 [H, n, 128] = decode of rows ``rows`` of stream ``s`` of sequence ``b``
        (code * scale + minimum in float32, rounded: flashloop/packing.py:108-132)."""

        codes = self._rows(self._k_codes if kind == "k" else self._v_codes, s, b).index_select(1, rows)  # [H, n, 16 * bits]
        per_byte = 8 // self.bits
        shifts = torch.arange(per_byte, device=self._device, dtype=torch.uint8) * self.bits
        values = ((codes.unsqueeze(-1) >> shifts) & ((1 << self.bits) - 1)).reshape(self.heads, -1, HEAD_DIM).float()
        if kind == "k":
            groups = rows // GROUP
            minimum = self._rows(self._k_min, s, b, GROUP).index_select(1, groups).float()
            scale = self._rows(self._k_scale, s, b, GROUP).index_select(1, groups).float()
        else:
            record = self._rows(self._v_meta, s, b).index_select(1, rows).float()  # [H, n, 4]: min0 min1 scale0 scale1
            minimum = record[..., 0:2].repeat_interleave(GROUP, dim=-1)
            scale = record[..., 2:4].repeat_interleave(GROUP, dim=-1)
        return (values * scale + minimum).to(torch.bfloat16)

    def gather(self, loop: int, indices: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        """The reconstructed K and V rows of ``loop`` at one-dimensional logical ``indices``
        (flashloop/cache.py:1114-1200): bfloat16 [B, H, n, 128].  An audit path in tensor ops
        (every sum is rounded to bfloat16 as there); the readers never go through it."""

        loop = int(loop)
        if loop not in range(4):
            raise ValueError("loop must be in [0, 3]")
        if indices.ndim != 1:
            raise ValueError("indices must be one-dimensional")
        indices = indices.to(device=self._device, dtype=torch.long)
        counts = self.token_counts()
        if indices.numel() and (int(indices.min()) < 0 or int(indices.max()) >= min(counts)):
            raise IndexError("cache index is outside the logical sequence")
        out_k = torch.empty((self.batch, self.heads, int(indices.numel()), HEAD_DIM), dtype=torch.bfloat16,
                            device=self._device)
        out_v = torch.empty_like(out_k)
        for b in range(self.batch):
            quant, start = self.quantized_tokens_of(b), int(self._state_host[b, _native.STATE_TAIL_START])
            inside = torch.nonzero(indices < quant).flatten()
            if inside.numel():
                rows = indices.index_select(0, inside)
                k = self._decode_rows(0, b, rows, "k")
                v = self._decode_rows(0, b, rows, "v")
                for s in range(1, loop + 1):
                    if s == 1:
                        k = k + self._decode_rows(1, b, rows, "k")
                        v = v + self._decode_rows(1, b, rows, "v")
                        continue
                    base = self._rank_base_host[b]
                    ranks = self._rank[s - 2][base:base + quant].index_select(0, rows)
                    held = torch.nonzero(ranks >= 0).flatten()
                    if held.numel():
                        compact = ranks.index_select(0, held).long()
                        k.index_add_(1, held, self._decode_rows(s, b, compact, "k"))
                        v.index_add_(1, held, self._decode_rows(s, b, compact, "v"))
                out_k[b].index_copy_(1, inside, k)
                out_v[b].index_copy_(1, inside, v)
            outside = torch.nonzero(indices >= quant).flatten()
            if outside.numel():
                slots = (start + indices.index_select(0, outside) - quant) % TAIL_CAPACITY
                sl = slice(b * self.heads, (b + 1) * self.heads)
                out_k[b].index_copy_(1, outside, self._tail_k[loop, sl].index_select(1, slots))
                out_v[b].index_copy_(1, outside, self._tail_v[loop, sl].index_select(1, slots))
        return out_k, out_v

    # ------------------------------------------------------------------ readers

    def _check_vectors(self, *vectors: torch.Tensor) -> None:
        expected = (self.batch, self.heads, 1, HEAD_DIM)
        for v in vectors:
            if tuple(v.shape) != expected:
                raise ValueError("attention vectors differ from this cache layer")
            if v.dtype != torch.bfloat16:
                raise ValueError("fused attention specializes BF16 vectors")
        _native.require_cuda(*vectors)

    def _workspace(self) -> torch.Tensor:
        return self._ws

    def reader_status(self) -> int:
        """Synchronise and return the readers' status word: 0, or 1 when a reader gave up
        waiting for one of its own asynchronous copies (its output is then undefined)."""

        ws = self._workspace()
        flag = C.c_int32(0)
        _native.check(_native.load().fl_workspace_status(
            _native.ptr(ws), self.batch * self.heads, C.byref(flag), _native.current_stream(self._device)),
            "fl_workspace_status")
        return int(flag.value)

    def dense_source_attention(self, loop: int, *, query: torch.Tensor, current_key: torch.Tensor,
                               current_value: torch.Tensor, scaling: float, return_logits: bool,
                               out: torch.Tensor | None = None, logits_out: torch.Tensor | None = None):
        """Attention of one query per head over every cached token of ``loop`` plus the
        current token (flashloop/cache.py:1644-1756).  Returns (output float32
        [B, H, 1, 128], scaled logits float32 [B, H, 1, N + 1] or None); for a ragged
        batch N is the longest context and shorter rows are padded with -inf."""

        loop = int(loop)
        if loop not in range(4):
            raise ValueError("loop must be in [0, 3]")
        self._check_vectors(query, current_key, current_value)
        q, k, v = query.contiguous(), current_key.contiguous(), current_value.contiguous()
        max_ctx = self.max_context_tokens
        if out is None:
            out = torch.empty((self.batch, self.heads, 1, HEAD_DIM), dtype=torch.float32, device=self._device)
        logits = None
        stride = 0
        if return_logits:
            stride = _round_up(max_ctx + 1, 4)
            if logits_out is not None:
                logits = logits_out
                stride = int(logits.shape[-1])
            elif self.batch == 1 or len(set(self.token_counts())) == 1:
                logits = torch.empty((self.batch, self.heads, 1, stride), dtype=torch.float32, device=self._device)
            else:
                logits = torch.full((self.batch, self.heads, 1, stride), float("-inf"),
                                    dtype=torch.float32, device=self._device)
        ws = self._workspace()
        lib = _native.load()
        _native.check(lib.fl_dense_source_attention(
            C.byref(self._native), loop, _native.ptr(q), _native.ptr(k), _native.ptr(v), float(scaling),
            _native.ptr(out), _native.ptr(logits), stride, max_ctx, _native.ptr(ws), ws.numel(),
            _native.current_stream(self._device)), "fl_dense_source_attention")
        if logits is not None and logits_out is None:
            logits = logits[..., :max_ctx + 1]
        return out, logits

    def select_decode_keys(self, logits: torch.Tensor, *, fraction: float) -> PaddedDecodeSelection:
        """The loop-2 selection of flashloop/engine.py:438-481 from the scaled logits
        returned by :meth:`dense_source_attention`."""

        return select_decode_keys_padded(logits, fraction=fraction, values_are_logits=True,
                                         seq_state=self._seq_state, max_keys=self.max_context_tokens + 1)

    def cached_mass_sparse_attention_delta(self, loop: int, *, query: torch.Tensor,
                                           current_key: torch.Tensor, current_value: torch.Tensor,
                                           indices: torch.Tensor, valid: torch.Tensor,
                                           source_selected_output: torch.Tensor, global_mass: torch.Tensor,
                                           scaling: float, current_position: int | None = None,
                                           out: torch.Tensor | None = None,
                                           current_logits_out: torch.Tensor | None = None) -> torch.Tensor:
        """The cached-mass late-loop attention correction
        (flashloop/cache.py:1517-1642): ``global_mass * (subset-softmax target -
        source_selected_output)`` over the valid selected indices.  The current token
        is index quant + tail of each sequence; ``current_position`` is accepted for
        interface compatibility and checked against it for a batch of one.
        ``current_logits_out`` (float32 [batch*heads]) receives the scaled logit of the current
        token of the heads that selected it (kivi_outer_gemv_cuda.cu:1826-1835)."""

        loop = int(loop)
        if loop not in (2, 3):
            raise ValueError("cached-mass sparse attention is only valid for Loop 3/4")
        self._check_vectors(query, current_key, current_value)
        if tuple(source_selected_output.shape) != (self.batch, self.heads, 1, HEAD_DIM):
            raise ValueError("attention vectors differ from this cache layer")
        if indices.ndim == 4 and indices.shape[-2] == 1:
            indices = indices.squeeze(-2)
        if indices.ndim != 3 or tuple(indices.shape[:2]) != (self.batch, self.heads):
            raise ValueError("indices must have shape [batch, heads, selected]")
        if tuple(valid.shape) != tuple(indices.shape):
            raise ValueError("valid mask must match selected indices")
        if tuple(global_mass.shape) != (self.batch, self.heads, 1, 1):
            raise ValueError("global mass must have shape [batch, heads, 1, 1]")
        if current_position is not None and self.batch == 1 and int(current_position) != self.token_count:
            raise ValueError("current_position differs from the cache's token count")
        idx = indices.to(device=self._device, dtype=torch.int32).contiguous()
        val = valid.to(device=self._device).contiguous()
        val = val.view(torch.uint8) if val.dtype == torch.bool else val.to(torch.uint8)
        src = source_selected_output.float().contiguous()
        mass = global_mass.float().contiguous()
        if out is None:
            out = torch.empty((self.batch, self.heads, 1, HEAD_DIM), dtype=torch.float32, device=self._device)
        ws = self._workspace()
        lib = _native.load()
        _native.check(lib.fl_sparse_attention_delta(
            C.byref(self._native), loop, _native.ptr(query.contiguous()),
            _native.ptr(current_key.contiguous()), _native.ptr(current_value.contiguous()),
            _native.ptr(idx), _native.ptr(val), int(idx.shape[-1]), _native.ptr(src), _native.ptr(mass),
            float(scaling), _native.ptr(out), _native.ptr(current_logits_out), _native.ptr(ws), ws.numel(),
            _native.current_stream(self._device)), "fl_sparse_attention_delta")
        return out

    def _normalize_indices(self, indices: torch.Tensor) -> torch.Tensor:
        if indices.ndim == 1:
            indices = indices[None, None, :].expand(self.batch, self.heads, -1)
        elif indices.ndim == 4 and indices.shape[-2] == 1:
            indices = indices.squeeze(-2)
        if indices.ndim != 3 or tuple(indices.shape[:2]) != (self.batch, self.heads):
            raise ValueError("indices must have shape [selected] or [batch, heads, selected]")
        return indices.to(device=self._device, dtype=torch.int32).contiguous()

    def qk(self, loop: int, query: torch.Tensor, indices: torch.Tensor, *,
           validate_indices: bool = True, current_key: torch.Tensor | None = None) -> torch.Tensor:
        """Unscaled logits of selected logical rows (flashloop/cache.py:1202-1356)."""

        loop = int(loop)
        if loop not in range(4):
            raise ValueError("loop must be in [0, 3]")
        self._check_vectors(query)
        idx = self._normalize_indices(indices)
        if validate_indices and idx.numel() and (int(idx.min()) < 0 or int(idx.max()) >= self.max_context_tokens):
            raise IndexError("cache index is outside the logical sequence")
        out = torch.empty((self.batch, self.heads, 1, idx.shape[-1]), dtype=torch.float32, device=self._device)
        lib = _native.load()
        _native.check(lib.fl_selected_qk(
            C.byref(self._native), loop, _native.ptr(query.contiguous()), _native.ptr(idx), None,
            int(idx.shape[-1]), _native.ptr(current_key.contiguous()) if current_key is not None else None,
            _native.ptr(out), _native.current_stream(self._device)), "fl_selected_qk")
        return out

    def pv(self, loop: int, weights: torch.Tensor, indices: torch.Tensor, *,
           validate_indices: bool = True, current_value: torch.Tensor | None = None,
           valid: torch.Tensor | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
        """Probability-weighted V of selected logical rows (flashloop/cache.py:1358-1515).
        With ``current_value`` the row of index quant + tail is the current token's value,
        which folds FlashLoopEngine._selected_value_aggregate (engine.py:346-371) into
        the same launch."""

        loop = int(loop)
        if loop not in range(4):
            raise ValueError("loop must be in [0, 3]")
        idx = self._normalize_indices(indices)
        if tuple(weights.shape) != (self.batch, self.heads, 1, idx.shape[-1]):
            raise ValueError("weights must match [batch, heads, 1, selected]")
        if validate_indices and idx.numel() and (int(idx.min()) < 0 or int(idx.max()) > self.max_context_tokens):
            raise IndexError("cache index is outside the logical sequence")
        w = weights.float().contiguous()
        val = None
        if valid is not None:
            val = valid.contiguous()
            val = val.view(torch.uint8) if val.dtype == torch.bool else val.to(torch.uint8)
        if out is None:
            out = torch.empty((self.batch, self.heads, 1, HEAD_DIM), dtype=torch.float32, device=self._device)
        ws = self._workspace()
        lib = _native.load()
        _native.check(lib.fl_selected_pv(
            C.byref(self._native), loop, _native.ptr(w), _native.ptr(idx), _native.ptr(val),
            int(idx.shape[-1]), _native.ptr(current_value.contiguous()) if current_value is not None else None,
            _native.ptr(out), _native.ptr(ws), ws.numel(), _native.current_stream(self._device)),
            "fl_selected_pv")
        return out

    # ------------------------------------------------------------------ append / rollover

    def append_decode_token(self, keys: Sequence[torch.Tensor], values: Sequence[torch.Tensor]) -> None:
        """Append the four loops' K/V of one decoded token per sequence to the BF16 tail
        and roll the oldest 64 tail tokens into the packed streams when the tail reaches
        128 (flashloop/cache.py:1758-1838).  Three launches of ``fl_append_decode_token``,
        no host synchronisation: the device advances ``seq_state`` itself and the host
        mirror below follows by the same arithmetic."""

        shape = _validate_loop_tensors(keys, values)
        if shape != (self.batch, self.heads, 1, HEAD_DIM):
            raise ValueError("decode K/V shape does not match the cache")
        if keys[0].dtype != torch.bfloat16:
            raise ValueError("decode K/V must be bfloat16")
        _native.require_cuda(*keys, *values)
        full = self.residual_length + self.group_size
        for b in range(self.batch):
            st = self._state_host[b]
            if int(st[_native.STATE_TAIL_LEN]) + 1 >= full:
                room = (int(st[_native.STATE_QUANT_TOKENS]) + GROUP <= self._caps[0][b]
                        and int(st[_native.STATE_ROWS2]) + GROUP <= self._caps[2][b]
                        and int(st[_native.STATE_ROWS3]) + GROUP <= self._caps[3][b])
                if not room:
                    raise RuntimeError("the preallocated cache is full; raise max_new_tokens")
        ks = [k.contiguous() for k in keys]
        vs = [v.contiguous() for v in values]
        key_table = (C.c_void_p * 4)(*[k.data_ptr() for k in ks])
        value_table = (C.c_void_p * 4)(*[v.data_ptr() for v in vs])
        _native.check(_native.load().fl_append_decode_token(
            C.byref(self._native), key_table, value_table, _native.current_stream(self._device)),
            "fl_append_decode_token")
        self.advance_host_state()

    def advance_host_state(self) -> None:
        """Host mirror of what one ``fl_append_decode_token`` does to ``seq_state``.  Called
        by :meth:`append_decode_token`; a caller that replays a captured decode step calls
        it once per replay."""

        full = self.residual_length + self.group_size
        for b in range(self.batch):
            st = self._state_host[b]
            for i in range(2):
                self._tail_active_host[b][i].append(True)
            st[_native.STATE_TAIL_LEN] += 1
            if int(st[_native.STATE_TAIL_LEN]) >= full:
                for i in range(2):
                    flags = self._tail_active_host[b][i]
                    self._compact_counts[b][i] += sum(flags[:GROUP])
                    del flags[:GROUP]
                st[_native.STATE_QUANT_TOKENS] += GROUP
                st[_native.STATE_ROWS2] += GROUP
                st[_native.STATE_ROWS3] += GROUP
                st[_native.STATE_TAIL_LEN] -= GROUP
                st[_native.STATE_TAIL_START] = (int(st[_native.STATE_TAIL_START]) + GROUP) % TAIL_CAPACITY


class CrossLoopKVLayerBuilder:
    """Build one physical cache layer loop by loop, so that a prefill can drop every loop's dense
    K/V as soon as it is packed (flashloop/cache.py:315-625): ``from_loop1`` packs the anchor,
    ``add_loop2`` the delta against its decode, ``finalize`` the compact Loop-3/4 deltas against
    the reconstruction read back from the packed streams.  Batched: all tensors carry B sequences
    of equal prompt length; compact tensors hold the retained rows in position order, positions
    are int32 ``[B, rows]`` (ascending, padded with -1; one-dimensional for a batch of one).

    One ``fl_encode_prefill_stage`` launch per stage; the codes are the same bits as the
    reference's builder produces (and as :meth:`CrossLoopKVLayer.from_prefill`)."""

    def __init__(self) -> None:
        self.group_size = 0
        self.residual_length = 0
        self.packed_tokens = 0
        self.reader_backend = "kivi_outer"
        self.absolute_late_overrides = False
        self._layer: CrossLoopKVLayer | None = None
        self._tokens = 0
        self._extra = 0
        self._has_loop2 = False

    @property
    def retains_dense_loop1_prefix(self) -> bool:
        """Audit flag (flashloop/cache.py:399-403): nothing dense is kept between the stages."""

        return False

    @classmethod
    def from_loop1(cls, loop1_key: torch.Tensor, loop1_value: torch.Tensor, *, group_size: int = 64,
                   residual_length: int = 64, absolute_late_overrides: bool = False,
                   absolute_override_dtype: str = "int4", reader_backend: str = "kivi_outer", bits: int = 4,
                   max_new_tokens: int = 0) -> "CrossLoopKVLayerBuilder":
        shape = tuple(int(v) for v in loop1_key.shape)
        if len(shape) != 4 or loop1_value.shape != loop1_key.shape:
            raise ValueError("Loop-1 K/V must match [batch, heads, tokens, channels]")
        if loop1_value.dtype != loop1_key.dtype or loop1_value.device != loop1_key.device:
            raise ValueError("Loop-1 K/V must share dtype and device")
        if int(group_size) <= 0 or int(residual_length) < 0:
            raise ValueError("invalid group_size or residual_length")
        if absolute_late_overrides or absolute_override_dtype != "int4":
            raise ValueError("the CUDA cache supports additive cross-loop deltas only")
        if reader_backend not in {"kivi_outer", "triton_row"}:
            raise ValueError("unknown KV reader backend")
        batch, heads, tokens, channels = shape
        if channels != HEAD_DIM:
            raise ValueError("the CUDA cache specializes head_dim=128")
        _native.require_cuda(loop1_key, loop1_value)
        self = cls()
        self.group_size, self.residual_length = int(group_size), int(residual_length)
        self.reader_backend = reader_backend
        self._tokens = tokens
        self.packed_tokens = packed = max(0, ((tokens - self.residual_length) // self.group_size) * self.group_size)
        if tokens - packed > TAIL_CAPACITY:
            raise RuntimeError("tail longer than the ring")
        self._extra = _round_up(max_new_tokens, GROUP) + 2 * GROUP
        layer = CrossLoopKVLayer(batch=batch, heads=heads, token_capacities=[packed + self._extra] * batch,
                                 compact_capacities=None, bits=bits, group_size=group_size,
                                 residual_length=residual_length, device=loop1_key.device, dtype=loop1_key.dtype)
        st = layer._state_host
        st[:, _native.STATE_QUANT_TOKENS] = packed
        st[:, _native.STATE_TAIL_LEN] = tokens - packed
        layer._push_state()
        self._layer = layer
        self._stage(0, loop1_key, loop1_value)
        return self

    def _stage(self, stage: int, keys: torch.Tensor, values: torch.Tensor, positions: torch.Tensor | None = None) -> None:
        layer = self._layer
        keys, values = keys.contiguous(), values.contiguous()
        rows = int(keys.shape[2])
        if stage < 2:
            tail = self._tokens - self.packed_tokens
            bh = layer.batch * layer.heads
            layer._tail_k[stage, :, :tail].copy_(keys[:, :, self.packed_tokens:].reshape(bh, tail, HEAD_DIM))
            layer._tail_v[stage, :, :tail].copy_(values[:, :, self.packed_tokens:].reshape(bh, tail, HEAD_DIM))
            if not self.packed_tokens:
                return
        elif not self.packed_tokens or rows == 0:
            return
        _native.check(_native.load().fl_encode_prefill_stage(
            C.byref(layer._native), 0, layer.batch, rows, stage, _native.ptr(keys), _native.ptr(values),
            _native.ptr(positions), 0 if positions is None else int(positions.shape[1]), 0 if stage < 2 else 1,
            _native.current_stream(layer._device)), "fl_encode_prefill_stage")

    def _check_dense(self, key: torch.Tensor, value: torch.Tensor, label: str) -> None:
        layer = self._layer
        expected = (layer.batch, layer.heads, self._tokens, HEAD_DIM)
        if tuple(key.shape) != expected or value.shape != key.shape:
            raise ValueError(f"{label} K/V shape differs from Loop 1")
        if key.dtype != layer._dtype or value.dtype != layer._dtype:
            raise ValueError(f"{label} K/V dtype differs from Loop 1")
        if key.device != layer._device or value.device != layer._device:
            raise ValueError(f"{label} K/V device differs from Loop 1")

    def add_loop2(self, loop2_key: torch.Tensor, loop2_value: torch.Tensor) -> None:
        if self._has_loop2:
            raise RuntimeError("Loop 2 is already installed")
        self._check_dense(loop2_key, loop2_value, "Loop-2")
        self._stage(1, loop2_key, loop2_value)
        self._has_loop2 = True

    def _check_updates(self, positions: torch.Tensor, key: torch.Tensor, value: torch.Tensor, label: str):
        """Positions as int32 [B, rows] on the device, the number of retained rows per sequence."""

        layer = self._layer
        logical = positions.to(device=layer._device, dtype=torch.int32)
        if logical.ndim == 1:
            logical = logical[None].expand(layer.batch, -1) if layer.batch == 1 else None
        if logical is None or logical.ndim != 2 or logical.shape[0] != layer.batch:
            raise ValueError(f"{label} positions must have shape [batch, rows]")
        logical = logical.contiguous()
        held = logical >= 0
        count = held.sum(1)
        rows = int(logical.shape[1])
        if rows:
            ordered = (logical[:, 1:] > logical[:, :-1]) | ~held[:, 1:]
            padded_last = held[:, :-1] | ~held[:, 1:]  # no position after a -1
            if not bool(ordered.all()) or not bool(padded_last.all()):
                raise ValueError(f"{label} positions must be strictly sorted")
            if int(logical.max()) >= self._tokens:
                raise IndexError(f"{label} update is outside the prompt")
        expected = (layer.batch, layer.heads, rows, HEAD_DIM)
        if tuple(key.shape) != expected or value.shape != key.shape:
            raise ValueError(f"{label} compact K/V shape differs from its positions")
        if key.dtype != layer._dtype or value.dtype != layer._dtype:
            raise ValueError(f"{label} compact K/V dtype differs from Loop 1")
        if key.device != layer._device or value.device != layer._device:
            raise ValueError(f"{label} compact K/V device differs from Loop 1")
        return logical, count

    def finalize(self, *, loop3_positions: torch.Tensor, loop3_keys: torch.Tensor, loop3_values: torch.Tensor,
                 loop4_positions: torch.Tensor, loop4_keys: torch.Tensor,
                 loop4_values: torch.Tensor) -> CrossLoopKVLayer:
        if not self._has_loop2:
            raise RuntimeError("Loop 2 must be installed before finalization")
        layer, packed, tokens = self._layer, self.packed_tokens, self._tokens
        pos3, _ = self._check_updates(loop3_positions, loop3_keys, loop3_values, "Loop-3")
        pos4, _ = self._check_updates(loop4_positions, loop4_keys, loop4_values, "Loop-4")
        device = layer._device
        member3 = torch.zeros((layer.batch, tokens + 1), dtype=torch.bool, device=device)
        member3.scatter_(1, torch.where(pos3 >= 0, pos3, tokens).long(), True)
        if pos4.numel() and not bool(member3.gather(1, torch.where(pos4 >= 0, pos4, tokens).long())[pos4 >= 0].all()):
            raise ValueError("Loop-4 positions must be nested in Loop-3 positions")
        inside = [((p >= 0) & (p < packed)) for p in (pos3, pos4)]
        counts = [m.sum(1).tolist() for m in inside]
        layer._allocate_compact([(_round_up(n3, GROUP) + self._extra, _round_up(n4, GROUP) + self._extra)
                                 for n3, n4 in zip(*counts)])
        # rank maps: logical prefix token -> its row in the compact stream (positions are ascending,
        # so the i-th retained position inside the prefix is row i)
        for i, (pos, mask) in enumerate(zip((pos3, pos4), inside)):
            ranks = torch.cumsum(mask.to(torch.int32), 1, dtype=torch.int32) - 1
            for b in range(layer.batch):
                base = layer._rank_base_host[b]
                view = layer._rank[i][base:base + packed]
                view.fill_(-1)
                view[pos[b][mask[b]].long()] = ranks[b][mask[b]]
        for b in range(layer.batch):
            st = layer._state_host[b]
            st[_native.STATE_ROWS2] = _round_up(int(counts[0][b]), GROUP)
            st[_native.STATE_ROWS3] = _round_up(int(counts[1][b]), GROUP)
            layer._compact_counts[b] = [int(counts[0][b]), int(counts[1][b])]
        layer._push_state()
        self._stage(2, loop3_keys, loop3_values, pos3)
        self._stage(3, loop4_keys, loop4_values, pos4)
        # tails of loops 3 and 4: the tail before, with the retained tail tokens replaced
        tail = tokens - packed
        bh = layer.batch * layer.heads
        for i, (pos, key, value) in enumerate(((pos3, loop3_keys, loop3_values), (pos4, loop4_keys, loop4_values))):
            loop = 2 + i
            layer._tail_k[loop, :, :tail].copy_(layer._tail_k[loop - 1, :, :tail])
            layer._tail_v[loop, :, :tail].copy_(layer._tail_v[loop - 1, :, :tail])
            flags = torch.zeros((layer.batch, TAIL_CAPACITY), dtype=torch.uint8, device=device)
            for b in range(layer.batch):
                late = torch.nonzero(pos[b] >= packed).flatten()
                if late.numel():
                    slots = pos[b][late].long() - packed
                    sl = slice(b * layer.heads, (b + 1) * layer.heads)
                    layer._tail_k[loop, sl].index_copy_(1, slots, key[b].index_select(1, late))
                    layer._tail_v[loop, sl].index_copy_(1, slots, value[b].index_select(1, late))
                    flags[b, slots] = 1
            layer._tail_active[i].copy_(flags)
            host = flags[:, :tail].bool().tolist()
            for b in range(layer.batch):
                layer._tail_active_host[b][i] = host[b]
        self._layer = None
        return layer


class CrossLoopKVCache:
    """Layer-indexed owner for physical Cross-Loop KV storage (flashloop/cache.py:1841-1950)."""

    def __init__(self, *, num_layers: int) -> None:
        num_layers = int(num_layers)
        if num_layers <= 0:
            raise ValueError("num_layers must be positive")
        self.layers: list[CrossLoopKVLayer | None] = [None] * num_layers

    def set_layer(self, layer_index: int, layer: CrossLoopKVLayer) -> None:
        layer_index = int(layer_index)
        if layer_index not in range(len(self.layers)):
            raise IndexError("layer index is outside the cache")
        if self.layers[layer_index] is not None:
            raise RuntimeError("physical cache layer is already installed")
        self.layers[layer_index] = layer

    def _require_layer(self, layer_index: int) -> CrossLoopKVLayer:
        layer_index = int(layer_index)
        if layer_index not in range(len(self.layers)):
            raise IndexError("layer index is outside the cache")
        layer = self.layers[layer_index]
        if layer is None:
            raise RuntimeError("physical cache layer has not been installed")
        return layer

    def physical_layout_audit(self) -> dict:
        installed = [layer for layer in self.layers if layer is not None]
        return {"installed_layers": len(installed), "reader_backends": ["kivi_outer"] if installed else [],
                "kivi_packed_streams": 0, "row_packed_streams": 8 * len(installed),
                "bf16_cross_loop_layers": 0}

    def qk(self, layer_index, loop, query, indices, *, validate_indices=True):
        return self._require_layer(layer_index).qk(loop, query, indices, validate_indices=validate_indices)

    def pv(self, layer_index, loop, weights, indices, *, validate_indices=True, **kwargs):
        return self._require_layer(layer_index).pv(loop, weights, indices,
                                                   validate_indices=validate_indices, **kwargs)

    def cached_mass_sparse_attention_delta(self, layer_index, loop, **kwargs):
        return self._require_layer(layer_index).cached_mass_sparse_attention_delta(loop, **kwargs)

    def dense_source_attention(self, layer_index, loop, **kwargs):
        return self._require_layer(layer_index).dense_source_attention(loop, **kwargs)

    @property
    def storage_bytes(self) -> int:
        return sum(layer.storage_bytes for layer in self.layers if layer is not None)
