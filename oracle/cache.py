"""Anchor + delta cross-loop KV layer (numpy oracle, one sequence).

Restates flashloop/cache.py for the packed path with additive deltas:

* prefix encoding of the four loops (``from_prefill`` / ``_encode_initial_prefix``,
  cache.py:752-817, 1008-1074): anchor = pack(X1); d2 = pack(X2 - dec(anchor));
  d3/d4 = pack of the active rows' residual against the running bf16
  reconstruction; every subtraction and addition is a bfloat16 tensor operation;
* the BF16 tail, decode append and the 64-token rollover (cache.py:1758-1838) with
  the row layout's append rule (cache.py:202-242: new rows keep their own
  metadata group);
* the readers: ``gather`` (cache.py:1114-1200), ``qk``/``pv`` (cache.py:1202-1515,
  Torch branches), ``dense_source_attention`` (cache.py:1745-1756) and
  ``cached_mass_sparse_attention_delta`` (cache.py:1619-1642).

Arrays are float32 holding bf16-representable values with layout [1, H, n, D].
Reader arithmetic runs in float64 so that the oracle is the more accurate side of
every tolerance comparison.
"""

from __future__ import annotations

import numpy as np

from . import bf16
from .packing import PackedRows, concat_rows, pack_k_rows, pack_v_rows
from .selection import positions_and_rank_map


class LayerOracle:
    def __init__(self) -> None:
        self.group_size = 64
        self.residual_length = 64
        self.bits = 4
        self.quantized_tokens = 0
        self.keys: list[PackedRows | None] = [None] * 4
        self.values: list[PackedRows | None] = [None] * 4
        self.override_indices = (np.zeros(0, np.int32), np.zeros(0, np.int32))
        self.rank_maps = (np.zeros(0, np.int32), np.zeros(0, np.int32))
        self.tail_keys: list[np.ndarray] = []
        self.tail_values: list[np.ndarray] = []
        self.tail_active = [np.zeros(0, bool), np.zeros(0, bool)]
        self.heads = 0
        self.channels = 0

    # ------------------------------------------------------------------ construction

    @classmethod
    def from_prefill(cls, keys, values, *, mask_loop3, mask_loop4, group_size=64,
                     residual_length=64, bits=4) -> "LayerOracle":
        """cache.py:752-817.  keys/values: four arrays [1,H,T,D]; masks bool [T]."""

        self = cls()
        _, heads, tokens, channels = keys[0].shape
        self.heads, self.channels = heads, channels
        self.group_size, self.residual_length, self.bits = group_size, residual_length, bits
        mask3 = np.asarray(mask_loop3, bool).reshape(-1)
        mask4 = np.asarray(mask_loop4, bool).reshape(-1)
        if np.any(mask4 & ~mask3):
            raise ValueError("Loop-4 overrides must be nested in Loop-3 overrides")
        packed = max(0, ((tokens - residual_length) // group_size) * group_size)
        self.quantized_tokens = packed
        if packed:
            self._encode_prefix([k[:, :, :packed] for k in keys], [v[:, :, :packed] for v in values],
                                mask3[:packed], mask4[:packed])
        self.tail_keys = [np.array(k[:, :, packed:], np.float32) for k in keys]
        self.tail_values = [np.array(v[:, :, packed:], np.float32) for v in values]
        self.tail_active = [mask3[packed:].copy(), mask4[packed:].copy()]
        return self

    def _encode_prefix(self, keys, values, mask3, mask4) -> None:
        """cache.py:1008-1074."""

        tokens = keys[0].shape[2]
        g, b = self.group_size, self.bits
        self.keys[0] = pack_k_rows(keys[0], group_size=g, bits=b)
        self.values[0] = pack_v_rows(values[0], group_size=g, bits=b)
        recon_k = self.keys[0].decode()
        recon_v = self.values[0].decode()
        self.keys[1] = pack_k_rows(bf16.sub(keys[1], recon_k), group_size=g, bits=b)
        self.values[1] = pack_v_rows(bf16.sub(values[1], recon_v), group_size=g, bits=b)
        recon_k = bf16.add(recon_k, self.keys[1].decode())
        recon_v = bf16.add(recon_v, self.values[1].decode())
        pos3, rank3 = positions_and_rank_map(mask3, tokens)
        pos4, rank4 = positions_and_rank_map(mask4, tokens)
        self.override_indices = (pos3, pos4)
        self.rank_maps = (rank3, rank4)
        for stream, (tk, tv, pos) in enumerate(((keys[2], values[2], pos3),
                                                (keys[3], values[3], pos4)), start=2):
            if pos.size == 0:
                continue
            sel = pos.astype(np.int64)
            dk = bf16.sub(tk[:, :, sel], recon_k[:, :, sel])
            dv = bf16.sub(tv[:, :, sel], recon_v[:, :, sel])
            self.keys[stream] = pack_k_rows(dk, group_size=g, bits=b)
            self.values[stream] = pack_v_rows(dv, group_size=g, bits=b)
            recon_k = recon_k.copy()
            recon_v = recon_v.copy()
            recon_k[:, :, sel] = bf16.add(recon_k[:, :, sel], self.keys[stream].decode())
            recon_v[:, :, sel] = bf16.add(recon_v[:, :, sel], self.values[stream].decode())

    # ------------------------------------------------------------------ bookkeeping

    @property
    def tail_tokens(self) -> int:
        return int(self.tail_keys[0].shape[2]) if self.tail_keys else 0

    @property
    def token_count(self) -> int:
        return self.quantized_tokens + self.tail_tokens

    def stream_tokens(self) -> tuple:
        return tuple(0 if s is None else s.shape[2] for s in self.keys)

    # ------------------------------------------------------------------ append / rollover

    def append_decode_token(self, keys, values) -> None:
        """cache.py:1758-1776.  keys/values: four arrays [1,H,1,D]."""

        self.tail_keys = [np.concatenate([t, np.asarray(k, np.float32)], axis=2)
                          for t, k in zip(self.tail_keys, keys)]
        self.tail_values = [np.concatenate([t, np.asarray(v, np.float32)], axis=2)
                            for t, v in zip(self.tail_values, values)]
        self.tail_active = [np.concatenate([a, np.ones(1, bool)]) for a in self.tail_active]
        while self.tail_tokens >= self.residual_length + self.group_size:
            self._roll_one_group()

    def _roll_one_group(self) -> None:
        """cache.py:1778-1838: quantise the oldest ``group_size`` tail tokens of all four
        loops into new stream segments and shift the tail."""

        w = self.group_size
        block = LayerOracle.from_prefill(
            [t[:, :, :w] for t in self.tail_keys], [t[:, :, :w] for t in self.tail_values],
            mask_loop3=self.tail_active[0][:w], mask_loop4=self.tail_active[1][:w],
            group_size=w, residual_length=0, bits=self.bits)
        old = self.quantized_tokens
        for s in range(4):
            self.keys[s] = concat_rows(self.keys[s], block.keys[s])
            self.values[s] = concat_rows(self.values[s], block.values[s])
        self.override_indices = tuple(
            np.concatenate([cur, add + np.int32(old)]).astype(np.int32)
            for cur, add in zip(self.override_indices, block.override_indices))
        self.quantized_tokens += w
        ranks = []
        for pos in self.override_indices:
            rank = np.full((self.quantized_tokens,), -1, np.int32)
            rank[pos] = np.arange(pos.size, dtype=np.int32)
            ranks.append(rank)
        self.rank_maps = tuple(ranks)
        self.tail_keys = [t[:, :, w:] for t in self.tail_keys]
        self.tail_values = [t[:, :, w:] for t in self.tail_values]
        self.tail_active = [a[w:] for a in self.tail_active]

    # ------------------------------------------------------------------ readers

    def _prefix_rows(self, loop: int, indices: np.ndarray, *, chain_bf16):
        """K and V of prefix tokens ``indices`` at ``loop``: sum over streams <= loop.

        The reference combines the streams in three slightly different ways, all inside
        the BF16 tolerance of one another; ``chain_bf16`` picks one:

        * ``True``  -- cache.py:1134-1182 (``gather``): every decoded stream is a bf16
          tensor and the additions are bf16 operations;
        * ``"streams"`` -- cache.py:1308-1340 / kivi_backend.py:1024-1046 (``qk``/``pv``
          Torch branches): every stream is decoded to bf16, the per-stream products are
          summed in float32;
        * ``False`` -- flashloop/csrc/kivi_outer_gemv_cuda.cu:782-806 (fused readers):
          float32 ``scale * code + zero`` summed without intermediate rounding."""

        idx = indices.astype(np.int64)
        outs = []
        for streams in (self.keys, self.values):
            dec = (lambda p: p.decode_f32()) if chain_bf16 is False else (lambda p: p.decode())
            combine = bf16.add if chain_bf16 is True else (lambda a, b: a + b)
            total = dec(streams[0])[:, :, idx].astype(np.float32)
            for s in range(1, loop + 1):
                packed = streams[s]
                if packed is None:
                    continue
                if s == 1:
                    total = combine(total, dec(packed)[:, :, idx])
                    continue
                ranks = self.rank_maps[s - 2][idx]
                active = np.nonzero(ranks >= 0)[0]
                if active.size:
                    total = total.copy()
                    total[:, :, active] = combine(total[:, :, active],
                                                  dec(packed)[:, :, ranks[active].astype(np.int64)])
            outs.append(total)
        return outs[0], outs[1]

    def gather(self, loop: int, indices: np.ndarray, *, chain_bf16: bool = True):
        """cache.py:1114-1200: logical K/V rows of ``loop`` for 1-D ``indices``."""

        indices = np.asarray(indices, np.int64)
        out_k = np.zeros((1, self.heads, indices.size, self.channels), np.float32)
        out_v = np.zeros_like(out_k)
        prefix = np.nonzero(indices < self.quantized_tokens)[0]
        if prefix.size:
            k, v = self._prefix_rows(loop, indices[prefix], chain_bf16=chain_bf16)
            out_k[:, :, prefix] = k
            out_v[:, :, prefix] = v
        tail = np.nonzero(indices >= self.quantized_tokens)[0]
        if tail.size:
            t = indices[tail] - self.quantized_tokens
            out_k[:, :, tail] = self.tail_keys[loop][:, :, t]
            out_v[:, :, tail] = self.tail_values[loop][:, :, t]
        return out_k, out_v

    def dense_source_attention(self, loop, *, query, current_key, current_value, scaling,
                               chain_bf16=False):
        """cache.py:1745-1756.  Returns (output [1,H,1,D] f32, scaled logits [1,H,1,N+1])."""

        k, v = self.gather(loop, np.arange(self.token_count), chain_bf16=chain_bf16)
        k = np.concatenate([k, current_key.astype(np.float32)], axis=2).astype(np.float64)
        v = np.concatenate([v, current_value.astype(np.float32)], axis=2).astype(np.float64)
        logits = np.einsum("bhqd,bhnd->bhqn", query.astype(np.float64), k) * float(scaling)
        w = np.exp(logits - logits.max(axis=-1, keepdims=True))
        w /= w.sum(axis=-1, keepdims=True)
        out = np.einsum("bhqn,bhnd->bhqd", w, v)
        return out.astype(np.float32), logits.astype(np.float32)

    def _gather_per_head(self, loop, indices, *, chain_bf16):
        """Per-head logical rows: indices [1,H,S] -> K, V [1,H,S,D]."""

        heads, sel = indices.shape[1], indices.shape[2]
        k = np.zeros((1, heads, sel, self.channels), np.float32)
        v = np.zeros_like(k)
        for h in range(heads):
            kh, vh = self.gather(loop, indices[0, h], chain_bf16=chain_bf16)
            k[0, h] = kh[0, h]
            v[0, h] = vh[0, h]
        return k, v

    def qk(self, loop, query, indices, *, chain_bf16=False):
        """cache.py:1202-1356 (unscaled logits of selected logical rows)."""

        k, _ = self._gather_per_head(loop, np.asarray(indices), chain_bf16=chain_bf16)
        return np.einsum("bhqd,bhnd->bhqn", query.astype(np.float64),
                         k.astype(np.float64)).astype(np.float32)

    def pv(self, loop, weights, indices, *, chain_bf16=False):
        """cache.py:1358-1515 (probability-weighted V of selected logical rows)."""

        _, v = self._gather_per_head(loop, np.asarray(indices), chain_bf16=chain_bf16)
        return np.einsum("bhqn,bhnd->bhqd", weights.astype(np.float64),
                         v.astype(np.float64)).astype(np.float32)

    def selected_value_aggregate(self, loop, *, selected_indices, selected_weights,
                                 current_value, past_tokens):
        """flashloop/engine.py:346-371."""

        is_current = selected_indices == past_tokens
        safe = np.where(is_current, 0, selected_indices)
        past = selected_weights * (~is_current)[:, :, None, :]
        out = self.pv(loop, past, safe).astype(np.float64)
        out += (selected_weights * is_current[:, :, None, :]).sum(axis=-1, keepdims=True) \
            * current_value.astype(np.float64)
        return out.astype(np.float32)

    def cached_mass_sparse_attention_delta(self, loop, *, query, current_key, current_value,
                                           current_position, indices, valid,
                                           source_selected_output, global_mass, scaling):
        """cache.py:1619-1642: mass * (subset-softmax target - cached source subset)."""

        indices = np.asarray(indices)
        valid = np.asarray(valid, bool)
        is_current = valid & (indices == int(current_position))
        safe = np.where(is_current | ~valid, 0, indices)
        logits = self.qk(loop, query, safe).astype(np.float64)
        cur = np.einsum("bhqd,bhnd->bhqn", query.astype(np.float64), current_key.astype(np.float64))
        logits = np.where(is_current[:, :, None, :], cur, logits) * float(scaling)
        logits = np.where(valid[:, :, None, :], logits, -np.inf)
        w = np.exp(logits - logits.max(axis=-1, keepdims=True))
        w /= w.sum(axis=-1, keepdims=True)
        target = self.pv(loop, (w * (~is_current)[:, :, None, :]).astype(np.float32), safe)
        target = target.astype(np.float64) + (w * is_current[:, :, None, :]).sum(
            axis=-1, keepdims=True) * current_value.astype(np.float64)
        out = global_mass.astype(np.float64) * (target - source_selected_output.astype(np.float64))
        return out.astype(np.float32)

    # ------------------------------------------------------------------ accounting

    @property
    def storage_bytes(self) -> int:
        """cache.py:1084-1101."""

        total = sum(s.storage_bytes for s in (*self.keys, *self.values) if s is not None)
        total += sum(2 * t.size for t in (*self.tail_keys, *self.tail_values))
        total += sum(a.nbytes for a in (*self.override_indices, *self.rank_maps))
        total += sum(a.size for a in self.tail_active)
        return int(total)
