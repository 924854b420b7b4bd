"""Batched Ouro-style four-loop inference orchestration.

Mirrors flashloop/engine.py:112-607 (``FlashLoopEngine.prefill / decode / generate / reset``,
``EngineState``, ``PrefillOutput``, ``DecodeOutput``, ``DecodeReceipt``) with a batch dimension:
the reference is batch-one (engine.py:176-177, 376-377); here every sequence of the batch has
its own cache state inside one ``CrossLoopKVLayer`` per physical layer and all sequences share
every launch.  Prompts of one call have equal length.

Decode per layer and loop (engine.py:393-537): loops 1-2 run the dense reader; after loop 2 the
top ``decode_key_fraction`` keys are selected from its logits and their loop-2 value aggregate
is cached; loops 3-4 run the cached-mass sparse reader over those keys and add the projected
correction to the loop-2 attention output.  After the four loops the token's K/V of every loop
are appended (``fl_append_decode_token``).  With ``use_cuda_graph=True`` the whole decode step
(model GEMMs included) is recorded once and replayed.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from .cache import CrossLoopKVCache, CrossLoopKVLayer, CrossLoopKVLayerBuilder
from .compaction import RetainedTokens, hidden_delta_score, retain_tokens
from .config import FlashLoopConfig, validate_ouro_model
from .selection import decode_budget
from .prefill import PrefillReceipt, apply_rope, dense_prefill_loop, sparse_prefill_loop
from . import step_ops
from .tensor_parallel import PartialSum, PeerAllReduce
from .weights import fused_mlp, project_qkv, project_value, repack_projection_weights


@dataclass(frozen=True)
class EngineState:
    cache: CrossLoopKVCache
    next_position: int
    mask_loop3: torch.Tensor
    mask_loop4: torch.Tensor
    prefill_receipts: tuple


@dataclass(frozen=True)
class PrefillOutput:
    logits: torch.Tensor
    state: EngineState


@dataclass(frozen=True)
class DecodeReceipt:
    dense_attention_calls: int
    sparse_attention_calls: int
    dense_late_loop_calls: int
    selected_keys_per_layer: tuple


@dataclass(frozen=True)
class DecodeOutput:
    logits: torch.Tensor
    state: EngineState
    receipt: DecodeReceipt


class FlashLoopEngine:
    """Narrow adapter that reuses an Ouro-style model's weights without copying them."""

    def __init__(self, model: torch.nn.Module, *, config: FlashLoopConfig | None = None,
                 validate_model: bool = True, max_new_tokens: int = 512, use_cuda_graph: bool = False,
                 reference_loop4_scores: bool = True, fuse_decode_ops: bool = True, tp_group=None,
                 tp_allreduce: str = "peer", tp_wait_limit: int = 0, stream_projections: bool = True) -> None:
        if validate_model:
            validate_ouro_model(model)
        elif int(getattr(model.config, "total_ut_steps", 0)) != 4:
            raise ValueError("FlashLoop requires exactly four recurrent loops")
        self.model = model.eval()
        self.config = config or FlashLoopConfig()
        self.layers = self.model.model.layers
        self.backbone = self.model.model
        if self.config.fuse_projection_weights:
            repack_projection_weights(self.layers)
        self.max_new_tokens = int(max_new_tokens)
        self.use_cuda_graph = bool(use_cuda_graph)
        self.reference_loop4_scores = bool(reference_loop4_scores)
        # tensor parallelism: the model holds this rank's heads / FFN columns (see tensor_parallel.py)
        # and the partial o_proj / down_proj outputs are summed over ``tp_group``: with NCCL in
        # prefill, and in a decode step either with NCCL (tp_allreduce="nccl", eager launches only)
        # or inside the norm launch over peer memory (tp_allreduce="peer", recordable in a graph)
        if tp_allreduce not in ("peer", "nccl"):
            raise ValueError("tp_allreduce is 'peer' or 'nccl'")
        if tp_group is not None and use_cuda_graph and tp_allreduce != "peer":
            raise ValueError("with NCCL all-reduces the tensor-parallel decode step is launched eagerly: "
                             "use_cuda_graph=False or tp_allreduce='peer'")
        self.tp_group = tp_group
        self.tp_allreduce = tp_allreduce
        self.tp_wait_limit = int(tp_wait_limit)
        self._peer: PeerAllReduce | None = None
        self._reduce = PartialSum(tp_group) if tp_group is not None else (lambda t: t)
        self.fuse_decode_ops = bool(fuse_decode_ops) and self._modules_are_fusable()
        # the projections of a decode step of at most 16 sequences through this library's weight-
        # streaming kernel (step_ops.linear) instead of the framework's GEMM
        self.stream_projections = bool(stream_projections)
        self._reuse = self.config.reuse_selected_probabilities and self.config.enable_sparse_decode
        self._state: EngineState | None = None
        self._graph = None
        self._graph_io = None
        self._graph_warm = False
        self._decode_limit = 0

    @classmethod
    def from_pretrained(cls, model_path: str, *, config: FlashLoopConfig | None = None,
                        torch_dtype: torch.dtype = torch.bfloat16, device: str | torch.device = "cuda",
                        **kwargs) -> "FlashLoopEngine":
        """engine.py:134-150: load an Ouro checkpoint with its remote modelling code."""

        from transformers import AutoModelForCausalLM

        model = AutoModelForCausalLM.from_pretrained(model_path, trust_remote_code=True,
                                                     torch_dtype=torch_dtype).to(device)
        return cls(model, config=config, validate_model=True, **kwargs)

    @property
    def state(self) -> EngineState:
        if self._state is None:
            raise RuntimeError("engine cache is not initialized")
        return self._state

    def reset(self) -> None:
        self._state = None
        self._graph = None
        self._graph_io = None
        self._graph_warm = False
        self._decode_limit = 0

    # ------------------------------------------------------------------ prefill

    def _retain(self, loop: int, scores: torch.Tensor, fraction: float,
                eligible: torch.Tensor | None) -> RetainedTokens:
        """Retention decision of ``loop`` (3 or 4); a subclass may substitute its own policy."""

        return retain_tokens(scores, fraction=fraction, eligible=eligible)

    @torch.inference_mode()
    def prefill(self, input_ids: torch.Tensor, attention_mask: torch.Tensor | None = None) -> PrefillOutput:
        """engine.py:162-344 for a batch of equally long prompts [B, T]."""

        if self._state is not None:
            raise RuntimeError("engine cache is already initialized; call reset()")
        if input_ids.ndim != 2 or input_ids.shape[1] <= 0:
            raise ValueError("prefill requires input_ids [batch, tokens] with at least one token")
        if attention_mask is not None and not bool(attention_mask.bool().all().item()):
            raise ValueError("padding is not supported: prompts of one call have equal length")
        batch, tokens = (int(v) for v in input_ids.shape)
        hidden = self.backbone.embed_tokens(input_ids)
        positions = torch.arange(tokens, device=input_ids.device).unsqueeze(0).expand(batch, -1)
        rope = self.backbone.rotary_emb(hidden, positions)
        norm = self.backbone.norm

        # Every loop's dense K/V is packed as soon as the loop ends and dropped (engine.py:204-260):
        # Loop 1 goes into the anchor streams before Loop 2 runs, Loop 2 into the delta-2 streams,
        # and the late loops write their retained rows into the Loop-2 composite in place and hand
        # the cache only those rows.  At most one full-size composite is alive at any time.
        loop1 = dense_prefill_loop(self.layers, hidden, position_embeddings=rope, final_norm=norm, loop=1,
                                   reduce=self._reduce)
        builders = []
        for index in range(len(self.layers)):
            builders.append(CrossLoopKVLayerBuilder.from_loop1(
                loop1.composite_cache.keys[index], loop1.composite_cache.values[index],
                group_size=self.config.group_size, residual_length=self.config.residual_length,
                bits=self.config.kv_bits, max_new_tokens=self.max_new_tokens))
            loop1.composite_cache.keys[index] = None
            loop1.composite_cache.values[index] = None
        loop2 = dense_prefill_loop(self.layers, loop1.hidden_states, position_embeddings=rope, final_norm=norm,
                                   loop=2, reduce=self._reduce)
        for index, builder in enumerate(builders):
            builder.add_loop2(loop2.composite_cache.keys[index], loop2.composite_cache.values[index])
        fraction3, fraction4 = self.config.effective_prefill_fractions
        keep3 = self._retain(3, hidden_delta_score(loop2.hidden_states, loop1.hidden_states), fraction3, None)
        loop3 = sparse_prefill_loop(self.layers, loop2.hidden_states, retained=keep3,
                                    composite_cache=loop2.composite_cache, position_embeddings=rope,
                                    final_norm=norm, loop=3, reduce=self._reduce, consume_inputs=True)
        if self.reference_loop4_scores:
            # engine.py:258-275 runs Loop 3 with consume_inputs=True, so prefill.py:236-237,254
            # write the Loop-3 rows into the Loop-2 tensor itself and the score of
            # engine.py:271-272 compares that tensor with itself: every Loop-4 score is 0 and
            # the retained set is decided by the tie rule alone (here: lowest positions first).
            score4 = torch.zeros((batch, tokens), dtype=torch.float32, device=input_ids.device)
        else:
            score4 = hidden_delta_score(loop3.hidden_states, loop2.hidden_states)
        keep4 = self._retain(4, score4, fraction4, keep3.mask)
        loop4 = sparse_prefill_loop(self.layers, loop3.hidden_states, retained=keep4,
                                    composite_cache=loop3.composite_cache, position_embeddings=rope,
                                    final_norm=norm, loop=4, reduce=self._reduce, consume_inputs=True)

        physical = CrossLoopKVCache(num_layers=len(self.layers))
        loops = (loop1, loop2, loop3, loop4)
        rows3, rows4 = int(keep3.count[0]), int(keep4.count[0])
        for index, builder in enumerate(builders):
            physical.set_layer(index, builder.finalize(
                loop3_positions=keep3.positions[:, :rows3], loop3_keys=loop3.updates[index][0],
                loop3_values=loop3.updates[index][1], loop4_positions=keep4.positions[:, :rows4],
                loop4_keys=loop4.updates[index][0], loop4_values=loop4.updates[index][1]))
            loop4.composite_cache.keys[index] = None  # the composite of this layer (shared by loops 2-4)
            loop4.composite_cache.values[index] = None
        self._decode_limit = tokens + self.max_new_tokens
        if (self.tp_group is not None and self.tp_allreduce == "peer" and input_ids.is_cuda
                and (self._peer is None or self._peer.rows_max < batch)):
            # collective over the group: every rank reaches this point of prefill
            self._peer = PeerAllReduce(self.tp_group, rows_max=batch, width=int(hidden.shape[-1]),
                                       device=input_ids.device, wait_limit=self.tp_wait_limit)
        self._state = EngineState(cache=physical, next_position=tokens, mask_loop3=keep3.mask,
                                  mask_loop4=keep4.mask,
                                  prefill_receipts=tuple(lp.receipt for lp in loops))
        logits = self.model.lm_head(loop4.hidden_states[:, -1]).float()
        return PrefillOutput(logits=logits, state=self._state)

    # ------------------------------------------------------------------ decode

    @staticmethod
    def _norm_eps(norm) -> float | None:
        for name in ("eps", "variance_epsilon"):
            if hasattr(norm, name):
                return float(getattr(norm, name))
        return None

    def _modules_are_fusable(self) -> bool:
        """True when every layer is the plain Ouro block the one-launch glue kernels restate:
        weight-only RMSNorms, repacked bias-free projections, SiLU-gated MLP, equal Q/K/V widths."""

        norms = [self.backbone.norm]
        for layer in self.layers:
            attention, mlp = layer.self_attn, layer.mlp
            if not hasattr(attention, "_flashloop_qkv_weight") or not hasattr(mlp, "_flashloop_gate_up_weight"):
                return False
            if len(set(attention._flashloop_qkv_splits)) != 1 or len(set(mlp._flashloop_gate_up_splits)) != 1:
                return False
            if int(attention.head_dim) != 128 or "silu" not in type(mlp.act_fn).__name__.lower():
                return False
            if attention.o_proj.bias is not None or mlp.down_proj.bias is not None:
                return False
            norms += [layer.input_layernorm, layer.input_layernorm_2, layer.post_attention_layernorm,
                      layer.post_attention_layernorm_2]
        for norm in norms:
            weight = getattr(norm, "weight", None)
            if weight is None or weight.dtype != torch.bfloat16 or getattr(norm, "bias", None) is not None:
                return False
            if self._norm_eps(norm) is None or len(list(norm.parameters())) != 1:
                return False
        return True

    def _decode_step(self, token_ids: torch.Tensor, position_ids: torch.Tensor) -> torch.Tensor:
        """The device work of one decode step; returns float32 logits [B, vocab]."""

        if self.fuse_decode_ops and token_ids.is_cuda:
            return self._decode_step_fused(token_ids, position_ids)
        return self._decode_step_modules(token_ids, position_ids)

    def _attend(self, loop: int, index: int, q, k, v, scaling: float, sources: list, o_proj, batch: int,
                convert: bool = True):
        """The cache-facing part of one layer and loop (engine.py:422-531).  Returns (partial,
        addend, keep): the projected attention output [B, 1, hidden] is ``[addend +] sum over the
        tensor-parallel ranks of partial`` (one rank: partial itself), and with ``keep`` the caller
        stores that output in ``sources[index][0]`` for the late loops.  With ``convert`` False the
        readers' float32 output goes to ``o_proj`` as it is (a projection that rounds on load)."""

        def cast(t, dtype):
            return t.to(dtype) if convert else t

        physical = self.state.cache.layers[index]
        if loop < 2 or not self.config.enable_sparse_decode:
            want_logits = loop == 1 and self.config.enable_sparse_decode
            out, logits = physical.dense_source_attention(loop, query=q, current_key=k, current_value=v,
                                                          scaling=scaling, return_logits=want_logits)
            partial = o_proj(cast(out, q.dtype).view(batch, 1, -1))
            if want_logits:
                sel = physical.select_decode_keys(logits, fraction=self.config.effective_decode_key_fraction)
                aggregate = physical.pv(1, sel.selected_weights, sel.indices, current_value=v,
                                        valid=sel.valid, validate_indices=False)
                sources[index] = [None, sel, aggregate]
            return partial, None, want_logits
        projected0, sel, aggregate = sources[index]
        if self.config.reuse_selected_probabilities:
            # engine.py:502-513: the loop-2 probabilities are reused, only V is read
            target = physical.pv(loop, sel.selected_weights, sel.indices, current_value=v, valid=sel.valid,
                                 validate_indices=False)
            delta = sel.global_mass.view(batch, -1, 1, 1) * (target - aggregate)
            return o_proj(cast(delta, v.dtype).view(batch, 1, -1)), projected0, False
        delta = physical.cached_mass_sparse_attention_delta(
            loop, query=q, current_key=k, current_value=v, indices=sel.indices, valid=sel.valid,
            source_selected_output=aggregate, global_mass=sel.global_mass, scaling=scaling)
        return o_proj(cast(delta, v.dtype).view(batch, 1, -1)), projected0, False

    def _linear(self, x: torch.Tensor, weight: torch.Tensor, *, swiglu: bool = False,
                to_norm: bool = False) -> torch.Tensor:
        """A bias-free projection of the fused decode step (and, with ``swiglu``, the gated
        activation of a fused gate/up weight).  With ``to_norm`` the result goes straight to
        :meth:`_sum_norm`, which on one GPU also takes the float32 partial sums
        [splits, rows, 1, out] of ``step_ops.linear_partial``."""

        if (to_norm and self.stream_projections and self._peer is None and self.tp_group is None
                and step_ops.linear_partial_fits(x, weight)):
            return step_ops.linear_partial(x, weight)
        if self.stream_projections and step_ops.linear_fits(x, weight):
            return step_ops.linear(x, weight, swiglu=swiglu)
        y = torch.nn.functional.linear(x.to(weight.dtype), weight)
        return step_ops.swiglu(y) if swiglu else y

    def _decode_reduce(self, partial: torch.Tensor) -> torch.Tensor:
        """Sum of a decode step's partial outputs over the tensor-parallel ranks."""

        if self._peer is not None:
            return self._peer(partial.contiguous())
        return self._reduce(partial)

    def _sum_norm(self, partial, addend, norm, norm2, residual, want_sum: bool):
        """``s = [addend +] sum over ranks of partial``; ``hidden = residual + norm(s)``;
        ``x = norm2(hidden)``: one launch (with peer tensor parallelism the sum over the ranks
        happens inside it).  Returns (hidden, x, s or None)."""

        eps = self._norm_eps
        if partial.dtype == torch.float32 and partial.ndim == 4:  # step_ops.linear_partial's slices
            hidden, x, total = step_ops.rmsnorm_partial(
                partial, norm.weight, eps(norm), residual=residual, weight2=norm2.weight, eps2=eps(norm2),
                addend=addend, want_sum=want_sum and addend is None)
            return hidden, x, total
        if self._peer is not None:
            return self._peer.reduce_norm(partial.contiguous(), norm.weight, eps(norm), residual=residual,
                                          weight2=norm2.weight, eps2=eps(norm2), addend=addend, want_sum=want_sum)
        total = self._reduce(partial)
        hidden, x = step_ops.rmsnorm(total, norm.weight, eps(norm), residual=residual, weight2=norm2.weight,
                                     eps2=eps(norm2), addend=addend)
        return hidden, x, (total if addend is None else None)

    def _decode_step_fused(self, token_ids: torch.Tensor, position_ids: torch.Tensor) -> torch.Tensor:
        """One decode step with the elementwise glue as one-launch kernels (``step_ops``): per layer
        and loop four GEMMs, the Q/K/V split + RoPE, the readers, two add + norm launches and
        SwiGLU.  Same arithmetic, op by op, as :meth:`_decode_step_modules`."""

        F = torch.nn.functional
        cache = self.state.cache
        hidden = self.backbone.embed_tokens(token_ids)
        batch = int(token_ids.shape[0])
        cos, sin = self.backbone.rotary_emb(hidden, position_ids)
        cos, sin = cos.contiguous(), sin.contiguous()
        n_layers = len(self.layers)
        keys = [[None] * 4 for _ in range(n_layers)]
        values = [[None] * 4 for _ in range(n_layers)]
        sources = [None] * n_layers
        eps = self._norm_eps
        first = self.layers[0].input_layernorm
        for loop in range(4):
            x = step_ops.rmsnorm(hidden, first.weight, eps(first))
            for index, layer in enumerate(self.layers):
                attention, mlp = layer.self_attn, layer.mlp
                if loop >= 2 and self._reuse:
                    # engine.py:401-408: no Q/K in the late loops; the loop-2 key stands in for the append
                    v = project_value(attention, x).view(batch, -1, 1, 128)
                    q, k = None, keys[index][1]
                else:
                    weight, heads = attention._flashloop_qkv_weight, attention._flashloop_qkv_splits[0] // 128
                    if self.stream_projections and step_ops.linear_fits(x, weight):
                        q, k, v = step_ops.qkv_rope(x, weight, cos, sin, heads=heads)
                    else:
                        q, k, v = F.linear(x, weight).split(attention._flashloop_qkv_splits, dim=-1)
                        q, k, v = step_ops.rope_split(q, k, v, cos, sin, heads=heads)
                keys[index][loop], values[index][loop] = k, v
                partial, addend, keep = self._attend(loop, index, q, k, v, float(attention.scaling), sources,
                                                     lambda t, w=attention.o_proj.weight: self._linear(t, w, to_norm=True),
                                                     batch, convert=False)
                n2, n3, n4 = layer.input_layernorm_2, layer.post_attention_layernorm, layer.post_attention_layernorm_2
                hidden, x, projected = self._sum_norm(partial, addend, n2, n3, hidden, keep)
                if keep:
                    sources[index][0] = projected
                m = self._linear(self._linear(x, mlp._flashloop_gate_up_weight, swiglu=True), mlp.down_proj.weight,
                                 to_norm=True)
                following = self.backbone.norm if index == n_layers - 1 else self.layers[index + 1].input_layernorm
                hidden, x, _ = self._sum_norm(m, None, n4, following, hidden, False)
            hidden = x  # the final norm of this loop
        for index in range(n_layers):
            cache.layers[index].append_decode_token(keys[index], values[index])
        return self.model.lm_head(hidden[:, -1]).float()  # 200 MB of weights: the library GEMM streams them at 0.88 of peak

    def _decode_step_modules(self, token_ids: torch.Tensor, position_ids: torch.Tensor) -> torch.Tensor:
        """One decode step through the model's own modules (any Ouro-style block)."""

        cache = self.state.cache
        hidden = self.backbone.embed_tokens(token_ids)
        batch = int(token_ids.shape[0])
        cos, sin = self.backbone.rotary_emb(hidden, position_ids)
        n_layers = len(self.layers)
        keys = [[None] * 4 for _ in range(n_layers)]
        values = [[None] * 4 for _ in range(n_layers)]
        sources = [None] * n_layers
        for loop in range(4):
            for index, layer in enumerate(self.layers):
                attention = layer.self_attn
                head_dim = int(attention.head_dim)
                if loop >= 2 and self._reuse:
                    v = project_value(attention, layer.input_layernorm(hidden))
                    v = v.view(batch, 1, -1, head_dim).transpose(1, 2).contiguous()
                    q, k = None, keys[index][1]
                else:
                    q, k, v = project_qkv(attention, layer.input_layernorm(hidden))
                    heads = q.shape[-1] // head_dim
                    q = q.view(batch, 1, heads, head_dim).transpose(1, 2)
                    k = k.view(batch, 1, heads, head_dim).transpose(1, 2)
                    v = v.view(batch, 1, heads, head_dim).transpose(1, 2).contiguous()
                    q, k = apply_rope(q, k, cos, sin)
                    q, k = q.contiguous(), k.contiguous()
                keys[index][loop], values[index][loop] = k, v
                partial, addend, keep = self._attend(loop, index, q, k, v, float(attention.scaling), sources,
                                                     attention.o_proj, batch)
                projected = self._decode_reduce(partial)
                if addend is not None:
                    projected = addend + projected
                if keep:
                    sources[index][0] = projected
                residual = hidden
                hidden = residual + layer.input_layernorm_2(projected)
                hidden = hidden + layer.post_attention_layernorm_2(
                    self._decode_reduce(fused_mlp(layer.mlp, layer.post_attention_layernorm(hidden))))
            hidden = self.backbone.norm(hidden)
        for index in range(n_layers):
            cache.layers[index].append_decode_token(keys[index], values[index])
        return self.model.lm_head(hidden[:, -1]).float()

    def _graph_decode(self, token_ids: torch.Tensor) -> torch.Tensor:
        """Decode through a recorded CUDA graph.  The first call runs eagerly with the launch
        geometry fixed to the longest context this engine can reach (it creates every lazily
        allocated buffer), the second records the step, later ones replay it."""

        state = self.state
        layers = state.cache.layers
        if self._graph_io is None:
            for layer in layers:
                layer.context_bound = self._decode_limit
            self._graph_io = (token_ids.clone(), torch.empty_like(token_ids, dtype=torch.long), None)
        static_ids, static_pos, static_logits = self._graph_io
        static_ids.copy_(token_ids)
        static_pos.fill_(state.next_position)
        if self._graph is None and not self._graph_warm:
            self._graph_warm = True
            return self._decode_step(static_ids, static_pos)
        if self._graph is None:
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                static_logits = self._decode_step(static_ids, static_pos)
            # recording advanced the host mirror of the cache state but ran nothing on the
            # device: one replay brings the device in line
            graph.replay()
            self._graph = graph
            self._graph_io = (static_ids, static_pos, static_logits)
            return static_logits.clone()
        self._graph.replay()
        for layer in layers:
            layer.advance_host_state()
        return static_logits.clone()

    @torch.inference_mode()
    def decode(self, token_ids: torch.Tensor) -> DecodeOutput:
        """engine.py:373-570 for one token per sequence, token_ids [B, 1]."""

        state = self.state
        layers = state.cache.layers
        batch = layers[0].batch
        if tuple(token_ids.shape) != (batch, 1):
            raise ValueError("decode requires exactly one token per sequence")
        if state.next_position >= self._decode_limit:
            raise RuntimeError("the preallocated cache is full; raise max_new_tokens")
        if self.use_cuda_graph:
            logits = self._graph_decode(token_ids)
        else:
            position_ids = torch.full((batch, 1), state.next_position, device=token_ids.device, dtype=torch.long)
            logits = self._decode_step(token_ids, position_ids)
        self._state = EngineState(cache=state.cache, next_position=state.next_position + 1,
                                  mask_loop3=state.mask_loop3, mask_loop4=state.mask_loop4,
                                  prefill_receipts=state.prefill_receipts)
        sparse = self.config.enable_sparse_decode
        n = len(self.layers)
        budget = decode_budget(state.next_position + 1, self.config.effective_decode_key_fraction)
        receipt = DecodeReceipt(dense_attention_calls=(2 if sparse else 4) * n,
                                sparse_attention_calls=(2 if sparse else 0) * n,
                                dense_late_loop_calls=(0 if sparse else 2) * n,
                                selected_keys_per_layer=tuple([budget] * n) if sparse else ())
        return DecodeOutput(logits=logits, state=self._state, receipt=receipt)

    # ------------------------------------------------------------------ generate

    @torch.inference_mode()
    def generate(self, input_ids: torch.Tensor, *, max_new_tokens: int, eos_token_id: int | None = None,
                 stop_token_sequences: tuple = ()) -> torch.Tensor:
        """Greedy generation (engine.py:572-607).  With a batch, generation stops when every
        sequence has produced ``eos_token_id`` (finished sequences keep emitting it)."""

        if int(max_new_tokens) <= 0:
            raise ValueError("max_new_tokens must be positive")
        if int(max_new_tokens) > self.max_new_tokens:
            raise ValueError("max_new_tokens exceeds the room preallocated by the engine")
        if eos_token_id is None:
            eos_token_id = getattr(self.model.config, "eos_token_id", None)
        logits = self.prefill(input_ids).logits
        generated = input_ids
        finished = torch.zeros(input_ids.shape[0], dtype=torch.bool, device=input_ids.device)
        completions: list[list[int]] = [[] for _ in range(input_ids.shape[0])] if stop_token_sequences else []
        for step in range(int(max_new_tokens)):
            next_token = torch.argmax(logits, dim=-1, keepdim=True)
            if eos_token_id is not None:
                next_token = torch.where(finished[:, None], torch.full_like(next_token, int(eos_token_id)), next_token)
                finished = finished | (next_token[:, 0] == int(eos_token_id))
            generated = torch.cat([generated, next_token], dim=1)
            if stop_token_sequences:
                for b, tok in enumerate(next_token[:, 0].tolist()):
                    completions[b].append(tok)
                    if any(seq and tuple(completions[b][-len(seq):]) == tuple(seq) for seq in stop_token_sequences):
                        finished[b] = True
            if (eos_token_id is not None or stop_token_sequences) and bool(finished.all().item()):
                break
            if step + 1 < int(max_new_tokens):
                logits = self.decode(next_token).logits
        return generated
