"""Generate tests/golden/engine_vectors.npz by running the reference's FlashLoopEngine on CPU.

Run in a checkout that has the reference next to it:

    FLASHLOOP_REFERENCE=/path/to/FlashLoop python tests/golden/make_engine_golden.py

The model is the tiny Ouro-shaped stand-in of tests/helpers.py (weights from numpy's
RandomState, so they need not be stored).  For each of two prompts the reference engine
(flashloop/engine.py, validate_model=False, Torch reader path on CPU) prefills 200 tokens and
greedily decodes 70 tokens, which crosses one 64-token rollover.  Stored: prompts, retention
masks, prefill logits, decoded tokens and the logits of every decode step.

For prompt 0 the script also records a trace of everything that crosses the cache boundary:
the four loops' prefill K/V handed to the cache builder (cache.py:343-398, 415-439, 510-560),
and for every decode step, layer and loop the query / key / value vectors and the results of
``dense_source_attention``, the loop-2 selection with its value aggregate, and
``cached_mass_sparse_attention_delta``.  Replaying that trace through the CUDA cache compares
the hot path with the reference engine's own trajectory without any GEMM rounding in between.
"""

from __future__ import annotations

import os
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parents[1]))
ref_root = os.environ.get("FLASHLOOP_REFERENCE", "/root/reference")
sys.path.insert(0, ref_root)

import flashloop.cache as ref_cache  # noqa: E402
from flashloop.engine import FlashLoopEngine as RefEngine  # noqa: E402
from tests.helpers import tiny_ouro_model  # noqa: E402

PROMPT_TOKENS = 200
DECODE_STEPS = 70
torch.set_num_threads(8)

out: dict[str, np.ndarray] = {}
trace: dict[str, np.ndarray] = {}
tracing = {"on": False, "step": 0, "layer": 0}


def bits(t: torch.Tensor) -> np.ndarray:
    """bf16 tensors are stored as their uint16 bit patterns."""

    t = t.detach().contiguous()
    return t.view(torch.int16).numpy().view(np.uint16) if t.dtype == torch.bfloat16 else t.numpy()


# --- record what the engine hands to the cache builder during prefill ----------------------
Builder = ref_cache.CrossLoopKVLayerBuilder
_from_loop1, _add_loop2, _finalize = Builder.from_loop1.__func__, Builder.add_loop2, Builder.finalize


def from_loop1(cls, key, value, **kwargs):
    if tracing["on"]:
        index = tracing["layer"]
        tracing["layer"] += 1
        trace[f"prefill.l{index}.k1"], trace[f"prefill.l{index}.v1"] = bits(key), bits(value)
    builder = _from_loop1(cls, key, value, **kwargs)
    builder._trace_index = tracing["layer"] - 1
    return builder


def add_loop2(self, key, value):
    if tracing["on"]:
        trace[f"prefill.l{self._trace_index}.k2"], trace[f"prefill.l{self._trace_index}.v2"] = bits(key), bits(value)
    return _add_loop2(self, key, value)


def finalize(self, **kw):
    if tracing["on"]:
        i = self._trace_index
        for name in ("loop3_keys", "loop3_values", "loop4_keys", "loop4_values"):
            trace[f"prefill.l{i}.{name}"] = bits(kw[name])
    return _finalize(self, **kw)


Builder.from_loop1 = classmethod(from_loop1)
Builder.add_loop2 = add_loop2
Builder.finalize = finalize


def trace_decode(engine) -> None:
    """Wrap the cache-facing calls of one engine so that each records its inputs and outputs."""

    cache = engine.state.cache
    dense, sparse, aggregate = (cache.dense_source_attention, cache.cached_mass_sparse_attention_delta,
                                engine._selected_value_aggregate)

    def key(layer, loop, name):
        return f"s{tracing['step']}.l{layer}.r{loop}.{name}"

    def traced_dense(layer, loop, **kw):
        result, logits = dense(layer, loop, **kw)
        for name in ("query", "current_key", "current_value"):
            trace[key(layer, loop, name)] = bits(kw[name])
        trace[key(layer, loop, "out")] = bits(result.float())
        if logits is not None:
            trace[key(layer, loop, "logits")] = bits(logits.float())
        return result, logits

    def traced_aggregate(**kw):
        result = aggregate(**kw)
        layer = kw["layer_index"]
        trace[key(layer, 1, "sel_indices")] = bits(kw["selected_indices"].to(torch.int32))
        trace[key(layer, 1, "sel_weights")] = bits(kw["selected_weights"].float())
        trace[key(layer, 1, "sel_output")] = bits(result.float())
        return result

    def traced_sparse(layer, loop, **kw):
        result = sparse(layer, loop, **kw)
        for name in ("query", "current_key", "current_value"):
            trace[key(layer, loop, name)] = bits(kw[name])
        if loop == 2:
            trace[key(layer, 1, "sel_valid")] = bits(kw["valid"])
            trace[key(layer, 1, "sel_mass")] = bits(kw["global_mass"].float())
        trace[key(layer, loop, "out")] = bits(result.float())
        return result

    cache.dense_source_attention = traced_dense
    cache.cached_mass_sparse_attention_delta = traced_sparse
    engine._selected_value_aggregate = traced_aggregate

rng = np.random.RandomState(5)
prompts = rng.randint(0, 256, size=(2, PROMPT_TOKENS)).astype(np.int64)
out["prompts"] = prompts
for p in range(2):
    engine = RefEngine(tiny_ouro_model(), validate_model=False)
    tracing.update(on=(p == 0), step=0, layer=0)
    pre = engine.prefill(torch.from_numpy(prompts[p:p + 1]))
    if p == 0:
        trace_decode(engine)
    out[f"p{p}.prefill_logits"] = pre.logits.float().reshape(-1).numpy()
    out[f"p{p}.mask3"] = pre.state.mask_loop3.reshape(-1).numpy()
    out[f"p{p}.mask4"] = pre.state.mask_loop4.reshape(-1).numpy()
    logits = pre.logits.reshape(1, -1)
    tokens, step_logits, selected = [], [], []
    for step in range(DECODE_STEPS):
        tracing["step"] = step
        token = logits.argmax(-1, keepdim=True)
        tokens.append(int(token))
        dec = engine.decode(token.view(1, 1))
        logits = dec.logits.reshape(1, -1)
        step_logits.append(logits.float().reshape(-1).numpy())
        selected.append(dec.receipt.selected_keys_per_layer[0])
    out[f"p{p}.tokens"] = np.asarray(tokens, dtype=np.int64)
    out[f"p{p}.decode_logits"] = np.stack(step_logits)
    out[f"p{p}.selected"] = np.asarray(selected, dtype=np.int64)
    layer0 = engine.state.cache.layers[0]
    out[f"p{p}.final_quantized_tokens"] = np.asarray(layer0.quantized_tokens)
    out[f"p{p}.final_tail_tokens"] = np.asarray(layer0.tail_tokens)

# --- the reuse_selected_probabilities option (engine.py:401-408, 502-513): prompt 0, 24 steps ---
from flashloop.config import FlashLoopConfig as RefConfig  # noqa: E402

tracing.update(on=False)
engine = RefEngine(tiny_ouro_model(), validate_model=False, config=RefConfig(reuse_selected_probabilities=True))
logits = engine.prefill(torch.from_numpy(prompts[0:1])).logits.reshape(1, -1)
tokens, step_logits = [], []
for _ in range(24):
    token = logits.argmax(-1, keepdim=True)
    tokens.append(int(token))
    logits = engine.decode(token.view(1, 1)).logits.reshape(1, -1)
    step_logits.append(logits.float().reshape(-1).numpy())
out["reuse.tokens"] = np.asarray(tokens, dtype=np.int64)
out["reuse.decode_logits"] = np.stack(step_logits)

np.savez_compressed(HERE / "engine_vectors.npz", **out)
np.savez_compressed(HERE / "engine_trace.npz", **trace)
print("trace:", len(trace), "arrays,", (HERE / "engine_trace.npz").stat().st_size / 1e6, "MB")
print("wrote", len(out), "arrays,", (HERE / "engine_vectors.npz").stat().st_size / 1e3, "kB")
for p in range(2):
    print(p, "logit std", out[f"p{p}.decode_logits"].std(), "mask3", out[f"p{p}.mask3"].sum(),
          "mask4", out[f"p{p}.mask4"].sum(), out[f"p{p}.final_quantized_tokens"], out[f"p{p}.final_tail_tokens"])
