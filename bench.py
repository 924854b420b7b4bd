#!/usr/bin/env python3
"""Decode benchmark: tokens/s of the four-loop decoder over the int4 KV-residual cache.

Default workload (BASELINE configs[3], the configuration the metric is quoted on): the
Ouro-1.4B-shaped random-init bf16 model (24 layers x 4 loops, hidden 2048, 16 heads x 128,
SwiGLU 5632, vocab 49152) decoding through ``FlashLoopEngine`` at batch 16 per GPU after
2048-token random prompts: loops 1-2 dense, 25 % / 10 % token retention, 10 % key retention,
4-bit K/V in groups of 64 with a 64-token BF16 tail.  One step = one decoded token per sequence
(embed, 4 x 24 layers of norm / QKV / RoPE / reader / o_proj / MLP, append, lm_head).

``--workload hotpath`` is the reader-only step of BASELINE configs[1] (batch 8, context 8192,
the KV-attention kernels of 24 layers on synthetic vectors), ``ragged`` configs[2], ``kernels`` a
per-kernel table.  Every line carries ``roofline`` (the dominant kernel of the timed step) and
``roofline_dense`` / ``roofline_sparse``: the dense loop-2 reader and the loop-4 sparse reader at
the configs[1] shapes (batch 8 x 16 heads x 8192, 820 selected keys), the shapes the 70 %
HBM target is quoted on.

Prints ONE JSON line (rank 0).  ``--impl reference`` times the CPU port of the same step on the
host cores instead.
"""

from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import tempfile
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

HEADS, HEAD_DIM, CONTEXT, LAYERS, BATCH = 16, 128, 8192, 24, 8
KEY_FRACTION = 0.10
SCALING = HEAD_DIM ** -0.5
METRIC = "decode tok/s (Ouro-1.4B-shape R4)"
METRIC_HOTPATH = "decode tok/s of the KV-attention path alone (configs[1] reader step, no model)"
# Measured DRAM traffic of the readers: written by `python bench.py --update-traffic <ncu raw csv>`
# from an ncu capture of a small case, with the commit it was captured at.
TRAFFIC_FILE = ROOT / "profiles" / "reader_traffic.json"


def measured_traffic(kernel: str, algorithmic_bytes: float):
    """DRAM bytes per launch of ``kernel`` ("dense_reader" / "selected_reader"): the ncu capture's
    traffic-to-algorithmic ratio (every packed byte is read once, so traffic grows in proportion
    to the algorithmic bytes) times this launch's algorithmic bytes; (None, why) without a
    capture."""

    if not TRAFFIC_FILE.exists():
        return None, "no ncu capture recorded in profiles/reader_traffic.json"
    entry = json.loads(TRAFFIC_FILE.read_text()).get(kernel)
    if not entry:
        return None, f"no ncu capture of {kernel} recorded"
    ratio = entry["dram_bytes_per_launch"] / entry["algorithmic_bytes_per_launch"]
    return ratio * algorithmic_bytes, (f"ncu dram__bytes_read+write of the capture at commit {entry['commit']} "
                                       f"({entry['case']}): {ratio:.3f} x algorithmic, scaled to this launch")


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="e2e", choices=["hotpath", "ragged", "e2e", "e2e-2.6b", "kernels"],
                    help="e2e (default): configs[3], the Ouro-1.4B-shaped model decoding through the engine; "
                         "hotpath: configs[1], the KV-attention path of every layer on synthetic vectors; "
                         "ragged: configs[2], the same path over 32 sequences of 1024..32768 tokens (one layer); "
                         "kernels: every kernel of the path alone at the configs[1] shapes, with its bytes and fraction of peak; "
                         "e2e-2.6b: one GPU's share of configs[4] (48 layers, 8 of the 64 sequences, 8192-token prompts)")
    ap.add_argument("--layers", type=int, default=None, help="physical layers (default 24; 1 for ragged)")
    ap.add_argument("--batch", type=int, default=None, help="sequences per GPU (default 8 hotpath, 16 e2e)")
    ap.add_argument("--context", type=int, default=None, help="context / prompt length (default 8192 hotpath, 2048 e2e)")
    ap.add_argument("--bits", type=int, default=4)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--tp", action="store_true",
                    help="e2e workload: make the headline one model sharded by heads and FFN columns over the ranks "
                         "(strong scaling) instead of one replica per rank; without it an N>1 line still carries that "
                         "measurement as `tensor_parallel`")
    ap.add_argument("--tp-allreduce", default="peer", choices=["peer", "nccl"],
                    help="decode-step sum over the ranks: peer = this library's one-launch all-reduce + norm over "
                         "peer memory, replayed from a CUDA graph; nccl = NCCL all-reduces, launched eagerly")
    ap.add_argument("--no-tp-probe", action="store_true", help="N>1 replica runs: skip the tensor-parallel measurement")
    ap.add_argument("--no-graph", action="store_true", help="launch every step eagerly instead of replaying a CUDA graph")
    ap.add_argument("--no-probes", action="store_true",
                    help="skip the configs[1]-shaped reader probes behind roofline_dense / roofline_sparse")
    ap.add_argument("--update-traffic", metavar="CSV", nargs="+", default=None,
                    help="read `ncu -i <rep> --page raw --csv` exports of reader captures and record their DRAM "
                         "traffic in profiles/reader_traffic.json (no GPU needed)")
    args = ap.parse_args()
    args.config_index = 3
    if args.workload == "e2e-2.6b":
        args.workload, args.config_index = "e2e", 4
        args.layers = args.layers or 48
        args.batch = args.batch or 8
        args.context = args.context or 8192
    if args.batch is None:
        args.batch = {"hotpath": BATCH, "ragged": 32, "e2e": 16, "kernels": BATCH}[args.workload]
    if args.context is None:
        args.context = {"hotpath": CONTEXT, "ragged": 32768, "e2e": 2048, "kernels": CONTEXT}[args.workload]
    if args.layers is None:
        args.layers = 1 if args.workload == "ragged" else LAYERS
    return args


def workload_name(args) -> str:
    if args.workload == "e2e":
        which = ("configs[3] end-to-end Ouro-1.4B-shaped decoder" if args.config_index == 3 else
                 "configs[4] Ouro-2.6B-shaped decoder, one GPU's share of the batch of 64,")
        return (f"{which} (random-init bf16, {args.layers} layers x 4 loops, "
                f"hidden 2048, {HEADS} heads x {HEAD_DIM}, SwiGLU 5632, vocab 49152): batch {args.batch}/GPU, "
                f"{args.context}-token random prompts, greedy decode, loops 1-2 dense, 25%/10% token retention, "
                f"10% key retention, {args.bits}-bit K/V group 64")
    if args.workload == "ragged":
        return (f"configs[2] ragged batched decode: batch {args.batch}/GPU, context lengths uniform in "
                f"[1024, {args.context}] (seeded), {HEADS} heads x {HEAD_DIM}, 4 loops, {args.bits}-bit K/V group 64, "
                f"64-token BF16 tail, top-10% keys in loops 3-4, {args.layers} layer(s)")
    return (f"configs[1] sparse late-loop decode: batch {args.batch}/GPU, {HEADS} heads x {HEAD_DIM}, "
            f"context {args.context}, 4 loops, {args.bits}-bit K/V group 64, 64-token BF16 tail, "
            f"top-10% keys in loops 3-4, {args.layers} layers")


def bench_config(args) -> dict:
    """The ``config`` object of the JSON line; both arms print the same one for the same flags."""

    world = max(1, int(args.gpus))
    tp = bool(getattr(args, "tp", False)) and world > 1
    if args.workload == "e2e":
        l2 = "inputs larger than L2: each step streams the layer weights four times and the packed cache"
        parallelism = (f"tensor parallel x{world}: heads and FFN columns sharded, all-reduce after o_proj and the MLP"
                       if tp else f"batch-data-parallel replicas x{world}, no data-path collective")
    else:
        l2 = "inputs larger than L2: each step streams the packed cache of every layer"
        parallelism = f"batch-sharded x{world}, no data-path collective"
    return {"workload": workload_name(args), "global_batch": args.batch if tp else args.batch * world, "l2": l2,
            "parallelism": parallelism,
            "launch": ("eager" if args.no_graph or (tp and getattr(args, "tp_allreduce", "peer") == "nccl")
                       else "one CUDA graph replay per step")}


# ----------------------------------------------------------------------------- algorithmic bytes


def stream_bytes_per_token(bits: int) -> int:
    """K codes + V codes + K metadata (512 B per 64 tokens) + V metadata (8 B) per token."""
    return 2 * 16 * bits + 8 + 8


def dense_bytes(batch_heads: int, loop: int, quant: int, tail: int, bits: int) -> int:
    """Dense reader, loop index 0..3: streams 0..loop of the packed prefix, K+V tail rows,
    query / current K / current V (bf16) and the float32 output."""
    return batch_heads * ((loop + 1) * stream_bytes_per_token(bits) * quant + tail * 512 + 1280)


def sparse_bytes(batch_heads: int, loop: int, keys: int, quant: int, bits: int) -> int:
    """Gathered reader: selected rows of every stream (codes + V metadata), the K metadata of
    every group, 13 B of index / validity / rank lookups per key, vectors in and out."""
    per_stream = keys * (2 * 16 * bits + 8) + 512 * (quant // 64)
    return batch_heads * ((loop + 1) * per_stream + keys * 13 + 1280)


# ----------------------------------------------------------------------------- clocks


class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.path = tempfile.NamedTemporaryFile(prefix="fl_clocks_", suffix=".csv", delete=False).name
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in Path(self.path).read_text().splitlines():
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, value in zip(names, parts[3:7]):
                if value.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.path)
        if sm:
            out.update(sm_mhz=statistics.median(sm), sm_max_mhz=max(mx), reasons=sorted(reasons), samples=len(sm))
        return out


# ----------------------------------------------------------------------------- reader probes


def load_peak():
    peaks_path = ROOT / "MEASURED_PEAKS.json"
    peaks = json.loads(peaks_path.read_text()) if peaks_path.exists() else {}
    peak = float(peaks.get("hbm_gbs", 6650.0))
    return peak, ("measured (MEASURED_PEAKS.json hbm_gbs)" if peaks else "fallback 6650 GB/s")


def roofline_object(kernel: str, traffic_key: str, algorithmic_bytes: float, launch_ms: list, peak: float,
                    peak_kind: str, timing: str) -> dict:
    avg_ms = statistics.mean(launch_ms) if launch_ms else float("nan")
    achieved = algorithmic_bytes / (avg_ms * 1e-3) / 1e9
    traffic, source = measured_traffic(traffic_key, algorithmic_bytes)
    return {"bound": "hbm", "kernel": kernel, "achieved": achieved, "peak": peak, "unit": "GB/s",
            "frac": achieved / peak, "frac_of_nominal_8000": achieved / 8000.0, "peak_source": peak_kind,
            "algorithmic_bytes_per_launch": algorithmic_bytes, "avg_launch_ms": avg_ms,
            "launches_timed": len(launch_ms), "timing": timing, "traffic": traffic, "traffic_source": source}


def probe_configs1_readers(device, bits: int, layers_n: int = 4) -> dict:
    """The two readers at the shapes the HBM target is quoted on (BASELINE configs[1]: batch 8,
    16 heads x 128, context 8192, residuals on every token, 820 selected keys): the dense loop-2
    reader and the loop-4 cached-mass sparse reader, each timed with CUDA events around a graph of
    twelve launches that cycle over ``layers_n`` layers, so that no launch finds its input in L2.
    Returns {"roofline_dense": ..., "roofline_sparse": ...}."""

    import torch

    from flashloop_b200.cache import CrossLoopKVLayer
    from flashloop_b200.synthetic import make_loop_kv

    B, H, T = BATCH, HEADS, CONTEXT
    peak, peak_kind = load_peak()
    ones = torch.ones(B, T, dtype=torch.bool, device=device)
    layers = []
    for li in range(layers_n):
        keys, values = [[] for _ in range(4)], [[] for _ in range(4)]
        for b in range(B):
            k, v = make_loop_kv(H, T, seed=7000 + li * 100 + b, device=device)
            for r in range(4):
                keys[r].append(k[r])
                values[r].append(v[r])
        layers.append(CrossLoopKVLayer.from_prefill([torch.cat(k) for k in keys], [torch.cat(v) for v in values],
                                                    mask_loop3=ones, mask_loop4=ones, bits=bits))
        del keys, values
    quant, tail = layers[0].quantized_tokens, layers[0].tail_tokens
    gen = torch.Generator(device=device).manual_seed(1)
    q, ck, cv = (torch.randn(B, H, 1, HEAD_DIM, generator=gen, device=device).to(torch.bfloat16) for _ in range(3))
    out = torch.empty(B, H, 1, HEAD_DIM, device=device)
    logits = [layer.dense_source_attention(1, query=q, current_key=ck, current_value=cv, scaling=SCALING,
                                           return_logits=True)[1].clone() for layer in layers]
    sels = [layer.select_decode_keys(lg, fraction=KEY_FRACTION) for layer, lg in zip(layers, logits)]
    srcs = [layer.pv(1, sel.selected_weights, sel.indices, current_value=cv, valid=sel.valid, validate_indices=False)
            for layer, sel in zip(layers, sels)]
    keys_n = math.ceil((quant + tail + 1) * KEY_FRACTION)

    def timeit(fn, reps: int = 12, rounds: int = 5) -> list:
        for i in range(layers_n):
            fn(i)
        torch.cuda.synchronize(device)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for i in range(reps):
                fn(i)
        graph.replay()
        torch.cuda.synchronize(device)
        ms = []
        for _ in range(rounds):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            graph.replay()
            e1.record()
            torch.cuda.synchronize(device)
            ms.append(e0.elapsed_time(e1) / reps)
        return ms

    lg_out = torch.empty_like(logits[0])
    dense_ms = timeit(lambda i: layers[i % layers_n].dense_source_attention(
        1, query=q, current_key=ck, current_value=cv, scaling=SCALING, return_logits=True, out=out, logits_out=lg_out))
    sparse_ms = timeit(lambda i: layers[i % layers_n].cached_mass_sparse_attention_delta(
        3, query=q, current_key=ck, current_value=cv, indices=sels[i % layers_n].indices,
        valid=sels[i % layers_n].valid, source_selected_output=srcs[i % layers_n],
        global_mass=sels[i % layers_n].global_mass, scaling=SCALING, out=out))
    status = max(layer.reader_status() for layer in layers)
    timing = (f"CUDA events around a graph of 12 launches cycling over {layers_n} layers of batch {B} x {H} heads x "
              f"context {T} (inputs larger than L2), 5 replays")
    return {
        "roofline_dense": roofline_object(
            f"dense_reader_kernel<{bits},1> (loop 2: anchor + delta-2 streams) at configs[1] shapes", "dense_reader",
            dense_bytes(B * H, 1, quant, tail, bits), dense_ms, peak, peak_kind, timing),
        "roofline_sparse": roofline_object(
            f"selected_reader_kernel<{bits},delta,4> (loop 4: cached-mass sparse reader, {keys_n} keys of {quant + tail + 1}) "
            "at configs[1] shapes", "selected_reader", sparse_bytes(B * H, 3, keys_n, quant, bits), sparse_ms, peak,
            peak_kind, timing),
        "probe_reader_status": status,
    }


def probe_projection(model, rows: int, device) -> dict:
    """The largest launch group of the end-to-end step by time: the fused gate/up projection with
    SwiGLU (``fl_linear_rows``), timed with CUDA events around a graph that walks the layers' own
    weights (24 x 46 MB, so no launch finds its weights in L2).  Algorithmic bytes = the weight, once.
    Returns {"roofline_projection": ...} or {} when the step does not use the kernel at this batch."""

    import torch

    from flashloop_b200 import step_ops

    weights = [layer.mlp._flashloop_gate_up_weight for layer in model.model.layers
               if hasattr(layer.mlp, "_flashloop_gate_up_weight")]
    if not weights:
        return {}
    x = torch.randn(rows, 1, weights[0].shape[1], device=device).to(torch.bfloat16)
    if not step_ops.linear_fits(x, weights[0]):
        return {}
    for w in weights:
        step_ops.linear(x, w, swiglu=True)
    torch.cuda.synchronize(device)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for w in weights:
            step_ops.linear(x, w, swiglu=True)
    graph.replay()
    torch.cuda.synchronize(device)
    ms = []
    for _ in range(5):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        graph.replay()
        e1.record()
        torch.cuda.synchronize(device)
        ms.append(e0.elapsed_time(e1) / len(weights))
    peak, peak_kind = load_peak()
    out_f, in_f = (int(v) for v in weights[0].shape)
    obj = roofline_object(
        f"linear_ring_kernel<2,1> (gate/up projection + SwiGLU, {rows} rows x [{out_f} x {in_f}] bfloat16 weight), the "
        "largest launch group of the step by time", "projection", float(weights[0].numel() * 2), ms, peak, peak_kind,
        f"CUDA events around a graph of {len(weights)} launches over the layers' own weights, 5 replays")
    return {"roofline_projection": obj}


# ----------------------------------------------------------------------------- the CPU oracle leg


def _oracle_head_step(seed: int, context: int, bits: int) -> float:
    """One head of one sequence of one layer through the oracle's decode step; returns seconds.
    (The only place outside tests/ where the oracle runs: it is the CPU baseline.)"""

    import numpy as np

    from flashloop_b200.synthetic import make_loop_kv, make_query
    from oracle import selection as osel
    from oracle.cache import LayerOracle

    keys, values = make_loop_kv(1, context, seed=seed)
    import torch

    torch.set_num_threads(1)
    to_np = lambda t: t.float().numpy()
    ones = np.ones(context, bool)
    layer = LayerOracle.from_prefill([to_np(k) for k in keys], [to_np(v) for v in values],
                                     mask_loop3=ones, mask_loop4=ones, bits=bits)
    q, ck, cv = (to_np(t) for t in make_query(1, seed=seed))
    start = time.perf_counter()
    layer.dense_source_attention(0, query=q, current_key=ck, current_value=cv, scaling=SCALING)
    _, logits = layer.dense_source_attention(1, query=q, current_key=ck, current_value=cv, scaling=SCALING)
    sel = osel.select_from_logits(logits, fraction=KEY_FRACTION)
    src = layer.selected_value_aggregate(1, selected_indices=sel["indices"], selected_weights=sel["selected_weights"],
                                         current_value=cv, past_tokens=context)
    for loop in (2, 3):
        layer.cached_mass_sparse_attention_delta(
            loop, query=q, current_key=ck, current_value=cv, current_position=context, indices=sel["indices"],
            valid=sel["valid"], source_selected_output=src, global_mass=sel["global_mass"], scaling=SCALING)
    layer.append_decode_token([ck] * 4, [cv] * 4)
    return time.perf_counter() - start


def cpu_pool():
    """One worker process per host core (at most 32).  spawn, not fork: the parent may hold a CUDA
    context and OpenMP threads."""

    import multiprocessing
    from concurrent.futures import ProcessPoolExecutor

    cores = min(os.cpu_count() or 1, 32)
    return ProcessPoolExecutor(max_workers=cores, mp_context=multiprocessing.get_context("spawn")), cores


def cpu_oracle_tokens_per_second(args, tasks_per_core: int = 3, pool=None) -> dict:
    """Time the oracle on every host core at once (one head-step task per core per round) and
    scale to whole decode tokens: one token = HEADS heads x layers."""

    own = pool is None
    if own:
        pool = cpu_pool()
    executor, cores = pool
    tasks = cores * tasks_per_core
    start = time.perf_counter()
    try:
        seconds = list(executor.map(_oracle_head_step, range(tasks), [args.context] * tasks, [args.bits] * tasks))
    finally:
        if own:
            executor.shutdown()
    wall = time.perf_counter() - start
    # all workers run at once: aggregate rate = workers / mean seconds per head-step
    head_steps_per_s = cores / (sum(seconds) / len(seconds))
    return {
        "value": head_steps_per_s / (HEADS * args.layers),
        "unit": "tok/s",
        "cores": cores,
        "kind": "port",
        "sample": (f"{tasks} head-steps (1 sequence x 1 head x 1 layer each, context {args.context}) on {cores} "
                   f"processes, mean {sum(seconds) / len(seconds):.2f} s per head-step (cache build excluded, "
                   f"{wall:.1f} s wall with it), scaled by {HEADS} heads x {args.layers} layers per token"),
    }


def run_reference_kernels(args) -> None:
    """``--impl reference --workload kernels``: the reference's own CUDA readers (its extension
    ``flashloop_kivi_gemv``, built unmodified from the reference checkout by oracle/build_ref.py into
    oracle/_ref/) on this GPU, at the shapes of the kernel table: the dense reader of loops 1 and 2
    and the cached-mass sparse reader of loops 3 and 4, called with the tensors the reference's
    ``kivi_backend`` hands them.  One JSON line with a row per kernel; the algorithmic bytes are
    those of this library's table, so the fractions compare like with like."""

    import torch

    if int(os.environ.get("RANK", "0")) != 0:
        return
    module_dir = ROOT / "oracle" / "_ref"
    if not (module_dir / "flashloop_kivi_gemv.so").exists():
        print(json.dumps({"impl": "reference", "workload": "kernels",
                          "unavailable": "oracle/_ref/flashloop_kivi_gemv.so is not built (python oracle/build_ref.py)"}))
        return
    sys.path.insert(0, str(module_dir))
    import flashloop_kivi_gemv as reference_extension

    from flashloop_b200 import kivi_backend as kb
    from flashloop_b200.synthetic import make_loop_kv

    device = torch.device("cuda", 0)
    B, H, T = args.batch, HEADS, args.context
    quant = ((T - 64) // 64) * 64
    tail = T - quant
    keys, values = [[] for _ in range(4)], [[] for _ in range(4)]
    for b in range(B):
        k, v = make_loop_kv(H, T, seed=7000 + b, device=device)
        for r in range(4):
            keys[r].append(k[r])
            values[r].append(v[r])
    keys = [torch.cat(k) for k in keys]
    values = [torch.cat(v) for v in values]
    # the residual chain of the reference's cache builder (flashloop/cache.py:415-439): every stream
    # packs what the streams before it leave of that loop's tensor
    k_streams, v_streams = [], []
    base_k = base_v = None
    for r in range(4):
        dk = keys[r][:, :, :quant] if base_k is None else keys[r][:, :, :quant] - base_k
        dv = values[r][:, :, :quant] if base_v is None else values[r][:, :, :quant] - base_v
        k_streams.append(kb.pack_kivi_k_per_channel(dk.contiguous()))
        v_streams.append(kb.pack_kivi_v_per_token(dv.contiguous()))
        base_k = k_streams[-1].decode() if base_k is None else base_k + k_streams[-1].decode()
        base_v = v_streams[-1].decode() if base_v is None else base_v + v_streams[-1].decode()
    del base_k, base_v
    tails_k = [k[:, :, quant:].contiguous() for k in keys]
    tails_v = [v[:, :, quant:].contiguous() for v in values]
    del keys, values
    identity = torch.arange(quant, dtype=torch.int32, device=device)
    gen = torch.Generator(device=device).manual_seed(1)
    q, ck, cv = (torch.randn(B, H, 1, HEAD_DIM, generator=gen, device=device).to(torch.bfloat16) for _ in range(3))

    class Recorder:
        """Stands in for the extension: runs it and keeps the arguments of the call."""

        def __init__(self):
            self.calls = {}

        def __getattr__(self, name):
            def call(*a):
                self.calls[name] = a
                return getattr(reference_extension, name)(*a)
            return call

    recorder = Recorder()
    rows = []
    peak, peak_kind = load_peak()

    def timed(name: str, call_args, reps: int = 5) -> float:
        fn = getattr(reference_extension, name)
        fn(*call_args)
        torch.cuda.synchronize(device)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn(*call_args)
        e1.record()
        torch.cuda.synchronize(device)
        return e0.elapsed_time(e1) / reps * 1e3

    logits = None
    for loop in (0, 1):
        _, lg = kb.kivi_fused_dense_source_attention(
            query=q, current_key=ck, current_value=cv, key_streams=k_streams, value_streams=v_streams,
            rank_maps=(identity, identity), tail_key=tails_k[loop], tail_value=tails_v[loop], scaling=SCALING,
            loop=loop, extension=recorder, return_logits=True)
        logits = lg
        us = timed("dense_source_attention_cuda", recorder.calls["dense_source_attention_cuda"])
        mb = dense_bytes(B * H, loop, quant, tail, 4) / 1e6
        rows.append({"kernel": f"reference dense_source_attention_cuda, loop {loop + 1} (3 launches)", "us": us,
                     "algorithmic_MB": mb, "GBps": mb / us * 1e3, "frac_of_peak": mb / us * 1e3 / peak})
    # the selection of flashloop/engine.py:438-498 in tensor ops: top 10 % of the loop-2 softmax, ascending
    weights = torch.softmax(logits.float(), dim=-1)[:, :, 0]
    total = weights.shape[-1]
    budget = min(total, max(1, math.ceil(total * KEY_FRACTION)))
    top = torch.topk(weights, budget, dim=-1)
    indices = torch.sort(top.indices, dim=-1).values
    mass = top.values.sum(-1)
    capacity = (budget // 64 + 1) * 64
    padded = torch.zeros(B, H, capacity, dtype=torch.int32, device=device)
    padded[..., :budget] = indices.to(torch.int32)
    valid = torch.zeros(B, H, capacity, dtype=torch.bool, device=device)
    valid[..., :budget] = True
    source = torch.zeros(B, H, 1, HEAD_DIM, device=device)
    for loop in (2, 3):
        kb.kivi_fused_sparse_attention_delta(
            query=q, current_key=ck, current_value=cv, key_streams=k_streams, value_streams=v_streams,
            rank_maps=(identity, identity), tail_key=tails_k[loop], tail_value=tails_v[loop], indices=padded,
            valid=valid, source_selected_output=source, global_mass=mass.view(B, H, 1, 1), current_position=quant + tail,
            scaling=SCALING, loop=loop, extension=recorder)
        us = timed("sparse_attention_delta_cuda", recorder.calls["sparse_attention_delta_cuda"])
        mb = sparse_bytes(B * H, loop, budget, quant, 4) / 1e6
        rows.append({"kernel": f"reference sparse_attention_delta_cuda, loop {loop + 1}, {budget} keys (3 launches)",
                     "us": us, "algorithmic_MB": mb, "GBps": mb / us * 1e3, "frac_of_peak": mb / us * 1e3 / peak})
    print(json.dumps({
        "impl": "reference", "metric": "kernel table: the reference's CUDA readers on this GPU", "unit": "GB/s",
        "n_gpus": 1, "peak_GBps": peak, "peak_source": peak_kind,
        "config": {"workload": f"the reference extension's readers alone at batch {B}, {H} heads x {HEAD_DIM}, context {T}, "
                               "4-bit KIVI words, all-token residuals; CUDA events around five eager calls of each "
                               "entry point (its output and scratch allocations included, as its callers pay them)"},
        "kind": "reference-cuda", "rows": rows}))


def run_reference(args) -> None:
    """The CPU arm: the port of the reference's path on the host cores.  One step is one bounded
    sample of the workload (one head-step of the KV-attention path per core, plus, for the
    end-to-end workload, the projections and MLP of two layers in float32 Torch); ``warmup``
    samples are discarded, ``steps`` samples are timed.  ``steps`` and ``ms_per_step`` describe
    the samples that really ran; ``value`` extrapolates them to whole decode steps (the line says
    so: "extrapolated")."""

    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    e2e = args.workload == "e2e"
    measure = cpu_e2e_tokens_per_second if e2e else cpu_oracle_tokens_per_second
    pool = cpu_pool()
    for _ in range(args.warmup):
        measure(args, tasks_per_core=1, pool=pool)
    results, walls = [], []
    for _ in range(args.steps):
        t0 = time.perf_counter()
        results.append(measure(args, tasks_per_core=1, pool=pool))
        walls.append(time.perf_counter() - t0)
    pool[0].shutdown()
    value = statistics.mean(r["value"] for r in results)
    best = dict(results[0])
    best["value"] = value
    best["sample"] = f"{args.steps} timed samples after {args.warmup} warm-up samples, each: " + results[0]["sample"]
    line = {
        "impl": "reference", "metric": METRIC if e2e else METRIC_HOTPATH, "value": value, "unit": "tok/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * statistics.mean(walls), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic", "extrapolated": True,
        "ms_per_full_step_extrapolated": 1e3 / value,
        "config": bench_config(args), "cpu_baseline": best,
        "e2e": {"value": value, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ----------------------------------------------------------------------------- the GPU leg


def run_b200(args) -> None:
    import torch
    import torch.distributed as dist

    from flashloop_b200 import _native, sharding
    from flashloop_b200.cache import CrossLoopKVLayer
    from flashloop_b200.synthetic import make_loop_kv

    _native.load()  # fail loudly when the CUDA library is missing
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)

    B, H, T, NL = args.batch, HEADS, args.context, args.layers
    steps_total = args.warmup + args.steps
    # ---- build the cache: NL layers, B sequences (seed distinct per rank / sequence / layer)
    layers = []
    if args.workload == "ragged":
        lengths = torch.randint(1024, T + 1, (B,), generator=torch.Generator().manual_seed(rank)).tolist()
    else:
        lengths = [T] * B
    for layer_index in range(NL):
        sequences = []
        for b in range(B):
            k, v = make_loop_kv(H, lengths[b], seed=sharding.sequence_seed(rank, layer_index, b), device=device)
            ones = torch.ones(lengths[b], dtype=torch.bool, device=device)
            sequences.append((k, v, ones, ones))
        layers.append(CrossLoopKVLayer.from_prefill_ragged(sequences, bits=args.bits,
                                                           max_new_tokens=2 * steps_total + 192))
        del sequences
    quants = [layers[0].quantized_tokens_of(b) for b in range(B)]
    tails = [layers[0].tail_tokens_of(b) for b in range(B)]

    # ---- per-step inputs: query / current K / current V of every (layer, loop), bf16
    gen = torch.Generator(device="cpu").manual_seed(1234 + rank)
    host_inputs = torch.randn((3, NL, 4, B, H, 1, HEAD_DIM), generator=gen).to(torch.bfloat16).pin_memory()
    dev_inputs = host_inputs.to(device)
    out = torch.empty((NL, 4, B, H, 1, HEAD_DIM), dtype=torch.float32, device=device)
    host_out = torch.empty(out.shape, dtype=torch.float32).pin_memory()
    probe = []  # CUDA event pairs around the dominant kernel (dense reader, loop 2)

    bound = max(lengths) + steps_total + 64
    for layer in layers:
        layer.context_bound = bound  # fixed launch geometry: the step can be replayed as a CUDA graph

    def step(inputs, advance_host: bool = True) -> None:
        q_all, k_all, v_all = inputs[0], inputs[1], inputs[2]
        for li, layer in enumerate(layers):
            q, k, v = q_all[li], k_all[li], v_all[li]
            layer.dense_source_attention(0, query=q[0], current_key=k[0], current_value=v[0], scaling=SCALING,
                                         return_logits=False, out=out[li, 0])
            _, logits = layer.dense_source_attention(1, query=q[1], current_key=k[1], current_value=v[1],
                                                     scaling=SCALING, return_logits=True, out=out[li, 1])
            sel = layer.select_decode_keys(logits, fraction=KEY_FRACTION)
            src = layer.pv(1, sel.selected_weights, sel.indices, current_value=v[1], valid=sel.valid,
                           validate_indices=False)
            for loop in (2, 3):
                layer.cached_mass_sparse_attention_delta(
                    loop, query=q[loop], current_key=k[loop], current_value=v[loop], indices=sel.indices,
                    valid=sel.valid, source_selected_output=src, global_mass=sel.global_mass, scaling=SCALING,
                    out=out[li, loop])
            layer.append_decode_token([k[r] for r in range(4)], [v[r] for r in range(4)])

    def barrier():
        sharding.barrier(device)

    def timed(fn, count: int) -> float:
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(count):
            fn()
        e1.record()
        barrier()
        return sharding.max_over_ranks(e0.elapsed_time(e1), device)

    # ---- warm-up (eager; the launches of one step are counted), then record one step as a CUDA
    # graph over static input buffers
    for i in range(max(1, args.warmup)):
        if i == 0:
            _native.count_launches(True)
        step(dev_inputs)
        if i == 0:
            launch_counts = _native.count_launches(False)
    launches_per_step = sum(launch_counts.values())
    graph = None
    if not args.no_graph:
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            step(dev_inputs)  # recorded, not run: the host mirror advanced, the device did not
        # undo nothing: replaying once now brings the device in line with the host mirror
        graph.replay()
        torch.cuda.synchronize()

    def run_step():
        if graph is None:
            step(dev_inputs)
        else:
            graph.replay()
            for layer in layers:
                layer.advance_host_state()

    # ---- device-resident leg
    sampler = ClockSampler(local) if rank == 0 else None
    torch.cuda.profiler.start()  # lets `ncu --profile-from-start off` see the timed region only
    ms_total = timed(run_step, args.steps)
    torch.cuda.profiler.stop()
    clocks = sampler.stop() if sampler else {}
    timed_launches = launches_per_step * args.steps
    # every rank decodes its own B sequences: tokens of all ranks over the slowest rank's time
    value = sharding.sum_over_ranks(B * args.steps, device) / (ms_total * 1e-3)

    # ---- the dominant kernel alone: the loop-2 dense reader of every layer, same arguments as in
    # the step, timed with CUDA events on the launching stream right after the timed region
    # (events cannot be recorded inside a replayed graph)
    probe_ms = []
    q1, k1, v1 = dev_inputs[0][:, 1], dev_inputs[1][:, 1], dev_inputs[2][:, 1]
    for rep in range(3):
        for li, layer in enumerate(layers):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            layer.dense_source_attention(1, query=q1[li], current_key=k1[li], current_value=v1[li],
                                         scaling=SCALING, return_logits=True, out=out[li, 1])
            e1.record()
            if rep:
                probe.append((e0, e1))
    torch.cuda.synchronize()
    probe_ms = [a.elapsed_time(b) for a, b in probe]

    # ---- end-to-end leg: the same step through the public API with HOST buffers
    def e2e_step():
        dev_inputs.copy_(host_inputs, non_blocking=True)
        run_step()
        host_out.copy_(out, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    e2e_steps = max(2, min(args.steps, 16))
    e2e_step()
    e2e_ms = timed(e2e_step, e2e_steps)
    e2e_value = sharding.sum_over_ranks(B * e2e_steps, device) / (e2e_ms * 1e-3)
    status = max(layer.reader_status() for layer in layers)

    # ---- the loop-4 sparse reader of every layer, same arguments as in the step
    sparse_probe = []
    q3, k3, v3 = dev_inputs[0][:, 3], dev_inputs[1][:, 3], dev_inputs[2][:, 3]
    for rep in range(3):
        for li, layer in enumerate(layers):
            _, lg = layer.dense_source_attention(1, query=q1[li], current_key=k1[li], current_value=v1[li],
                                                 scaling=SCALING, return_logits=True, out=out[li, 1])
            sel = layer.select_decode_keys(lg, fraction=KEY_FRACTION)
            src = layer.pv(1, sel.selected_weights, sel.indices, current_value=v1[li], valid=sel.valid,
                           validate_indices=False)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            layer.cached_mass_sparse_attention_delta(3, query=q3[li], current_key=k3[li], current_value=v3[li],
                                                     indices=sel.indices, valid=sel.valid, source_selected_output=src,
                                                     global_mass=sel.global_mass, scaling=SCALING, out=out[li, 3])
            e1.record()
            if rep:
                sparse_probe.append((e0, e1))
    torch.cuda.synchronize()
    sparse_ms = [a.elapsed_time(b) for a, b in sparse_probe]
    status = max(status, max(layer.reader_status() for layer in layers))

    if rank == 0:
        peak, peak_kind = load_peak()
        algo = sum(dense_bytes(H, 1, q_, t_, args.bits) for q_, t_ in zip(quants, tails))
        sparse_algo = sum(sparse_bytes(H, 3, math.ceil((q_ + t_ + 1) * KEY_FRACTION), q_, args.bits)
                          for q_, t_ in zip(quants, tails))
        step_bytes = 0
        for q_, t_ in zip(quants, tails):
            keys = math.ceil((q_ + t_ + 1) * KEY_FRACTION)
            step_bytes += NL * (dense_bytes(H, 0, q_, t_, args.bits) + dense_bytes(H, 1, q_, t_, args.bits)
                                + sparse_bytes(H, 1, keys, q_, args.bits) - H * 1280  # selected PV, loop 2
                                + sparse_bytes(H, 2, keys, q_, args.bits) + sparse_bytes(H, 3, keys, q_, args.bits))
        in_step = "CUDA events around single launches with the step's own arguments, right after the timed region"
        line = {
            "metric": METRIC_HOTPATH, "value": value, "unit": "tok/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_total / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": bench_config(args),
            "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": "tok/s", "h2d_bytes_per_step": int(host_inputs.numel() * 2),
                    "d2h_bytes_per_step": int(host_out.numel() * 4), "steps": e2e_steps},
            "gpu_launches": timed_launches,
            "gpu_launches_source": f"{launches_per_step} launches of this library's kernels counted in one step "
                                   f"({launch_counts}) x {args.steps} timed steps",
            "roofline": roofline_object(f"dense_reader_kernel<{args.bits},1> (loop 2: anchor + delta-2 streams)",
                                        "dense_reader", algo, probe_ms, peak, peak_kind, in_step),
            "roofline_sparse": roofline_object(
                f"selected_reader_kernel<{args.bits},delta,4> (loop 4: cached-mass sparse reader)", "selected_reader",
                sparse_algo, sparse_ms, peak, peak_kind, in_step),
            "step_algorithmic_GBps": step_bytes / (ms_total / args.steps * 1e-3) / 1e9,
            "reader_status": status,
        }
        # codes are dequantised and multiplied in float16 pairs, accumulated in float32
        if not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_oracle_tokens_per_second(args)
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


# ----------------------------------------------------------------------------- per-kernel table


def run_kernel_table(args) -> None:
    """Every kernel of the path timed alone (CUDA events around a graph of back-to-back launches
    over six different layers, so that no launch finds its input in L2), with its algorithmic
    bytes and the fraction of the measured copy bandwidth.  One JSON line."""

    import torch

    from flashloop_b200 import _native
    from flashloop_b200.cache import CrossLoopKVLayer
    from flashloop_b200.compaction import gather_rows, hidden_delta_score, retain_tokens, scatter_rows
    from flashloop_b200.kivi_backend import kivi_to_rows, pack_kivi_k_per_channel, pack_kivi_v_per_token
    from flashloop_b200.packing import pack_k_per_channel, pack_v_per_token
    from flashloop_b200.synthetic import make_loop_kv

    _native.load()
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    B, H, T, bits, NL = args.batch, HEADS, args.context, args.bits, 6
    peaks_path = ROOT / "MEASURED_PEAKS.json"
    peaks = json.loads(peaks_path.read_text()) if peaks_path.exists() else {}
    peak = float(peaks.get("hbm_gbs", 6650.0))
    rows = []

    def timeit(fn, reps: int = 12) -> float:
        for i in range(3):
            fn(i)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for i in range(reps):
                fn(i)
        graph.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(3):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / (3 * reps) * 1e3

    def add(name: str, us: float, nbytes: float, note: str = "") -> None:
        gbs = nbytes / us / 1e3
        rows.append({"kernel": name, "us": round(us, 1), "algorithmic_MB": round(nbytes / 1e6, 1),
                     "GBps": round(gbs), "frac_of_peak": round(gbs / peak, 3), "note": note})

    # ---- inputs: NL layers of B sequences
    ones = torch.ones(B, T, dtype=torch.bool, device=device)
    kv = []
    for layer_index in range(NL):
        keys, values = [[] for _ in range(4)], [[] for _ in range(4)]
        for b in range(B):
            k, v = make_loop_kv(H, T, seed=layer_index * 100 + b, device=device)
            for r in range(4):
                keys[r].append(k[r])
                values[r].append(v[r])
        kv.append(([torch.cat(k) for k in keys], [torch.cat(v) for v in values]))
    elems = B * H * T * HEAD_DIM
    # ---- codecs (per launch: one [B,H,T,128] bf16 tensor in, packed codes + metadata out)
    code_bytes = elems * bits / 8
    add("pack_k rows (fl_pack_k_rows)", timeit(lambda i: pack_k_per_channel(kv[i % NL][0][0], bits=bits)),
        2 * elems + code_bytes + elems / 64 * 4)
    add("pack_v rows (fl_pack_v_rows)", timeit(lambda i: pack_v_per_token(kv[i % NL][1][0], bits=bits)),
        2 * elems + code_bytes + elems / 64 * 4)
    if bits == 4:
        add("pack_k KIVI words (fl_pack_kivi_k)", timeit(lambda i: pack_kivi_k_per_channel(kv[i % NL][0][0])),
            2 * elems + code_bytes + elems / 64 * 4)
        add("pack_v KIVI words (fl_pack_kivi_v)", timeit(lambda i: pack_kivi_v_per_token(kv[i % NL][1][0])),
            2 * elems + code_bytes + elems / 64 * 4)
        packed = [pack_kivi_k_per_channel(kv[i][0][0]) for i in range(NL)]
        add("KIVI words -> rows, K (fl_kivi_to_rows_k)", timeit(lambda i: kivi_to_rows(packed[i % NL])), 2 * code_bytes)
        del packed
    # ---- prefill encoder: four loops of K and V in, all streams out
    def build(i):
        return CrossLoopKVLayer.from_prefill(kv[i % NL][0], kv[i % NL][1], mask_loop3=ones, mask_loop4=ones, bits=bits,
                                             max_new_tokens=256)
    layers = [build(i) for i in range(NL)]  # also the warm-up of the encoder
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    rebuilt = [build(i) for i in range(NL)]
    torch.cuda.synchronize()
    add("prefill residual encoder, all-token masks (fl_encode_prefill + rank maps + tails)",
        (time.perf_counter() - t0) / NL * 1e6, 8 * 2 * elems + 4 * 2 * (code_bytes + elems / 64 * 4),
        "wall clock per layer: three encoder launches, two retention launches, tail copies and the Python around them")
    del rebuilt
    quant, tail = layers[0].quantized_tokens, layers[0].tail_tokens
    for layer in layers:
        layer.context_bound = T + 256
    bh = B * H
    gen = torch.Generator(device=device).manual_seed(1)
    q, ck, cv = (torch.randn(B, H, 1, HEAD_DIM, generator=gen, device=device).to(torch.bfloat16) for _ in range(3))
    out = torch.empty(B, H, 1, HEAD_DIM, device=device)
    for loop in range(4):
        us = timeit(lambda i: layers[i % NL].dense_source_attention(loop, query=q, current_key=ck, current_value=cv,
                                                                   scaling=SCALING, return_logits=loop == 1, out=out))
        add(f"dense reader loop {loop + 1} (fl_dense_source_attention)", us, dense_bytes(bh, loop, quant, tail, bits))
    _, logits = layers[0].dense_source_attention(1, query=q, current_key=ck, current_value=cv, scaling=SCALING,
                                                 return_logits=True)
    keys_n = math.ceil((T + 1) * KEY_FRACTION)
    add("decode key selection (fl_select_decode_keys)",
        timeit(lambda i: layers[0].select_decode_keys(logits, fraction=KEY_FRACTION)), bh * (4 * (T + 1) + 6 * keys_n),
        "latency bound: one CTA per head")
    sel = layers[0].select_decode_keys(logits, fraction=KEY_FRACTION)
    pv_bytes = bh * (2 * keys_n * (16 * bits + 8) + keys_n * 13 + 1280)
    add("selected value aggregate, loop 2 (fl_selected_pv)",
        timeit(lambda i: layers[i % NL].pv(1, sel.selected_weights, sel.indices, current_value=cv, valid=sel.valid,
                                           validate_indices=False, out=out)), pv_bytes)
    add("selected logits, loop 2 (fl_selected_qk)",
        timeit(lambda i: layers[i % NL].qk(1, q, sel.indices, validate_indices=False, current_key=ck)),
        bh * (2 * (keys_n * 16 * bits + 512 * (quant // 64)) + keys_n * 8 + 512))
    src = layers[0].pv(1, sel.selected_weights, sel.indices, current_value=cv, valid=sel.valid, validate_indices=False)
    for loop in (2, 3):
        us = timeit(lambda i: layers[i % NL].cached_mass_sparse_attention_delta(
            loop, query=q, current_key=ck, current_value=cv, indices=sel.indices, valid=sel.valid,
            source_selected_output=src, global_mass=sel.global_mass, scaling=SCALING, out=out))
        add(f"sparse delta loop {loop + 1} (fl_sparse_attention_delta)", us, sparse_bytes(bh, loop, keys_n, quant, bits))
    # ---- append: plain step, and the step that rolls 64 tokens over (timed once per layer, eagerly)
    k4, v4 = [ck] * 4, [cv] * 4
    def graph_of_appends(layer, count: int):
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for _ in range(count):
                layer.append_decode_token(k4, v4)  # recorded, not run: the host mirror runs ahead of the device
        return graph

    def replay_us(graph) -> float:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        graph.replay()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1e3

    plain, rolled = [], []
    for layer in layers:
        layer.append_decode_token(k4, v4)  # warm-up, tail 64 -> 65
        torch.cuda.synchronize()
        eight = graph_of_appends(layer, 8)
        replay_us(eight)                                  # tail -> 73
        plain.append(min(replay_us(eight) for _ in range(3)) / 8)   # tail -> 97
        one = graph_of_appends(layer, 1)
        for _ in range(30):
            one.replay()                                  # tail -> 127
        torch.cuda.synchronize()
        rolled.append(replay_us(one))                     # tail 127 -> 128: the rollover
    add("append, no rollover (fl_append_decode_token, 3 launches)", statistics.median(plain), bh * 8 * 256 * 2)
    add("append with 64-token rollover (3 launches)", statistics.median(rolled),
        bh * (4 * 2 * 64 * 256 + 4 * 64 * (2 * 16 * bits + 24)), "one graph launch of three kernels")
    # ---- token retention (prefill time): hidden [B, T, 2048]
    h1 = torch.randn(B, T, 2048, generator=gen, device=device).to(torch.bfloat16)
    h2 = (h1.float() + 0.1 * torch.randn(B, T, 2048, generator=gen, device=device)).to(torch.bfloat16)
    add("hidden-delta score (fl_hidden_delta_score)", timeit(lambda i: hidden_delta_score(h2, h1)), 2 * h1.numel() * 2)
    score = hidden_delta_score(h2, h1)
    add("token retention (fl_select_prefill_tokens)", timeit(lambda i: retain_tokens(score, fraction=0.25)),
        B * T * (4 + 1 + 4 + 4), "latency bound: one CTA per sequence")
    kept = retain_tokens(score, fraction=0.25)
    n = int(kept.count[0])
    compact = gather_rows(h2, kept.positions, kept.count, rows=n)
    add("gather retained rows (fl_gather_rows)", timeit(lambda i: gather_rows(h2, kept.positions, kept.count, rows=n)),
        2 * compact.numel() * 2)
    add("scatter retained rows (fl_scatter_rows)", timeit(lambda i: scatter_rows(h2, compact, kept.positions, kept.count)),
        2 * compact.numel() * 2)
    line = {"metric": "kernel table: achieved GB/s per kernel of the path", "unit": "GB/s", "n_gpus": 1,
            "peak_GBps": peak, "peak_source": "measured (MEASURED_PEAKS.json hbm_gbs)" if peaks else "fallback 6650 GB/s",
            "config": {"workload": f"every kernel alone at batch {B}, {H} heads x {HEAD_DIM}, context {T}, {bits}-bit, "
                                   f"all-token masks; timed as graphs of 12 launches over 6 layers"},
            "kernels": rows}
    print(json.dumps(line))


# ----------------------------------------------------------------------------- the end-to-end workload


def cpu_e2e_tokens_per_second(args, tasks_per_core: int = 3, pool=None) -> dict:
    """CPU stand-in for one decode token of the model: the oracle's KV-attention step (per head,
    scaled) plus the projection / MLP GEMVs of two Ouro-shaped layers in torch on the host cores
    (scaled to ``layers`` x 4 loops)."""

    import torch

    from flashloop_b200.ouro_shape import OuroShapedConfig, OuroShapedForCausalLM
    from flashloop_b200.weights import fused_mlp, project_qkv

    kv = cpu_oracle_tokens_per_second(args, tasks_per_core=tasks_per_core, pool=pool)
    torch.set_num_threads(os.cpu_count() or 1)
    model = OuroShapedForCausalLM(OuroShapedConfig(num_hidden_layers=2, vocab_size=1024), dtype=torch.float32)
    x = torch.randn(1, 1, 2048)
    with torch.inference_mode():
        def layers_once():
            h = x
            for layer in model.model.layers:
                q, _, _ = project_qkv(layer.self_attn, layer.input_layernorm(h))
                h = h + layer.input_layernorm_2(layer.self_attn.o_proj(q))
                h = h + layer.post_attention_layernorm_2(fused_mlp(layer.mlp, layer.post_attention_layernorm(h)))
            return h
        layers_once()
        start = time.perf_counter()
        reps = 5
        for _ in range(reps):
            layers_once()
        per_layer = (time.perf_counter() - start) / reps / 2
    seconds = 1.0 / kv["value"] + per_layer * args.layers * 4
    return {"value": 1.0 / seconds, "unit": "tok/s", "cores": kv["cores"], "kind": "port",
            "sample": (f"KV attention: {kv['sample']}; model side: float32 torch GEMVs of 2 layers on "
                       f"{os.cpu_count()} threads, {per_layer * 1e3:.2f} ms per layer, scaled by {args.layers} layers x 4 loops")}


def run_e2e(args) -> None:
    import torch
    import torch.distributed as dist

    from flashloop_b200 import FlashLoopConfig, FlashLoopEngine, _native, sharding
    from flashloop_b200.ouro_shape import OuroShapedConfig, OuroShapedForCausalLM
    from flashloop_b200.tensor_parallel import shard_ouro_model

    _native.load()  # fail loudly when the CUDA library is missing
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    B, T, NL = args.batch, args.context, args.layers
    e2e_steps = max(2, min(args.steps, 16))
    budget = max(2, args.warmup) + args.steps + e2e_steps + 8
    cfg = OuroShapedConfig(num_hidden_layers=NL)
    model = OuroShapedForCausalLM(cfg, seed=0, device=device)
    tp = args.tp and world > 1
    if tp:
        shard_ouro_model(model, rank, world)  # this rank's heads and FFN columns
    graph_ok = not args.no_graph and not (tp and args.tp_allreduce == "nccl")
    engine = FlashLoopEngine(model, config=FlashLoopConfig(kv_bits=args.bits), validate_model=False,
                             max_new_tokens=budget, use_cuda_graph=graph_ok,
                             tp_group=dist.group.WORLD if tp else None, tp_allreduce=args.tp_allreduce)
    gen = torch.Generator().manual_seed(100 + (0 if tp else rank))
    prompts = torch.randint(0, cfg.vocab_size, (B, T), generator=gen).to(device)
    torch.cuda.synchronize()
    torch.cuda.reset_peak_memory_stats(device)
    before_prefill = torch.cuda.memory_allocated(device)
    t0 = time.perf_counter()
    logits = engine.prefill(prompts).logits
    torch.cuda.synchronize()
    prefill_s = time.perf_counter() - t0
    prefill_peak = torch.cuda.max_memory_allocated(device) - before_prefill
    state = {"token": logits.argmax(-1, keepdim=True)}

    def run_step():
        state["token"] = engine.decode(state["token"]).logits.argmax(-1, keepdim=True)

    def timed(fn, count: int) -> float:
        sharding.barrier(device)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(count):
            fn()
        e1.record()
        sharding.barrier(device)
        return sharding.max_over_ranks(e0.elapsed_time(e1), device)

    # the engine runs its first decode eagerly (the launches of that step are counted), records the
    # second as a CUDA graph and replays it from then on
    _native.count_launches(True)
    run_step()
    launch_counts = _native.count_launches(False)
    launches_per_step = sum(launch_counts.values())
    for _ in range(max(2, args.warmup) - 1):
        run_step()
    sampler = ClockSampler(local) if rank == 0 else None
    torch.cuda.profiler.start()
    ms_total = timed(run_step, args.steps)
    torch.cuda.profiler.stop()
    clocks = sampler.stop() if sampler else {}
    job_tokens = (lambda n: float(B * n)) if tp else (lambda n: sharding.sum_over_ranks(B * n, device))
    value = job_tokens(args.steps) / (ms_total * 1e-3)

    # ---- end to end: token ids come from pinned host memory, the chosen token goes back to it
    host_token = state["token"].cpu().pin_memory()
    dev_token = torch.empty_like(state["token"])

    def e2e_step():
        dev_token.copy_(host_token, non_blocking=True)
        out = engine.decode(dev_token).logits.argmax(-1, keepdim=True)
        host_token.copy_(out, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    e2e_ms = timed(e2e_step, e2e_steps)
    e2e_value = job_tokens(e2e_steps) / (e2e_ms * 1e-3)

    # ---- the dominant kernel of the path alone: the loop-2 dense reader of every layer
    layers = engine.state.cache.layers
    H = cfg.num_attention_heads // (world if tp else 1)
    q, k, v = (torch.randn((B, H, 1, HEAD_DIM), device=device).to(torch.bfloat16) for _ in range(3))
    # one pass over the layers, captured as a graph like the step itself and replayed between two
    # events, every layer's cache being a different 230 MB
    first_out, first_logits = layers[0].dense_source_attention(1, query=q, current_key=k, current_value=v,
                                                               scaling=SCALING, return_logits=True)
    out_buf, logits_buf = torch.empty_like(first_out), torch.empty_like(first_logits)

    def reader_pass():
        for layer in layers:
            layer.dense_source_attention(1, query=q, current_key=k, current_value=v, scaling=SCALING,
                                         return_logits=True, out=out_buf, logits_out=logits_buf)

    reader_pass()
    torch.cuda.synchronize()
    reader_graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(reader_graph):
        reader_pass()
    probe = []
    for rep in range(4):
        a, b_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        reader_graph.replay()
        b_.record()
        if rep:
            probe.append((a, b_))
    torch.cuda.synchronize()
    probe_ms = [a.elapsed_time(b_) / len(layers) for a, b_ in probe]
    status = max(layer.reader_status() for layer in layers)
    quant, tail = layers[0].quantized_tokens, layers[0].tail_tokens

    # ---- the two readers at the shapes the HBM target is quoted on (rank 0 only: a probe, not part
    # of the job's throughput)
    probes = {}
    if rank == 0 and not args.no_probes:
        probes = probe_configs1_readers(device, args.bits)
        probes.update(probe_projection(model, B, device))
    if world > 1:
        dist.barrier()

    # ---- N>1 replica runs: the same model once more, sharded over the ranks (strong scaling)
    tensor_parallel = None
    if world > 1 and not tp and not args.no_tp_probe:
        # every rank takes the same branch at every step: a rank that fails tells the others before the
        # next collective, so nobody is left waiting in one
        def all_ok(ok: bool) -> bool:
            flag = torch.tensor([0 if ok else 1], device=device)
            dist.all_reduce(flag)
            return int(flag.item()) == 0

        failure, tp_engine, tp_ms, peer_status = None, None, None, None
        try:
            tp_model = OuroShapedForCausalLM(cfg, seed=0, device=device)
            shard_ouro_model(tp_model, rank, world)
            tp_engine = FlashLoopEngine(tp_model, config=FlashLoopConfig(kv_bits=args.bits), validate_model=False,
                                        max_new_tokens=budget, use_cuda_graph=not args.no_graph,
                                        tp_group=dist.group.WORLD, tp_allreduce="peer")
        except Exception as exc:  # noqa: BLE001 - reported in the line, the replica numbers stand
            failure = f"{type(exc).__name__}: {exc}"
        if all_ok(failure is None):
            shared = torch.randint(0, cfg.vocab_size, (B, T), generator=torch.Generator().manual_seed(100)).to(device)
            tp_state = {"token": tp_engine.prefill(shared).logits.argmax(-1, keepdim=True)}

            def tp_step():
                tp_state["token"] = tp_engine.decode(tp_state["token"]).logits.argmax(-1, keepdim=True)

            for _ in range(max(3, args.warmup)):
                tp_step()
            tp_ms = timed(tp_step, args.steps)
            peer_status = tp_engine._peer.status()
            tensor_parallel = {
                "value": B * args.steps / (tp_ms * 1e-3), "unit": "tok/s", "ms_per_step": tp_ms / args.steps,
                "scaling": "strong", "global_batch": B, "parallelism": f"tp{world}",
                "all_reduce": "fl_allreduce_rmsnorm (one launch per sum, peer stores over NVLink, fused with the "
                              "residual add and the RMSNorms), whole step replayed from a CUDA graph",
                "peer_status": peer_status}
        else:
            tensor_parallel = {"unavailable": failure or "another rank could not build the tensor-parallel engine"}
        dist.barrier()

    if rank == 0:
        peak, peak_kind = load_peak()
        algo = dense_bytes(B * H, 1, quant, tail, args.bits)
        weights = sum(p.numel() for n, p in model.named_parameters() if "embed" not in n) * 2
        line = {
            "metric": METRIC, "value": value, "unit": "tok/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_total / args.steps, "higher_is_better": True,
            "scaling": "strong" if tp else "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": bench_config(args),
            "details": {"prefill_seconds": prefill_s, "prefill_peak_bytes_above_model": prefill_peak,
                        "cache_storage_bytes": engine.state.cache.storage_bytes, "context_at_end": quant + tail,
                        "weight_bytes_streamed_per_step": 4 * weights},
            "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": "tok/s", "h2d_bytes_per_step": int(host_token.numel() * 8),
                    "d2h_bytes_per_step": int(host_token.numel() * 8), "steps": e2e_steps},
            "gpu_launches": launches_per_step * args.steps,
            "gpu_launches_source": f"{launches_per_step} launches of this library's kernels counted in one eager "
                                   f"decode step ({launch_counts}) x {args.steps} timed steps; the framework's own "
                                   f"launches (embedding, lm_head GEMM, argmax) are not counted",
            "roofline": roofline_object(
                f"dense_reader_kernel<{args.bits},1> (loop 2: anchor + delta-2 streams), the dominant kernel of "
                f"this library in the step, at the step's shapes ({B * H} heads x {quant + tail} tokens)",
                "dense_reader", algo, probe_ms, peak, peak_kind,
                "CUDA events around a graph of one launch per cache layer of the engine (24 launches, each layer a "
                "different cache), replayed right after the timed region"),
            "reader_status": status,
        }
        line.update(probes)
        if tensor_parallel is not None:
            line["tensor_parallel"] = tensor_parallel
        if tp:
            line["tensor_parallel_all_reduce"] = args.tp_allreduce
            line["peer_status"] = engine._peer.status() if engine._peer is not None else None
        if not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_e2e_tokens_per_second(args)
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def update_traffic(args) -> None:
    """Record the measured DRAM traffic of the readers from `ncu -i <report> --page raw --csv`
    exports (no GPU needed).  The captures are of the hotpath workload at ``--batch`` x 16 heads x
    ``--context`` (all-token residuals, top 10 % keys); per kernel the launches found are averaged.
    Writes profiles/reader_traffic.json with the commit the files were captured at."""

    import csv

    scale = {"byte": 1.0, "Kbyte": 1e3, "Mbyte": 1e6, "Gbyte": 1e9}
    B, H, T, bits = args.batch, HEADS, args.context, args.bits
    quant = ((T - 64) // 64) * 64
    tail = T - quant
    keys_n = math.ceil((T + 1) * KEY_FRACTION)
    wanted = {
        "dense_reader": (f"dense_reader_kernel<{bits}, 1>", dense_bytes(B * H, 1, quant, tail, bits)),
        "selected_reader": (f"selected_reader_kernel<{bits}, 0, 4>", sparse_bytes(B * H, 3, keys_n, quant, bits)),
    }
    found = {k: [] for k in wanted}
    for path in args.update_traffic:
        rows = list(csv.reader(open(path)))
        start = next(i for i, row in enumerate(rows) if "Kernel Name" in row)
        header, units = rows[start], rows[start + 1]
        name_at = header.index("Kernel Name")
        cols = [header.index(m) for m in ("dram__bytes_read.sum", "dram__bytes_write.sum")]
        for row in rows[start + 2:]:
            if len(row) <= max(cols):
                continue
            for key, (pattern, _) in wanted.items():
                if pattern.replace(" ", "") in row[name_at].replace(" ", ""):
                    found[key].append(sum(float(row[c].replace(",", "")) * scale[units[c]] for c in cols))
    commit = subprocess.run(["git", "rev-parse", "--short", "HEAD"], cwd=ROOT, capture_output=True, text=True).stdout.strip()
    record = json.loads(TRAFFIC_FILE.read_text()) if TRAFFIC_FILE.exists() else {}
    for key, values in found.items():
        if values:
            record[key] = {"kernel": wanted[key][0], "dram_bytes_per_launch": statistics.mean(values),
                           "algorithmic_bytes_per_launch": wanted[key][1], "launches": len(values),
                           "case": f"batch {B} x {H} heads x context {T}, {bits}-bit, {keys_n} selected keys",
                           "commit": commit, "files": [Path(f).name for f in args.update_traffic]}
    TRAFFIC_FILE.write_text(json.dumps(record, indent=1) + "\n")
    print(json.dumps(record, indent=1))


def main() -> None:
    args = parse_args()
    if args.update_traffic:
        update_traffic(args)
    elif args.impl == "reference" and args.workload == "kernels":
        run_reference_kernels(args)
    elif args.impl == "reference":
        run_reference(args)
    elif args.workload == "e2e":
        run_e2e(args)
    elif args.workload == "kernels":
        run_kernel_table(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
