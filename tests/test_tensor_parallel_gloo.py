"""Tensor-parallel host logic on CPU: two ``gloo`` ranks shard the tiny Ouro-shaped model by head
and FFN column, run a dense prefill loop with the all-reduce hook, and must reproduce the
unsharded loop."""

from __future__ import annotations

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from flashloop_b200.prefill import dense_prefill_loop
from flashloop_b200.tensor_parallel import PartialSum, shard_ouro_model, shard_range
from tests.helpers import tiny_ouro_model


def test_shard_range_and_shapes():
    assert shard_range(16, 8, 3) == (6, 8)
    with pytest.raises(ValueError):
        shard_range(10, 4, 0)
    model = shard_ouro_model(tiny_ouro_model(), rank=1, world=2)
    layer = model.model.layers[0]
    assert layer.self_attn.q_proj.weight.shape == (128, 256) and layer.self_attn.o_proj.weight.shape == (256, 128)
    assert layer.mlp.gate_proj.weight.shape == (192, 256) and layer.mlp.down_proj.weight.shape == (256, 192)
    full = tiny_ouro_model().model.layers[0]
    assert torch.equal(layer.self_attn.k_proj.weight, full.self_attn.k_proj.weight[128:256])
    assert torch.equal(layer.mlp.down_proj.weight, full.mlp.down_proj.weight[:, 192:384])
    assert shard_ouro_model(tiny_ouro_model(), 0, 1) is not None and PartialSum(None).world == 1


def _loop(model, ids, reduce):
    backbone = model.model
    hidden = backbone.embed_tokens(ids)
    positions = torch.arange(ids.shape[1]).unsqueeze(0).expand(ids.shape[0], -1)
    rope = backbone.rotary_emb(hidden, positions)
    with torch.inference_mode():
        return dense_prefill_loop(backbone.layers, hidden, position_embeddings=rope, final_norm=backbone.norm,
                                  loop=1, reduce=reduce)


def _worker(rank: int, world: int, port: int, results) -> None:
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.set_num_threads(2)
        ids = torch.randint(0, 256, (2, 40), generator=torch.Generator().manual_seed(3))
        sharded = _loop(shard_ouro_model(tiny_ouro_model(), rank, world), ids, PartialSum(None))
        out = {"hidden": sharded.hidden_states.float(), "k_shape": tuple(sharded.composite_cache.keys[0].shape)}
        if rank == 0:
            whole = _loop(tiny_ouro_model(), ids, lambda t: t)
            out["reference"] = whole.hidden_states.float()
            out["k_local_matches"] = torch.equal(sharded.composite_cache.keys[0], whole.composite_cache.keys[0][:, :1])
        results[rank] = out
    finally:
        dist.destroy_process_group()


def test_two_ranks_reproduce_the_unsharded_loop():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    results = ctx.Manager().dict()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, results)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(180)
        assert p.exitcode == 0
    a, b = results[0], results[1]
    assert torch.equal(a["hidden"], b["hidden"])                 # every rank holds the same residual stream
    assert a["k_shape"] == (2, 1, 40, 128)                        # one of the two heads per rank
    assert a["k_local_matches"]                                   # layer-0 keys of the local head: no sum involved
    ref = a["reference"]
    err = (a["hidden"] - ref).abs()
    assert float(err.max()) < 0.06 * float(ref.abs().max()) and float(err.mean()) < 0.01 * float(ref.abs().mean()) + 1e-3
