"""GPU parity of the KIVI-layout reader surface (flashloop_b200.kivi_backend and the
``flashloop_kivi_gemv`` stand-in behind it) against vectors produced by the reference's own
``kivi_outer`` cache layer, and against plain Torch arithmetic on the decoded streams.

The streams are the reference's packed KIVI words (tests/golden/reference_vectors.npz,
``layer.kivi_outer.*``), handed to the readers exactly as the reference's cache hands them to
its extension (flashloop/cache.py:1265-1285, 1421-1441, 1607-1625, 1681-1700)."""

from __future__ import annotations

import numpy as np
import pytest
import torch

from tests.gpu_util import assert_bf16_tolerance, bf16_tensor, max_err
from tests.helpers import bf, golden_inputs, golden_stream

pytestmark = pytest.mark.gpu

SCALING = 128 ** -0.5


@pytest.fixture(scope="module")
def kb():
    from flashloop_b200 import _native, kivi_backend

    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    _native.load()
    return kivi_backend


def _stream(kb, golden, prefix: str, axis: str):
    ref = golden_stream(golden, prefix)
    assert ref is not None, prefix
    return kb.KiviPacked4Bit(payload=torch.from_numpy(ref["payload"].copy()).cuda(),
                             minimum=torch.from_numpy(ref["minimum"].copy()).cuda(),
                             scale=torch.from_numpy(ref["scale"].copy()).cuda(), original_shape=ref["shape"],
                             original_dtype=torch.bfloat16, axis=axis, group_size=64)


@pytest.fixture()
def streams(kb, golden):
    from flashloop_b200 import flashloop_kivi_gemv

    flashloop_kivi_gemv.forget()
    keys = tuple(_stream(kb, golden, f"layer.kivi_outer.k{s}", "per_channel") for s in range(4))
    values = tuple(_stream(kb, golden, f"layer.kivi_outer.v{s}", "per_token") for s in range(4))
    ranks = (torch.from_numpy(golden["layer.kivi_outer.rank3"]).cuda(),
             torch.from_numpy(golden["layer.kivi_outer.rank4"]).cuda())
    tails = ([bf16_tensor(bf(golden[f"layer.tail_k{r}"])) for r in range(4)],
             [bf16_tensor(bf(golden[f"layer.tail_v{r}"])) for r in range(4)])
    return keys, values, ranks, tails


def test_extension_object_exports_the_reference_names(kb):
    ext = kb.load_kivi_outer_extension()
    for name in ("gemv_forward_cuda_outer_dim_logical", "qk_selected_cuda", "pv_selected_cuda",
                 "qk_cross_loop_cuda", "pv_cross_loop_cuda", "sparse_attention_delta_cuda",
                 "dense_source_attention_cuda"):
        assert callable(getattr(ext, name)), name


def test_fused_dense_source_attention_vs_reference_vectors(kb, golden, streams):
    keys, values, ranks, (tail_k, tail_v) = streams
    *_, q, ck, cv = golden_inputs(golden)
    ext = kb.load_kivi_outer_extension()
    for loop in (0, 1):
        out, logits = kb.kivi_fused_dense_source_attention(
            query=bf16_tensor(q), current_key=bf16_tensor(ck), current_value=bf16_tensor(cv), key_streams=keys,
            value_streams=values, rank_maps=ranks, tail_key=tail_k[loop], tail_value=tail_v[loop], scaling=SCALING,
            loop=loop, extension=ext, return_logits=True)
        assert tuple(logits.shape) == (1, 2, 1, 201)
        assert_bf16_tolerance(out.cpu().numpy(), golden[f"dense.kivi_outer.loop{loop}.out"], what=f"dense loop {loop}")
        assert max_err(logits.cpu().numpy(), golden[f"dense.kivi_outer.loop{loop}.logits"]) < 5e-2
        out_only, none = kb.kivi_fused_dense_source_attention(
            query=bf16_tensor(q), current_key=bf16_tensor(ck), current_value=bf16_tensor(cv), key_streams=keys,
            value_streams=values, rank_maps=ranks, tail_key=tail_k[loop], tail_value=tail_v[loop], scaling=SCALING,
            loop=loop)
        assert none is None and torch.equal(out_only, out)
    with pytest.raises(ValueError):
        kb.kivi_fused_dense_source_attention(
            query=bf16_tensor(q), current_key=bf16_tensor(ck), current_value=bf16_tensor(cv), key_streams=keys,
            value_streams=values, rank_maps=ranks, tail_key=tail_k[2], tail_value=tail_v[2], scaling=SCALING, loop=2)


def test_fused_sparse_attention_delta_vs_reference_vectors(kb, golden, streams):
    keys, values, ranks, (tail_k, tail_v) = streams
    idx = torch.from_numpy(golden["select.padded"]).cuda()
    valid = torch.from_numpy(golden["select.valid"]).cuda()
    q3, k3, v3 = (bf16_tensor(bf(golden[f"sparse.{n}"])) for n in ("query", "cur_k", "cur_v"))
    for loop in (2, 3):
        # the reference hands over its whole tail buffer and says where the tail ends
        pad = torch.zeros(1, 2, 128 - tail_k[loop].shape[2], 128, dtype=torch.bfloat16, device="cuda")
        delta, current = kb.kivi_fused_sparse_attention_delta(
            query=q3, current_key=k3, current_value=v3, key_streams=keys, value_streams=values, rank_maps=ranks,
            tail_key=torch.cat([tail_k[loop], pad], 2), tail_value=torch.cat([tail_v[loop], pad], 2), indices=idx,
            valid=valid, source_selected_output=torch.from_numpy(golden["select.selected_output"]).cuda(),
            global_mass=torch.from_numpy(golden["select.mass"]).cuda(), current_position=200, scaling=SCALING,
            loop=loop, return_current_logits=True)
        assert_bf16_tolerance(delta.cpu().numpy(), golden[f"sparse.kivi_outer.loop{loop}"], what=f"sparse loop {loop}")
        # heads that selected the current token report its scaled logit, the others NaN
        picked = ((idx == 200) & valid).any(-1)[0]
        want = (q3.float() * k3.float()).sum(-1)[0, :, 0] * SCALING
        assert torch.isnan(current[0][~picked]).all()
        assert torch.allclose(current[0][picked], want[picked], atol=1e-3)
    with pytest.raises(ValueError):
        kb.kivi_fused_sparse_attention_delta(
            query=q3, current_key=k3, current_value=v3, key_streams=keys, value_streams=values, rank_maps=ranks,
            tail_key=tail_k[2], tail_value=tail_v[2], indices=idx, valid=valid,
            source_selected_output=torch.from_numpy(golden["select.selected_output"]).cuda(),
            global_mass=torch.from_numpy(golden["select.mass"]).cuda(), current_position=999, scaling=SCALING, loop=2)


def test_cross_loop_qk_pv_fused_and_unfused(kb, golden, streams):
    """Fused readers against (a) the reference layer's qk on the packed prefix and (b) the un-fused
    composition over plain Torch GEMVs on the decoded streams."""

    keys, values, ranks, _ = streams
    *_, q, _, _ = golden_inputs(golden)
    query = bf16_tensor(q)
    padded = torch.from_numpy(golden["select.padded"]).cuda()
    inside = padded < 128
    safe = torch.where(inside, padded, torch.zeros_like(padded))
    weights = torch.from_numpy(golden["select.selected_weights"]).cuda() * inside[:, :, None, :]
    for loop in range(4):
        got = kb.kivi_fused_cross_loop_qk(query, keys, ranks, safe, loop=loop)
        ref = torch.from_numpy(golden[f"qk.kivi_outer.loop{loop}"]).cuda()
        assert float(((got - ref).abs() * inside[:, :, None, :]).max()) < 0.2
        assert torch.allclose(got * inside[:, :, None, :], ref * inside[:, :, None, :], rtol=1e-2, atol=5e-2)
        plain = kb.kivi_cross_loop_qk(query, keys, ranks, safe, loop=loop, gemv=kb.outer_matmul_reference)
        assert torch.allclose(got, plain, rtol=1e-2, atol=5e-2), float((got - plain).abs().max())
        picked = kb.kivi_cross_loop_qk(query, keys, ranks, safe, loop=loop, gemv=kb.outer_matmul_reference,
                                       selected_gemv=lambda x, s, i: kb.kivi_selected_qk(x, s, i))
        assert torch.allclose(picked, plain, rtol=1e-2, atol=5e-2)
        out = kb.kivi_fused_cross_loop_pv(weights, values, ranks, safe, loop=loop)
        plain_v = kb.kivi_cross_loop_pv(weights, values, ranks, safe, loop=loop, gemv=kb.outer_matmul_reference)
        assert_bf16_tolerance(out.cpu().numpy(), plain_v.cpu().numpy(), what=f"pv loop {loop}")
        picked_v = kb.kivi_cross_loop_pv(weights, values, ranks, safe, loop=loop, gemv=kb.outer_matmul_reference,
                                         selected_gemv=lambda x, s, i: kb.kivi_selected_pv(x, s, i))
        assert_bf16_tolerance(picked_v.cpu().numpy(), plain_v.cpu().numpy(), what=f"selected pv loop {loop}")


def test_outer_gemv_and_selected_readers_vs_decoded_streams(kb, golden, streams):
    keys, values, _, _ = streams
    gen = torch.Generator().manual_seed(8)
    for stream in (keys[0], keys[2]):  # the anchor and a compact stream with a partial last group
        tokens = stream.original_shape[2]
        x = torch.randn(1, 2, 2, 128, generator=gen).to(torch.bfloat16).cuda()
        got = kb.kivi_outer_gemv(x, stream)
        want = kb.outer_matmul_reference(x, stream)
        assert tuple(got.shape) == (1, 2, 2, tokens)
        # unscaled logits reach +-60 with the outlier channels; 0.2 absolute is the bound the
        # selected-QK reader is held to elsewhere
        assert torch.allclose(got, want, rtol=1e-2, atol=0.2), float((got - want).abs().max())
        idx = torch.randint(0, tokens, (1, 2, 17), generator=gen).cuda()
        sel = kb.kivi_selected_qk(x[:, :, :1], stream, idx)
        assert torch.allclose(sel, torch.gather(want[:, :, :1], -1, idx[:, :, None, :]), rtol=1e-2, atol=0.2)
    for stream in (values[0], values[3]):
        tokens = stream.original_shape[2]
        w = torch.rand(1, 2, 1, tokens, generator=gen).cuda() / tokens
        got = kb.kivi_outer_gemv(w, stream)
        want = kb.outer_matmul_reference(w, stream)
        assert_bf16_tolerance(got.cpu().numpy(), want.cpu().numpy(), what="V gemv")
        idx = torch.randint(0, tokens, (1, 2, 9), generator=gen).cuda()
        ws = torch.rand(1, 2, 1, 9, generator=gen).cuda() / 9
        spread = torch.zeros(1, 2, 1, tokens, device="cuda").scatter_add_(-1, idx[:, :, None, :], ws)
        assert_bf16_tolerance(kb.kivi_selected_pv(ws, stream, idx).cpu().numpy(),
                              kb.outer_matmul_reference(spread, stream).cpu().numpy(), what="selected V")
    with pytest.raises(ValueError):
        kb.kivi_selected_qk(torch.zeros(1, 2, 1, 128, device="cuda"), values[0], torch.zeros(3, dtype=torch.long))
    with pytest.raises(RuntimeError):
        kb.kivi_outer_gemv(torch.zeros(1, 2, 1, 128), keys[0])


def test_adopted_streams_follow_in_place_updates(kb, golden, streams):
    """The converted copy is found again for unchanged tensors and rebuilt after an in-place
    update, and a freed tensor's address cannot alias a cached entry."""

    from flashloop_b200 import flashloop_kivi_gemv as ext

    keys, values, ranks, (tail_k, tail_v) = streams
    *_, q, ck, cv = golden_inputs(golden)
    args = dict(query=bf16_tensor(q), current_key=bf16_tensor(ck), current_value=bf16_tensor(cv), key_streams=keys,
                value_streams=values, rank_maps=ranks, tail_key=tail_k[1], tail_value=tail_v[1], scaling=SCALING,
                loop=1)
    first, _ = kb.kivi_fused_dense_source_attention(**args)
    entries = len(ext._ADOPTED)
    again, _ = kb.kivi_fused_dense_source_attention(**args)
    assert len(ext._ADOPTED) == entries and torch.equal(first, again)
    values[0].scale.mul_(2.0)  # same storage, new contents
    changed, _ = kb.kivi_fused_dense_source_attention(**args)
    assert len(ext._ADOPTED) == entries + 1
    assert float((changed - first).abs().max()) > 1e-2
    ext.forget()
    fresh, _ = kb.kivi_fused_dense_source_attention(**args)
    assert torch.equal(fresh, changed)
    ext.set_cache_capacity(1)
    kb.kivi_fused_cross_loop_qk(args["query"], keys, ranks, torch.arange(5, device="cuda"), loop=0)
    assert len(ext._ADOPTED) == 1
    ext.set_cache_capacity(64)
