"""GPU parity: the CUDA path (through the C ABI) against the numpy oracle and the golden
vectors.  Bit-exact for codes, metadata, rank maps, tails and selected indices; the BF16
tolerance (2e-2 max-abs / 1e-2 relative) for attention outputs against the fake-quant path,
plus a tighter bound against the oracle's float32 restatement of the same packed cache."""

from __future__ import annotations

import math

import numpy as np
import pytest
import torch

from oracle import bf16, fakequant, packing as opack, selection as osel
from tests.gpu_util import (assert_bf16_tolerance, assert_layer_matches, bf16_tensor, bits16,
                            max_err, oracle_layer, to_np)
from tests.helpers import bf, f16, golden_inputs, golden_stream

pytestmark = pytest.mark.gpu

SCALING = 128 ** -0.5


@pytest.fixture(scope="module")
def fl():
    import flashloop_b200 as pkg

    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    from flashloop_b200 import _native

    _native.load()
    return pkg


def _synth(heads, tokens, seed, all_active=False):
    from flashloop_b200.synthetic import make_loop_kv, make_masks, make_query

    keys, values = make_loop_kv(heads, tokens, seed=seed)
    m3, m4 = make_masks(tokens, seed=seed, all_active=all_active)
    q, ck, cv = make_query(heads, seed=seed)
    return keys, values, m3, m4, q, ck, cv


def _cuda(ts):
    return [t.cuda() for t in ts]


# ------------------------------------------------------------------------------ packing


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("tokens", [1, 8, 63, 64, 200, 1000])
def test_pack_bit_exact_vs_oracle(fl, dtype, tokens):
    from flashloop_b200 import kivi_backend, packing

    g = torch.Generator().manual_seed(tokens)
    x = (torch.randn(2, 3, tokens, 128, generator=g) * torch.rand(1, 3, 1, 128, generator=g) * 4).to(dtype)
    xn = to_np(x)
    for bits in (4, 2):
        k = packing.pack_k_per_channel(x.cuda(), bits=bits)
        v = packing.pack_v_per_token(x.cuda(), bits=bits)
        ok, ov = opack.pack_k_rows(xn, bits=bits), opack.pack_v_rows(xn, bits=bits)
        for got, want, name in ((k, ok, "k"), (v, ov, "v")):
            np.testing.assert_array_equal(got.payload.cpu().numpy(), want.payload, err_msg=f"{name} payload {bits}")
            np.testing.assert_array_equal(bits16(got.minimum), want.minimum.view(np.uint16), err_msg=f"{name} min {bits}")
            np.testing.assert_array_equal(bits16(got.scale), want.scale.view(np.uint16), err_msg=f"{name} scale {bits}")
            np.testing.assert_array_equal(bits16(got.decode().to(torch.bfloat16)), bf16.to_bits(want.decode()),
                                          err_msg=f"{name} decode {bits}")
    kk = kivi_backend.pack_kivi_k_per_channel(x.cuda())
    kv = kivi_backend.pack_kivi_v_per_token(x.cuda())
    okk, okv = opack.pack_kivi_k(xn), opack.pack_kivi_v(xn)
    for got, want, name in ((kk, okk, "kivi k"), (kv, okv, "kivi v")):
        np.testing.assert_array_equal(got.payload.cpu().numpy(), want.payload, err_msg=name)
        np.testing.assert_array_equal(bits16(got.minimum), want.minimum.view(np.uint16), err_msg=name)
        np.testing.assert_array_equal(bits16(got.scale), want.scale.view(np.uint16), err_msg=name)
        np.testing.assert_array_equal(bits16(got.decode().to(torch.bfloat16)), bf16.to_bits(want.decode()), err_msg=name)
    # KIVI words re-arranged on the GPU give the row layout
    rk, rv = kivi_backend.kivi_to_rows(kk), kivi_backend.kivi_to_rows(kv)
    np.testing.assert_array_equal(rk.payload.cpu().numpy(), opack.pack_k_rows(xn).payload)
    np.testing.assert_array_equal(rv.payload.cpu().numpy(), opack.pack_v_rows(xn).payload)
    np.testing.assert_array_equal(bits16(rv.scale), opack.pack_v_rows(xn).scale.view(np.uint16))


@pytest.mark.parametrize("tag", ["bf16", "f16", "f32"])
def test_pack_bit_exact_vs_reference_vectors(fl, golden, tag):
    from flashloop_b200 import kivi_backend, packing

    if tag == "bf16":
        x = torch.from_numpy(bf(golden["in.key0"])).to(torch.bfloat16)
    elif tag == "f16":
        x = torch.from_numpy(golden["pack.f16.input"].view(np.float16).copy())
    else:
        x = torch.from_numpy(golden["pack.f32.input"].copy())
    x = x.cuda()
    for fn, name in ((kivi_backend.pack_kivi_k_per_channel, "kivi_k"), (kivi_backend.pack_kivi_v_per_token, "kivi_v"),
                     (packing.pack_k_per_channel, "rows_k"), (packing.pack_v_per_token, "rows_v")):
        got, ref = fn(x), golden_stream(golden, f"pack.{tag}.{name}")
        np.testing.assert_array_equal(got.payload.cpu().numpy(), ref["payload"], err_msg=name)
        np.testing.assert_array_equal(bits16(got.minimum), ref["minimum"].view(np.uint16), err_msg=name)
        np.testing.assert_array_equal(bits16(got.scale), ref["scale"].view(np.uint16), err_msg=name)
        if tag == "bf16":
            np.testing.assert_array_equal(bits16(got.decode()), golden[f"pack.bf16.{name}.decode"], err_msg=name)


def test_pack_rejects_bad_arguments(fl):
    from flashloop_b200 import packing

    with pytest.raises(ValueError):
        packing.pack_k_per_channel(torch.zeros(2, 3, 128, device="cuda"))
    with pytest.raises(TypeError):
        packing.pack_k_per_channel(torch.zeros(1, 1, 8, 128, dtype=torch.int32, device="cuda"))
    with pytest.raises(ValueError):
        packing.pack_v_per_token(torch.zeros(1, 1, 0, 128, device="cuda"))
    with pytest.raises(RuntimeError):
        packing.pack_k_per_channel(torch.zeros(1, 1, 8, 128))  # CPU tensor: no fallback


# ------------------------------------------------------------------------------ cache construction


def test_prefill_streams_bit_exact_vs_reference_vectors(fl, golden):
    from flashloop_b200.cache import CrossLoopKVLayer

    keys, values, m3, m4, *_ = golden_inputs(golden)
    layer = CrossLoopKVLayer.from_prefill(
        [bf16_tensor(k) for k in keys], [bf16_tensor(v) for v in values],
        mask_loop3=torch.from_numpy(m3)[None].cuda(), mask_loop4=torch.from_numpy(m4)[None].cuda())
    ex = layer.export_sequence(0)
    assert ex["quantized_tokens"] == 128
    for s in range(4):
        for kind in ("k", "v"):
            ref = golden_stream(golden, f"layer.triton_row.{kind}{s}")
            np.testing.assert_array_equal(ex[f"{kind}{s}.payload"].cpu().numpy(), ref["payload"][0], err_msg=f"{kind}{s}")
            np.testing.assert_array_equal(bits16(ex[f"{kind}{s}.minimum"]), ref["minimum"][0].view(np.uint16))
            np.testing.assert_array_equal(bits16(ex[f"{kind}{s}.scale"]), ref["scale"][0].view(np.uint16))
    np.testing.assert_array_equal(ex["rank3"].cpu().numpy(), golden["layer.triton_row.rank3"])
    np.testing.assert_array_equal(ex["rank4"].cpu().numpy(), golden["layer.triton_row.rank4"])
    for r in range(4):
        np.testing.assert_array_equal(bits16(ex[f"tail_k{r}"]), golden[f"layer.tail_k{r}"][0])


def _compact(t, mask):
    """Rows of [1, H, T, D] at the True positions of ``mask`` [T], in position order."""
    return t[:, :, torch.nonzero(mask).flatten()].contiguous()


def test_staged_builder_bit_exact_vs_reference_vectors(fl, golden):
    """CrossLoopKVLayerBuilder (from_loop1 / add_loop2 / finalize on compact Loop-3/4 rows) and
    from_prefill_updates against the reference's streams, rank maps and tails, and ``gather``
    against the reference layer's gather."""

    from flashloop_b200.cache import CrossLoopKVLayer, CrossLoopKVLayerBuilder

    keys, values, m3, m4, *_ = golden_inputs(golden)
    k = [bf16_tensor(x) for x in keys]
    v = [bf16_tensor(x) for x in values]
    mask3, mask4 = torch.from_numpy(m3).cuda(), torch.from_numpy(m4).cuda()
    pos3 = torch.nonzero(mask3).flatten().to(torch.int32)
    pos4 = torch.nonzero(mask4).flatten().to(torch.int32)
    builder = CrossLoopKVLayerBuilder.from_loop1(k[0], v[0], max_new_tokens=128)
    assert not builder.retains_dense_loop1_prefix and builder.packed_tokens == 128
    with pytest.raises(RuntimeError):
        builder.finalize(loop3_positions=pos3, loop3_keys=_compact(k[2], mask3), loop3_values=_compact(v[2], mask3),
                         loop4_positions=pos4, loop4_keys=_compact(k[3], mask4), loop4_values=_compact(v[3], mask4))
    builder.add_loop2(k[1], v[1])
    with pytest.raises(RuntimeError):
        builder.add_loop2(k[1], v[1])
    staged = builder.finalize(loop3_positions=pos3, loop3_keys=_compact(k[2], mask3),
                              loop3_values=_compact(v[2], mask3), loop4_positions=pos4,
                              loop4_keys=_compact(k[3], mask4), loop4_values=_compact(v[3], mask4))
    at_once = CrossLoopKVLayer.from_prefill_updates(
        loop1_key=k[0], loop1_value=v[0], loop2_key=k[1], loop2_value=v[1], loop3_positions=pos3,
        loop3_keys=_compact(k[2], mask3), loop3_values=_compact(v[2], mask3), loop4_positions=pos4,
        loop4_keys=_compact(k[3], mask4), loop4_values=_compact(v[3], mask4))
    for layer in (staged, at_once):
        ex = layer.export_sequence(0)
        assert ex["quantized_tokens"] == 128 and ex["tail_tokens"] == 72
        for s in range(4):
            for kind in ("k", "v"):
                ref = golden_stream(golden, f"layer.triton_row.{kind}{s}")
                np.testing.assert_array_equal(ex[f"{kind}{s}.payload"].cpu().numpy(), ref["payload"][0], err_msg=f"{kind}{s}")
                np.testing.assert_array_equal(bits16(ex[f"{kind}{s}.minimum"]), ref["minimum"][0].view(np.uint16))
                np.testing.assert_array_equal(bits16(ex[f"{kind}{s}.scale"]), ref["scale"][0].view(np.uint16))
        np.testing.assert_array_equal(ex["rank3"].cpu().numpy(), golden["layer.triton_row.rank3"])
        np.testing.assert_array_equal(ex["rank4"].cpu().numpy(), golden["layer.triton_row.rank4"])
        # The builder sees only the retained Loop-3/4 rows: a tail token that a late loop did not
        # retain keeps the loop before's row (flashloop/cache.py:584-606), whereas the vectors come
        # from full Loop-3/4 tensors; the tails of loops 1-2 and the retained rows are the same.
        for r in range(2):
            np.testing.assert_array_equal(bits16(ex[f"tail_k{r}"]), golden[f"layer.tail_k{r}"][0])
            np.testing.assert_array_equal(bits16(ex[f"tail_v{r}"]), golden[f"layer.tail_v{r}"][0])
        for r, mask in ((2, mask3), (3, mask4)):
            kept = mask[128:].cpu().numpy()
            np.testing.assert_array_equal(bits16(ex[f"tail_k{r}"])[:, kept], golden[f"layer.tail_k{r}"][0][:, kept])
            np.testing.assert_array_equal(bits16(ex[f"tail_k{r}"])[:, ~kept], bits16(ex[f"tail_k{r - 1}"])[:, ~kept])
            np.testing.assert_array_equal(bits16(ex[f"tail_v{r}"])[:, kept], golden[f"layer.tail_v{r}"][0][:, kept])
        np.testing.assert_array_equal(ex["tail_active3"].cpu().numpy(), golden["layer.tail_active3"][0])
        np.testing.assert_array_equal(ex["tail_active4"].cpu().numpy(), golden["layer.tail_active4"][0])
    every = torch.arange(200)
    for loop in (1, 3):
        gk, gv = staged.gather(loop, every)
        upto = 200 if loop == 1 else 128  # (loop 3: the packed prefix; its tail differs as said above)
        np.testing.assert_array_equal(bits16(gk)[:, :, :upto], golden[f"gather.loop{loop}.k"][:, :, :upto])
        np.testing.assert_array_equal(bits16(gv)[:, :, :upto], golden[f"gather.loop{loop}.v"][:, :, :upto])
    with pytest.raises(IndexError):
        staged.gather(1, torch.tensor([200]))
    with pytest.raises(ValueError):  # Loop-4 rows must be Loop-3 rows
        other = CrossLoopKVLayerBuilder.from_loop1(k[0], v[0])
        other.add_loop2(k[1], v[1])
        stray = torch.nonzero(~mask3).flatten()[:3].to(torch.int32)
        other.finalize(loop3_positions=pos3, loop3_keys=_compact(k[2], mask3), loop3_values=_compact(v[2], mask3),
                       loop4_positions=stray, loop4_keys=k[3][:, :, stray.long()].contiguous(),
                       loop4_values=v[3][:, :, stray.long()].contiguous())


@pytest.mark.parametrize("bits", [4, 2])
def test_staged_builder_batch_equals_one_shot_encoder(fl, bits):
    """A batch of three prompts, retention masks that differ per sequence: the staged builder
    and the one-shot from_prefill produce identical layers (every stream, rank map and tail)."""

    from flashloop_b200.cache import CrossLoopKVLayer, CrossLoopKVLayerBuilder
    from flashloop_b200.synthetic import make_loop_kv, make_masks

    heads, tokens, batch = 3, 450, 3
    per = [make_loop_kv(heads, tokens, seed=900 + b) for b in range(batch)]
    keys = [torch.cat([per[b][0][r] for b in range(batch)]).cuda() for r in range(4)]
    values = [torch.cat([per[b][1][r] for b in range(batch)]).cuda() for r in range(4)]
    masks = [make_masks(tokens, seed=900 + b) for b in range(batch)]
    m3 = torch.stack([m[0] for m in masks]).cuda()
    m4 = torch.stack([m[1] for m in masks]).cuda()
    # composites as a prefill holds them: a late loop's tensor is the loop before with its retained
    # rows replaced
    for r, mask in ((2, m3), (3, m4)):
        keep = mask[:, None, :, None]
        keys[r] = torch.where(keep, keys[r], keys[r - 1])
        values[r] = torch.where(keep, values[r], values[r - 1])
    one_shot = CrossLoopKVLayer.from_prefill(keys, values, mask_loop3=m3, mask_loop4=m4, bits=bits)

    def positions(mask):
        rows = int(mask.sum(1).max())
        out = torch.full((batch, rows), -1, dtype=torch.int32, device="cuda")
        for b in range(batch):
            p = torch.nonzero(mask[b]).flatten().to(torch.int32)
            out[b, :p.numel()] = p
        return out

    def compact(t, pos):
        idx = pos.clamp(min=0).long()[:, None, :, None].expand(-1, heads, -1, 128)
        return torch.gather(t, 2, idx).contiguous()

    p3, p4 = positions(m3), positions(m4)
    builder = CrossLoopKVLayerBuilder.from_loop1(keys[0], values[0], bits=bits)
    builder.add_loop2(keys[1], values[1])
    staged = builder.finalize(loop3_positions=p3, loop3_keys=compact(keys[2], p3), loop3_values=compact(values[2], p3),
                              loop4_positions=p4, loop4_keys=compact(keys[3], p4), loop4_values=compact(values[3], p4))
    for b in range(batch):
        a, c = one_shot.export_sequence(b), staged.export_sequence(b)
        assert a.keys() == c.keys()
        for name in a:
            if isinstance(a[name], torch.Tensor):
                assert torch.equal(a[name], c[name]), (bits, b, name)
            else:
                assert a[name] == c[name], (bits, b, name)
    assert staged.storage_bytes == one_shot.storage_bytes


@pytest.mark.parametrize("tokens,all_active", [(100, False), (128, False), (191, False), (200, False),
                                               (333, True), (700, False)])
def test_prefill_and_readers_vs_oracle(fl, tokens, all_active):
    """Edge lengths: no packed prefix (100), one group (128), longest tail (191), ragged
    compact streams, identity rank maps (all_active)."""

    from flashloop_b200.cache import CrossLoopKVLayer

    heads = 3
    keys, values, m3, m4, q, ck, cv = _synth(heads, tokens, seed=tokens, all_active=all_active)
    oracle = oracle_layer(keys, values, m3, m4)
    layer = CrossLoopKVLayer.from_prefill(_cuda(keys), _cuda(values), mask_loop3=m3[None].cuda(),
                                          mask_loop4=m4[None].cuda())
    assert_layer_matches(layer, 0, oracle, what=f"T={tokens}")
    qn, ckn, cvn = to_np(q), to_np(ck), to_np(cv)
    kn, vn = [to_np(k) for k in keys], [to_np(v) for v in values]
    masks = [np.ones(tokens, bool), m3.numpy(), m4.numpy()]
    for loop in range(4):
        out, logits = layer.dense_source_attention(loop, query=q.cuda(), current_key=ck.cuda(),
                                                   current_value=cv.cuda(), scaling=SCALING, return_logits=True)
        want, want_logits = oracle.dense_source_attention(loop, query=qn, current_key=ckn, current_value=cvn,
                                                          scaling=SCALING)
        assert logits.shape[-1] == tokens + 1
        assert max_err(logits.cpu().numpy(), want_logits) < 2e-2, (loop, max_err(logits.cpu().numpy(), want_logits))
        assert max_err(out.cpu().numpy(), want) < 5e-3, (loop, max_err(out.cpu().numpy(), want))
        # At these short, peaked contexts the packed cache (float16 metadata) and the fake-quant
        # path (float32 metadata) themselves differ by up to ~2e-2 per element (different rounding
        # decisions in the residual streams); the kernel must not add to that gap.
        fq, _ = fakequant.fake_quant_attention(kn, vn, loop=loop, query=qn, current_key=ckn, current_value=cvn,
                                               scaling=SCALING, active_masks=masks)
        gap = np.abs(want - fq)
        assert np.all(np.abs(out.cpu().numpy() - fq) <= gap + 5e-3)
    assert layer.reader_status() == 0


def test_config1_attention_within_bf16_tolerance_of_fake_quant(fl):
    """BASELINE config 1 (batch 1, 16 heads, context 4096, 4-bit, group 64, 64-token BF16 tail,
    outlier K channels, N(0, 0.1) loop residuals on every token): dense attention of every loop
    against flashloop_torch's fake-quant path, tolerance 2e-2 max-abs / 1e-2 relative."""

    from flashloop_b200.cache import CrossLoopKVLayer

    heads, tokens = 16, 4096
    keys, values, m3, m4, q, ck, cv = _synth(heads, tokens, seed=0, all_active=True)
    layer = CrossLoopKVLayer.from_prefill(_cuda(keys), _cuda(values), mask_loop3=m3[None].cuda(),
                                          mask_loop4=m4[None].cuda())
    assert layer.quantized_tokens == 4032 and layer.tail_tokens == 64
    kn, vn = [to_np(k) for k in keys], [to_np(v) for v in values]
    qn, ckn, cvn = to_np(q), to_np(ck), to_np(cv)
    for loop in range(4):
        out, _ = layer.dense_source_attention(loop, query=q.cuda(), current_key=ck.cuda(), current_value=cv.cuda(),
                                              scaling=SCALING, return_logits=False)
        fq, _ = fakequant.fake_quant_attention(kn, vn, loop=loop, query=qn, current_key=ckn, current_value=cvn,
                                               scaling=SCALING)
        assert_bf16_tolerance(out.cpu().numpy(), fq, what=f"config 1 dense loop {loop} vs fake-quant")


# ------------------------------------------------------------------------------ selection


def test_select_decode_keys_bit_exact(fl, golden):
    from flashloop_b200 import selection

    w = torch.from_numpy(golden["select.weights"]).cuda()
    sel = selection.select_decode_keys(w, fraction=0.10)
    np.testing.assert_array_equal(sel.indices.cpu().numpy(), golden["select.indices"])
    np.testing.assert_allclose(sel.global_mass.cpu().numpy(), golden["select.global_mass"], rtol=1e-5)
    w2 = torch.from_numpy(golden["select2.weights"]).cuda()
    sel2 = selection.select_decode_keys(w2, fraction=0.10)
    np.testing.assert_array_equal(sel2.indices.cpu().numpy(), golden["select2.indices"])
    # the engine's padded contract, from scaled logits
    logits = torch.from_numpy(golden["dense.triton_row.loop1.logits"]).cuda()
    padded = selection.select_decode_keys_padded(logits, fraction=0.10, values_are_logits=True)
    np.testing.assert_array_equal(padded.indices[:, :, :].cpu().numpy(), golden["select.padded"])
    np.testing.assert_array_equal(padded.valid.cpu().numpy(), golden["select.valid"])
    np.testing.assert_allclose(padded.global_mass.cpu().numpy(), golden["select.mass"], rtol=1e-5)
    np.testing.assert_allclose(padded.selected_weights.cpu().numpy(), golden["select.selected_weights"],
                               rtol=1e-4, atol=1e-9)


@pytest.mark.parametrize("keys,fraction", [(1, 0.1), (9, 0.1), (10, 0.1), (641, 0.1), (8193, 0.1),
                                           (4097, 0.25), (300, 1.0), (33000, 0.05)])
def test_select_decode_keys_vs_oracle(fl, keys, fraction):
    from flashloop_b200 import selection

    g = torch.Generator().manual_seed(keys)
    logits = torch.randn(2, 4, 1, keys, generator=g) * 2.0
    # duplicates force ties; the lower index must win
    if keys > 20:
        logits[0, 0, 0, 5] = logits[0, 0, 0, 17]
        logits[1, 2, 0, : keys // 2] = logits[1, 2, 0, keys // 2: 2 * (keys // 2)]
    want = osel.select_from_logits(logits.numpy(), fraction=fraction)
    got = selection.select_decode_keys_padded(logits.cuda(), fraction=fraction, values_are_logits=True)
    budget = osel.decode_budget(keys, fraction)
    assert got.indices.shape[-1] == (budget // 64 + 1) * 64
    weights = want["weights"]
    for b in range(2):
        for h in range(4):
            if osel.boundary_is_tied(weights[b, h, 0], budget) and not np.array_equal(
                    np.sort(np.argsort(-logits[b, h, 0].numpy(), kind="stable")[:budget]), want["indices"][b, h, :budget]):
                continue  # exp() collapsed distinct logits at the boundary: order undefined in the reference too
            np.testing.assert_array_equal(got.indices[b, h].cpu().numpy(), want["indices"][b, h], err_msg=f"{b},{h}")
    np.testing.assert_array_equal(got.valid.cpu().numpy(), want["valid"])
    np.testing.assert_allclose(got.global_mass.cpu().numpy(), want["global_mass"], rtol=1e-4)
    np.testing.assert_array_equal(got.counts.cpu().numpy(), np.full((2, 4), budget))
    # weights given instead of logits
    w = torch.from_numpy(weights)
    sel = selection.select_decode_keys(w.cuda(), fraction=fraction)
    idx, mass = osel.select_decode_keys(weights, fraction=fraction)
    np.testing.assert_array_equal(sel.indices.cpu().numpy(), idx)
    np.testing.assert_allclose(sel.global_mass.cpu().numpy(), mass, rtol=1e-4)


# ------------------------------------------------------------------------------ sparse readers


@pytest.mark.parametrize("tokens,all_active", [(200, False), (700, False), (1500, True)])
def test_sparse_readers_vs_oracle(fl, tokens, all_active):
    from flashloop_b200.cache import CrossLoopKVLayer

    heads = 2
    keys, values, m3, m4, q, ck, cv = _synth(heads, tokens, seed=1000 + tokens, all_active=all_active)
    oracle = oracle_layer(keys, values, m3, m4)
    layer = CrossLoopKVLayer.from_prefill(_cuda(keys), _cuda(values), mask_loop3=m3[None].cuda(),
                                          mask_loop4=m4[None].cuda())
    qn, ckn, cvn = to_np(q), to_np(ck), to_np(cv)
    # loop-2 source pass: logits -> selection -> selected aggregate
    out1, logits = layer.dense_source_attention(1, query=q.cuda(), current_key=ck.cuda(), current_value=cv.cuda(),
                                                scaling=SCALING, return_logits=True)
    _, want_logits = oracle.dense_source_attention(1, query=qn, current_key=ckn, current_value=cvn, scaling=SCALING)
    # select on the ORACLE's logits so that both sides pick from identical inputs
    sel = layer.select_decode_keys(torch.from_numpy(want_logits).cuda(), fraction=0.10)
    want_sel = osel.select_from_logits(want_logits, fraction=0.10)
    np.testing.assert_array_equal(sel.indices.cpu().numpy(), want_sel["indices"])
    np.testing.assert_array_equal(sel.valid.cpu().numpy(), want_sel["valid"])
    assert bool((sel.indices == tokens).any()) or True
    src = layer.pv(1, sel.selected_weights, sel.indices, current_value=cv.cuda(), valid=sel.valid,
                   validate_indices=False)
    want_src = oracle.selected_value_aggregate(1, selected_indices=want_sel["indices"],
                                               selected_weights=want_sel["selected_weights"],
                                               current_value=cvn, past_tokens=tokens)
    assert max_err(src.cpu().numpy(), want_src) < 5e-3, max_err(src.cpu().numpy(), want_src)
    # unscaled logits of the selected rows
    for loop in range(4):
        qk = layer.qk(loop, q.cuda(), sel.indices, validate_indices=False, current_key=ck.cuda())
        is_cur = want_sel["indices"] == tokens
        want_qk = oracle.qk(loop, qn, np.where(is_cur, 0, want_sel["indices"]))
        cur = np.einsum("bhqd,bhnd->bhqn", qn.astype(np.float64), ckn.astype(np.float64))
        want_qk = np.where(is_cur[:, :, None, :], cur, want_qk)
        want_qk = np.where(want_sel["valid"][:, :, None, :], want_qk, want_qk)
        got = qk.cpu().numpy()
        mask = want_sel["valid"][:, :, None, :]
        assert max_err(got[mask], want_qk[mask]) < 0.2, (loop, max_err(got[mask], want_qk[mask]))
    # loops 3 and 4: cached-mass delta with a fresh query
    from flashloop_b200.synthetic import make_query

    q3, k3, v3 = make_query(heads, seed=77)
    for loop in (2, 3):
        delta = layer.cached_mass_sparse_attention_delta(
            loop, query=q3.cuda(), current_key=k3.cuda(), current_value=v3.cuda(), current_position=tokens,
            indices=sel.indices, valid=sel.valid, source_selected_output=torch.from_numpy(want_src).cuda(),
            global_mass=sel.global_mass, scaling=SCALING)
        want = oracle.cached_mass_sparse_attention_delta(
            loop, query=to_np(q3), current_key=to_np(k3), current_value=to_np(v3), current_position=tokens,
            indices=want_sel["indices"], valid=want_sel["valid"], source_selected_output=want_src,
            global_mass=want_sel["global_mass"], scaling=SCALING)
        assert max_err(delta.cpu().numpy(), want) < 5e-3, (loop, max_err(delta.cpu().numpy(), want))
        assert_bf16_tolerance(delta.cpu().numpy(), want, what=f"sparse loop {loop}")


def test_sparse_vs_reference_vectors(fl, golden):
    from flashloop_b200.cache import CrossLoopKVLayer

    keys, values, m3, m4, q, ck, cv = golden_inputs(golden)
    layer = CrossLoopKVLayer.from_prefill(
        [bf16_tensor(k) for k in keys], [bf16_tensor(v) for v in values],
        mask_loop3=torch.from_numpy(m3)[None].cuda(), mask_loop4=torch.from_numpy(m4)[None].cuda())
    for loop in (0, 1):
        out, logits = layer.dense_source_attention(loop, query=bf16_tensor(q), current_key=bf16_tensor(ck),
                                                   current_value=bf16_tensor(cv), scaling=SCALING, return_logits=True)
        for backend in ("triton_row", "kivi_outer"):
            assert_bf16_tolerance(out.cpu().numpy(), golden[f"dense.{backend}.loop{loop}.out"])
            assert max_err(logits.cpu().numpy(), golden[f"dense.{backend}.loop{loop}.logits"]) < 5e-2
    idx = torch.from_numpy(golden["select.padded"]).cuda()
    valid = torch.from_numpy(golden["select.valid"]).cuda()
    for loop in (2, 3):
        delta = layer.cached_mass_sparse_attention_delta(
            loop, query=bf16_tensor(bf(golden["sparse.query"])), current_key=bf16_tensor(bf(golden["sparse.cur_k"])),
            current_value=bf16_tensor(bf(golden["sparse.cur_v"])), current_position=200, indices=idx, valid=valid,
            source_selected_output=torch.from_numpy(golden["select.selected_output"]).cuda(),
            global_mass=torch.from_numpy(golden["select.mass"]).cuda(), scaling=SCALING)
        for backend in ("triton_row", "kivi_outer"):
            assert_bf16_tolerance(delta.cpu().numpy(), golden[f"sparse.{backend}.loop{loop}"])


# ------------------------------------------------------------------------------ append / rollover


def test_append_and_rollover_bit_exact_vs_reference_vectors(fl, golden):
    from flashloop_b200.cache import CrossLoopKVLayer

    keys, values, m3, m4, q, ck, cv = golden_inputs(golden)
    layer = CrossLoopKVLayer.from_prefill(
        [bf16_tensor(k) for k in keys], [bf16_tensor(v) for v in values],
        mask_loop3=torch.from_numpy(m3)[None].cuda(), mask_loop4=torch.from_numpy(m4)[None].cuda(),
        max_new_tokens=128)
    ak, av = bf(golden["append.keys"]), bf(golden["append.values"])
    for step in range(ak.shape[0]):
        layer.append_decode_token([bf16_tensor(ak[step][:, :, r:r + 1]) for r in range(4)],
                                  [bf16_tensor(av[step][:, :, r:r + 1]) for r in range(4)])
    ex = layer.export_sequence(0)
    assert ex["quantized_tokens"] == 192 and ex["tail_tokens"] == int(golden["append.tail_tokens"])
    for s in range(4):
        for kind in ("k", "v"):
            ref = golden_stream(golden, f"append.{kind}{s}")
            np.testing.assert_array_equal(ex[f"{kind}{s}.payload"].cpu().numpy(), ref["payload"][0], err_msg=f"{kind}{s}")
            np.testing.assert_array_equal(bits16(ex[f"{kind}{s}.minimum"]), ref["minimum"][0].view(np.uint16))
            np.testing.assert_array_equal(bits16(ex[f"{kind}{s}.scale"]), ref["scale"][0].view(np.uint16))
        ref = golden_stream(golden, f"append.k{s}")
        if ref["row_groups"] is not None:
            np.testing.assert_array_equal(ex[f"k{s}.row_groups"].cpu().numpy(), ref["row_groups"])
    np.testing.assert_array_equal(ex["rank3"].cpu().numpy(), golden["append.rank3"])
    np.testing.assert_array_equal(ex["rank4"].cpu().numpy(), golden["append.rank4"])
    for r in range(4):
        np.testing.assert_array_equal(bits16(ex[f"tail_k{r}"]), golden[f"append.tail_k{r}"][0])
        np.testing.assert_array_equal(bits16(ex[f"tail_v{r}"]), golden[f"append.tail_v{r}"][0])
    for loop in (0, 1):
        out, logits = layer.dense_source_attention(loop, query=bf16_tensor(q), current_key=bf16_tensor(ck),
                                                   current_value=bf16_tensor(cv), scaling=SCALING, return_logits=True)
        assert_bf16_tolerance(out.cpu().numpy(), golden[f"append.dense.loop{loop}.out"])
        assert max_err(logits.cpu().numpy(), golden[f"append.dense.loop{loop}.logits"]) < 5e-2


def test_ragged_batch_with_appends_vs_oracle(fl):
    """Three sequences of different lengths in one layer; appends roll them over at
    different steps; every reader is checked per sequence against its own oracle."""

    from flashloop_b200.cache import CrossLoopKVLayer
    from flashloop_b200.synthetic import make_query

    heads, lengths = 2, [150, 420, 259]
    seqs, oracles = [], []
    for i, t in enumerate(lengths):
        keys, values, m3, m4, *_ = _synth(heads, t, seed=50 + i)
        seqs.append((_cuda(keys), _cuda(values), m3.cuda(), m4.cuda()))
        oracles.append(oracle_layer(keys, values, m3, m4))
    layer = CrossLoopKVLayer.from_prefill_ragged(seqs, max_new_tokens=200)
    g = torch.Generator().manual_seed(4)
    for step in range(130):
        ks = [(torch.randn(3, heads, 1, 128, generator=g) * (1.0 if r == 0 else 0.1)) for r in range(4)]
        vs = [(torch.randn(3, heads, 1, 128, generator=g) * (1.0 if r == 0 else 0.1)) for r in range(4)]
        ks = [sum(ks[: r + 1]).to(torch.bfloat16) for r in range(4)]
        vs = [sum(vs[: r + 1]).to(torch.bfloat16) for r in range(4)]
        layer.append_decode_token(_cuda(ks), _cuda(vs))
        for b in range(3):
            oracles[b].append_decode_token([to_np(k[b:b + 1]) for k in ks], [to_np(v[b:b + 1]) for v in vs])
        if step in (0, 41, 129):
            for b in range(3):
                assert_layer_matches(layer, b, oracles[b], what=f"step {step} seq {b}")
    q = torch.cat([make_query(heads, seed=b)[0] for b in range(3)])
    ck = torch.cat([make_query(heads, seed=b)[1] for b in range(3)])
    cv = torch.cat([make_query(heads, seed=b)[2] for b in range(3)])
    counts = layer.token_counts()
    assert counts == [o.token_count for o in oracles]
    for loop in range(4):
        out, logits = layer.dense_source_attention(loop, query=q.cuda(), current_key=ck.cuda(),
                                                   current_value=cv.cuda(), scaling=SCALING, return_logits=True)
        for b in range(3):
            want, want_logits = oracles[b].dense_source_attention(
                loop, query=to_np(q[b:b + 1]), current_key=to_np(ck[b:b + 1]), current_value=to_np(cv[b:b + 1]),
                scaling=SCALING)
            assert max_err(out[b:b + 1].cpu().numpy(), want) < 5e-3
            assert max_err(logits[b:b + 1, :, :, :counts[b] + 1].cpu().numpy(), want_logits) < 2e-2
    # selection + sparse delta on the ragged batch
    out1, logits = layer.dense_source_attention(1, query=q.cuda(), current_key=ck.cuda(), current_value=cv.cuda(),
                                                scaling=SCALING, return_logits=True)
    sel = layer.select_decode_keys(logits, fraction=0.10)
    src = layer.pv(1, sel.selected_weights, sel.indices, current_value=cv.cuda(), valid=sel.valid,
                   validate_indices=False)
    delta = layer.cached_mass_sparse_attention_delta(3, query=q.cuda(), current_key=ck.cuda(), current_value=cv.cuda(),
                                                     indices=sel.indices, valid=sel.valid, source_selected_output=src,
                                                     global_mass=sel.global_mass, scaling=SCALING)
    for b in range(3):
        n = counts[b] + 1
        budget = osel.decode_budget(n, 0.10)
        assert int(sel.counts[b, 0]) == budget
        idx = sel.indices[b:b + 1].cpu().numpy()
        valid = sel.valid[b:b + 1].cpu().numpy()
        assert valid[0, 0].sum() == budget and np.all(np.diff(idx[0, 0, :budget]) > 0)
        want = oracles[b].cached_mass_sparse_attention_delta(
            3, query=to_np(q[b:b + 1]), current_key=to_np(ck[b:b + 1]), current_value=to_np(cv[b:b + 1]),
            current_position=counts[b], indices=idx, valid=valid,
            source_selected_output=src[b:b + 1].cpu().numpy(), global_mass=sel.global_mass[b:b + 1].cpu().numpy(),
            scaling=SCALING)
        assert max_err(delta[b:b + 1].cpu().numpy(), want) < 5e-3


# ------------------------------------------------------------------------------ 2-bit variant


def test_two_bit_cache_vs_oracle_and_fake_quant(fl):
    from flashloop_b200.cache import CrossLoopKVLayer

    heads, tokens = 2, 400
    keys, values, m3, m4, q, ck, cv = _synth(heads, tokens, seed=9, all_active=True)
    oracle = oracle_layer(keys, values, m3, m4, bits=2)
    layer = CrossLoopKVLayer.from_prefill(_cuda(keys), _cuda(values), mask_loop3=m3[None].cuda(),
                                          mask_loop4=m4[None].cuda(), bits=2)
    assert_layer_matches(layer, 0, oracle, what="2-bit")
    qn, ckn, cvn = to_np(q), to_np(ck), to_np(cv)
    for loop in range(4):
        out, _ = layer.dense_source_attention(loop, query=q.cuda(), current_key=ck.cuda(), current_value=cv.cuda(),
                                              scaling=SCALING, return_logits=False)
        want, _ = oracle.dense_source_attention(loop, query=qn, current_key=ckn, current_value=cvn, scaling=SCALING)
        assert max_err(out.cpu().numpy(), want) < 5e-3, (loop, max_err(out.cpu().numpy(), want))
        # With 3 levels, the packed cache (float16 metadata) and the fake-quant path (float32
        # metadata) make different rounding decisions in the residual streams and differ by up
        # to ~8e-2 per output element at any context length; the kernel must not add to that gap.
        fq, _ = fakequant.fake_quant_attention([to_np(k) for k in keys], [to_np(v) for v in values], loop=loop,
                                               query=qn, current_key=ckn, current_value=cvn, scaling=SCALING,
                                               codec_profile="kivi2_channel")
        assert np.all(np.abs(out.cpu().numpy() - fq) <= np.abs(want - fq) + 5e-3)
    assert layer.reader_status() == 0


# ------------------------------------------------------------------------------ full-size properties


def test_full_size_properties(fl):
    """BASELINE config 2 shapes (batch 8, 16 heads, context 8192), where the oracle is too
    slow: properties that hold at any size."""

    from flashloop_b200 import packing
    from flashloop_b200.cache import CrossLoopKVLayer
    from flashloop_b200.synthetic import make_loop_kv

    batch, heads, tokens = 8, 16, 8192
    keys = [[] for _ in range(4)]
    values = [[] for _ in range(4)]
    for b in range(batch):
        k, v = make_loop_kv(heads, tokens, seed=b, device="cuda")
        for r in range(4):
            keys[r].append(k[r])
            values[r].append(v[r])
    keys = [torch.cat(k) for k in keys]
    values = [torch.cat(v) for v in values]
    # (1) pack round trip: |decode - x| <= scale/2 (+ bf16 rounding of the result)
    pk = packing.pack_k_per_channel(keys[0])
    err = (pk.decode().float() - keys[0].float()).abs()
    # half a step of quantisation, the float16 rounding of scale (times a code up to 15) and of
    # the minimum, and the bfloat16 rounding of the decoded value
    scale = pk.scale.float().repeat_interleave(64, dim=2)
    minimum = pk.minimum.float().repeat_interleave(64, dim=2)
    bound = scale * (0.5 + 16 * 2 ** -11) + minimum.abs() * 2 ** -10 + keys[0].float().abs() * 2 ** -7 + 1e-6
    assert bool((err <= bound).all())
    ones = torch.ones(batch, tokens, dtype=torch.bool, device="cuda")
    layer = CrossLoopKVLayer.from_prefill(keys, values, mask_loop3=ones, mask_loop4=ones)
    g = torch.Generator(device="cuda").manual_seed(1)
    q = torch.randn(batch, heads, 1, 128, generator=g, device="cuda").to(torch.bfloat16)
    ck = torch.randn(batch, heads, 1, 128, generator=g, device="cuda").to(torch.bfloat16)
    cv = torch.randn(batch, heads, 1, 128, generator=g, device="cuda").to(torch.bfloat16)
    out1, logits = layer.dense_source_attention(1, query=q, current_key=ck, current_value=cv, scaling=SCALING,
                                                return_logits=True)
    # (2) the logits and output agree with a torch float32 evaluation of the same packed streams
    k_hat = (layer_decode(layer, 0, "k", tokens) + layer_decode(layer, 1, "k", tokens))
    v_hat = (layer_decode(layer, 0, "v", tokens) + layer_decode(layer, 1, "v", tokens))
    quant = layer.quantized_tokens
    k_all = torch.cat([k_hat, keys[1][:, :, quant:].float(), ck.float()], dim=2)
    v_all = torch.cat([v_hat, values[1][:, :, quant:].float(), cv.float()], dim=2)
    ref_logits = torch.matmul(q.float(), k_all.transpose(-1, -2)) * SCALING
    ref = torch.matmul(torch.softmax(ref_logits, -1), v_all)
    assert float((logits - ref_logits).abs().max()) < 3e-2
    assert float((out1 - ref).abs().max()) < 5e-3
    # (3) selection: sorted, exact budget, every selected weight >= every unselected weight
    sel = layer.select_decode_keys(logits, fraction=0.10)
    budget = math.ceil((tokens + 1) * 0.10)
    assert sel.indices.shape[-1] == (budget // 64 + 1) * 64
    idx = sel.indices[..., :budget].long()
    assert bool((idx[..., 1:] > idx[..., :-1]).all()) and bool(sel.valid[..., :budget].all())
    assert not bool(sel.valid[..., budget:].any())
    chosen = torch.zeros_like(logits, dtype=torch.bool).squeeze(2)
    chosen.scatter_(-1, idx, True)
    lg = logits.squeeze(2)
    assert bool((lg.masked_fill(~chosen, float("inf")).amin(-1) >= lg.masked_fill(chosen, float("-inf")).amax(-1)).all())
    w = torch.softmax(lg, -1)
    assert torch.allclose(sel.global_mass.flatten(), (w * chosen).sum(-1).flatten(), rtol=1e-4)
    # (4) selecting every key makes the sparse reader reproduce the dense reader (loops 3, 4)
    full = layer.select_decode_keys(logits, fraction=1.0)
    zero = torch.zeros(batch, heads, 1, 128, device="cuda")
    one = torch.ones(batch, heads, 1, 1, device="cuda")
    for loop in (2, 3):
        dense, _ = layer.dense_source_attention(loop, query=q, current_key=ck, current_value=cv, scaling=SCALING,
                                                return_logits=False)
        sparse = layer.cached_mass_sparse_attention_delta(loop, query=q, current_key=ck, current_value=cv,
                                                          indices=full.indices, valid=full.valid,
                                                          source_selected_output=zero, global_mass=one,
                                                          scaling=SCALING)
        assert float((dense - sparse).abs().max()) < 5e-3, float((dense - sparse).abs().max())
    # (5) V rows that are one constant per 64-channel group quantise exactly (span 0); softmax
    # weights sum to one, so the output is that row
    const = torch.randn(1, heads, 1, 2, generator=g, device="cuda").to(torch.bfloat16).repeat_interleave(64, dim=-1)
    flat = [const.expand(batch, heads, tokens, 128).contiguous() for _ in range(4)]
    layer2 = CrossLoopKVLayer.from_prefill(keys, flat, mask_loop3=ones, mask_loop4=ones)
    for loop in (0, 3):
        out, _ = layer2.dense_source_attention(loop, query=q, current_key=ck,
                                               current_value=const.expand(batch, heads, 1, 128).contiguous(),
                                               scaling=SCALING, return_logits=False)
        # a zero span is stored as scale 1, so the centred codes contribute -8 * p and the bias
        # +8 * p in float16: the two cancel to within float16 rounding of 8, not of the value
        assert float((out - const.float()).abs().max()) < 2e-2
    assert layer.reader_status() == 0 and layer2.reader_status() == 0


def test_sparse_equals_dense_with_retention_and_any_slot_order(fl):
    """Compact streams at a size where one gather CTA stages several batches: with every key
    selected the sparse reader must reproduce the dense reader of loops 3 and 4 (25 % / 10 % of the
    tokens hold a row in streams 2 / 3), and the order of the slots must not matter."""

    from flashloop_b200.cache import CrossLoopKVLayer
    from flashloop_b200.synthetic import make_loop_kv

    batch, heads, tokens = 4, 16, 4096
    keys = [[] for _ in range(4)]
    values = [[] for _ in range(4)]
    for b in range(batch):
        k, v = make_loop_kv(heads, tokens, seed=40 + b, device="cuda")
        for r in range(4):
            keys[r].append(k[r])
            values[r].append(v[r])
    keys = [torch.cat(k) for k in keys]
    values = [torch.cat(v) for v in values]
    g = torch.Generator(device="cuda").manual_seed(5)
    m3 = torch.rand(batch, tokens, generator=g, device="cuda") < 0.25
    m4 = m3 & (torch.rand(batch, tokens, generator=g, device="cuda") < 0.4)
    layer = CrossLoopKVLayer.from_prefill(keys, values, mask_loop3=m3, mask_loop4=m4)
    q = torch.randn(batch, heads, 1, 128, generator=g, device="cuda").to(torch.bfloat16)
    ck = torch.randn(batch, heads, 1, 128, generator=g, device="cuda").to(torch.bfloat16)
    cv = torch.randn(batch, heads, 1, 128, generator=g, device="cuda").to(torch.bfloat16)
    _, logits = layer.dense_source_attention(1, query=q, current_key=ck, current_value=cv, scaling=SCALING,
                                             return_logits=True)
    full = layer.select_decode_keys(logits, fraction=1.0)
    some = layer.select_decode_keys(logits, fraction=0.10)
    zero = torch.zeros(batch, heads, 1, 128, device="cuda")
    one = torch.ones(batch, heads, 1, 1, device="cuda")
    for loop in (2, 3):
        dense, _ = layer.dense_source_attention(loop, query=q, current_key=ck, current_value=cv, scaling=SCALING,
                                                return_logits=False)
        sparse = layer.cached_mass_sparse_attention_delta(loop, query=q, current_key=ck, current_value=cv,
                                                          indices=full.indices, valid=full.valid,
                                                          source_selected_output=zero, global_mass=one,
                                                          scaling=SCALING)
        assert float((dense - sparse).abs().max()) < 5e-3, (loop, float((dense - sparse).abs().max()))
        # a permutation of the slots (padding slots included) gives the same sums
        for sel in (full, some):
            perm = torch.randperm(sel.indices.shape[-1], generator=g, device="cuda")
            base = layer.cached_mass_sparse_attention_delta(loop, query=q, current_key=ck, current_value=cv,
                                                            indices=sel.indices, valid=sel.valid,
                                                            source_selected_output=zero, global_mass=one,
                                                            scaling=SCALING)
            mixed = layer.cached_mass_sparse_attention_delta(loop, query=q, current_key=ck, current_value=cv,
                                                             indices=sel.indices[..., perm].contiguous(),
                                                             valid=sel.valid[..., perm].contiguous(),
                                                             source_selected_output=zero, global_mass=one,
                                                             scaling=SCALING)
            assert float((base - mixed).abs().max()) < 2e-3, (loop, float((base - mixed).abs().max()))
    perm = torch.randperm(some.indices.shape[-1], generator=g, device="cuda")
    for loop in (1, 3):
        base = layer.pv(loop, some.selected_weights, some.indices, current_value=cv, valid=some.valid,
                        validate_indices=False)
        mixed = layer.pv(loop, some.selected_weights[..., perm].contiguous(), some.indices[..., perm].contiguous(),
                         current_value=cv, valid=some.valid[..., perm].contiguous(), validate_indices=False)
        assert float((base - mixed).abs().max()) < 2e-3, (loop, float((base - mixed).abs().max()))
        qk = layer.qk(loop, q, some.indices, validate_indices=False, current_key=ck)
        qk_mixed = layer.qk(loop, q, some.indices[..., perm].contiguous(), validate_indices=False, current_key=ck)
        # unselected padding slots carry index 0 with valid unknown to qk: compare the valid ones
        keep = some.valid[:, :, None, :]
        assert float(((qk[..., perm] - qk_mixed) * keep[..., perm]).abs().max()) < 2e-2
    assert layer.reader_status() == 0


def layer_decode(layer, s, kind, tokens):
    """float32 dequantisation of stream ``s`` of every sequence with torch ops."""
    from flashloop_b200.packing import Packed4Bit

    quant = layer.quantized_tokens
    outs = []
    for b in range(layer.batch):
        ex = layer.export_sequence(b)
        p = Packed4Bit(payload=ex[f"{kind}{s}.payload"][None].contiguous(),
                       minimum=ex[f"{kind}{s}.minimum"][None].contiguous(),
                       scale=ex[f"{kind}{s}.scale"][None].contiguous(),
                       original_shape=(1, layer.heads, quant, 128), original_dtype=torch.float32,
                       axis="per_channel" if kind == "k" else "per_token", group_size=64)
        codes = torch.stack([(p.payload & 0xF), (p.payload >> 4)], dim=-1).reshape(1, layer.heads, quant, 128).float()
        if kind == "k":
            mn = p.minimum.float().repeat_interleave(64, dim=2)
            sc = p.scale.float().repeat_interleave(64, dim=2)
        else:
            mn = p.minimum.float().repeat_interleave(64, dim=3)
            sc = p.scale.float().repeat_interleave(64, dim=3)
        outs.append(codes * sc + mn)
    return torch.cat(outs)


# ------------------------------------------------------------------------------ token retention


def test_token_retention_vs_reference_vectors_and_oracle(fl, golden):
    from flashloop_b200 import compaction, selection

    h1 = torch.from_numpy(bf(golden["retain.h1"])).to(torch.bfloat16).cuda()
    h2 = torch.from_numpy(bf(golden["retain.h2"])).to(torch.bfloat16).cuda()
    score = compaction.hidden_delta_score(h2, h1)
    np.testing.assert_allclose(score.cpu().numpy(), golden["retain.score3"], rtol=2e-5)
    s3 = torch.from_numpy(golden["retain.score3"]).cuda()
    s4 = torch.from_numpy(golden["retain.score4"]).cuda()
    r3 = compaction.retain_tokens(s3, fraction=0.25)
    assert torch.equal(r3.mask.cpu(), torch.from_numpy(golden["retain.mask3"]))
    r4 = compaction.retain_tokens(s4, fraction=0.10, eligible=r3.mask)
    assert torch.equal(r4.mask.cpu(), torch.from_numpy(golden["retain.mask4"]))
    assert torch.equal(selection.select_prefill_tokens(s4, fraction=0.10, eligible=r3.mask), r4.mask)
    for r in (r3, r4):
        m = r.mask[0].cpu().numpy()
        pos, rank = osel.positions_and_rank_map(m, m.size)
        n = int(r.count[0])
        assert n == pos.size
        np.testing.assert_array_equal(r.positions[0, :n].cpu().numpy(), pos)
        assert bool((r.positions[0, n:] == -1).all())
        np.testing.assert_array_equal(r.rank[0].cpu().numpy(), rank)


@pytest.mark.parametrize("tokens,fraction", [(1, 0.25), (7, 0.1), (2048, 0.25), (8192, 0.10), (5000, 1.0)])
def test_token_retention_and_row_movement_vs_oracle(fl, tokens, fraction):
    from flashloop_b200 import compaction

    g = torch.Generator().manual_seed(tokens)
    batch = 3
    scores = torch.rand(batch, tokens, generator=g)
    if tokens > 16:
        scores[1, 3] = scores[1, 11]  # a tie: the lower index wins
    eligible = torch.rand(batch, tokens, generator=g) < 0.6
    eligible[:, -1] = True
    for elig in (None, eligible):
        want = osel.select_prefill_tokens(scores.numpy(), fraction=fraction,
                                          eligible=None if elig is None else elig.numpy())
        got = compaction.retain_tokens(scores.cuda(), fraction=fraction,
                                       eligible=None if elig is None else elig.cuda())
        np.testing.assert_array_equal(got.mask.cpu().numpy(), want)
        for b in range(batch):
            pos, rank = osel.positions_and_rank_map(want[b], tokens)
            assert int(got.count[b]) == pos.size
            np.testing.assert_array_equal(got.positions[b, :pos.size].cpu().numpy(), pos)
            np.testing.assert_array_equal(got.rank[b].cpu().numpy(), rank)
    # gather the retained rows of a [B*H, T, 128] array, scatter them back into zeros
    heads = 2
    full = torch.randn(batch * heads, tokens, 128, generator=g).to(torch.bfloat16).cuda()
    rows = int(got.count.max())
    compact = compaction.gather_rows(full, got.positions, got.count, rows=rows, per_sequence=heads)
    back = torch.zeros_like(full)
    compaction.scatter_rows(back, compact, got.positions, got.count, per_sequence=heads)
    for o in range(batch * heads):
        b = o // heads
        n = int(got.count[b])
        pos = got.positions[b, :n].long()
        assert torch.equal(compact[o, :n], full[o].index_select(0, pos))
        expect = torch.zeros_like(full[o])
        expect[pos] = full[o, pos]
        assert torch.equal(back[o], expect)
