"""Pins the numpy oracle to vectors produced by the reference's own CPU code.

Bit-exact where the contract is integer/byte work (codes, float16 metadata, rank maps,
selected indices); float32 tolerance where the reference sums in a different order.
"""

from __future__ import annotations

import numpy as np
import pytest

from oracle import bf16, fakequant, packing, selection
from oracle.cache import LayerOracle
from tests.helpers import (assert_kivi_equal, assert_rows_equal, bf, f16, golden_inputs,
                           golden_stream)

SCALING = 128 ** -0.5


def _pack_input(g, tag):
    if tag == "bf16":
        return bf(g["in.key0"])
    if tag == "f16":
        return g["pack.f16.input"].view(np.float16).astype(np.float32)
    return g["pack.f32.input"]


@pytest.mark.parametrize("tag", ["bf16", "f16", "f32"])
def test_pack_both_layouts_bit_exact(golden, tag):
    x = _pack_input(golden, tag)
    assert_kivi_equal(packing.pack_kivi_k(x), golden_stream(golden, f"pack.{tag}.kivi_k"), what="kivi k")
    assert_kivi_equal(packing.pack_kivi_v(x), golden_stream(golden, f"pack.{tag}.kivi_v"), what="kivi v")
    assert_rows_equal(packing.pack_k_rows(x), golden_stream(golden, f"pack.{tag}.rows_k"), what="rows k")
    assert_rows_equal(packing.pack_v_rows(x), golden_stream(golden, f"pack.{tag}.rows_v"), what="rows v")


def test_decode_bit_exact_and_layouts_agree(golden):
    x = bf(golden["in.key0"])
    for name, packed in (("kivi_k", packing.pack_kivi_k(x)), ("kivi_v", packing.pack_kivi_v(x)),
                         ("rows_k", packing.pack_k_rows(x)), ("rows_v", packing.pack_v_rows(x))):
        np.testing.assert_array_equal(bf16.to_bits(packed.decode()),
                                      golden[f"pack.bf16.{name}.decode"], err_msg=name)
    k = packing.kivi_to_rows(packing.pack_kivi_k(x))
    assert_rows_equal(k, golden_stream(golden, "pack.bf16.rows_k"), what="kivi->rows k")
    v = packing.kivi_to_rows(packing.pack_kivi_v(x))
    assert_rows_equal(v, golden_stream(golden, "pack.bf16.rows_v"), what="kivi->rows v")


@pytest.fixture(scope="module")
def layer(golden):
    keys, values, m3, m4, *_ = golden_inputs(golden)
    return LayerOracle.from_prefill(keys, values, mask_loop3=m3, mask_loop4=m4)


def test_residual_chain_streams_bit_exact(golden, layer):
    assert layer.quantized_tokens == int(golden["layer.triton_row.quantized_tokens"]) == 128
    for s in range(4):
        assert_rows_equal(layer.keys[s], golden_stream(golden, f"layer.triton_row.k{s}"), what=f"k{s}")
        assert_rows_equal(layer.values[s], golden_stream(golden, f"layer.triton_row.v{s}"), what=f"v{s}")
        # the reference's default backend holds the same codes in the KIVI word layout
        ref = golden_stream(golden, f"layer.kivi_outer.k{s}")
        kivi = packing.PackedKivi(ref["payload"], ref["minimum"], ref["scale"], ref["shape"], "per_channel")
        assert_rows_equal(packing.kivi_to_rows(kivi), golden_stream(golden, f"layer.triton_row.k{s}"))
        ref = golden_stream(golden, f"layer.kivi_outer.v{s}")
        kivi = packing.PackedKivi(ref["payload"], ref["minimum"], ref["scale"], ref["shape"], "per_token")
        assert_rows_equal(packing.kivi_to_rows(kivi), golden_stream(golden, f"layer.triton_row.v{s}"))
    for i, name in enumerate(("pos3", "pos4")):
        np.testing.assert_array_equal(layer.override_indices[i], golden[f"layer.triton_row.{name}"])
    for i, name in enumerate(("rank3", "rank4")):
        np.testing.assert_array_equal(layer.rank_maps[i], golden[f"layer.triton_row.{name}"])
    for r in range(4):
        np.testing.assert_array_equal(bf16.to_bits(layer.tail_keys[r]), golden[f"layer.tail_k{r}"])
        np.testing.assert_array_equal(bf16.to_bits(layer.tail_values[r]), golden[f"layer.tail_v{r}"])
    np.testing.assert_array_equal(layer.tail_active[0], golden["layer.tail_active3"][0])
    np.testing.assert_array_equal(layer.tail_active[1], golden["layer.tail_active4"][0])


def test_gather_matches_reference_bf16_chain(golden, layer):
    for loop in (1, 3):
        k, v = layer.gather(loop, np.arange(layer.token_count), chain_bf16=True)
        np.testing.assert_array_equal(bf16.to_bits(k), golden[f"gather.loop{loop}.k"])
        np.testing.assert_array_equal(bf16.to_bits(v), golden[f"gather.loop{loop}.v"])


@pytest.mark.parametrize("loop", [0, 1])
def test_dense_source_attention(golden, layer, loop):
    *_, q, ck, cv = golden_inputs(golden)
    out, logits = layer.dense_source_attention(loop, query=q, current_key=ck, current_value=cv,
                                               scaling=SCALING, chain_bf16=True)
    np.testing.assert_allclose(out, golden[f"dense.triton_row.loop{loop}.out"], rtol=2e-5, atol=2e-6)
    np.testing.assert_allclose(logits, golden[f"dense.triton_row.loop{loop}.logits"], rtol=2e-5, atol=2e-5)
    # float32 stream sums (what the fused readers compute) stay inside the BF16 tolerance
    out32, _ = layer.dense_source_attention(loop, query=q, current_key=ck, current_value=cv,
                                            scaling=SCALING, chain_bf16=False)
    for backend in ("triton_row", "kivi_outer"):
        np.testing.assert_allclose(out32, golden[f"dense.{backend}.loop{loop}.out"], rtol=1e-2, atol=2e-2)


def test_decode_key_selection_bit_exact(golden):
    w = golden["select.weights"]
    assert not selection.boundary_is_tied(w[0, 0, 0], golden["select.indices"].shape[-1])
    idx, mass = selection.select_decode_keys(w, fraction=0.10)
    np.testing.assert_array_equal(idx, golden["select.indices"])
    np.testing.assert_allclose(mass, golden["select.global_mass"], rtol=1e-6)
    w2 = golden["select2.weights"]
    idx2, mass2 = selection.select_decode_keys(w2, fraction=0.10)
    np.testing.assert_array_equal(idx2, golden["select2.indices"])
    np.testing.assert_allclose(mass2, golden["select2.global_mass"], rtol=1e-6)
    sel = selection.select_from_logits(golden["dense.triton_row.loop1.logits"], fraction=0.10)
    np.testing.assert_array_equal(sel["indices"], golden["select.padded"])
    np.testing.assert_array_equal(sel["valid"], golden["select.valid"])
    np.testing.assert_allclose(sel["global_mass"], golden["select.mass"], rtol=1e-5)
    np.testing.assert_allclose(sel["selected_weights"], golden["select.selected_weights"], rtol=1e-4, atol=1e-9)


def test_selected_qk_pv_and_aggregate(golden, layer):
    *_, q, ck, cv = golden_inputs(golden)
    padded, valid = golden["select.padded"], golden["select.valid"]
    sel_w = golden["select.selected_weights"]
    past = layer.token_count
    is_cur = padded == past
    safe = np.where(is_cur, 0, padded)
    for loop in range(4):
        qk = layer.qk(loop, q, safe, chain_bf16="streams")
        np.testing.assert_allclose(qk, golden[f"qk.triton_row.loop{loop}"], rtol=1e-5, atol=1e-4)
        np.testing.assert_allclose(layer.qk(loop, q, safe), golden[f"qk.kivi_outer.loop{loop}"],
                                   rtol=1e-2, atol=0.25)
        pv = layer.pv(loop, sel_w * (~is_cur)[:, :, None, :], safe, chain_bf16="streams")
        np.testing.assert_allclose(pv, golden[f"pv.triton_row.loop{loop}"], rtol=1e-4, atol=1e-5)
    agg = layer.selected_value_aggregate(1, selected_indices=padded, selected_weights=sel_w,
                                         current_value=cv, past_tokens=past)
    np.testing.assert_allclose(agg, golden["select.selected_output"], rtol=1e-2, atol=5e-3)


@pytest.mark.parametrize("loop", [2, 3])
def test_cached_mass_sparse_delta(golden, layer, loop):
    q, ck, cv = bf(golden["sparse.query"]), bf(golden["sparse.cur_k"]), bf(golden["sparse.cur_v"])
    delta = layer.cached_mass_sparse_attention_delta(
        loop, query=q, current_key=ck, current_value=cv, current_position=layer.token_count,
        indices=golden["select.padded"], valid=golden["select.valid"],
        source_selected_output=golden["select.selected_output"],
        global_mass=golden["select.mass"], scaling=SCALING)
    for backend in ("triton_row", "kivi_outer"):
        np.testing.assert_allclose(delta, golden[f"sparse.{backend}.loop{loop}"], rtol=1e-2, atol=2e-2)


def test_append_and_rollover_bit_exact(golden):
    keys, values, m3, m4, q, ck, cv = golden_inputs(golden)
    layer = LayerOracle.from_prefill(keys, values, mask_loop3=m3, mask_loop4=m4)
    ak, av = bf(golden["append.keys"]), bf(golden["append.values"])  # [70,1,H,4,D]
    for step in range(ak.shape[0]):
        layer.append_decode_token([ak[step][:, :, r:r + 1] for r in range(4)],
                                  [av[step][:, :, r:r + 1] for r in range(4)])
    assert layer.quantized_tokens == int(golden["append.quantized_tokens"]) == 192
    assert layer.tail_tokens == int(golden["append.tail_tokens"])
    for s in range(4):
        ref = golden_stream(golden, f"append.k{s}")
        assert_rows_equal(layer.keys[s], ref, what=f"k{s}")
        if ref["row_groups"] is not None and layer.keys[s].row_groups is not None:
            np.testing.assert_array_equal(layer.keys[s].row_groups, ref["row_groups"])
        assert_rows_equal(layer.values[s], golden_stream(golden, f"append.v{s}"), what=f"v{s}")
    np.testing.assert_array_equal(layer.rank_maps[0], golden["append.rank3"])
    np.testing.assert_array_equal(layer.rank_maps[1], golden["append.rank4"])
    np.testing.assert_array_equal(layer.override_indices[0], golden["append.pos3"])
    for r in range(4):
        np.testing.assert_array_equal(bf16.to_bits(layer.tail_keys[r]), golden[f"append.tail_k{r}"])
        np.testing.assert_array_equal(bf16.to_bits(layer.tail_values[r]), golden[f"append.tail_v{r}"])
    for loop in (0, 1):
        out, logits = layer.dense_source_attention(loop, query=q, current_key=ck, current_value=cv,
                                                   scaling=SCALING, chain_bf16=True)
        np.testing.assert_allclose(out, golden[f"append.dense.loop{loop}.out"], rtol=2e-5, atol=2e-6)
        np.testing.assert_allclose(logits, golden[f"append.dense.loop{loop}.logits"], rtol=2e-5, atol=2e-5)


@pytest.mark.parametrize("profile", ["kivi4_channel", "kivi2_channel"])
def test_fake_quant_codec_bit_exact(golden, profile):
    keys, values, m3, m4, *_ = golden_inputs(golden)
    tq = 128
    rk, rv = fakequant.encode_temporal_group(
        [k[:, :, :tq] for k in keys], [v[:, :, :tq] for v in values],
        active_masks=[np.ones(tq, bool), m3[:tq], m4[:tq]], codec_profile=profile)
    for loop in (1, 3):
        np.testing.assert_array_equal(bf16.to_bits(rk[loop]), golden[f"fq.{profile}.k{loop}"])
        np.testing.assert_array_equal(bf16.to_bits(rv[loop]), golden[f"fq.{profile}.v{loop}"])


def test_packed_cache_within_tolerance_of_fake_quant(golden, layer):
    """The packed cache (float16 metadata) vs the fake-quant path (float32 metadata):
    the BF16 tolerance the readers are held to."""

    keys, values, m3, m4, q, ck, cv = golden_inputs(golden)
    for loop in range(4):
        out, _ = layer.dense_source_attention(loop, query=q, current_key=ck, current_value=cv, scaling=SCALING)
        ref, _ = fakequant.fake_quant_attention(keys, values, loop=loop, query=q, current_key=ck,
                                                current_value=cv, scaling=SCALING,
                                                active_masks=[np.ones(200, bool), m3, m4])
        np.testing.assert_allclose(out, ref, rtol=1e-2, atol=2e-2)


def test_fake_quant_sparse_delta_matches_reference(golden):
    """The oracle's fake-quant definition of the sparse late-loop output against the reference's
    own mass_scaled_sparse_output (flashloop_torch/attention_utils.py:216-248)."""

    keys, values, m3, m4, q, ck, cv = golden_inputs(golden)
    q3, k3, v3 = bf(golden["sparse.query"]), bf(golden["sparse.cur_k"]), bf(golden["sparse.cur_v"])
    got = fakequant.fake_quant_sparse_deltas(
        keys, values, loops=(2, 3), source_query=q, source_current_key=ck, source_current_value=cv,
        query=q3, current_key=k3, current_value=v3, scaling=SCALING, active_masks=[np.ones(200, bool), m3, m4])
    np.testing.assert_array_equal(got["mask"], golden["fqsparse.mask"])
    np.testing.assert_allclose(got["mass"], golden["fqsparse.mass"], rtol=1e-5)
    np.testing.assert_allclose(got["source_subset"], golden["fqsparse.source_subset"], rtol=1e-4, atol=1e-5)
    for loop in (2, 3):
        np.testing.assert_allclose(got["delta"][loop], golden[f"fqsparse.loop{loop}.delta"], rtol=1e-4, atol=1e-5)


def test_packed_sparse_delta_within_tolerance_of_fake_quant(golden, layer):
    """The oracle's exact evaluation of the packed cache against the fake-quant sparse output, on
    the keys, source aggregate and mass of the fake-quant path: the BF16 tolerance the sparse
    reader is held to."""

    keys, values, m3, m4, q, ck, cv = golden_inputs(golden)
    q3, k3, v3 = bf(golden["sparse.query"]), bf(golden["sparse.cur_k"]), bf(golden["sparse.cur_v"])
    ref = fakequant.fake_quant_sparse_deltas(
        keys, values, loops=(2, 3), source_query=q, source_current_key=ck, source_current_value=cv,
        query=q3, current_key=k3, current_value=v3, scaling=SCALING, active_masks=[np.ones(200, bool), m3, m4])
    idx, valid = selection.pad_selected(ref["mask"])
    for loop in (2, 3):
        out = layer.cached_mass_sparse_attention_delta(
            loop, query=q3, current_key=k3, current_value=v3, current_position=200, indices=idx, valid=valid,
            source_selected_output=ref["source_subset"], global_mass=ref["mass"], scaling=SCALING)
        np.testing.assert_allclose(out, ref["delta"][loop], rtol=1e-2, atol=2e-2)


def test_token_retention_bit_exact(golden):
    h1, h2, h3 = bf(golden["retain.h1"]), bf(golden["retain.h2"]), bf(golden["retain.h3"])
    s3 = selection.hidden_delta_score(h2, h1)
    np.testing.assert_allclose(s3, golden["retain.score3"], rtol=1e-5)
    m3 = selection.select_prefill_tokens(golden["retain.score3"], fraction=0.25)
    np.testing.assert_array_equal(m3, golden["retain.mask3"])
    m4 = selection.select_prefill_tokens(golden["retain.score4"], fraction=0.10, eligible=m3)
    np.testing.assert_array_equal(m4, golden["retain.mask4"])
    assert m3.sum() == 75 and m4.sum() == 30 and m3[0, -1] and m4[0, -1]
    assert not np.any(m4 & ~m3)
