"""GPU parity at the sizes of the BASELINE configurations, against independent references:

* the sparse late-loop reader against flashloop_torch's fake-quant definition of the sparse
  output (``oracle.fakequant.fake_quant_sparse_deltas``, pinned to the reference's
  ``mass_scaled_sparse_output`` by tests/test_oracle_golden.py), config 1 (16 heads x 4096) and one
  8192-token sequence of config 2 (820 keys), tolerance 2e-2 max-abs / 1e-2 relative;
* two (sequence, head) pairs of the batch-8 x 8192 layer of config 2 against the numpy oracle:
  dense loops 1-4, the selected key indices, the loop-2 aggregate and both sparse loops;
* config 3: a ragged batch holding a 32768-token and a 1024-token sequence, 4-bit and 2-bit,
  two heads each against the oracle.
"""

from __future__ import annotations

import numpy as np
import pytest
import torch

from oracle import fakequant, selection as osel
from oracle.cache import LayerOracle
from tests.gpu_util import assert_bf16_tolerance, max_err, to_np

pytestmark = pytest.mark.gpu

SCALING = 128 ** -0.5


@pytest.fixture(scope="module")
def fl():
    import flashloop_b200 as pkg
    from flashloop_b200 import _native

    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    _native.load()
    return pkg


def _cuda(ts):
    return [t.cuda() for t in ts]


def _sparse_vs_fake_quant(heads: int, tokens: int, seed: int, what: str):
    from flashloop_b200.cache import CrossLoopKVLayer
    from flashloop_b200.synthetic import make_loop_kv, make_masks, make_query

    keys, values = make_loop_kv(heads, tokens, seed=seed)
    m3, m4 = make_masks(tokens, seed=seed, all_active=True)
    q, ck, cv = make_query(heads, seed=seed)
    q3, k3, v3 = make_query(heads, seed=seed + 1)
    layer = CrossLoopKVLayer.from_prefill(_cuda(keys), _cuda(values), mask_loop3=m3[None].cuda(),
                                          mask_loop4=m4[None].cuda())
    kn, vn = [to_np(k) for k in keys], [to_np(v) for v in values]
    ref = fakequant.fake_quant_sparse_deltas(
        kn, vn, loops=(2, 3), source_query=to_np(q), source_current_key=to_np(ck), source_current_value=to_np(cv),
        query=to_np(q3), current_key=to_np(k3), current_value=to_np(v3), scaling=SCALING)
    idx, valid = osel.pad_selected(ref["mask"])
    assert int(valid[0, 0].sum()) == osel.decode_budget(tokens + 1, 0.10)
    for loop in (2, 3):
        delta = layer.cached_mass_sparse_attention_delta(
            loop, query=q3.cuda(), current_key=k3.cuda(), current_value=v3.cuda(),
            indices=torch.from_numpy(idx).cuda(), valid=torch.from_numpy(valid).cuda(),
            source_selected_output=torch.from_numpy(ref["source_subset"]).cuda(),
            global_mass=torch.from_numpy(ref["mass"]).cuda(), scaling=SCALING)
        assert_bf16_tolerance(delta.cpu().numpy(), ref["delta"][loop], what=f"{what} sparse loop {loop + 1} vs fake-quant")
    assert layer.reader_status() == 0


def test_config1_sparse_delta_within_bf16_tolerance_of_fake_quant(fl):
    """BASELINE config 1 (batch 1, 16 heads, context 4096): loops 3 and 4 through the sparse reader
    against flashloop_torch's fake-quant sparse output on the same keys, source aggregate and mass."""

    _sparse_vs_fake_quant(16, 4096, seed=0, what="config 1")


def test_config2_sequence_sparse_delta_within_bf16_tolerance_of_fake_quant(fl):
    """One sequence of BASELINE config 2 (16 heads, context 8192, 820 selected keys)."""

    _sparse_vs_fake_quant(16, 8192, seed=2, what="config 2")


def test_config2_batch_pairs_vs_oracle(fl):
    """The batch-8 x 16-head x 8192-token layer of BASELINE config 2 on the GPU; sequences 5 / 2,
    heads 3 / 11 are rebuilt as one-head oracles and every reader of the decode step is compared
    for them: dense loops 1-4, the loop-2 selection, its value aggregate and the sparse loops."""

    from flashloop_b200.cache import CrossLoopKVLayer
    from flashloop_b200.synthetic import make_loop_kv

    batch, heads, tokens = 8, 16, 8192
    per_seq = [make_loop_kv(heads, tokens, seed=b, device="cuda") for b in range(batch)]
    keys = [torch.cat([per_seq[b][0][r] for b in range(batch)]) for r in range(4)]
    values = [torch.cat([per_seq[b][1][r] for b in range(batch)]) for r in range(4)]
    gen = torch.Generator().manual_seed(12)
    m3 = torch.rand(batch, tokens, generator=gen) < 0.25
    m4 = m3 & (torch.rand(batch, tokens, generator=gen) < 0.4)
    m3[:, -1] = True
    m4[:, -1] = True
    layer = CrossLoopKVLayer.from_prefill(keys, values, mask_loop3=m3.cuda(), mask_loop4=m4.cuda())
    q, ck, cv = (torch.randn(batch, heads, 1, 128, generator=gen).to(torch.bfloat16) for _ in range(3))
    q3, k3, v3 = (torch.randn(batch, heads, 1, 128, generator=gen).to(torch.bfloat16) for _ in range(3))
    outs, logits = {}, None
    for loop in range(4):
        outs[loop], lg = layer.dense_source_attention(loop, query=q.cuda(), current_key=ck.cuda(),
                                                      current_value=cv.cuda(), scaling=SCALING, return_logits=loop == 1)
        logits = lg if loop == 1 else logits
    for b, h in ((5, 3), (2, 11)):
        pick = lambda t: to_np(t[b:b + 1, h:h + 1])
        oracle = LayerOracle.from_prefill([to_np(per_seq[b][0][r][:, h:h + 1]) for r in range(4)],
                                          [to_np(per_seq[b][1][r][:, h:h + 1]) for r in range(4)],
                                          mask_loop3=m3[b].numpy(), mask_loop4=m4[b].numpy())
        want_logits = None
        for loop in range(4):
            want, wl = oracle.dense_source_attention(loop, query=pick(q), current_key=pick(ck), current_value=pick(cv),
                                                     scaling=SCALING)
            assert max_err(outs[loop][b:b + 1, h:h + 1].cpu().numpy(), want) < 5e-3, (b, h, loop)
            if loop == 1:
                want_logits = wl
                assert max_err(logits[b:b + 1, h:h + 1].cpu().numpy(), wl) < 2e-2
        # selection on the oracle's logits, so that both sides choose from identical inputs
        full_logits = logits.clone()
        full_logits[b, h] = torch.from_numpy(want_logits[0, 0]).cuda()
        sel = layer.select_decode_keys(full_logits, fraction=0.10)
        want_sel = osel.select_from_logits(want_logits, fraction=0.10)
        np.testing.assert_array_equal(sel.indices[b, h].cpu().numpy(), want_sel["indices"][0, 0])
        np.testing.assert_array_equal(sel.valid[b, h].cpu().numpy(), want_sel["valid"][0, 0])
        assert int(want_sel["valid"].sum()) == 820
        src = layer.pv(1, sel.selected_weights, sel.indices, current_value=cv.cuda(), valid=sel.valid,
                       validate_indices=False)
        want_src = oracle.selected_value_aggregate(1, selected_indices=want_sel["indices"],
                                                   selected_weights=want_sel["selected_weights"],
                                                   current_value=pick(cv), past_tokens=tokens)
        assert max_err(src[b:b + 1, h:h + 1].cpu().numpy(), want_src) < 5e-3
        for loop in (2, 3):
            delta = layer.cached_mass_sparse_attention_delta(
                loop, query=q3.cuda(), current_key=k3.cuda(), current_value=v3.cuda(), indices=sel.indices,
                valid=sel.valid, source_selected_output=src, global_mass=sel.global_mass, scaling=SCALING)
            want = oracle.cached_mass_sparse_attention_delta(
                loop, query=pick(q3), current_key=pick(k3), current_value=pick(v3), current_position=tokens,
                indices=want_sel["indices"], valid=want_sel["valid"],
                source_selected_output=src[b:b + 1, h:h + 1].cpu().numpy(),
                global_mass=sel.global_mass[b:b + 1, h:h + 1].cpu().numpy(), scaling=SCALING)
            assert max_err(delta[b:b + 1, h:h + 1].cpu().numpy(), want) < 5e-3, (b, h, loop)
            assert_bf16_tolerance(delta[b:b + 1, h:h + 1].cpu().numpy(), want, what=f"config 2 sparse loop {loop + 1}")
    assert layer.reader_status() == 0


@pytest.mark.parametrize("bits", [4, 2])
def test_config3_ragged_long_and_short_vs_oracle(fl, bits):
    """BASELINE config 3 extremes in one ragged layer: a 32768-token, a 1024-token and a
    5000-token sequence, two heads each, loop residuals on every token; every stream bit-exact and
    every reader (dense loops 1-4, selection, aggregate, sparse loops) against the oracle."""

    from flashloop_b200.cache import CrossLoopKVLayer
    from flashloop_b200.synthetic import make_loop_kv, make_query
    from tests.gpu_util import assert_layer_matches, oracle_layer

    heads, lengths = 2, [32768, 1024, 5000]
    seqs, oracles = [], []
    for i, t in enumerate(lengths):
        keys, values = make_loop_kv(heads, t, seed=300 + i)
        ones = torch.ones(t, dtype=torch.bool)
        seqs.append((_cuda(keys), _cuda(values), ones.cuda(), ones.cuda()))
        oracles.append(oracle_layer(keys, values, ones, ones, bits=bits))
    layer = CrossLoopKVLayer.from_prefill_ragged(seqs, bits=bits)
    for b in range(3):
        assert_layer_matches(layer, b, oracles[b], what=f"{bits}-bit seq {b}")
    q = torch.cat([make_query(heads, seed=40 + b)[0] for b in range(3)])
    ck = torch.cat([make_query(heads, seed=40 + b)[1] for b in range(3)])
    cv = torch.cat([make_query(heads, seed=40 + b)[2] for b in range(3)])
    q3 = torch.cat([make_query(heads, seed=50 + b)[0] for b in range(3)])
    want_logits = []
    logits = None
    for loop in range(4):
        out, lg = layer.dense_source_attention(loop, query=q.cuda(), current_key=ck.cuda(), current_value=cv.cuda(),
                                               scaling=SCALING, return_logits=loop == 1)
        logits = lg if loop == 1 else logits
        for b in range(3):
            want, wl = oracles[b].dense_source_attention(loop, query=to_np(q[b:b + 1]), current_key=to_np(ck[b:b + 1]),
                                                         current_value=to_np(cv[b:b + 1]), scaling=SCALING)
            assert max_err(out[b:b + 1].cpu().numpy(), want) < 5e-3, (bits, loop, b)
            if loop == 1:
                want_logits.append(wl)
                assert max_err(lg[b:b + 1, :, :, :lengths[b] + 1].cpu().numpy(), wl) < 2e-2
    # selection over the oracle's logits (ragged: rows beyond a sequence's keys stay -inf)
    merged = torch.full_like(logits, float("-inf"))
    for b in range(3):
        merged[b, :, :, :lengths[b] + 1] = torch.from_numpy(want_logits[b][0]).cuda()
    sel = layer.select_decode_keys(merged, fraction=0.10)
    src = layer.pv(1, sel.selected_weights, sel.indices, current_value=cv.cuda(), valid=sel.valid,
                   validate_indices=False)
    deltas = {loop: layer.cached_mass_sparse_attention_delta(
        loop, query=q3.cuda(), current_key=ck.cuda(), current_value=cv.cuda(), indices=sel.indices, valid=sel.valid,
        source_selected_output=src, global_mass=sel.global_mass, scaling=SCALING) for loop in (2, 3)}
    for b in range(3):
        want_sel = osel.select_from_logits(want_logits[b], fraction=0.10)
        cap = want_sel["indices"].shape[-1]
        np.testing.assert_array_equal(sel.indices[b, :, :cap].cpu().numpy(), want_sel["indices"][0])
        np.testing.assert_array_equal(sel.valid[b, :, :cap].cpu().numpy(), want_sel["valid"][0])
        assert not bool(sel.valid[b, :, cap:].any())
        want_src = oracles[b].selected_value_aggregate(1, selected_indices=want_sel["indices"],
                                                       selected_weights=want_sel["selected_weights"],
                                                       current_value=to_np(cv[b:b + 1]), past_tokens=lengths[b])
        assert max_err(src[b:b + 1].cpu().numpy(), want_src) < 5e-3, (bits, b)
        for loop in (2, 3):
            want = oracles[b].cached_mass_sparse_attention_delta(
                loop, query=to_np(q3[b:b + 1]), current_key=to_np(ck[b:b + 1]), current_value=to_np(cv[b:b + 1]),
                current_position=lengths[b], indices=want_sel["indices"], valid=want_sel["valid"],
                source_selected_output=src[b:b + 1].cpu().numpy(),
                global_mass=sel.global_mass[b:b + 1].cpu().numpy(), scaling=SCALING)
            assert max_err(deltas[loop][b:b + 1].cpu().numpy(), want) < 5e-3, (bits, loop, b)
    assert layer.reader_status() == 0
