"""Generate the golden vectors that pin the oracle to the reference's own code.

Run here (needs the reference checkout; it is never needed at test time):

    python tests/golden/make_golden.py <path of the reference checkout>

It imports the reference's ``flashloop`` and ``flashloop_torch`` packages, runs
their CPU/Torch code on small seeded inputs and writes ``reference_vectors.npz``
next to this script.  Every stored array is an output of unmodified reference code
(or an input fed to it); nothing is computed by this repository's own codecs.
"""

from __future__ import annotations

import math
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parents[1]))
ref_root = sys.argv[1] if len(sys.argv) > 1 else "/root/reference"
sys.path.insert(0, ref_root)

from flashloop_b200.synthetic import make_loop_kv, make_masks, make_query  # noqa: E402

import flashloop  # noqa: E402  (the reference)
from flashloop import cache as ref_cache  # noqa: E402
from flashloop import engine as ref_engine  # noqa: E402
from flashloop import kivi_backend as ref_kivi  # noqa: E402
from flashloop import packing as ref_packing  # noqa: E402
from flashloop import selection as ref_selection  # noqa: E402
from flashloop_torch import kv_quantization as ref_fq  # noqa: E402

assert Path(flashloop.__file__).resolve().is_relative_to(Path(ref_root).resolve())

out: dict[str, np.ndarray] = {}


def bits(t: torch.Tensor) -> np.ndarray:
    """bf16/f16 tensor -> uint16 bit patterns."""
    return t.contiguous().view(torch.int16).numpy().view(np.uint16).copy()


def put(name: str, t) -> None:
    if isinstance(t, torch.Tensor):
        if t.dtype in (torch.bfloat16, torch.float16):
            out[name] = bits(t)
        elif t.dtype == torch.bool:
            out[name] = t.numpy().copy()
        else:
            out[name] = t.contiguous().numpy().copy()
    else:
        out[name] = np.asarray(t)


def put_stream(prefix: str, packed) -> None:
    if packed is None:
        out[prefix + ".none"] = np.ones(1, np.uint8)
        return
    put(prefix + ".payload", packed.payload)
    put(prefix + ".minimum", packed.minimum)
    put(prefix + ".scale", packed.scale)
    put(prefix + ".shape", np.asarray(packed.original_shape, np.int64))
    groups = getattr(packed, "row_groups", None)
    if groups is not None:
        put(prefix + ".row_groups", groups)


torch.manual_seed(0)
torch.set_num_threads(4)
H, T, D = 2, 200, 128
keys, values = make_loop_kv(H, T, seed=11)
mask3, mask4 = make_masks(T, seed=11)
query, cur_k, cur_v = make_query(H, seed=11)
scaling = D ** -0.5
for r in range(4):
    put(f"in.key{r}", keys[r])
    put(f"in.value{r}", values[r])
put("in.mask3", mask3)
put("in.mask4", mask4)
put("in.query", query)
put("in.cur_k", cur_k)
put("in.cur_v", cur_v)

# --- A. plain packing, both layouts, three dtypes -------------------------------------
for tag, x in (("bf16", keys[0]), ("f16", keys[1][:, :1, :70].to(torch.float16)),
               ("f32", values[2][:, :1, :70].float() * 1.3)):
    if tag != "bf16":
        put(f"pack.{tag}.input", x if x.dtype != torch.float16 else x)
    put_stream(f"pack.{tag}.kivi_k", ref_kivi.pack_kivi_k_per_channel(x))
    put_stream(f"pack.{tag}.kivi_v", ref_kivi.pack_kivi_v_per_token(x))
    put_stream(f"pack.{tag}.rows_k", ref_packing.pack_k_per_channel(x))
    put_stream(f"pack.{tag}.rows_v", ref_packing.pack_v_per_token(x))
put("pack.bf16.kivi_k.decode", ref_kivi.pack_kivi_k_per_channel(keys[0]).decode())
put("pack.bf16.kivi_v.decode", ref_kivi.pack_kivi_v_per_token(keys[0]).decode())
put("pack.bf16.rows_k.decode", ref_packing.pack_k_per_channel(keys[0]).decode())
put("pack.bf16.rows_v.decode", ref_packing.pack_v_per_token(keys[0]).decode())


# --- B. cache layer construction, both backends ---------------------------------------
def build(backend: str):
    return ref_cache.CrossLoopKVLayer.from_prefill(
        keys, values, mask_loop3=mask3[None], mask_loop4=mask4[None],
        group_size=64, residual_length=64, reader_backend=backend)


layers = {b: build(b) for b in ("triton_row", "kivi_outer")}
for backend, layer in layers.items():
    for s in range(4):
        put_stream(f"layer.{backend}.k{s}", layer._packed_keys[s])
        put_stream(f"layer.{backend}.v{s}", layer._packed_values[s])
    put(f"layer.{backend}.pos3", layer.override_indices[0])
    put(f"layer.{backend}.pos4", layer.override_indices[1])
    put(f"layer.{backend}.rank3", layer.rank_maps[0])
    put(f"layer.{backend}.rank4", layer.rank_maps[1])
    put(f"layer.{backend}.quantized_tokens", np.int64(layer.quantized_tokens))
    put(f"layer.{backend}.storage_bytes", np.int64(layer.storage_bytes))
row = layers["triton_row"]
for r in range(4):
    put(f"layer.tail_k{r}", row._tail_keys[r])
    put(f"layer.tail_v{r}", row._tail_values[r])
put("layer.tail_active3", row._tail_active[0])
put("layer.tail_active4", row._tail_active[1])

# --- C. dense source attention (loops 0, 1) and logical gather --------------------------
for backend, layer in layers.items():
    for loop in (0, 1):
        o, lg = layer.dense_source_attention(loop, query=query, current_key=cur_k,
                                             current_value=cur_v, scaling=scaling,
                                             return_logits=True)
        put(f"dense.{backend}.loop{loop}.out", o)
        put(f"dense.{backend}.loop{loop}.logits", lg)
for loop in (1, 3):
    gk, gv = row.gather(loop, torch.arange(row.token_count))
    put(f"gather.loop{loop}.k", gk)
    put(f"gather.loop{loop}.v", gv)

# --- D. decode key selection (engine.py:438-481 run through the reference helpers) ------
logits1 = torch.from_numpy(out["dense.triton_row.loop1.logits"])
weights = torch.softmax(logits1, dim=-1, dtype=torch.float32)
past = row.token_count
sel = ref_selection.select_decode_keys(weights, fraction=0.10)
put("select.weights", weights)
put("select.indices", sel.indices)
put("select.global_mass", sel.global_mass)
budget = min(past + 1, max(1, math.ceil((past + 1) * 0.10)))
idx = sel.indices.squeeze(-2)
padded, valid = ref_engine._pad_decode_indices(idx)
sel_global = torch.gather(weights, -1, sel.indices.long())
pg = torch.zeros((*sel_global.shape[:-1], padded.shape[-1]))
pg[..., :budget] = sel_global
mass = pg.sum(dim=-1, keepdim=True)
sel_w = pg / mass
put("select.padded", padded)
put("select.valid", valid)
put("select.mass", mass)
put("select.selected_weights", sel_w)
# a second selection problem with a current-token hit and a tail hit guaranteed
w2 = torch.rand(1, H, 1, 777, generator=torch.Generator().manual_seed(5))
w2 = w2 / w2.sum(-1, keepdim=True)
s2 = ref_selection.select_decode_keys(w2, fraction=0.10)
put("select2.weights", w2)
put("select2.indices", s2.indices)
put("select2.global_mass", s2.global_mass)

# --- E. selected QK / PV and the loop-2 selected aggregate -------------------------------
is_cur = padded == past
safe = torch.where(is_cur, torch.zeros_like(padded), padded)
for backend, layer in layers.items():
    for loop in range(4):
        put(f"qk.{backend}.loop{loop}", layer.qk(loop, query, safe, validate_indices=False))
        put(f"pv.{backend}.loop{loop}",
            layer.pv(loop, sel_w * (~is_cur)[:, :, None, :], safe, validate_indices=False))
sel_out = row.pv(1, sel_w * (~is_cur)[:, :, None, :], safe, validate_indices=False)
sel_out = sel_out + torch.sum(sel_w * is_cur[:, :, None, :], dim=-1, keepdim=True) * cur_v.float()
put("select.selected_output", sel_out)

# --- F. cached-mass sparse delta (loops 2, 3) --------------------------------------------
q3, k3, v3 = make_query(H, seed=12)
put("sparse.query", q3)
put("sparse.cur_k", k3)
put("sparse.cur_v", v3)
for backend, layer in layers.items():
    for loop in (2, 3):
        delta = layer.cached_mass_sparse_attention_delta(
            loop, query=q3, current_key=k3, current_value=v3, current_position=past,
            indices=padded, valid=valid, source_selected_output=sel_out,
            global_mass=mass, scaling=scaling)
        put(f"sparse.{backend}.loop{loop}", delta)

# --- G. decode appends across one rollover (row-layout append rule) ----------------------
gen = torch.Generator().manual_seed(99)
appended = []
for step in range(70):
    ks = [(torch.randn(1, H, 1, D, generator=gen) * (1.0 if r == 0 else 0.1)) for r in range(4)]
    vs = [(torch.randn(1, H, 1, D, generator=gen) * (1.0 if r == 0 else 0.1)) for r in range(4)]
    ks = [sum(ks[: r + 1]).to(torch.bfloat16) for r in range(4)]
    vs = [sum(vs[: r + 1]).to(torch.bfloat16) for r in range(4)]
    appended.append((ks, vs))
    row.append_decode_token(ks, vs)
put("append.keys", torch.stack([torch.cat(k, dim=2) for k, _ in appended], dim=0))  # [70,1,H,4,D]
put("append.values", torch.stack([torch.cat(v, dim=2) for _, v in appended], dim=0))
for s in range(4):
    put_stream(f"append.k{s}", row._packed_keys[s])
    put_stream(f"append.v{s}", row._packed_values[s])
put("append.pos3", row.override_indices[0])
put("append.pos4", row.override_indices[1])
put("append.rank3", row.rank_maps[0])
put("append.rank4", row.rank_maps[1])
put("append.quantized_tokens", np.int64(row.quantized_tokens))
put("append.tail_tokens", np.int64(row.tail_tokens))
for r in range(4):
    put(f"append.tail_k{r}", row._tail_keys[r][:, :, : row.tail_tokens])
    put(f"append.tail_v{r}", row._tail_values[r][:, :, : row.tail_tokens])
for loop in (0, 1):
    o, lg = row.dense_source_attention(loop, query=query, current_key=cur_k, current_value=cur_v,
                                       scaling=scaling, return_logits=True)
    put(f"append.dense.loop{loop}.out", o)
    put(f"append.dense.loop{loop}.logits", lg)

# --- H. fake-quant codec (tolerance oracle) ----------------------------------------------
Tq = 128  # the quantised prefix of the 200-token prompt (before the appends of section G)
for profile in ("kivi4_channel", "kivi2_channel"):
    res = ref_fq.encode_temporal_group(
        [k[:, :, :Tq] for k in keys], [v[:, :, :Tq] for v in values],
        active_masks=[torch.ones(1, Tq, dtype=torch.bool), mask3[None, :Tq], mask4[None, :Tq]],
        group_size=64, codec_profile=profile)
    for loop in (1, 3):
        put(f"fq.{profile}.k{loop}", res.reconstructed_keys[loop])
        put(f"fq.{profile}.v{loop}", res.reconstructed_values[loop])
    if profile != "kivi4_channel":
        continue
    # --- J. the sparse late-loop output in the fake-quant domain: the reference's own
    # mass_scaled_sparse_output on its own reconstructions (prefix), BF16 tail and current token.
    # Source = loop 2 with the query / current K,V of section C; targets = loops 3, 4 with those
    # of section F; selection = top 10 % of the source weights; both scales = the selected mass.
    from flashloop_torch import attention_utils as ref_au  # noqa: E402

    def full(rec, loop_tensors, current, loop):
        return torch.cat([rec[loop].float(), loop_tensors[loop][:, :, Tq:].float(), current.float()], dim=2)

    src_k = full(res.reconstructed_keys, keys, cur_k, 1)
    src_v = full(res.reconstructed_values, values, cur_v, 1)
    src_logits = torch.matmul(query.float(), src_k.transpose(-1, -2)) * scaling
    fq_mask = ref_au.make_decode_topk_mask(torch.softmax(src_logits, dim=-1), 0.10)
    fq_mass = ref_au.selected_attention_mass(src_logits, fq_mask)
    put("fqsparse.mask", fq_mask)
    put("fqsparse.mass", fq_mass)
    put("fqsparse.source_subset", torch.matmul(ref_au.masked_subset_softmax(src_logits, fq_mask), src_v))
    zero = torch.zeros(1, H, 1, D)
    for loop in (2, 3):
        tgt_k = full(res.reconstructed_keys, keys, k3, loop)
        tgt_v = full(res.reconstructed_values, values, v3, loop)
        tgt_logits = torch.matmul(q3.float(), tgt_k.transpose(-1, -2)) * scaling
        put(f"fqsparse.loop{loop}.delta",
            ref_au.mass_scaled_sparse_output(zero, src_logits, tgt_logits, src_v, tgt_v, fq_mask, fq_mass, fq_mass))

# --- I. token retention -------------------------------------------------------------------
g2 = torch.Generator().manual_seed(3)
h1 = torch.randn(1, 300, 256, generator=g2).to(torch.bfloat16)
h2 = (h1.float() + 0.3 * torch.randn(1, 300, 256, generator=g2) * torch.rand(1, 300, 1, generator=g2)).to(torch.bfloat16)
h3 = (h2.float() + 0.2 * torch.randn(1, 300, 256, generator=g2) * torch.rand(1, 300, 1, generator=g2)).to(torch.bfloat16)
put("retain.h1", h1)
put("retain.h2", h2)
put("retain.h3", h3)
score3 = ref_engine._hidden_delta_score(h2, h1)
m3 = ref_selection.select_prefill_tokens(score3, fraction=0.25)
score4 = ref_engine._hidden_delta_score(h3, h2)
m4 = ref_selection.select_prefill_tokens(score4, fraction=0.10, eligible=m3)
put("retain.score3", score3)
put("retain.mask3", m3)
put("retain.score4", score4)
put("retain.mask4", m4)

np.savez_compressed(HERE / "reference_vectors.npz", **out)
total = sum(v.nbytes for v in out.values())
print(f"wrote {len(out)} arrays, {total/1e6:.2f} MB raw ->",
      (HERE / "reference_vectors.npz").stat().st_size / 1e6, "MB")
