"""The one-launch decode-step glue kernels against the tensor ops they restate, and the engine's
fused decode step against its module-by-module step."""

from __future__ import annotations

from pathlib import Path

import numpy as np
import pytest
import torch

from flashloop_b200 import FlashLoopEngine, step_ops
from flashloop_b200.ouro_shape import RMSNorm
from flashloop_b200.prefill import apply_rope
from tests.helpers import tiny_ouro_model

pytestmark = pytest.mark.gpu


def _ulp_close(a: torch.Tensor, b: torch.Tensor, *, ulps: int = 1, exact_fraction: float = 0.98):
    """bfloat16 results may differ by a rounding flip where the float32 reduction order differs."""

    a, b = a.float(), b.float()
    tol = ulps * torch.maximum(a.abs(), b.abs()) * 2.0 ** -7 + 1e-30
    assert bool(((a - b).abs() <= tol).all()), float((a - b).abs().max())
    assert float((a == b).float().mean()) >= exact_fraction


@pytest.mark.parametrize("rows,width", [(1, 256), (16, 2048), (5, 5632), (3, 8192)])
def test_rmsnorm_variants(rows, width):
    g = torch.Generator(device="cuda").manual_seed(rows * 7 + width)
    x = (torch.randn(rows, 1, width, generator=g, device="cuda") * 3).to(torch.bfloat16)
    res = torch.randn(rows, 1, width, generator=g, device="cuda").to(torch.bfloat16)
    n1, n2 = RMSNorm(width, 1e-6).cuda().to(torch.bfloat16), RMSNorm(width, 1e-5).cuda().to(torch.bfloat16)
    with torch.no_grad():
        n1.weight.copy_(1 + 0.1 * torch.randn(width, generator=g, device="cuda"))
        n2.weight.copy_(1 + 0.1 * torch.randn(width, generator=g, device="cuda"))
        _ulp_close(step_ops.rmsnorm(x, n1.weight, n1.eps), n1(x))
        summed = res + n1(x)
        _ulp_close(step_ops.rmsnorm(x, n1.weight, n1.eps, residual=res), summed)
        out, out2 = step_ops.rmsnorm(x, n1.weight, n1.eps, residual=res, weight2=n2.weight, eps2=n2.eps)
        _ulp_close(out, summed)
        _ulp_close(out2, n2(out))  # the second norm of the kernel's own sum


def test_rmsnorm_rejects():
    x = torch.zeros(2, 1, 100, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError, match="multiple of 8"):
        step_ops.rmsnorm(x, torch.ones(100, dtype=torch.bfloat16, device="cuda"), 1e-6)
    with pytest.raises(TypeError):
        step_ops.rmsnorm(x.float(), torch.ones(100, device="cuda"), 1e-6)


@pytest.mark.parametrize("batch,heads,fused", [(1, 2, True), (16, 16, True), (3, 16, False)])
def test_rope_split_matches_tensor_ops(batch, heads, fused):
    g = torch.Generator(device="cuda").manual_seed(batch + heads)
    width = heads * 128
    qkv = torch.randn(batch, 1, 3 * width, generator=g, device="cuda").to(torch.bfloat16)
    q, k, v = qkv.split(width, dim=-1)
    if not fused:
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    pos = torch.randint(0, 5000, (batch, 1), generator=g, device="cuda")
    inv = 1.0 / (10000.0 ** (torch.arange(0, 128, 2, device="cuda").float() / 128))
    emb = torch.cat([pos[..., None].float() * inv] * 2, dim=-1)
    cos, sin = emb.cos().to(torch.bfloat16), emb.sin().to(torch.bfloat16)
    heads_view = lambda t: t.reshape(batch, 1, heads, 128).transpose(1, 2)
    want_q, want_k = apply_rope(heads_view(q), heads_view(k), cos, sin)
    got_q, got_k, got_v = step_ops.rope_split(q, k, v, cos, sin, heads=heads)
    assert torch.equal(got_q, want_q) and torch.equal(got_k, want_k)
    assert torch.equal(got_v, heads_view(v)) and got_v.is_contiguous()


@pytest.mark.parametrize("rows,width", [(1, 384), (16, 5632)])
def test_swiglu_matches_tensor_ops(rows, width):
    g = torch.Generator(device="cuda").manual_seed(width)
    gu = (torch.randn(rows, 1, 2 * width, generator=g, device="cuda") * 2).to(torch.bfloat16)
    gate, up = gu.split(width, dim=-1)
    want = torch.nn.functional.silu(gate) * up
    _ulp_close(step_ops.swiglu(gu), want, exact_fraction=0.995)


def test_fused_decode_step_follows_module_step():
    eg = np.load(Path(__file__).parent / "golden" / "engine_vectors.npz")
    prompts = torch.from_numpy(eg["prompts"]).cuda()
    logits = []
    for fuse in (True, False):
        engine = FlashLoopEngine(tiny_ouro_model().cuda(), validate_model=False, max_new_tokens=16,
                                 fuse_decode_ops=fuse)
        assert engine.fuse_decode_ops == fuse
        engine.prefill(prompts)
        steps = []
        for s in range(12):
            token = torch.tensor([[eg["p0.tokens"][s]], [eg["p1.tokens"][s]]], device="cuda")
            steps.append(engine.decode(token).logits.cpu().numpy())
        logits.append(np.stack(steps))
    # same arithmetic op by op; float32 reduction order inside the norms differs, and a flipped
    # bfloat16 rounding can flip a selected key (see test_gpu_engine), so compare statistically
    err = np.abs(logits[0] - logits[1]).mean(axis=(1, 2))
    assert np.median(err) < 0.03 and err.max() < 0.3, err
    assert np.corrcoef(logits[0].ravel(), logits[1].ravel())[0, 1] > 0.995


def test_unfusable_model_falls_back_to_modules():
    model = tiny_ouro_model().cuda()
    model.model.layers[0].mlp.act_fn = torch.nn.GELU()
    assert FlashLoopEngine(model, validate_model=False).fuse_decode_ops is False



@pytest.mark.parametrize("rows,out_features,in_features", [(16, 6144, 2048), (16, 2048, 5632), (2, 768, 256),
                                                           (5, 256, 384), (1, 49152, 2048), (16, 4128, 1056),
                                                           (5, 8192, 1056)])
def test_linear_rows_matches_float32_product(rows, out_features, in_features):
    g = torch.Generator(device="cuda").manual_seed(rows + out_features)
    x = torch.randn(rows, 1, in_features, generator=g, device="cuda").to(torch.bfloat16)
    w = (torch.randn(out_features, in_features, generator=g, device="cuda") * 0.05).to(torch.bfloat16)
    assert step_ops.linear_fits(x, w)
    got = step_ops.linear(x, w)
    want = (x.float() @ w.float().T)
    # float32 accumulation in another order, then one rounding to bfloat16
    assert got.shape == (rows, 1, out_features) and got.dtype == torch.bfloat16
    # float32 accumulation in another order, then one rounding to bfloat16: half an ulp of the
    # result plus the float32 noise of a sum of in_features terms (visible where the terms cancel)
    err = (got.float() - want).abs()
    bound = 2.0 ** -8 * want.abs() + 1e-5 * float((x.float().abs().max() * w.float().abs().max())) * in_features ** 0.5
    assert bool((err <= bound).all()), (float(err.max()), float(want.abs().max()))
    assert float((got == want.to(torch.bfloat16)).float().mean()) > 0.97


@pytest.mark.parametrize("rows,out_features,in_features,dtype", [(16, 2048, 2048, torch.float32),
                                                                  (16, 2048, 5632, torch.bfloat16),
                                                                  (3, 256, 384, torch.bfloat16),
                                                                  (1, 4096, 1024, torch.float32)])
def test_split_projection_and_its_norm(rows, out_features, in_features, dtype):
    """``linear_partial`` leaves float32 sums over four slices of in_features; their sum is the
    float32 product, and ``rmsnorm_partial`` equals ``rmsnorm`` of that sum rounded to bfloat16, bit
    for bit, with and without addend, residual and second norm."""

    g = torch.Generator(device="cuda").manual_seed(rows + out_features + in_features)
    x = torch.randn(rows, 1, in_features, generator=g, device="cuda").to(dtype)
    w = (torch.randn(out_features, in_features, generator=g, device="cuda") * 0.05).to(torch.bfloat16)
    assert step_ops.linear_partial_fits(x, w)
    partial = step_ops.linear_partial(x, w)
    assert partial.shape == (step_ops.LINEAR_SPLITS, rows, 1, out_features) and partial.dtype == torch.float32
    want = x.to(torch.bfloat16).float() @ w.float().T
    total = partial.sum(0)
    bound = 1e-5 * float(x.float().abs().max() * w.float().abs().max()) * in_features ** 0.5
    assert float((total - want).abs().max()) <= bound
    summed = total.to(torch.bfloat16)
    n1 = (1 + 0.1 * torch.randn(out_features, generator=g, device="cuda")).to(torch.bfloat16)
    n2 = (1 + 0.1 * torch.randn(out_features, generator=g, device="cuda")).to(torch.bfloat16)
    addend = torch.randn(rows, 1, out_features, generator=g, device="cuda").to(torch.bfloat16)
    residual = torch.randn(rows, 1, out_features, generator=g, device="cuda").to(torch.bfloat16)
    out, out2, kept = step_ops.rmsnorm_partial(partial, n1, 1e-6, want_sum=True)
    assert out2 is None and torch.equal(kept, summed) and torch.equal(out, step_ops.rmsnorm(summed, n1, 1e-6))
    out, out2, kept = step_ops.rmsnorm_partial(partial, n1, 1e-6, residual=residual, weight2=n2, eps2=1e-5,
                                               addend=addend)
    want_out, want_out2 = step_ops.rmsnorm(summed, n1, 1e-6, residual=residual, weight2=n2, eps2=1e-5, addend=addend)
    assert kept is None and torch.equal(out, want_out) and torch.equal(out2, want_out2)


def test_split_projection_rejects_what_it_cannot_slice():
    x = torch.randn(2, 1, 96, device="cuda").to(torch.bfloat16)
    w = torch.randn(64, 96, device="cuda").to(torch.bfloat16)   # 96 is not four slices of chunks of 32
    assert not step_ops.linear_partial_fits(x, w)
    with pytest.raises(ValueError):
        step_ops.linear_partial(x, w)
    wide = torch.randn(8192, 128, device="cuda").to(torch.bfloat16)  # enough tiles for the other kernels
    assert not step_ops.linear_partial_fits(torch.randn(2, 1, 128, device="cuda").to(torch.bfloat16), wide)


@pytest.mark.parametrize("rows,width,in_features", [(16, 5632, 2048), (3, 192, 256)])
def test_linear_rows_with_swiglu(rows, width, in_features):
    g = torch.Generator(device="cuda").manual_seed(rows + width)
    x = torch.randn(rows, 1, in_features, generator=g, device="cuda").to(torch.bfloat16)
    w = (torch.randn(2 * width, in_features, generator=g, device="cuda") * 0.05).to(torch.bfloat16)
    got = step_ops.linear(x, w, swiglu=True)
    want = step_ops.swiglu(step_ops.linear(x, w))           # the two launches it replaces: same roundings
    assert got.shape == (rows, 1, width) and torch.equal(got, want)
    ref = torch.nn.functional.silu((x.float() @ w.float().T)[..., :width]) * (x.float() @ w.float().T)[..., width:]
    assert float((got.float() - ref).abs().max()) <= 2.0 ** -6 * float(ref.abs().max()) + 1e-5


def test_linear_rows_rejects():
    x = torch.zeros(17, 1, 256, dtype=torch.bfloat16, device="cuda")
    w = torch.zeros(256, 256, dtype=torch.bfloat16, device="cuda")
    assert not step_ops.linear_fits(x, w)
    with pytest.raises(RuntimeError, match="at most 16 rows"):
        step_ops.linear(x, w)
    assert not step_ops.linear_fits(x[:4], torch.zeros(256, 250, dtype=torch.bfloat16, device="cuda"))


def test_linear_rows_takes_float32_rows():
    g = torch.Generator(device="cuda").manual_seed(11)
    x = torch.randn(16, 1, 2048, generator=g, device="cuda")
    w = (torch.randn(2048, 2048, generator=g, device="cuda") * 0.05).to(torch.bfloat16)
    assert torch.equal(step_ops.linear(x, w), step_ops.linear(x.to(torch.bfloat16), w))


@pytest.mark.parametrize("batch,heads,hidden", [(16, 16, 2048), (3, 2, 256), (1, 8, 1024)])
def test_qkv_rope_equals_linear_then_rope_split(batch, heads, hidden):
    g = torch.Generator(device="cuda").manual_seed(batch + heads)
    x = torch.randn(batch, 1, hidden, generator=g, device="cuda").to(torch.bfloat16)
    w = (torch.randn(3 * heads * 128, hidden, generator=g, device="cuda") * 0.05).to(torch.bfloat16)
    pos = torch.randint(0, 5000, (batch, 1), generator=g, device="cuda")
    inv = 1.0 / (10000.0 ** (torch.arange(0, 128, 2, device="cuda").float() / 128))
    emb = torch.cat([pos[..., None].float() * inv] * 2, dim=-1)
    cos, sin = emb.cos().to(torch.bfloat16), emb.sin().to(torch.bfloat16)
    q, k, v = step_ops.linear(x, w).split(heads * 128, dim=-1)
    want = step_ops.rope_split(q, k, v, cos, sin, heads=heads)
    got = step_ops.qkv_rope(x, w, cos, sin, heads=heads)
    for a, b in zip(got, want):
        assert a.shape == b.shape and torch.equal(a, b)


def test_rmsnorm_addend_equals_separate_add():
    g = torch.Generator(device="cuda").manual_seed(4)
    x, a, res = ((torch.randn(16, 1, 2048, generator=g, device="cuda") * 2).to(torch.bfloat16) for _ in range(3))
    w1 = (1 + 0.1 * torch.randn(2048, generator=g, device="cuda")).to(torch.bfloat16)
    w2 = (1 + 0.1 * torch.randn(2048, generator=g, device="cuda")).to(torch.bfloat16)
    got = step_ops.rmsnorm(x, w1, 1e-6, residual=res, weight2=w2, eps2=1e-5, addend=a)
    want = step_ops.rmsnorm(a + x, w1, 1e-6, residual=res, weight2=w2, eps2=1e-5)
    assert torch.equal(got[0], want[0]) and torch.equal(got[1], want[1])
