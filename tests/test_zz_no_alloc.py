"""The scratch-free dense reader entry point, called straight through the C ABI.

Some hosts cannot allocate device memory where they call the reader (inside a stream
capture, or as a plugin in a process whose memory belongs to someone else's pool), so
``fl_dense_source_attention_static`` keeps its scratch in a static device array.  This test
calls it twice in a row on the same layer and compares each result with the ordinary entry
point, which takes a caller-provided workspace, and with the CPU oracle.
"""

from __future__ import annotations

import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_static_scratch_entry_matches_workspace_entry():
    from flashloop_b200 import _native
    from flashloop_b200.cache import CrossLoopKVLayer
    from flashloop_b200.synthetic import make_loop_kv, make_masks, make_query
    from oracle.cache import LayerOracle

    lib = _native.load()
    heads, tokens, scaling = 4, 1500, 128 ** -0.5
    keys, values = make_loop_kv(heads, tokens, seed=21)
    mask3, mask4 = make_masks(tokens, seed=21)
    layer = CrossLoopKVLayer.from_prefill([k.cuda() for k in keys], [v.cuda() for v in values],
                                          mask_loop3=mask3[None].cuda(), mask_loop4=mask4[None].cuda())
    f = lambda t: t.float().numpy()
    oracle = LayerOracle.from_prefill([f(k) for k in keys], [f(v) for v in values], mask_loop3=mask3.numpy(),
                                      mask_loop4=mask4.numpy())
    stream = _native.current_stream(torch.device("cuda"))
    workspace = layer._workspace()
    stride = tokens + 4
    for call in range(2):  # two calls in a row: the second one finds the first one's leftovers
        q, ck, cv = (t.cuda() for t in make_query(heads, seed=100 + call))
        for loop in (1, 3):
            want = torch.empty(1, heads, 1, 128, device="cuda")
            want_logits = torch.full((1, heads, 1, stride), float("-inf"), device="cuda")
            _native.check(lib.fl_dense_source_attention(
                C.byref(layer._native), loop, q.data_ptr(), ck.data_ptr(), cv.data_ptr(), scaling,
                want.data_ptr(), want_logits.data_ptr(), stride, tokens, workspace.data_ptr(),
                workspace.numel(), stream), "fl_dense_source_attention")
            got = torch.empty_like(want)
            got_logits = torch.full_like(want_logits, float("-inf"))
            _native.check(lib.fl_dense_source_attention_static(
                C.byref(layer._native), loop, q.data_ptr(), ck.data_ptr(), cv.data_ptr(), scaling,
                got.data_ptr(), got_logits.data_ptr(), stride, tokens, stream),
                "fl_dense_source_attention_static")
            torch.cuda.synchronize()
            # same kernel, same split points: logits are identical; outputs may differ in the
            # last bits because the partials merge in arrival order
            assert torch.equal(got_logits, want_logits), (call, loop)
            assert torch.allclose(got, want, rtol=1e-5, atol=1e-6), (call, loop, float((got - want).abs().max()))
            exact, _ = oracle.dense_source_attention(loop, query=f(q.cpu()), current_key=f(ck.cpu()),
                                                     current_value=f(cv.cpu()), scaling=scaling)
            assert float((got.cpu() - torch.from_numpy(exact)).abs().max()) < 5e-3, (call, loop)
    flag = C.c_int32(-1)
    _native.check(lib.fl_static_status(C.byref(flag), stream), "fl_static_status")
    assert flag.value == 0  # no bounded wait of the static entry point ran out
    # sizes beyond the built-in scratch are refused with a clear message
    status = lib.fl_dense_source_attention_static(
        C.byref(layer._native), 1, q.data_ptr(), ck.data_ptr(), cv.data_ptr(), scaling, got.data_ptr(), None, 0,
        1 << 20, stream)
    assert status == -4 and b"exceeds the built-in scratch" in lib.fl_last_error()
