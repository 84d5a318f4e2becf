"""GPU test of tris_moe_layer_forward_static, the entry point for callers that must not
allocate device memory (their pool owns the GPU, or their host framework forbids it).

It is called through the C ABI exactly like tris_moe_layer_forward, minus the workspace, and
must give the same output as that entry point - here on two calls in a row with different
inputs, because all calls share one built-in scratch array that keeps the previous call's
contents.  The file name sorts last so that a run that stops at the first failure has
already run every other test.
"""
import ctypes as C

import numpy as np
import pytest
import torch


pytestmark = pytest.mark.gpu



def _make_block(tm):
    from trismoe_b200 import synth

    shape = synth.LayerShape(256, 192, 8, 2, rank=96, group_size=32)
    layer = synth.synth_layer(shape, seed=21)
    for name in ("gate", "up", "down"):
        layer["shared_" + name] = (layer["shared_" + name].float() * 5.0).half()
    blk = tm.TrisSparseMoeBlock(shape.hidden_size, shape.intermediate_size, shape.num_experts, shape.top_k, True)
    blk.load_grouped_payloads(layer["gate"], layer["up"], layer["down"], layer["shared_gate"], layer["shared_up"],
                              layer["shared_down"], layer["router_weight"], device="cuda")
    return shape, blk


def _call(lib, tm, blk, x, logits, static):
    T = x.shape[0]
    y = torch.empty_like(x)
    stream = torch.cuda.current_stream().cuda_stream
    view = blk.layer_view()
    if static:
        st = lib.tris_moe_layer_forward_static(C.byref(view), x.data_ptr(), logits.data_ptr(), T, y.data_ptr(), None, stream)
    else:
        need = lib.tris_moe_layer_workspace_bytes(C.byref(view), T)
        ws = torch.empty((need,), dtype=torch.uint8, device="cuda")
        st = lib.tris_moe_layer_forward(C.byref(view), x.data_ptr(), logits.data_ptr(), T, y.data_ptr(), None,
                                        ws.data_ptr(), need, stream)
    tm._native.check(st, "static layer forward" if static else "layer forward")
    torch.cuda.synchronize()
    return y


def test_static_scratch_entry_matches_workspace_entry(lib):
    import trismoe_b200 as tm
    from trismoe_b200 import synth

    assert torch.cuda.is_available()
    shape, blk = _make_block(tm)
    for call, T in enumerate((7, 3)):  # two calls in a row; the second is smaller, so stale rows remain behind it
        x = synth.synth_activations(T, shape.hidden_size, seed=40 + call).cuda()
        logits = synth.synth_router_logits(T, shape.num_experts, seed=50 + call).cuda()
        want = _call(lib, tm, blk, x, logits, static=False)
        got = _call(lib, tm, blk, x, logits, static=True)
        assert torch.isfinite(got.float()).all()
        assert want.float().abs().mean().item() > 1e-4
        # Both entries run the identical launch sequence, so the outputs must be bit-identical: a
        # read of stale scratch from the previous call could otherwise hide inside a tolerance.
        assert torch.equal(got, want), call


def test_static_scratch_entry_rejects_oversized_batches(lib):
    import trismoe_b200 as tm

    shape, blk = _make_block(tm)
    view = blk.layer_view()
    T = 1
    while lib.tris_moe_layer_workspace_bytes(C.byref(view), T) <= tm._native.STATIC_SCRATCH_BYTES:
        T *= 2
    x = torch.zeros((T, shape.hidden_size), dtype=torch.float16, device="cuda")
    logits = torch.zeros((T, shape.num_experts), dtype=torch.float32, device="cuda")
    y = torch.empty_like(x)
    st = lib.tris_moe_layer_forward_static(C.byref(view), x.data_ptr(), logits.data_ptr(), T, y.data_ptr(), None,
                                           torch.cuda.current_stream().cuda_stream)
    assert st == 5  # TRIS_ERR_WORKSPACE
    msg = lib.tris_last_error().decode()
    assert "scratch" in msg and str(tm._native.STATIC_SCRATCH_BYTES) in msg
