"""GPU parity of the ordinary (non-expert) compact3 linears: attention-style projections whose
columns are the layer's input features (several 256-column chunks), fused q/k/v, the dual
gate/up of a dense MLP, input / output scale vectors and bias.  Results go through the C ABI
(grouped entry points with a single-expert payload) and are compared with the fp32 oracle built
from the oracle's own dequantised weights; the weights themselves are checked bit for bit."""
import numpy as np
import pytest
import torch

import trismoe_oracle as orc
from helpers import to_numpy_payload

pytestmark = pytest.mark.gpu
MAX_ABS, MEAN_REL = 2e-2, 1e-3


def _single(rng, out_features, in_features, group=128, unit_cols=False):
    from trismoe_b200 import synth

    raw = synth.raw_projection(rng, 1, out_features, in_features, group_size=group, col_scale_one=unit_cols)
    # weights of order 1/sqrt(K) so that outputs keep a healthy fp16 range
    for key in ("s_r1", "s_r2", "ns_d_r1", "ns_nd_r1"):
        raw[key] = (raw[key].astype(np.float32) * (2.0 / 0.02 / np.sqrt(in_features))).astype(np.float16)
    payload = synth.pack_projection(raw, use_block_gr=True, keep_sparse_gmap=True)
    weight = orc.dequantize_expert(to_numpy_payload(payload), 0)
    return payload, weight


def _check(y, ref):
    max_abs, mean_rel = orc.error_metrics(y.float().cpu().numpy(), ref)
    assert np.abs(ref).mean() > 1e-3
    assert max_abs <= MAX_ABS and mean_rel <= MEAN_REL, (max_abs, mean_rel)


@pytest.mark.parametrize("out_features,in_features,rows", [(192, 512, 1), (256, 1024, 7), (96, 320, 40), (128, 256, 130)])
def test_linear_matches_oracle(lib, out_features, in_features, rows):
    import trismoe_b200 as tm

    rng = np.random.default_rng(out_features + rows)
    payload, weight = _single(rng, out_features, in_features, group=64 if in_features % 128 else 128)
    lin = tm.Compact3Linear(payload, device="cuda")
    got_w = tm.dequantize_grouped_payload(lin.payload)[0].cpu().numpy()
    assert np.array_equal(orc.canonical_half_bits(got_w), orc.canonical_half_bits(weight))
    x = torch.from_numpy(rng.standard_normal((rows, in_features)).astype(np.float16))
    y = lin(x.cuda().view(1, rows, in_features))
    assert y.shape == (1, rows, out_features)
    _check(y.view(rows, -1), x.numpy().astype(np.float32) @ weight.astype(np.float32).T)


def test_linear_with_input_scale_output_scale_and_bias(lib):
    """ns_mode == 1 form: x scaled per input column (rounded to fp16, as the reference kernel does),
    y scaled per output row, plus a bias."""
    import trismoe_b200 as tm

    rng = np.random.default_rng(5)
    O, K, rows = 160, 512, 9
    payload, weight = _single(rng, O, K)
    col = torch.from_numpy((1.0 + 0.3 * rng.standard_normal(K)).astype(np.float16))
    row = torch.from_numpy((1.0 + 0.3 * rng.standard_normal(O)).astype(np.float16))
    bias = torch.from_numpy((0.1 * rng.standard_normal(O)).astype(np.float16))
    lin = tm.Compact3Linear(payload, bias=bias, ns_vector_row=row, ns_vector_col=col, device="cuda")
    x = torch.from_numpy(rng.standard_normal((rows, K)).astype(np.float16))
    y = lin(x.cuda())
    xs = (x * col).numpy().astype(np.float32)  # fp16 product, one rounding
    ref = (xs @ weight.astype(np.float32).T) * row.numpy().astype(np.float32) + bias.numpy().astype(np.float32)
    _check(y, ref)


def test_fused_qkv_and_dual_gate_up(lib):
    import trismoe_b200 as tm

    rng = np.random.default_rng(9)
    K, rows = 512, 5
    (pq, wq), (pk, wk), (pv, wv) = _single(rng, 256, K), _single(rng, 128, K), _single(rng, 128, K)
    q, k, v = (tm.Compact3Linear(p, device="cuda") for p in (pq, pk, pv))
    x = torch.from_numpy(rng.standard_normal((rows, K)).astype(np.float16))
    x32 = x.numpy().astype(np.float32)
    yq, yk, yv = tm.run_compact3_qkv_forward(q, k, v, x.cuda().view(1, rows, K))
    assert yq.shape == (1, rows, 256) and yk.shape == (1, rows, 128)
    for y, w in ((yq, wq), (yk, wk), (yv, wv)):
        _check(y.view(rows, -1), x32 @ w.astype(np.float32).T)
    # the single launches give the same numbers as the fused form
    assert torch.equal(yk, k(x.cuda().view(1, rows, K)))
    (pg, wg), (pu, wu) = _single(rng, 192, K), _single(rng, 192, K)
    gate, up = tm.Compact3Linear(pg, device="cuda"), tm.Compact3Linear(pu, device="cuda")
    act = tm.run_compact3_gate_up_forward(gate, up, x.cuda(), fuse_silu_mul=True)
    g32, u32 = x32 @ wg.astype(np.float32).T, x32 @ wu.astype(np.float32).T
    _check(act, g32 / (1.0 + np.exp(-g32)) * u32)
    a, b = tm.run_compact3_gate_up_forward(gate, up, x.cuda(), fuse_silu_mul=False)
    _check(a, g32)
    _check(b, u32)


def test_qwen2_block_with_shared_expert(lib):
    """Qwen2-MoE style block: routed experts + an always-on shared expert (compact3 gate/up/down) scaled
    by sigmoid(shared_expert_gate(x)), against the fp32 oracle."""
    import trismoe_b200 as tm
    from trismoe_b200 import synth

    shape = synth.LayerShape(256, 192, 8, 2, rank=96, group_size=32)
    layer = synth.synth_layer(shape, seed=41)
    rng = np.random.default_rng(41)
    g_pay, g_w = _single(rng, 320, 256)
    u_pay, u_w = _single(rng, 320, 256)
    d_pay, d_w = _single(rng, 256, 320, group=64)
    gate_w = (rng.standard_normal((1, 256)) / 16).astype(np.float16)
    blk = tm.TrisQwen2SparseMoeBlock(shape.hidden_size, shape.intermediate_size, shape.num_experts, shape.top_k, True)
    blk.load_grouped_payloads(layer["gate"], layer["up"], layer["down"], layer["shared_gate"], layer["shared_up"],
                              layer["shared_down"], layer["router_weight"], device="cuda")
    blk.load_shared_expert(g_pay, u_pay, d_pay, torch.from_numpy(gate_w))
    T = 11
    x = (synth.synth_activations(T, 256, seed=3).float() * 0.25).half()   # keeps the MLP outputs of order one
    logits = synth.synth_router_logits(T, shape.num_experts, seed=4)
    y, _ = blk(x.cuda().view(1, T, -1), router_logits=logits.cuda())
    weights = {n: [orc.dequantize_expert(to_numpy_payload(layer[n]), e) for e in range(shape.num_experts)] for n in ("gate", "up", "down")}
    shared = {n: layer["shared_" + n].numpy() for n in ("gate", "up", "down")}
    ref = orc.moe_layer_fp32(x.numpy(), logits.numpy(), weights, shared, shape.top_k, True)
    xf = x.numpy().astype(np.float32)
    gate_o, up_o = xf @ g_w.astype(np.float32).T, xf @ u_w.astype(np.float32).T
    mlp = gate_o / (1.0 + np.exp(-gate_o)) * up_o
    shared_out = mlp @ d_w.astype(np.float32).T
    ref = ref + 1.0 / (1.0 + np.exp(-(xf @ gate_w.astype(np.float32).T))) * shared_out
    _check(y.view(T, -1), ref)
