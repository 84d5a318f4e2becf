"""GPU parity of the GEMMs that read 4-bit packed matrices in place: the null-space compensation
of ns_mode == 2 experts (fixture written by the reference's own payload builder and per-segment
fallback), the packed backbone product, and their use inside the grouped operators and the MoE
block.  Everything goes through the C ABI (tris_packed4_grouped_forward, tris_moe_layer_forward);
weights are checked bit for bit, outputs against the fp32 oracle within the layer tolerance."""
import numpy as np
import pytest
import torch

import trismoe_oracle as orc
from helpers import load_golden, to_numpy_payload

pytestmark = pytest.mark.gpu
MAX_ABS, MEAN_REL = 2e-2, 1e-3


def _check(got, ref, floor=1e-3):
    got = got.float().cpu().numpy() if isinstance(got, torch.Tensor) else got
    assert np.abs(ref).mean() > floor
    max_abs, mean_rel = orc.error_metrics(got, ref)
    assert max_abs <= MAX_ABS and mean_rel <= MEAN_REL, (max_abs, mean_rel)


def _np_matrix(m):
    return (m["qweight"].numpy(), m["qzeros"].numpy(), m["scales"].numpy(), m["g_idx"].numpy(), int(m["rows"]), int(m["cols"]))


@pytest.mark.parametrize("tag", ["pc", "g64"])
def test_packed_linear_weights_bit_exact_vs_reference_dequantize(lib, tag):
    """y = I @ W^T through the 4-bit GEMM reproduces PackedQuantMatrix4bit.dequantize bit for bit
    (each output is a single product, so the fp32 sum and the final rounding are exact)."""
    import trismoe_b200 as tm

    z = load_golden("backbone4.npz")
    rows, cols, _ = (int(v) for v in z[f"{tag}_dims"])
    payload = {k: torch.from_numpy(z[f"{tag}_{k}"].copy()) for k in ("qweight", "qzeros", "scales", "g_idx")}
    payload.update(rows=rows, cols=cols)
    assert tm.Packed4Linear.supports(payload)
    lin = tm.Packed4Linear(payload, "cuda")
    y = lin(torch.eye(cols, dtype=torch.float16, device="cuda"))        # [cols, rows] = W^T
    assert np.array_equal(orc.canonical_half_bits(y.t().cpu().numpy()), orc.canonical_half_bits(z[f"{tag}_weight_f16"]))


def test_packed_linear_rejects_permuted_groups(lib):
    import trismoe_b200 as tm

    z = load_golden("backbone4.npz")
    rows, cols, _ = (int(v) for v in z["perm_dims"])
    payload = {k: torch.from_numpy(z[f"perm_{k}"].copy()) for k in ("qweight", "qzeros", "scales", "g_idx")}
    payload.update(rows=rows, cols=cols)
    assert not tm.Packed4Linear.supports(payload)
    with pytest.raises(RuntimeError):
        tm.Packed4Linear(payload, "cuda")


@pytest.mark.parametrize("rows,cols,T", [(2048, 2048, 1), (2048, 2048, 16), (512, 2048, 128), (1024, 1024, 300), (80, 200, 5)])
@pytest.mark.parametrize("layout", [0, 2, 3])
def test_packed_linear_matches_oracle(lib, rows, cols, T, layout):
    """Backbone-sized products against fp32 sums over the oracle's dequantised matrix, in the three
    output column orders the grouped kernels consume."""
    import trismoe_b200 as tm
    from trismoe_b200 import synth

    if layout and rows % 32:
        pytest.skip("permuted layouts need rows % 32 == 0")
    rng = np.random.default_rng(rows + T)
    m = synth.packed4_matrix(rng, rows, cols, group_size=128 if cols % 128 == 0 else cols, scale_std=2.0 / np.sqrt(cols) / 8)
    w = orc.dequantize_packed4(*_np_matrix(m))
    x = rng.standard_normal((T, cols)).astype(np.float16)
    lin = tm.Packed4Linear(m, "cuda")
    y = lin(torch.from_numpy(x).cuda(), layout)
    assert lin.nbytes < rows * cols            # a quarter of the fp16 bytes, plus scales and zeros
    want = tm.compute_shared_hidden(torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda(), layout=layout)
    ref = x.astype(np.float32) @ w.astype(np.float32).T
    _check(y, want.float().cpu().numpy())          # same column order on both sides
    if layout == 0:
        _check(y, ref)


def _fixture_payload(z):
    return {k[len("payload_"):]: (torch.from_numpy(z[k].copy()) if z[k].ndim else int(z[k])) for k in z.files if k.startswith("payload_")}


def test_ns_compensation_fixture(lib):
    """The payload the reference's builder wrote (ranks 16 / 0 / 24 / 16 / 40, one expert without a
    pair, one without rows): result vs the fp32 oracle and vs the reference's fp16 fallback."""
    import trismoe_b200 as tm

    z = load_golden("ns_compensation.npz")
    payload = _fixture_payload(z)
    x = torch.from_numpy(z["x"].copy()).cuda()
    route = {"expert_ids": torch.from_numpy(z["expert_ids"].copy()).cuda(), "segment_offsets": torch.from_numpy(z["segment_offsets"].copy()).cuda()}
    got = tm.run_grouped_ns_compensation_forward(payload, x, route)
    ref = orc.ns_compensation_fp32({k[len("payload_"):]: z[k] for k in z.files if k.startswith("payload_")}, z["x"], z["expert_ids"],
                                   z["segment_offsets"])
    _check(got, ref)
    _check(got, z["compensation_f16"].astype(np.float32))
    seg = z["segment_offsets"]
    assert not got[seg[1]:seg[2]].any()       # the expert without a pair: zeros
    # segment lengths + expert ids instead of a route dict, and the two halves separately
    lengths = np.diff(seg).tolist()
    again = tm.run_grouped_ns_compensation_forward(payload, x, lengths, expert_ids=z["expert_ids"].tolist())
    assert torch.equal(again, got)


def _ns_layer(rng, E, infeatures, outfeatures, ranks, group=128, share_c2=False):
    import trismoe_b200 as tm
    from trismoe_b200 import synth

    experts, shared_c2 = [], None
    for rank in ranks:
        if rank == 0:
            experts.append(None)
            continue
        if share_c2 and shared_c2 is not None:
            c2 = shared_c2
        else:
            c2 = synth.packed4_matrix(rng, rank, infeatures, group, scale_std=2.0 / np.sqrt(infeatures) / 8)
            shared_c2 = c2
        c1 = synth.packed4_matrix(rng, outfeatures, rank, group, scale_std=2.0 / np.sqrt(rank) / 8)
        experts.append({"c1": c1, "c2": c2})
    return tm.build_grouped_ns_compensation_payload(experts, "cpu", torch.float16, infeatures, outfeatures)


@pytest.mark.parametrize("share_c2", [False, True])
@pytest.mark.parametrize("tokens", [1, 16, 128])
def test_ns_compensation_olmoe_shape(lib, tokens, share_c2):
    """64 experts, in 2048, out 1024, ranks 0 / 32 / 64 (shared C2: every expert rank 32 on one C2),
    top-8 routing of `tokens` tokens; plain result, accumulate form and C1-only form."""
    import trismoe_b200 as tm

    rng = np.random.default_rng(tokens + 7 * share_c2)
    E, K, O, top_k = 64, 2048, 1024, 8
    ranks = [32] * E if share_c2 else [int(v) for v in rng.choice([0, 32, 64], size=E)]
    payload = _ns_layer(rng, E, K, O, ranks, share_c2=share_c2)
    np_payload = {k: (v.numpy() if isinstance(v, torch.Tensor) else v) for k, v in payload.items()}
    selected = np.stack([rng.choice(E, size=top_k, replace=False) for _ in range(tokens)]).astype(np.int32)
    route = tm.build_grouped_route(torch.from_numpy(selected).cuda(), E)
    tok = route["grouped_token_indices"].cpu().numpy()
    x = rng.standard_normal((tokens, K)).astype(np.float16)
    xg = x[tok]
    ids, seg = route["expert_ids"].cpu().numpy(), route["segment_offsets"].cpu().numpy()
    ref = orc.ns_compensation_fp32(np_payload, xg, ids, seg)
    got = tm.run_grouped_ns_compensation_forward(payload, torch.from_numpy(xg).cuda(), route)
    _check(got, ref)
    # accumulate: fp16(base + fp16(compensation)), exactly what out.add_(compensation) gives
    base = torch.from_numpy(rng.standard_normal((xg.shape[0], O)).astype(np.float16)).cuda()
    acc = base.clone()
    tm.run_grouped_ns_compensation_forward(payload, torch.from_numpy(xg).cuda(), route, out=acc, accumulate=True)
    assert torch.equal(acc, base + got)
    # rows gathered from the token-major activations inside the kernel
    route_g = dict(route)
    route_g["_row_gather"] = route["grouped_token_indices"].to(torch.int32)
    assert torch.equal(tm.run_grouped_ns_compensation_forward(payload, torch.from_numpy(x).cuda(), route_g), got)
    # second half alone on a precomputed C2 product (run_grouped_ns_c1_forward)
    hidden = np.zeros((xg.shape[0], max(ranks)), np.float16)
    for s, e in enumerate(ids):
        c1, c2 = orc.ns_expert_matrices(np_payload, int(e))
        if c2 is not None:
            hidden[seg[s]:seg[s + 1], : c2.shape[0]] = (xg[seg[s]:seg[s + 1]].astype(np.float32) @ c2.astype(np.float32).T).astype(np.float16)
    got_c1 = tm.run_grouped_ns_c1_forward(payload, torch.from_numpy(hidden).cuda(), route)
    _check(got_c1, ref)


def test_grouped_operators_add_compensation(lib):
    """run_grouped_structured_expert_forward / _pair_forward with an ns payload: out = fp16(out + comp)
    bit for bit; with fuse_silu_mul the compensation is added before the activation."""
    import trismoe_b200 as tm
    from trismoe_b200 import synth

    rng = np.random.default_rng(3)
    shape = synth.LayerShape(256, 192, 8, 2, rank=96, group_size=32)
    layer = synth.synth_layer(shape, seed=11)
    gate, up = tm.prepare_grouped_payload(layer["gate"], "cuda"), tm.prepare_grouped_payload(layer["up"], "cuda")
    ranks = [16, 0, 24, 16, 8, 40, 0, 16]
    ns_a = _ns_layer(rng, 8, 256, 192, ranks, group=128)
    ns_b = _ns_layer(rng, 8, 256, 192, ranks[::-1], group=128)
    T = 9
    selected = np.stack([rng.choice(8, size=2, replace=False) for _ in range(T)]).astype(np.int32)
    route = tm.build_grouped_route(torch.from_numpy(selected).cuda(), 8)
    tok = route["grouped_token_indices"]
    x = torch.from_numpy(rng.standard_normal((T, 256)).astype(np.float16)).cuda()
    xg = x.index_select(0, tok)
    hg = tm.compute_shared_hidden(x, layer["shared_gate"].cuda()).index_select(0, tok)
    hu = tm.compute_shared_hidden(x, layer["shared_up"].cuda()).index_select(0, tok)
    base = tm.run_grouped_structured_expert_forward(gate, hg, xg, route)
    comp = tm.run_grouped_ns_compensation_forward(ns_a, xg, route)
    assert comp.abs().float().mean() > 1e-3
    with_ns = tm.run_grouped_structured_expert_forward(gate, hg, xg, route, ns_payload=ns_a)
    assert torch.equal(with_ns, base + comp)
    a0, b0 = tm.run_grouped_structured_expert_pair_forward(gate, up, hg, hu, xg, route)
    comp_b = tm.run_grouped_ns_compensation_forward(ns_b, xg, route)
    a1, b1 = tm.run_grouped_structured_expert_pair_forward(gate, up, hg, hu, xg, route, ns_payload_a=ns_a, ns_payload_b=ns_b)
    assert torch.equal(a1, a0 + comp) and torch.equal(b1, b0 + comp_b)
    fused, none = tm.run_grouped_structured_expert_pair_forward(gate, up, hg, hu, xg, route, ns_payload_a=ns_a, ns_payload_b=ns_b,
                                                                fuse_silu_mul=True)
    assert none is None
    assert torch.equal(fused, (torch.nn.functional.silu(a1.float()) * b1.float()).half())


@pytest.mark.parametrize("tokens", [1, 24, 40, 300])
def test_moe_block_with_packed_backbones(lib, tokens):
    """A block whose three backbones arrive as 4-bit payloads: kept in their nibbles (decode batches
    run the 4-bit GEMM inside tris_moe_layer_forward, large batches expand into shared scratch) vs the
    same block with the backbones expanded at load, and vs the fp32 oracle."""
    import trismoe_b200 as tm
    from trismoe_b200 import synth

    shape = synth.LayerShape(256, 192, 8, 2, rank=96, group_size=32)
    layer = synth.synth_layer(shape, seed=21)
    rng = np.random.default_rng(tokens)
    packed = {"gate": synth.packed4_matrix(rng, 96, 256, 128, scale_std=0.02), "up": synth.packed4_matrix(rng, 96, 256, 128, scale_std=0.02),
              "down": synth.packed4_matrix(rng, 96, 192, 64, scale_std=0.02)}
    blocks = {}
    for mode in ("nibbles", "fp16"):
        blk = tm.TrisSparseMoeBlock(shape.hidden_size, shape.intermediate_size, shape.num_experts, shape.top_k, shape.norm_topk_prob)
        clone = lambda p: {k: (v.clone() if isinstance(v, torch.Tensor) else v) for k, v in p.items()}
        blk.load_grouped_payloads(clone(layer["gate"]), clone(layer["up"]), clone(layer["down"]), packed["gate"], packed["up"],
                                  packed["down"], layer["router_weight"], device="cuda", packed_backbone=mode)
        blocks[mode] = blk
    assert set(blocks["nibbles"].packed_backbones) == {"gate", "up", "down"} and not blocks["fp16"].packed_backbones
    assert blocks["nibbles"].shared_gate.numel() == 0
    x = synth.synth_activations(tokens, shape.hidden_size, seed=tokens).cuda()
    logits = synth.synth_router_logits(tokens, shape.num_experts, seed=5).cuda()
    y_n, _ = blocks["nibbles"](x.view(1, tokens, -1), router_logits=logits)
    y_f, _ = blocks["fp16"](x.view(1, tokens, -1), router_logits=logits)
    weights = {n: [orc.dequantize_expert(to_numpy_payload(layer[n]), e) for e in range(shape.num_experts)] for n in ("gate", "up", "down")}
    shared = {n: orc.dequantize_packed4(*_np_matrix(packed[n])) for n in ("gate", "up", "down")}
    ref = orc.moe_layer_fp32(x.cpu().numpy(), logits.cpu().numpy(), weights, shared, shape.top_k, shape.norm_topk_prob)
    _check(y_n.view(tokens, -1), ref, floor=1e-4)
    _check(y_f.view(tokens, -1), ref, floor=1e-4)
    y_ops, _ = blocks["nibbles"].forward_grouped_ops(x.view(1, tokens, -1), router_logits=logits)
    _check(y_ops.view(tokens, -1), ref, floor=1e-4)
    blocks["nibbles"].raise_on_kernel_status()


def test_moe_block_with_vector_and_matrix_null_space(lib):
    """A block as a real ns checkpoint hands it over: per-projection input scales (ns_mode == 1, with the
    row scale in the payload's output_scale) and null-space pairs (ns_mode == 2) - against the fp32
    oracle with the scales folded into the weights and the compensation added per projection."""
    import trismoe_b200 as tm
    from trismoe_b200 import synth

    rng = np.random.default_rng(9)
    shape = synth.LayerShape(256, 192, 8, 2, rank=96, group_size=32)
    layer = synth.synth_layer(shape, seed=51)
    E, H, I = shape.num_experts, shape.hidden_size, shape.intermediate_size
    in_scale = {"gate": (1 + 0.2 * rng.standard_normal(H)).astype(np.float16), "up": (1 + 0.2 * rng.standard_normal(H)).astype(np.float16),
                "down": (1 + 0.2 * rng.standard_normal(I)).astype(np.float16)}
    out_scale = {"gate": (1 + 0.2 * rng.standard_normal((E, I))).astype(np.float16), "up": (1 + 0.2 * rng.standard_normal((E, I))).astype(np.float16),
                 "down": (1 + 0.2 * rng.standard_normal((E, H))).astype(np.float16)}
    for n in ("gate", "up", "down"):
        layer[n]["output_scale"] = torch.from_numpy(out_scale[n])
        layer[n]["has_output_scale"] = True
    ranks = [16, 0, 24, 16, 8, 40, 0, 16]
    ns = {"gate": _ns_layer(rng, E, H, I, ranks), "up": _ns_layer(rng, E, H, I, ranks[::-1]), "down": _ns_layer(rng, E, I, H, ranks)}
    blk = tm.TrisSparseMoeBlock(H, I, E, shape.top_k, shape.norm_topk_prob)
    blk.load_grouped_payloads(layer["gate"], layer["up"], layer["down"], layer["shared_gate"], layer["shared_up"], layer["shared_down"],
                              layer["router_weight"], device="cuda", input_scales={n: torch.from_numpy(v) for n, v in in_scale.items()})
    blk.load_ns_compensation_payloads(ns["gate"], ns["up"], ns["down"])
    T = 13
    x = (synth.synth_activations(T, H, seed=2).float() * 0.25).half()   # keeps the outputs of order one
    logits = synth.synth_router_logits(T, E, seed=6)
    y, _ = blk(x.cuda().view(1, T, -1), router_logits=logits.cuda())

    # fp32 restatement of QuantLinear.forward (mode 5) per routed expert, qlinear_cuda.py:4692-4749
    w = {n: [orc.dequantize_expert(to_numpy_payload({k: v for k, v in layer[n].items() if k not in ("output_scale", "has_output_scale")}), e)
             .astype(np.float32) for e in range(E)] for n in ("gate", "up", "down")}
    sv = {n: layer["shared_" + n].numpy().astype(np.float32) for n in ("gate", "up", "down")}
    np_ns = {n: {k: (v.cpu().numpy() if isinstance(v, torch.Tensor) else v) for k, v in ns[n].items() if not k.startswith("_tris")} for n in ns}

    def linear(n, e, xin):
        out = ((xin * in_scale[n].astype(np.float32)) @ sv[n].T) @ w[n][e].T * out_scale[n][e].astype(np.float32)
        c1, c2 = orc.ns_expert_matrices(np_ns[n], e)
        if c1 is not None:
            out = out + (xin @ c2.astype(np.float32).T) @ c1.astype(np.float32).T
        return out

    xf = x.numpy().astype(np.float32)
    sel, wts = orc.router_topk(logits.numpy(), shape.top_k, shape.norm_topk_prob)
    ref = np.zeros((T, H), np.float32)
    for t in range(T):
        for s in range(shape.top_k):
            e = int(sel[t, s])
            gate_o, up_o = linear("gate", e, xf[t:t + 1]), linear("up", e, xf[t:t + 1])
            mlp = gate_o / (1.0 + np.exp(-gate_o)) * up_o
            ref[t] += wts[t, s] * linear("down", e, mlp)[0]
    _check(y.view(T, -1), ref, floor=1e-4)
