"""GPU parity tests: every result comes from the CUDA library through its C ABI (via the
ctypes shim) and is compared with the CPU oracle / the reference-generated fixtures.

Bars: decoded bitmaps, dequantized fp16 weights, routes and top-k indices are bit-exact;
layer and operator outputs are within max-abs 2e-2 and mean-relative 1e-3 of the fp32
oracle (mean-relative = mean|y - y*| / mean|y*|).
"""
import ctypes as C
import math

import numpy as np
import pytest
import torch

import trismoe_oracle as orc
from helpers import golden_expert_payload, load_golden, to_numpy_payload

pytestmark = pytest.mark.gpu

MAX_ABS = 2e-2
MEAN_REL = 1e-3


@pytest.fixture(scope="module")
def tm(lib):
    import trismoe_b200

    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    return trismoe_b200


def _stack_golden(tm, z, E, prefix_fmt, use_block_gr=True):
    experts = [golden_expert_payload(z, prefix_fmt.format(e=e)) for e in range(E)]
    return tm.stack_expert_payloads(experts, use_block_gr=use_block_gr)


def _cuda_payload(tm, payload, **kw):
    p = {k: (v.clone() if isinstance(v, torch.Tensor) and not k.startswith("_") else v) for k, v in payload.items()}
    return tm.prepare_grouped_payload(p, "cuda", **kw)


def _oracle_weights_all(tm, layer, blk, name, experts):
    """fp16 oracle weights {e: [O, r]} of the given experts of projection ``name``.  The GPU's
    block-GR decode of the WHOLE projection is first checked bit for bit against the dense map
    the streams were encoded from (the generator keeps it), then the oracle dequantises every
    listed expert from those bits with vectorised numpy - no sampling."""
    p = layer[name]
    dense_ref = p["_dense_gmap_words"]
    if bool(p.get("compact3_use_block_gr", False)):
        dense_gpu = tm.decode_block_gr_gmap(blk._get_grouped_payload(name)).cpu()
        assert torch.equal(dense_gpu, dense_ref), name
    npp = to_numpy_payload(p)
    dense = dense_ref.numpy()
    r = int(npp["g_idx"].shape[1])
    out = {}
    for e in experts:
        out[e] = orc.dequantize_compact3(npp["qweight1"][e], npp["qweight2_sparse"][e], orc.unpack_rows(dense[e], r),
                                         npp["c_map"][e], npp["g_idx"][e], npp["col_pack3"][e], npp["row_pack3"][e], r)
    return out


def _assert_half_bits_equal(got, ref):
    assert got.shape == ref.shape
    a, b = orc.canonical_half_bits(got), orc.canonical_half_bits(ref)
    bad = np.flatnonzero(a.reshape(-1) != b.reshape(-1))
    assert bad.size == 0, f"{bad.size} of {a.size} fp16 weights differ, first at flat index {bad[:5]}"


# ---------------------------------------------------------------------------------------
# (1) block-GR decode and (2) dequantisation: bit-exact
# ---------------------------------------------------------------------------------------
@pytest.mark.parametrize("name", ["proj_ragged.npz", "proj_r256.npz"])
@pytest.mark.parametrize("sub", [1, 16, 32])
def test_decode_and_dequant_match_reference_fixtures(tm, name, sub):
    z = load_golden(name)
    E, O, r, _ = (int(v) for v in z["dims"])
    stacked = _stack_golden(tm, z, E, "ref{e}")
    # the host encoder reproduced the reference stream (checked on CPU); decode it on the GPU
    p = _cuda_payload(tm, stacked, gr_substreams=sub)
    dense = tm.decode_block_gr_gmap(p).cpu().numpy()
    for e in range(E):
        assert np.array_equal(dense[e], z[f"ref{e}_dense_gmap"]), f"expert {e}"
    w = tm.dequantize_grouped_payload(p).cpu().numpy()
    for e in range(E):
        _assert_half_bits_equal(w[e], z[f"ref{e}_weight_f16"])


def test_decode_sweep_every_k_raw_empty(tm):
    z = load_golden("block_gr_sweep.npz")
    for tag in ("a", "b", "braw"):
        dense = z["b_dense" if tag == "braw" else f"{tag}_dense"]
        pr, O = dense.shape
        r = pr * 32
        payload = {
            "qweight1": torch.zeros((1, pr, O), dtype=torch.int32),
            "qweight2_sparse": torch.zeros((1, 0, O), dtype=torch.int32),
            "qweight2_sparse_prefix": torch.zeros((1, pr + 1), dtype=torch.int32),
            "q_gmap_sparse": torch.zeros((1, 0, O), dtype=torch.int32),
            "q_gmap_sparse_prefix": torch.zeros((1, pr + 1), dtype=torch.int32),
            "q_gmap_gr_words": torch.from_numpy(z[f"{tag}_words"].copy())[None],
            "q_gmap_gr_offsets": torch.from_numpy(z[f"{tag}_offsets"].copy())[None],
            "q_gmap_gr_meta": torch.from_numpy(z[f"{tag}_meta"].copy())[None],
            "compact3_use_block_gr": True,
            "c_map": torch.zeros((1, pr), dtype=torch.int32),
            "g_idx": torch.zeros((1, r), dtype=torch.int32),
            "col_pack3": torch.zeros((1, r), dtype=torch.int64),
            "row_pack3": torch.zeros((1, O, 1), dtype=torch.int64),
        }
        for sub in (1, 4, 16):
            p = _cuda_payload(tm, payload, gr_substreams=sub)
            got = tm.decode_block_gr_gmap(p).cpu().numpy()[0]
            assert np.array_equal(got, dense), (tag, sub)


def test_corrupt_stream_is_rejected_at_prepare(tm):
    z = load_golden("proj_r256.npz")
    stacked = _stack_golden(tm, z, 2, "ref{e}")
    bad = {k: (v.clone() if isinstance(v, torch.Tensor) else v) for k, v in stacked.items()}
    bad["q_gmap_gr_offsets"][1, 3] = bad["q_gmap_gr_offsets"][1, 2] - 5  # non-monotone offsets
    with pytest.raises(RuntimeError, match="corrupt"):
        tm.prepare_grouped_payload(bad, "cuda")
    bad = {k: (v.clone() if isinstance(v, torch.Tensor) else v) for k, v in stacked.items()}
    bad["q_gmap_gr_meta"][0, 0] = 9 | (5 << 8)  # k = 9 > 7
    with pytest.raises(RuntimeError, match="corrupt"):
        tm.prepare_grouped_payload(bad, "cuda")
    bad = {k: (v.clone() if isinstance(v, torch.Tensor) else v) for k, v in stacked.items()}
    bad["g_idx"][0, 5] = 1  # group changes inside a 32-column word
    with pytest.raises(RuntimeError, match="g_idx"):
        tm.prepare_grouped_payload(bad, "cuda")


@pytest.fixture(scope="module")
def small_layer(tm):
    from trismoe_b200 import synth

    shape = synth.LayerShape(192, 160, 6, 2, rank=80, group_size=32, norm_topk_prob=True)
    layer = synth.synth_layer(shape, seed=5, keep_sparse_gmap=True)
    for name in ("gate", "up", "down"):  # larger backbones keep this tiny layer's outputs well inside fp16 range
        layer["shared_" + name] = (layer["shared_" + name].float() * 6.0).half()
    weights = {}
    for name in ("gate", "up", "down"):
        npp = to_numpy_payload(layer[name])
        weights[name] = [orc.dequantize_expert(npp, e) for e in range(shape.num_experts)]
    return shape, layer, weights


def test_dequant_synth_block_gr_and_sparse_formats(tm, small_layer):
    shape, layer, weights = small_layer
    for name in ("gate", "down"):
        ref = np.stack(weights[name])
        p = _cuda_payload(tm, layer[name])
        assert np.array_equal(tm.decode_block_gr_gmap(p).cpu().numpy(), layer[name]["_dense_gmap_words"].numpy())
        _assert_half_bits_equal(tm.dequantize_grouped_payload(p).cpu().numpy(), ref)
        # streaming format: sparse bitmap instead of the GR stream
        sparse = {k: v for k, v in layer[name].items()}
        sparse["compact3_use_block_gr"] = False
        p2 = _cuda_payload(tm, sparse)
        _assert_half_bits_equal(tm.dequantize_grouped_payload(p2).cpu().numpy(), ref)


def _grouped_reference(weights, hidden, route):
    return _grouped_reference_impl(weights, hidden, route)


def test_odd_shapes_take_the_unaligned_copy_path(tm):
    """Outputs not a multiple of 4 and rank not a multiple of 8: every staged row is
    misaligned for TMA, so the plain-load fallback of each copy is what runs."""
    from trismoe_b200 import synth

    shape = synth.LayerShape(70, 90, 3, 2, rank=44, group_size=32)
    layer = synth.synth_layer(shape, seed=9, keep_sparse_gmap=True)
    rng = np.random.default_rng(4)
    for name, O in (("gate", 90), ("down", 70)):
        npp = to_numpy_payload(layer[name])
        ref = np.stack([orc.dequantize_expert(npp, e) for e in range(3)])
        for fmt in ("block_gr", "sparse"):
            src = dict(layer[name])
            src["compact3_use_block_gr"] = fmt == "block_gr"
            p = _cuda_payload(tm, src)
            if fmt == "block_gr":
                assert np.array_equal(tm.decode_block_gr_gmap(p).cpu().numpy(), layer[name]["_dense_gmap_words"].numpy())
            _assert_half_bits_equal(tm.dequantize_grouped_payload(p).cpu().numpy(), ref)
            h = rng.standard_normal((7, 44)).astype(np.float16)
            out = tm.run_grouped_structured_expert_forward(p, torch.from_numpy(h).cuda(), None, [3, 0, 4])
            want = _grouped_reference(list(ref), h, {"expert_ids": np.array([0, 2]), "segment_offsets": np.array([0, 3, 7])})
            max_abs, mean_rel = orc.error_metrics(out.float().cpu().numpy(), want)
            assert max_abs <= MAX_ABS and mean_rel <= MEAN_REL, (max_abs, mean_rel)


# ---------------------------------------------------------------------------------------
# (3) backbone, (4) route, (5) router
# ---------------------------------------------------------------------------------------
@pytest.mark.parametrize("n,k,m", [(1, 2048, 256), (5, 1024, 256), (33, 512, 80), (130, 2048, 64), (1024, 1024, 256)])
def test_shared_hidden_vs_fp32(tm, n, k, m):
    g = torch.Generator().manual_seed(n * 7 + m)
    x = torch.randn((n, k), generator=g).half()
    sv = (0.02 * torch.randn((m, k), generator=g)).half()
    got = tm.compute_shared_hidden(x.cuda(), sv.cuda()).float().cpu().numpy()
    ref = (x.float() @ sv.float().T).numpy()
    max_abs, mean_rel = orc.error_metrics(got, ref)
    assert max_abs <= MAX_ABS and mean_rel <= MEAN_REL, (max_abs, mean_rel)


@pytest.mark.parametrize("T,k,E", [(1, 8, 64), (8, 8, 64), (128, 8, 64), (64, 2, 8), (16, 8, 256), (700, 2, 8),
                                   (700, 8, 64), (2048, 8, 64), (5000, 2, 8), (1111, 8, 256)])  # >= 8192 rows: multi-CTA sort
def test_route_matches_oracle(tm, T, k, E):
    rng = np.random.default_rng(T * 31 + E)
    sel = np.stack([rng.choice(E, size=k, replace=False) for _ in range(T)]).astype(np.int64)
    route = tm.build_grouped_route(torch.from_numpy(sel).cuda(), E)
    ref = orc.build_route(sel, E)
    for key in ("perm", "grouped_token_indices", "grouped_slots", "grouped_expert_ids", "expert_ids",
                "segment_offsets", "problem_offsets"):
        assert np.array_equal(route[key].cpu().numpy(), ref[key]), key
    assert route["total_problem_tiles_host"] == ref["total_problem_tiles_host"]
    inv = route["_row_of_flat"].cpu().numpy()
    assert np.array_equal(ref["perm"][inv], np.arange(T * k))
    assert route["perm"].dtype == torch.long and route["expert_ids"].dtype == torch.int32


def test_route_edge_cases(tm):
    empty = tm.build_grouped_route(torch.zeros((0, 8), dtype=torch.long, device="cuda"), 64)
    assert empty["grouped_token_indices"].numel() == 0 and empty["total_problem_tiles_host"] == 0
    assert tm.build_grouped_route(torch.zeros((8,), dtype=torch.long, device="cuda"), 64) is None
    # every token on one expert
    route = tm.build_grouped_route(torch.full((5, 1), 3, dtype=torch.long, device="cuda"), 4)
    assert route["expert_ids"].tolist() == [3] and route["segment_offsets"].tolist() == [0, 5]
    assert route["problem_offsets"].tolist() == [0, 2]


@pytest.mark.parametrize("T,E,k,norm", [(1, 64, 8, True), (37, 64, 8, False), (128, 8, 2, True), (16, 256, 8, True)])
def test_router_topk_matches_oracle(tm, T, E, k, norm):
    import ctypes as C

    rng = np.random.default_rng(E + T)
    logits = rng.standard_normal((T, E)).astype(np.float32)
    d = torch.from_numpy(logits).cuda()
    sel = torch.empty((T, k), dtype=torch.int32, device="cuda")
    w = torch.empty((T, k), dtype=torch.float32, device="cuda")
    lib = tm._native.load()
    tm._native.check(lib.tris_router_topk(d.data_ptr(), T, E, k, int(norm), sel.data_ptr(), w.data_ptr(),
                                          torch.cuda.current_stream().cuda_stream))
    rsel, rw = orc.router_topk(logits, k, norm)
    assert np.array_equal(sel.cpu().numpy(), rsel)
    assert np.allclose(w.cpu().numpy(), rw, rtol=1e-5, atol=1e-7)


# ---------------------------------------------------------------------------------------
# (6) grouped operators against the fp32 oracle
# ---------------------------------------------------------------------------------------
def _grouped_reference_impl(weights, hidden, route):
    out = np.zeros((hidden.shape[0], weights[0].shape[0]), dtype=np.float32)
    seg = route["segment_offsets"]
    for s, e in enumerate(route["expert_ids"]):
        rows = slice(int(seg[s]), int(seg[s + 1]))
        out[rows] = hidden[rows].astype(np.float32) @ weights[int(e)].astype(np.float32).T
    return out


@pytest.mark.parametrize("T", [1, 3, 20, 70])
@pytest.mark.parametrize("fmt", ["block_gr", "sparse"])
def test_grouped_forward_and_pair(tm, small_layer, T, fmt):
    shape, layer, weights = small_layer
    E, k, r = shape.num_experts, shape.top_k, shape.rank
    rng = np.random.default_rng(T)
    sel = np.stack([rng.choice(E, size=k, replace=False) for _ in range(T)]).astype(np.int64)
    route = tm.build_grouped_route(torch.from_numpy(sel).cuda(), E)
    oroute = orc.build_route(sel, E)
    R = T * k

    def payload(name):
        src = dict(layer[name])
        if fmt == "sparse":
            src["compact3_use_block_gr"] = False
        return _cuda_payload(tm, src)

    ha = rng.standard_normal((R, r)).astype(np.float16)
    hb = rng.standard_normal((R, r)).astype(np.float16)
    x_dummy = torch.zeros((R, 8), dtype=torch.float16, device="cuda")
    out = tm.run_grouped_structured_expert_forward(payload("down"), torch.from_numpy(ha).cuda(), x_dummy, route)
    ref = _grouped_reference(weights["down"], ha, oroute)
    max_abs, mean_rel = orc.error_metrics(out.float().cpu().numpy(), ref)
    assert max_abs <= MAX_ABS and mean_rel <= MEAN_REL, (max_abs, mean_rel)

    oa, ob = tm.run_grouped_structured_expert_pair_forward(payload("gate"), payload("up"), torch.from_numpy(ha).cuda(),
                                                           torch.from_numpy(hb).cuda(), x_dummy, route)
    ra = _grouped_reference(weights["gate"], ha, oroute)
    rb = _grouped_reference(weights["up"], hb, oroute)
    for got, want in ((oa, ra), (ob, rb)):
        max_abs, mean_rel = orc.error_metrics(got.float().cpu().numpy(), want)
        assert max_abs <= MAX_ABS and mean_rel <= MEAN_REL, (max_abs, mean_rel)
    fused, none = tm.run_grouped_structured_expert_pair_forward(
        payload("gate"), payload("up"), torch.from_numpy(ha).cuda(), torch.from_numpy(hb).cuda(), x_dummy, route,
        fuse_silu_mul=True)
    assert none is None
    want = ra / (1 + np.exp(-ra)) * rb
    max_abs, mean_rel = orc.error_metrics(fused.float().cpu().numpy(), want)
    assert max_abs <= MAX_ABS and mean_rel <= MEAN_REL, (max_abs, mean_rel)


def test_grouped_forward_from_segment_lengths_and_bad_args(tm, small_layer):
    shape, layer, weights = small_layer
    p = _cuda_payload(tm, layer["down"])
    r = shape.rank
    rng = np.random.default_rng(0)
    lengths = [2, 0, 5, 1, 0, 0]
    R = sum(lengths)
    h = rng.standard_normal((R, r)).astype(np.float16)
    out = tm.run_grouped_structured_expert_forward(p, torch.from_numpy(h).cuda(), None, lengths)
    route = {"expert_ids": np.array([0, 2, 3]), "segment_offsets": np.array([0, 2, 7, 8])}
    ref = _grouped_reference(weights["down"], h, route)
    max_abs, mean_rel = orc.error_metrics(out.float().cpu().numpy(), ref)
    assert max_abs <= MAX_ABS and mean_rel <= MEAN_REL
    # results sent to caller-chosen output rows: the same numbers, permuted
    scatter = torch.from_numpy(rng.permutation(R).astype(np.int32)).cuda()
    troute = {"expert_ids": torch.tensor([0, 2, 3], dtype=torch.int32, device="cuda"),
              "segment_offsets": torch.tensor([0, 2, 7, 8], dtype=torch.int32, device="cuda"),
              "_out_row_scatter": scatter}
    out2 = tm.run_grouped_structured_expert_forward(p, torch.from_numpy(h).cuda(), None, troute)
    assert torch.equal(out2[scatter.long()], out)
    # long segments (several passes of the 64-row variant) with scattered output rows
    big = [150, 0, 0, 70, 0, 9]
    Rb = sum(big)
    hb = torch.from_numpy(rng.standard_normal((Rb, r)).astype(np.float16)).cuda()
    plain = tm.run_grouped_structured_expert_forward(p, hb, None, big)
    sc = torch.from_numpy(rng.permutation(Rb).astype(np.int32)).cuda()
    broute = {"expert_ids": torch.tensor([0, 3, 5], dtype=torch.int32, device="cuda"),
              "segment_offsets": torch.tensor([0, 150, 220, 229], dtype=torch.int32, device="cuda"),
              "_max_rows_per_segment": 150, "_out_row_scatter": sc}
    scattered = tm.run_grouped_structured_expert_forward(p, hb, None, broute)
    assert torch.equal(scattered[sc.long()], plain)
    refb = _grouped_reference(weights["down"], hb.cpu().numpy(), {"expert_ids": np.array([0, 3, 5]),
                                                                  "segment_offsets": np.array([0, 150, 220, 229])})
    max_abs, mean_rel = orc.error_metrics(plain.float().cpu().numpy(), refb)
    assert max_abs <= MAX_ABS and mean_rel <= MEAN_REL
    # reference behaviour: wrong dtype / wrong rank -> None, not an exception
    assert tm.run_grouped_structured_expert_forward(p, torch.zeros((R, r), device="cuda"), None, lengths) is None
    assert tm.run_grouped_structured_expert_forward(p, torch.zeros((R, r + 8), dtype=torch.float16, device="cuda"), None, lengths) is None
    empty = tm.run_grouped_structured_expert_forward(p, torch.zeros((0, r), dtype=torch.float16, device="cuda"), None, [0] * 6)
    assert empty is None or empty.shape[0] == 0


# ---------------------------------------------------------------------------------------
# (7) whole block
# ---------------------------------------------------------------------------------------
def _block_from_layer(tm, shape, layer):
    blk = tm.TrisSparseMoeBlock(shape.hidden_size, shape.intermediate_size, shape.num_experts, shape.top_k,
                                shape.norm_topk_prob)
    cp = lambda p: {k: (v.clone() if isinstance(v, torch.Tensor) and not k.startswith("_") else v) for k, v in p.items()}
    blk.load_grouped_payloads(cp(layer["gate"]), cp(layer["up"]), cp(layer["down"]), layer["shared_gate"],
                              layer["shared_up"], layer["shared_down"], layer["router_weight"], device="cuda")
    return blk


@pytest.mark.parametrize("T", [1, 2, 9, 40, 128])
def test_layer_small_vs_fp32_oracle(tm, small_layer, T):
    from trismoe_b200 import synth

    shape, layer, weights = small_layer
    blk = _block_from_layer(tm, shape, layer)
    x = synth.synth_activations(T, shape.hidden_size, seed=T)
    logits = synth.synth_router_logits(T, shape.num_experts, seed=100 + T)
    shared = {n: layer["shared_" + n].numpy() for n in ("gate", "up", "down")}
    y, _ = blk(x.cuda().view(1, T, -1), router_logits=logits.cuda())
    ref = orc.moe_layer_fp32(x.numpy(), logits.numpy(), weights, shared, shape.top_k, shape.norm_topk_prob)
    max_abs, mean_rel = orc.error_metrics(y.view(T, -1).float().cpu().numpy(), ref)
    assert np.abs(ref).mean() > 0
    assert max_abs <= MAX_ABS and mean_rel <= MEAN_REL, (max_abs, mean_rel)
    # the operator-by-operator composition gives the same answer
    y2, _ = blk.forward_grouped_ops(x.cuda().view(1, T, -1), router_logits=logits.cuda())
    max_abs, mean_rel = orc.error_metrics(y2.view(T, -1).float().cpu().numpy(), ref)
    assert max_abs <= MAX_ABS and mean_rel <= 2 * MEAN_REL, (max_abs, mean_rel)


def test_layer_reference_fixture(tm):
    """Reference-built payloads and the reference block's own fp16 CPU output."""
    z = load_golden("moe_layer_small.npz")
    E, k, H, I, r, group, T = (int(v) for v in z["dims"])
    blk = tm.TrisSparseMoeBlock(H, I, E, k, True)
    payloads, weights = {}, {}
    for name in ("gate", "up", "down"):
        payloads[name] = _stack_golden(tm, z, E, name + "{e}")
        npp = to_numpy_payload(payloads[name])
        weights[name] = [orc.dequantize_expert(npp, e) for e in range(E)]
    blk.load_grouped_payloads(payloads["gate"], payloads["up"], payloads["down"], torch.from_numpy(z["shared_gate"].copy()),
                              torch.from_numpy(z["shared_up"].copy()), torch.from_numpy(z["shared_down"].copy()),
                              torch.from_numpy(z["router_weight"].copy()), device="cuda")
    x = torch.from_numpy(z["x"].copy()).cuda()
    y, logits = blk(x.view(1, T, H))
    # router computed on the GPU agrees with the reference's fp16 linear up to its rounding
    assert np.allclose(logits.cpu().numpy(), z["ref_router_logits_f16"].astype(np.float32), atol=2e-3, rtol=2e-3)
    shared = {n: z["shared_" + n] for n in ("gate", "up", "down")}
    ref32 = orc.moe_layer_fp32(z["x"], logits.cpu().numpy(), weights, shared, k, True)
    max_abs, mean_rel = orc.error_metrics(y.view(T, H).float().cpu().numpy(), ref32)
    assert max_abs <= MAX_ABS and mean_rel <= MEAN_REL, (max_abs, mean_rel)
    # and is as close to the reference's fp16 output as that output is to the fp32 oracle
    sel_mine, _ = orc.router_topk(logits.cpu().numpy(), k, True)
    if np.array_equal(np.sort(sel_mine, 1), np.sort(z["ref_selected"], 1)):
        max_abs, mean_rel = orc.error_metrics(y.view(T, H).float().cpu().numpy(), z["ref_y_f16"].astype(np.float32))
        assert max_abs <= MAX_ABS and mean_rel <= 5e-3, (max_abs, mean_rel)


@pytest.fixture(scope="module")
def olmoe_layer(tm):
    """Headline shape: 64 experts, top-8, hidden 2048, intermediate 1024, rank 256."""
    from trismoe_b200 import synth

    layer = synth.synth_layer(synth.OLMOE, seed=2026)
    blk = _block_from_layer(tm, synth.OLMOE, layer)
    return layer, blk


_OLMOE_ORACLE = {}


@pytest.mark.parametrize("T", [1, 8, 32, 128])
def test_layer_olmoe_shape_decode_batches(tm, olmoe_layer, T):
    """Full-size layer at decode batches 1/8/32/128: dequantised weights of EVERY expert the
    batch routes to bit-exact against the oracle, output against the fp32 oracle built from
    the oracle's own weights."""
    from trismoe_b200 import synth

    layer, blk = olmoe_layer
    shape = synth.OLMOE
    x = synth.synth_activations(T, shape.hidden_size, seed=T)
    logits = synth.synth_router_logits(T, shape.num_experts, seed=7 + T)
    sel, _ = orc.router_topk(logits.numpy(), shape.top_k, True)
    active = sorted(set(int(e) for e in sel.reshape(-1)))
    weights = {}
    for name in ("gate", "up", "down"):
        cache = _OLMOE_ORACLE.setdefault(name, {})
        cache.update(_oracle_weights_all(tm, layer, blk, name, [e for e in active if e not in cache]))
        got = tm.dequantize_grouped_payload(blk._get_grouped_payload(name))
        for e in active:
            _assert_half_bits_equal(got[e].cpu().numpy(), cache[e])
        weights[name] = cache
    shared = {n: layer["shared_" + n].numpy() for n in ("gate", "up", "down")}
    y, _ = blk(x.cuda().view(1, T, -1), router_logits=logits.cuda())
    ref = orc.moe_layer_fp32(x.numpy(), logits.numpy(), weights, shared, shape.top_k, True)
    max_abs, mean_rel = orc.error_metrics(y.view(T, -1).float().cpu().numpy(), ref)
    assert np.abs(ref).mean() > 1e-4
    assert max_abs <= MAX_ABS and mean_rel <= MEAN_REL, (max_abs, mean_rel)


_SHAPE_CACHE = {}


def _shape_layer(tm, shape_name, **kw):
    from trismoe_b200 import synth

    key = (shape_name, tuple(sorted(kw.items())))
    if key not in _SHAPE_CACHE:
        _SHAPE_CACHE.clear()  # one full-size layer at a time
        shape = getattr(synth, shape_name)
        layer = synth.synth_layer(shape, seed=77, **kw)
        _SHAPE_CACHE[key] = (layer, _block_from_layer(tm, shape, layer), {})
    return _SHAPE_CACHE[key]


@pytest.mark.parametrize("shape_name,T", [("MIXTRAL", 1), ("MIXTRAL", 64), ("QWEN35", 1), ("QWEN35", 16)])
def test_layer_other_baseline_shapes(tm, shape_name, T):
    """Mixtral-shaped (8 experts, top-2, hidden 4096, intermediate 14336) and Qwen3.5-shaped (256
    experts, top-8, hidden 2048, intermediate 512) layers at their decode batches: dequantized
    weights of every routed expert bit-exact against the oracle, output against the fp32 oracle."""
    from trismoe_b200 import synth

    shape = getattr(synth, shape_name)
    layer, blk, oracle_cache = _shape_layer(tm, shape_name)
    x = synth.synth_activations(T, shape.hidden_size, seed=3 + T)
    logits = synth.synth_router_logits(T, shape.num_experts, seed=11 + T)
    sel, _ = orc.router_topk(logits.numpy(), shape.top_k, shape.norm_topk_prob)
    active = sorted(set(int(e) for e in sel.reshape(-1)))
    weights = {}
    for name in ("gate", "up", "down"):
        cache = oracle_cache.setdefault(name, {})
        cache.update(_oracle_weights_all(tm, layer, blk, name, [e for e in active if e not in cache]))
        got = tm.dequantize_grouped_payload(blk._get_grouped_payload(name))
        for e in active:
            _assert_half_bits_equal(got[e].cpu().numpy(), cache[e])
        weights[name] = cache
        del got
    shared = {n: layer["shared_" + n].numpy() for n in ("gate", "up", "down")}
    y, _ = blk(x.cuda().view(1, T, -1), router_logits=logits.cuda())
    ref = orc.moe_layer_fp32(x.numpy(), logits.numpy(), weights, shared, shape.top_k, shape.norm_topk_prob)
    max_abs, mean_rel = orc.error_metrics(y.view(T, -1).float().cpu().numpy(), ref)
    assert np.abs(ref).mean() > 1e-4
    assert max_abs <= MAX_ABS and mean_rel <= MEAN_REL, (max_abs, mean_rel)


def test_full_size_properties(tm, olmoe_layer):
    """Size-independent properties at the headline size: GR decode of every block of every
    expert round-trips to the dense map it was encoded from; a token's output does not
    depend on what else is in the batch; the block is deterministic."""
    from trismoe_b200 import synth

    layer, blk = olmoe_layer
    for name in ("gate", "up", "down"):
        dense = tm.decode_block_gr_gmap(blk._get_grouped_payload(name)).cpu()
        assert torch.equal(dense, layer[name]["_dense_gmap_words"]), name
    T = 128
    x = synth.synth_activations(T, 2048, seed=1).cuda()
    logits = synth.synth_router_logits(T, 64, seed=2).cuda()
    y_all, _ = blk(x.view(1, T, -1), router_logits=logits)
    y_again, _ = blk(x.view(1, T, -1), router_logits=logits)
    assert torch.equal(y_all, y_again)
    for t in (0, 77):
        y_one, _ = blk(x[t: t + 1].view(1, 1, -1), router_logits=logits[t: t + 1])
        assert torch.allclose(y_one.view(-1).float(), y_all.view(T, -1)[t].float(), atol=2e-3, rtol=2e-3)


# ---------------------------------------------------------------------------------------
# (8) streaming: payloads paged from pinned host memory
# ---------------------------------------------------------------------------------------
@pytest.mark.parametrize("mode,fmt", [("bitmap", "sparse"), ("payload", "sparse"), ("payload", "block_gr")])
def test_streaming_forward_matches_oracle(tm, mode, fmt):
    """Payloads paged from pinned host memory: every layer's output is checked against the fp32
    oracle (weights dequantised by the oracle from the CPU payload), must be bit-identical from
    pass to pass and between eager launches and a CUDA-graph replay, and agrees with the
    resident block within the same tolerance (the resident block may run another kernel)."""
    from trismoe_b200 import staging, synth

    shape = synth.LayerShape(256, 192, 8, 2, rank=96, group_size=32)
    blocks, inputs, wants, refs = [], [], [], []
    for L in range(3):
        layer = synth.synth_layer(shape, seed=30 + L, keep_sparse_gmap=True)
        for name in ("gate", "up", "down"):
            layer["shared_" + name] = (layer["shared_" + name].float() * 5.0).half()
            if fmt == "sparse":
                layer[name]["compact3_use_block_gr"] = False
        blk = _block_from_layer(tm, shape, layer)
        T = 5 + 3 * L
        x = synth.synth_activations(T, shape.hidden_size, seed=L).cuda()
        logits = synth.synth_router_logits(T, shape.num_experts, seed=9 + L).cuda()
        want, _ = blk(x.view(1, T, -1), router_logits=logits)
        weights = {n: [orc.dequantize_expert(to_numpy_payload(layer[n]), e) for e in range(shape.num_experts)]
                   for n in ("gate", "up", "down")}
        shared = {n: layer["shared_" + n].numpy() for n in ("gate", "up", "down")}
        refs.append(orc.moe_layer_fp32(x.cpu().numpy(), logits.cpu().numpy(), weights, shared, shape.top_k, shape.norm_topk_prob))
        blocks.append(blk)
        inputs.append((x, logits))
        wants.append(want.clone())
    resident_before = sum(t.numel() * t.element_size() for b in blocks for p in ("gate", "up", "down")
                          for t in b._get_grouped_payload(p).values() if isinstance(t, torch.Tensor))
    manager = staging.GroupedQGmapCPUStagingManager(blocks, mode=mode)
    assert manager.initialize()
    resident_after = sum(t.numel() * t.element_size() for b in blocks for p in ("gate", "up", "down")
                         for t in b._get_grouped_payload(p).values() if isinstance(t, torch.Tensor))
    assert resident_after < resident_before
    streamed = [None] * 3
    for rep in range(2):  # second pass reuses the two staging slots
        for L, blk in enumerate(blocks):
            x, logits = inputs[L]
            got, _ = blk.forward_streaming(x.view(1, x.shape[0], -1), manager, L, router_logits=logits)
            torch.cuda.synchronize()
            T = x.shape[0]
            max_abs, mean_rel = orc.error_metrics(got.view(T, -1).float().cpu().numpy(), refs[L])
            assert np.abs(refs[L]).mean() > 1e-4
            assert max_abs <= MAX_ABS and mean_rel <= MEAN_REL, (mode, fmt, rep, L, max_abs, mean_rel)
            max_abs, mean_rel = orc.error_metrics(got.view(T, -1).float().cpu().numpy(), wants[L].view(T, -1).float().cpu().numpy())
            assert max_abs <= MAX_ABS and mean_rel <= MEAN_REL, (mode, fmt, rep, L, "vs resident", max_abs, mean_rel)
            if rep == 0:
                streamed[L] = got.clone()
            else:
                assert torch.equal(got, streamed[L]), (mode, fmt, rep, L)
    report = manager.overlap_report()
    assert report["layers"] == 6 and report["copy_ms"] > 0
    assert manager.pipeline_stats["calls"] == 6 and manager.pipeline_stats["slot_reuses"] >= 4
    # the same three-layer step as one CUDA graph: pager and compute streams, no host decisions
    manager.collect_timings = False
    outs = []

    def step():
        outs.clear()
        for L, blk in enumerate(blocks):
            x, logits = inputs[L]
            outs.append(blk.forward_streaming(x.view(1, x.shape[0], -1), manager, L, router_logits=logits)[0])

    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        step()
    for _ in range(2):
        for o in outs:
            o.zero_()
        graph.replay()
        torch.cuda.synchronize()
        for L in range(3):
            assert torch.equal(outs[L], streamed[L]), (mode, fmt, "graph", L)
    manager.collect_timings = True


@pytest.mark.parametrize("mode,fmt", [("bitmap", "sparse"), ("payload", "block_gr")])
def test_streaming_with_too_few_slots_reports_instead_of_reading_stale_slots(tm, mode, fmt):
    """A staging manager sized for fewer experts than a batch activates: the experts without a slot
    are marked "not paged" (-1) in the slot table, the grouped kernels skip their segments and the
    block reports TRIS_ERR_WORKSPACE - no output is silently computed from another expert's bytes.
    With enough slots the same call is clean."""
    from trismoe_b200 import staging, synth

    shape = synth.LayerShape(256, 192, 8, 2, rank=96, group_size=32)
    layer = synth.synth_layer(shape, seed=41, keep_sparse_gmap=True)
    if fmt == "sparse":
        for name in ("gate", "up", "down"):
            layer[name]["compact3_use_block_gr"] = False
    T = 12
    x = synth.synth_activations(T, shape.hidden_size, seed=3).cuda()
    logits = synth.synth_router_logits(T, shape.num_experts, seed=4).cuda()
    active = len(set(torch.topk(torch.softmax(logits.float(), 1), shape.top_k, -1)[1].reshape(-1).tolist()))
    assert active > 2
    for slots, expect in ((2, 5), (shape.num_experts, 0)):  # 5 = TRIS_ERR_WORKSPACE
        blk = _block_from_layer(tm, shape, layer)
        manager = staging.GroupedQGmapCPUStagingManager([blk], mode=mode, max_active_experts=slots)
        assert manager.initialize()
        blk.forward_streaming(x.view(1, T, -1), manager, 0, router_logits=logits)
        torch.cuda.synchronize()
        assert blk.last_kernel_status(clear=False) == expect, (slots, expect)
        if expect:
            with pytest.raises(RuntimeError, match="TRIS_ERR_WORKSPACE"):
                blk.raise_on_kernel_status()
        else:
            blk.raise_on_kernel_status()


@pytest.mark.parametrize("mode,fmt,T", [("bitmap", "sparse", 1), ("bitmap", "sparse", 16), ("payload", "block_gr", 1),
                                        ("payload", "block_gr", 16)])
def test_streaming_qwen35_shape_vs_oracle(tm, mode, fmt, T):
    """BASELINE config 4's shape (256 experts, top-8, hidden 2048, intermediate 512) in streaming
    mode at decode batch 1 and 16, both paging modes: output against the fp32 oracle whose weights
    are dequantised by the oracle for every routed expert."""
    from trismoe_b200 import staging, synth

    shape = synth.QWEN35
    kw = {"keep_sparse_gmap": True}
    layer, blk, oracle_cache = _shape_layer(tm, "QWEN35", **kw)
    x = synth.synth_activations(T, shape.hidden_size, seed=5 + T)
    logits = synth.synth_router_logits(T, shape.num_experts, seed=13 + T)
    sel, _ = orc.router_topk(logits.numpy(), shape.top_k, shape.norm_topk_prob)
    active = sorted(set(int(e) for e in sel.reshape(-1)))
    weights = {}
    for name in ("gate", "up", "down"):
        cache = oracle_cache.setdefault(name, {})
        cache.update(_oracle_weights_all(tm, layer, blk, name, [e for e in active if e not in cache]))
        weights[name] = cache
    shared = {n: layer["shared_" + n].numpy() for n in ("gate", "up", "down")}
    ref = orc.moe_layer_fp32(x.numpy(), logits.numpy(), weights, shared, shape.top_k, shape.norm_topk_prob)
    # a fresh block for the manager: it moves the paged tensors of its blocks to pinned host memory
    cp = lambda p: {k: (v.clone() if isinstance(v, torch.Tensor) else v) for k, v in p.items()}
    lay2 = {k: (cp(v) if isinstance(v, dict) else v) for k, v in layer.items()}
    if fmt == "sparse":
        for name in ("gate", "up", "down"):
            lay2[name]["compact3_use_block_gr"] = False
    sblk = _block_from_layer(tm, shape, lay2)
    manager = staging.GroupedQGmapCPUStagingManager([sblk], mode=mode)
    assert manager.initialize()
    for rep in range(2):
        got, _ = sblk.forward_streaming(x.cuda().view(1, T, -1), manager, 0, router_logits=logits.cuda())
        torch.cuda.synchronize()
        max_abs, mean_rel = orc.error_metrics(got.view(T, -1).float().cpu().numpy(), ref)
        assert np.abs(ref).mean() > 1e-4
        assert max_abs <= MAX_ABS and mean_rel <= MEAN_REL, (mode, fmt, T, rep, max_abs, mean_rel)
    del manager, sblk
    torch.cuda.empty_cache()


# ---------------------------------------------------------------------------------------
# (9) prefill-sized segments: tcgen05 / TMEM grouped kernel
# ---------------------------------------------------------------------------------------
@pytest.fixture
def tensor_core_from_64_rows(tm):
    """The launchers pick the tcgen05 kernel above a row count whose default lies beyond these
    tests' sizes; lower it so that the tensor-core kernel is what runs, and put it back."""
    lib = tm._native.load()
    previous = lib.tris_set_grouped_tc_min_rows(64)
    yield
    lib.tris_set_grouped_tc_min_rows(previous)


@pytest.mark.parametrize("rank,T", [(96, 200), (256, 150), (64, 700)])
def test_layer_prefill_rows_take_the_tensor_core_path(tm, tensor_core_from_64_rows, rank, T):
    """Few experts, many tokens: ~100+ rows per expert, rank a multiple of 32 -> the grouped
    kernels run their tcgen05 variant (weights unpacked once per tile into shared memory)."""
    from trismoe_b200 import synth

    shape = synth.LayerShape(256, 320, 4, 2, rank=rank, group_size=32)
    layer = synth.synth_layer(shape, seed=rank + T)
    for name in ("gate", "up", "down"):
        layer["shared_" + name] = (layer["shared_" + name].float() * 5.0).half()
    blk = _block_from_layer(tm, shape, layer)
    weights = {n: [orc.dequantize_expert(to_numpy_payload(layer[n]), e) for e in range(4)] for n in ("gate", "up", "down")}
    for name in ("gate", "up", "down"):  # the tile unpack of this path is the bit-exact one
        got = tm.dequantize_grouped_payload(blk._get_grouped_payload(name)).cpu().numpy()
        _assert_half_bits_equal(got, np.stack(weights[name]))
    x = synth.synth_activations(T, shape.hidden_size, seed=T)
    logits = synth.synth_router_logits(T, shape.num_experts, seed=T + 1)
    shared = {n: layer["shared_" + n].numpy() for n in ("gate", "up", "down")}
    y, _ = blk(x.cuda().view(1, T, -1), router_logits=logits.cuda())
    ref = orc.moe_layer_fp32(x.numpy(), logits.numpy(), weights, shared, shape.top_k, shape.norm_topk_prob)
    max_abs, mean_rel = orc.error_metrics(y.view(T, -1).float().cpu().numpy(), ref)
    assert np.abs(ref).mean() > 1e-4
    assert max_abs <= MAX_ABS and mean_rel <= MEAN_REL, (max_abs, mean_rel)
    # and agrees with the register (mma.sync) path, which the operator API takes for row-major input
    y2, _ = blk.forward_grouped_ops(x.cuda().view(1, T, -1), router_logits=logits.cuda())
    max_abs, mean_rel = orc.error_metrics(y2.view(T, -1).float().cpu().numpy(), ref)
    assert max_abs <= MAX_ABS and mean_rel <= 2 * MEAN_REL, (max_abs, mean_rel)


@pytest.mark.parametrize("kernel", ["register", "tensor_core"])
def test_layer_olmoe_shape_prefill_512(tm, olmoe_layer, kernel):
    """Headline shape, 512-token prefill (64 rows per expert on average)."""
    from trismoe_b200 import synth

    layer, blk = olmoe_layer
    T = 512
    x = synth.synth_activations(T, 2048, seed=3).cuda()
    logits = synth.synth_router_logits(T, 64, seed=4).cuda()
    lib = tm._native.load()
    previous = lib.tris_set_grouped_tc_min_rows(64 if kernel == "tensor_core" else 1 << 20)
    try:
        y, _ = blk(x.view(1, T, -1), router_logits=logits)
        torch.cuda.synchronize()
    finally:
        lib.tris_set_grouped_tc_min_rows(previous)
    y2, _ = blk.forward_grouped_ops(x.view(1, T, -1), router_logits=logits)
    ref = y2.view(T, -1).float().cpu().numpy()
    max_abs, mean_rel = orc.error_metrics(y.view(T, -1).float().cpu().numpy(), ref)
    assert np.abs(ref).mean() > 1e-4 and max_abs <= MAX_ABS and mean_rel <= 2 * MEAN_REL, (max_abs, mean_rel)
    # a single token of the batch, recomputed alone through the decode kernels
    for t in (5, 300):
        y_one, _ = blk(x[t: t + 1].view(1, 1, -1), router_logits=logits[t: t + 1])
        assert torch.allclose(y_one.view(-1).float(), y.view(T, -1)[t].float(), atol=3e-3, rtol=3e-3)


def test_row_split_of_long_segments_leaves_results_unchanged(tm):
    """Few experts with long, uneven segments (an expert-parallel rank's shape): the register-cached kernel
    shares a unit's 32-row passes among up to four CTAs.  With the split switched off the outputs are the same
    bits; segments of 1, 33, 70, 130 and 300 rows cover CTAs without a pass, a ragged last pass and CTAs with
    several passes; the result agrees with the fp32 oracle."""
    from trismoe_b200 import synth

    shape = synth.LayerShape(128, 192, 6, 1, rank=128, group_size=32)
    layer = synth.synth_layer(shape, seed=77)
    payloads = {n: tm.prepare_grouped_payload(layer[n], "cuda") for n in ("gate", "up", "down")}
    lengths = [1, 33, 0, 70, 130, 300]
    ids = np.concatenate([np.full(n, e, dtype=np.int64) for e, n in enumerate(lengths)])
    rng = np.random.default_rng(5)
    ids = ids[rng.permutation(ids.size)]
    R = int(ids.size)
    route = tm.build_grouped_route(torch.from_numpy(ids.reshape(R, 1)).cuda(), shape.num_experts)
    hg = (torch.randn((R, 128), generator=torch.Generator().manual_seed(1)) * 0.5).half().cuda()
    hu = (torch.randn((R, 128), generator=torch.Generator().manual_seed(2)) * 0.5).half().cuda()
    hd = (torch.randn((R, 128), generator=torch.Generator().manual_seed(3)) * 0.5).half().cuda()
    lib = tm._native.load()
    outs = {}
    previous = lib.tris_set_grouped_row_split_max(1)
    try:
        for limit in (1, 4, 16):
            lib.tris_set_grouped_row_split_max(limit)
            mlp, _ = tm.run_grouped_structured_expert_pair_forward(payloads["gate"], payloads["up"], hg, hu, None, route, fuse_silu_mul=True)
            down = tm.run_grouped_structured_expert_forward(payloads["down"], hd, None, route)
            torch.cuda.synchronize()
            outs[limit] = (mlp.clone(), down.clone())
    finally:
        lib.tris_set_grouped_row_split_max(previous)
    for limit in (4, 16):
        assert torch.equal(outs[limit][0], outs[1][0]) and torch.equal(outs[limit][1], outs[1][1]), limit
    # oracle: rows of the grouped order against the dequantized expert matrices
    order = route["grouped_token_indices"].cpu().numpy()
    w_down = [orc.dequantize_expert(to_numpy_payload(layer["down"]), e) for e in range(shape.num_experts)]
    hd_f32 = hd.cpu().numpy().astype(np.float32)  # row i of a grouped operand is grouped row i; its expert is that of flat entry order[i]
    ref = np.stack([hd_f32[i] @ w_down[int(ids[order[i]])].astype(np.float32).T for i in range(R)])
    max_abs, mean_rel = orc.error_metrics(outs[4][1].float().cpu().numpy(), ref)
    assert np.abs(ref).mean() > 1e-4 and max_abs <= MAX_ABS and mean_rel <= MEAN_REL, (max_abs, mean_rel)


# ---------------------------------------------------------------------------------------
# (10) expert-parallel exchange: a wait for a peer that never signals ends by itself
# ---------------------------------------------------------------------------------------
def test_peer_wait_times_out_and_reports(tm):
    """tris_ep_wait with counters nobody bumps: the one-CTA wait gives up after about two
    seconds, writes TRIS_ERR_TIMEOUT to the status word and still advances the step; with the
    counters at their target it returns at once and leaves the status alone.  The context stays
    usable (the next launches run)."""
    import time

    lib = tm._native.load()
    inc = lib.tris_ep_signal_increment()
    assert inc > 0
    flags = torch.zeros((64,), dtype=torch.int32, device="cuda")
    step = torch.zeros((1,), dtype=torch.int32, device="cuda")
    status = torch.zeros((1,), dtype=torch.int32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    t0 = time.perf_counter()
    tm._native.check(lib.tris_ep_wait(flags.data_ptr(), step.data_ptr(), 2, status.data_ptr(), stream), "ep_wait")
    torch.cuda.synchronize()
    waited = time.perf_counter() - t0
    assert 1.0 < waited < 10.0, waited
    assert int(status.item()) == 6 and int(step.item()) == 1  # TRIS_ERR_TIMEOUT
    status.zero_()
    flags[:2] = 2 * inc  # both peers have signalled step 2
    t0 = time.perf_counter()
    tm._native.check(lib.tris_ep_wait(flags.data_ptr(), step.data_ptr(), 2, status.data_ptr(), stream), "ep_wait")
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 1.0
    assert int(status.item()) == 0 and int(step.item()) == 2
    assert float((torch.ones(8, device="cuda") * 2).sum().item()) == 16.0


# ---------------------------------------------------------------------------------------
# (11) 4-bit packed backbone
# ---------------------------------------------------------------------------------------
def test_packed4_backbone_bit_exact_and_used_by_the_backbone_gemm(tm):
    """tris_packed4_dequantize against the reference's PackedQuantMatrix4bit.dequantize outputs
    (bit-exact), and ExpertSharedMatrix fed with the packed payload gives the backbone GEMM the
    same matrix as the fp16 path."""
    z = load_golden("backbone4.npz")
    for tag in ("pc", "g64", "perm"):
        rows, cols, _ = (int(v) for v in z[f"{tag}_dims"])
        payload = {"qweight": torch.from_numpy(z[f"{tag}_qweight"].copy()), "qzeros": torch.from_numpy(z[f"{tag}_qzeros"].copy()),
                   "scales": torch.from_numpy(z[f"{tag}_scales"].copy()), "g_idx": torch.from_numpy(z[f"{tag}_g_idx"].copy()),
                   "rows": torch.tensor(rows), "cols": torch.tensor(cols)}
        w = tm.dequantize_packed_4bit(payload, "cuda")
        _assert_half_bits_equal(w.cpu().numpy(), z[f"{tag}_weight_f16"])
        holder = tm.ExpertSharedMatrix().set_shared_sv(payload, device="cuda")
        assert holder.shared_sv_quant is not None and torch.equal(holder.shared_sv, w)
        x = torch.randn((5, cols), device="cuda").half()
        got = holder.compute_shared_hidden(x).float().cpu().numpy()
        ref = x.float().cpu().numpy() @ z[f"{tag}_weight_f16"].astype(np.float32).T
        assert np.abs(got - ref).max() <= 2e-2 * max(1.0, np.abs(ref).max())
    with pytest.raises(RuntimeError, match="inconsistent"):
        bad = dict(payload)
        bad["qzeros"] = payload["qzeros"][:, :-1]
        tm.dequantize_packed_4bit(bad, "cuda")


def test_input_projections_match_the_single_products(tm):
    """tris_input_projections (both backbones and the router logits in one launch) against
    three tris_shared_hidden_forward calls, decode-sized (mma.sync) and prefill-sized (tcgen05 +
    TMA) batches."""
    lib = tm._native.load()
    stream = torch.cuda.current_stream().cuda_stream
    H, r, E = 512, 96, 24
    g = torch.Generator().manual_seed(3)
    sg, su = (torch.randn((r, H), generator=g) * 0.05).half().cuda(), (torch.randn((r, H), generator=g) * 0.05).half().cuda()
    rw = (torch.randn((E, H), generator=g) * 0.05).half().cuda()
    for T in (3, 200):
        x = torch.randn((T, H), generator=g).half().cuda()
        hg, hu = torch.empty((T, r), dtype=torch.float16, device="cuda"), torch.empty((T, r), dtype=torch.float16, device="cuda")
        lg = torch.empty((T, E), dtype=torch.float32, device="cuda")
        tm._native.check(lib.tris_input_projections(x.data_ptr(), T, H, sg.data_ptr(), su.data_ptr(), r, rw.data_ptr(), E,
                                                    hg.data_ptr(), hu.data_ptr(), 2, lg.data_ptr(), stream), "input_projections")
        want = []
        for w, m, mode, dt in ((sg, r, 2, torch.float16), (su, r, 2, torch.float16), (rw, E, 1, torch.float32)):
            o = torch.empty((T, m), dtype=dt, device="cuda")
            tm._native.check(lib.tris_shared_hidden_forward(x.data_ptr(), None, T, None, H, w.data_ptr(), m, o.data_ptr(), mode,
                                                            stream), "shared_hidden")
            want.append(o)
        torch.cuda.synchronize()
        assert torch.equal(hg, want[0]) and torch.equal(hu, want[1]) and torch.equal(lg, want[2]), T
        ref = x.float() @ rw.float().T
        assert float((lg - ref).abs().max()) <= 2e-3 * max(1.0, float(ref.abs().max()))
    # without a router: two products, the logits pointer must be absent too
    tm._native.check(lib.tris_input_projections(x.data_ptr(), T, H, sg.data_ptr(), su.data_ptr(), r, None, 0,
                                                hg.data_ptr(), hu.data_ptr(), 0, None, stream), "input_projections")
    assert lib.tris_input_projections(x.data_ptr(), T, H, sg.data_ptr(), su.data_ptr(), r, rw.data_ptr(), E,
                                      hg.data_ptr(), hu.data_ptr(), 0, None, stream) == 1


def test_kernel_status_word_is_sticky_and_surfaces(tm, small_layer):
    """Status plumbing of the whole-layer entry point, without making a kernel time out: a preset
    TRIS_ERR_TIMEOUT in the workspace's status word survives forward calls (the kernels only set
    it), is returned by tris_moe_layer_last_status, raises through the block, and is cleared by
    the read; a clean run reports 0."""
    from trismoe_b200 import synth

    shape, layer, _ = small_layer
    blk = _block_from_layer(tm, shape, layer)
    x = synth.synth_activations(4, shape.hidden_size, seed=1).cuda()
    logits = synth.synth_router_logits(4, shape.num_experts, seed=2).cuda()
    blk(x.view(1, 4, -1), router_logits=logits)
    assert blk.last_kernel_status() == 0
    blk._workspace.view(torch.int32)[2] = 6  # TRIS_ERR_TIMEOUT, as a CTA whose wait ran out would leave it
    blk(x.view(1, 4, -1), router_logits=logits)  # a later call does not wipe the report
    assert blk.last_kernel_status(clear=False) == 6
    with pytest.raises(RuntimeError, match="TRIS_ERR_TIMEOUT"):
        blk.raise_on_kernel_status()
    assert blk.last_kernel_status() == 0  # the raise cleared it
    blk.raise_on_kernel_status()
    # the built-in scratch of the no-allocation entry has its own word
    word = C.c_int32(-1)
    lib = tm._native.load()
    tm._native.check(lib.tris_moe_layer_last_status(None, 1, torch.cuda.current_stream().cuda_stream, C.byref(word)), "status")
    assert word.value == 0


@pytest.mark.parametrize("slots,E,stride,offset", [(300, 8, 1, 0), (2048, 32, 260, 32), (9000, 8, 260, 56), (8192, 1, 7, 3)])
def test_route_reads_strided_offset_ids_in_place(tm, slots, E, stride, offset):
    """tris_build_grouped_route_ex on ids left behind exchange rows: entry f is ids[f * stride] - offset,
    negative and out-of-range entries are padding; large lists take the multi-CTA sort.  Against the
    oracle's route of the same ids (top_k = 1)."""
    rng = np.random.default_rng(slots + E)
    ids = rng.integers(-1, E, size=slots).astype(np.int32)          # -1: padding
    ids[rng.random(slots) < 0.05] = E + 3                              # out of range: padding as well
    raw = np.full((slots, stride), -7, np.int32)
    raw[:, 0] = np.where(ids >= 0, ids + offset, ids if offset == 0 else -1)
    dev = torch.from_numpy(raw).cuda()
    R = slots
    scratch_n = ((R + 2047) // 2048) * E
    buf = torch.empty((4 * R + 3 * E + 6 + scratch_n,), dtype=torch.int32, device="cuda")
    perm, tok, slot, rof = (buf[i * R:(i + 1) * R] for i in range(4))
    eids, seg = buf[4 * R: 4 * R + E], buf[4 * R + E: 4 * R + 2 * E + 1]
    prob, counts = buf[4 * R + 2 * E + 1: 4 * R + 3 * E + 2], buf[4 * R + 3 * E + 2: 4 * R + 3 * E + 6]
    lib = tm._native.load()
    tm._native.check(lib.tris_build_grouped_route_ex(dev.data_ptr(), stride, offset, R, 1, E, 4, perm.data_ptr(), tok.data_ptr(),
                                                     slot.data_ptr(), rof.data_ptr(), eids.data_ptr(), seg.data_ptr(), prob.data_ptr(),
                                                     counts.data_ptr(), buf[4 * R + 3 * E + 6:].data_ptr(), 4 * scratch_n,
                                                     torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    valid = (ids >= 0) & (ids < E)
    order = np.argsort(np.where(valid, ids, E), kind="stable")[: int(valid.sum())]   # stable by expert, padding dropped
    nseg = int(counts[0].item())
    present = sorted(set(ids[valid].tolist()))
    assert nseg == len(present)
    assert eids[:nseg].cpu().tolist() == present
    lengths = [int((ids[valid] == e).sum()) for e in present]
    assert seg[: nseg + 1].cpu().tolist() == np.concatenate([[0], np.cumsum(lengths)]).tolist()
    n_valid = int(valid.sum())
    assert np.array_equal(perm[:n_valid].cpu().numpy(), order)
    assert np.array_equal(tok[:n_valid].cpu().numpy(), order)
    inv = rof.cpu().numpy()
    assert np.all(inv[~valid] == -1)
    assert np.array_equal(order[inv[valid]], np.nonzero(valid)[0])
