"""CPU tests: the oracle and the host-side format code against fixtures produced by the
TriS-MoE reference's own Python code (tests/golden/make_golden.py)."""
import math

import numpy as np
import pytest
import torch

import trismoe_oracle as orc
from helpers import PAYLOAD_KEYS, golden_expert_payload, golden_raw_expert, load_golden, to_numpy_payload


@pytest.mark.parametrize("name", ["proj_ragged.npz", "proj_r256.npz"])
def test_packers_match_reference_payload(lib, name):
    import trismoe_b200 as tm

    z = load_golden(name)
    E, O, r, group = (int(v) for v in z["dims"])
    for e in range(E):
        raw = golden_raw_expert(z, e, O, r)
        mine = tm.build_compact3_packed_payload(
            b1=raw["b1"], b2=raw["b2"], g_map_non_salient=raw["g_map"], c_map=raw["c_map"], g_idx=raw["g_idx"],
            scales_s_r1=raw["s_r1"], scales_s_r2=raw["s_r2"], scales_ns_d_r1=raw["ns_d_r1"],
            scales_ns_nd_r1=raw["ns_nd_r1"], scales_s_c1=raw["s_c1"], scales_s_c2=raw["s_c2"],
            scales_ns_d_c1=raw["ns_d_c1"], scales_ns_nd_c1=raw["ns_nd_c1"])
        for k in PAYLOAD_KEYS:
            ref = z[f"ref{e}_{k}"]
            got = mine[k].numpy()
            assert got.dtype == ref.dtype, k
            assert got.shape == ref.shape, (k, got.shape, ref.shape)
            assert np.array_equal(got, ref), k
        dense = tm.dense_gmap_words(raw["g_map"], raw["c_map"]).numpy()
        assert np.array_equal(dense, z[f"ref{e}_dense_gmap"])


@pytest.mark.parametrize("name", ["proj_ragged.npz", "proj_r256.npz"])
def test_block_gr_encoder_and_oracle_decoder_match_reference(lib, name):
    import trismoe_b200 as tm

    z = load_golden(name)
    E, O, r, _ = (int(v) for v in z["dims"])
    pr = math.ceil(r / 32)
    for e in range(E):
        dense = z[f"ref{e}_dense_gmap"]
        words, offsets, meta = tm.block_gr_encode(torch.from_numpy(dense.copy()))
        assert np.array_equal(words.numpy(), z[f"ref{e}_gr_words"])
        assert np.array_equal(offsets.numpy(), z[f"ref{e}_gr_offsets"])
        assert np.array_equal(meta.numpy(), z[f"ref{e}_gr_meta"])
        decoded = orc.gr_decode_tensor(z[f"ref{e}_gr_words"], z[f"ref{e}_gr_offsets"], z[f"ref{e}_gr_meta"], pr, O)
        assert np.array_equal(decoded.view(np.int32), dense)


def test_block_gr_sweep_all_k_raw_and_empty(lib):
    import trismoe_b200 as tm

    z = load_golden("block_gr_sweep.npz")
    seen_k, raw_blocks, empty_blocks = set(), 0, 0
    for tag in ("a", "b", "braw"):
        dense = z["b_dense" if tag == "braw" else f"{tag}_dense"]
        words, offsets, meta = tm.block_gr_encode(torch.from_numpy(dense.copy()), force_raw=(tag == "braw"))
        assert np.array_equal(words.numpy(), z[f"{tag}_words"])
        assert np.array_equal(offsets.numpy(), z[f"{tag}_offsets"])
        assert np.array_equal(meta.numpy(), z[f"{tag}_meta"])
        decoded = orc.gr_decode_tensor(z[f"{tag}_words"], z[f"{tag}_offsets"], z[f"{tag}_meta"], *dense.shape)
        assert np.array_equal(decoded.view(np.int32), dense)
        for m in z[f"{tag}_meta"]:
            if int(m) & 16:
                raw_blocks += 1
            else:
                seen_k.add(int(m) & 15)
                empty_blocks += int(m) >> 8 == 0
    assert {0, 1, 2, 4, 5, 6, 7} <= seen_k
    assert raw_blocks >= 2 and empty_blocks >= 1


@pytest.mark.parametrize("name", ["proj_ragged.npz", "proj_r256.npz"])
def test_oracle_dequant_bit_exact_vs_reference(name):
    z = load_golden(name)
    E, O, r, _ = (int(v) for v in z["dims"])
    for e in range(E):
        sal = orc.unpack_vector(z[f"ref{e}_c_map_packed"], r)
        gbits = orc.restore_sparse(z[f"ref{e}_q_gmap_sparse"], ~sal, O)
        # the GR route to the same bits
        dense = orc.gr_decode_tensor(z[f"ref{e}_gr_words"], z[f"ref{e}_gr_offsets"], z[f"ref{e}_gr_meta"],
                                     math.ceil(r / 32), O)
        assert np.array_equal(orc.unpack_rows(dense, r), gbits)
        w = orc.dequantize_compact3(z[f"ref{e}_qweight1"], z[f"ref{e}_qweight2_sparse"], gbits,
                                    z[f"ref{e}_c_map_packed"], z[f"ref{e}_g_idx"], z[f"ref{e}_col_pack3"],
                                    z[f"ref{e}_row_pack3"], r)
        ref = z[f"ref{e}_weight_f16"]
        assert np.array_equal(orc.canonical_half_bits(w), orc.canonical_half_bits(ref))


def _layer_from_golden(z):
    import trismoe_b200 as tm

    E, k, H, I, r, group, T = (int(v) for v in z["dims"])
    payloads, weights, shared = {}, {}, {}
    for name in ("gate", "up", "down"):
        experts = [golden_expert_payload(z, f"{name}{e}") for e in range(E)]
        payloads[name] = tm.stack_expert_payloads(experts, use_block_gr=True)
        np_payload = to_numpy_payload(payloads[name])
        weights[name] = [orc.dequantize_expert(np_payload, e) for e in range(E)]
        shared[name] = z[f"shared_{name}"]
    return (E, k, H, I, r, group, T), payloads, weights, shared


def test_oracle_layer_matches_reference_block(lib):
    """fp32 oracle vs the reference's fp16 CPU block output: same routing, outputs within
    fp16 round-off of each other."""
    z = load_golden("moe_layer_small.npz")
    (E, k, H, I, r, group, T), payloads, weights, shared = _layer_from_golden(z)
    x = z["x"]
    logits = z["ref_router_logits_f16"].astype(np.float32)
    sel, _ = orc.router_topk(logits, k, True)
    assert np.array_equal(np.sort(sel, axis=1), np.sort(z["ref_selected"], axis=1))
    y = orc.moe_layer_fp32(x, logits, weights, shared, k, True)
    max_abs, mean_rel = orc.error_metrics(z["ref_y_f16"], y)
    assert np.abs(y).mean() > 1e-3  # the comparison is not vacuous
    assert max_abs <= 2e-2 and mean_rel <= 5e-3, (max_abs, mean_rel)
    route = orc.build_route(sel, E)
    for key in ("grouped_expert_ids", "expert_ids", "segment_offsets", "problem_offsets"):
        assert np.array_equal(route[key], z["ref_route_" + key]), key
    assert route["total_problem_tiles_host"] == int(z["ref_route_total_problem_tiles"][0])
    # rows of a segment: same token multiset as the reference's (its sort is not stable)
    seg = route["segment_offsets"]
    for s in range(len(seg) - 1):
        mine = np.sort(route["grouped_token_indices"][seg[s]: seg[s + 1]])
        ref = np.sort(z["ref_route_grouped_token_indices"][seg[s]: seg[s + 1]])
        assert np.array_equal(mine, ref)


def test_synth_payload_round_trip(lib):
    """Synthetic generator: GR streams decode back to the dense map, stacked tensors have
    the documented shapes, oracle weights are finite and non-trivial."""
    from trismoe_b200 import synth

    shape = synth.LayerShape(96, 160, 5, 2, rank=80, group_size=16)
    layer = synth.synth_layer(shape, seed=3, keep_sparse_gmap=True)
    for name, O in (("gate", 160), ("up", 160), ("down", 96)):
        p = layer[name]
        pr = 3
        assert tuple(p["qweight1"].shape) == (5, pr, O)
        assert tuple(p["q_gmap_gr_offsets"].shape) == (5, 2 * math.ceil(O / 64) + 1)
        npp = to_numpy_payload(p)
        for e in range(5):
            dense = orc.gr_decode_tensor(npp["q_gmap_gr_words"][e], npp["q_gmap_gr_offsets"][e], npp["q_gmap_gr_meta"][e], pr, O)
            assert np.array_equal(dense.view(np.int32), npp["_dense_gmap_words"][e])
            sal = orc.unpack_vector(npp["c_map"][e], 80)
            assert np.array_equal(orc.unpack_rows(dense, 80), orc.restore_sparse(npp["q_gmap_sparse"][e], ~sal, O))
        w = orc.dequantize_expert(npp, 0)
        assert np.isfinite(w.astype(np.float32)).all() and np.abs(w.astype(np.float32)).mean() > 1e-3


def test_packed4_backbone_matches_reference_dequantize():
    """4-bit packed backbone: the oracle against PackedQuantMatrix4bit.dequantize outputs
    (per-channel single group, 64-column groups, permuted group index)."""
    z = load_golden("backbone4.npz")
    for tag in ("pc", "g64", "perm"):
        rows, cols, _ = (int(v) for v in z[f"{tag}_dims"])
        w = orc.dequantize_packed4(z[f"{tag}_qweight"], z[f"{tag}_qzeros"], z[f"{tag}_scales"], z[f"{tag}_g_idx"], rows, cols)
        assert w.shape == (rows, cols)
        assert np.array_equal(w.view(np.uint16), z[f"{tag}_weight_f16"].view(np.uint16)), tag


# ---------------------------------------------------------------------------------------
# the timed CPU reference arm (oracle/cpu_reference_path.py) pinned to the same fixtures
# ---------------------------------------------------------------------------------------
@pytest.mark.parametrize("name", ["proj_ragged.npz", "proj_r256.npz"])
def test_cpu_reference_port_dequant_bit_exact_vs_reference(lib, name):
    """The torch-CPU port that bench.py times reproduces the reference's
    _dequantize_compact3_matrix weights bit for bit (modulo the sign of zero)."""
    import cpu_reference_path as cpu
    import trismoe_b200 as tm

    z = load_golden(name)
    E, O, r, _ = (int(v) for v in z["dims"])
    stacked = tm.stack_expert_payloads([golden_expert_payload(z, f"ref{e}") for e in range(E)], use_block_gr=False)
    for e in range(E):
        w = cpu.dequantize_expert(stacked, e).numpy()
        assert w.shape == (O, r)
        assert np.array_equal(orc.canonical_half_bits(w), orc.canonical_half_bits(z[f"ref{e}_weight_f16"])), e


def test_cpu_reference_port_block_matches_reference_block(lib):
    """...and its MoE block reproduces the output of the reference's own OlmoeSparseMoeBlock
    on CPU (moe_layer_small.npz: ref_y_f16), same routing, fp16 round-off apart."""
    import cpu_reference_path as cpu
    import trismoe_b200 as tm

    z = load_golden("moe_layer_small.npz")
    E, k, H, I, r, group, T = (int(v) for v in z["dims"])
    layer = {}
    for name in ("gate", "up", "down"):
        layer[name] = tm.stack_expert_payloads([golden_expert_payload(z, f"{name}{e}") for e in range(E)], use_block_gr=False)
        layer["shared_" + name] = torch.from_numpy(z["shared_" + name].copy())
    layer["router_weight"] = torch.from_numpy(z["router_weight"].copy())
    x = torch.from_numpy(z["x"].copy())
    y = cpu.moe_block_forward(x, layer, k, True).numpy()
    ref = z["ref_y_f16"]
    assert y.shape == ref.shape and np.abs(ref.astype(np.float32)).mean() > 1e-3
    # same tensor-op sequence as the reference: equal up to the accumulation order of index_add_ / F.linear
    max_abs, mean_rel = orc.error_metrics(y, ref)
    assert max_abs <= 4e-3 and mean_rel <= 1e-3, (max_abs, mean_rel)
    # the fp32 oracle sees both at the same distance
    logits = z["ref_router_logits_f16"].astype(np.float32)
    _, _, weights, shared = _layer_from_golden(z)
    y32 = orc.moe_layer_fp32(z["x"], logits, weights, shared, k, True)
    max_abs, mean_rel = orc.error_metrics(y, y32)
    assert max_abs <= 2e-2 and mean_rel <= 5e-3, (max_abs, mean_rel)


# ---------------------------------------------------------------------------------------
# null-space compensation (ns_mode == 2)
# ---------------------------------------------------------------------------------------
def _ns_payload(z):
    return {k[len("payload_"):]: z[k] for k in z.files if k.startswith("payload_")}


def test_ns_matrices_match_reference_dequantize():
    """Per-expert C1 / C2 sliced out of the reference's grouped compensation payload and dequantised
    by the oracle equal QuantLinear._get_ns_matrices (PackedQuantMatrix4bit.dequantize) bit for bit."""
    z = load_golden("ns_compensation.npz")
    payload = _ns_payload(z)
    for e, rank in enumerate(z["ranks"]):
        c1, c2 = orc.ns_expert_matrices(payload, e)
        if rank == 0:
            assert c1 is None and c2 is None
            continue
        assert np.array_equal(c1.view(np.uint16), z[f"c1_{e}"].view(np.uint16)), e
        assert np.array_equal(c2.view(np.uint16), z[f"c2_{e}"].view(np.uint16)), e


def test_ns_compensation_oracle_matches_reference_fallback():
    """The fp32 oracle against the reference's per-segment fallback (fp16 F.linear twice on CPU):
    within the layer tolerance; rows of the expert without a pair stay zero."""
    z = load_golden("ns_compensation.npz")
    got = orc.ns_compensation_fp32(_ns_payload(z), z["x"], z["expert_ids"], z["segment_offsets"])
    want = z["compensation_f16"].astype(np.float32)
    assert np.abs(want).mean() > 1e-3
    max_abs, mean_rel = orc.error_metrics(got, want)
    assert max_abs <= 2e-2 and mean_rel <= 1e-3, (max_abs, mean_rel)
    seg = z["segment_offsets"]
    assert not got[seg[1]:seg[2]].any() and not want[seg[1]:seg[2]].any()


def test_ns_payload_builder_matches_reference_layout():
    """build_grouped_ns_compensation_payload of the package reproduces the reference's payload
    tensors (offset tables, concatenated C2 / C1) from the per-expert matrices."""
    import torch

    import trismoe_b200 as tm

    z = load_golden("ns_compensation.npz")
    ref = _ns_payload(z)
    infeatures, outfeatures, group = int(ref["infeatures"]), int(ref["outfeatures"]), int(ref["group_size"])
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a))
    experts = []
    for e, rank in enumerate(int(r) for r in z["ranks"]):
        if rank == 0:
            experts.append(None)
            continue
        off, woff = int(ref["ns_c2_rank_offsets"][e]), int(ref["ns_c2_rank_word_offsets"][e])
        kw, go = int(ref["ns_c1_rank_word_offsets"][e]), int(ref["ns_c1_group_offsets"][e])
        zw, kwords = (rank + 7) // 8, (rank + 7) // 8
        c2 = {"qweight": t(ref["ns_c2_qweight"][:, off:off + rank]), "qzeros": t(ref["ns_c2_qzeros"][:, woff:woff + zw]),
              "scales": t(ref["ns_c2_scales"][:, off:off + rank]), "g_idx": t((np.arange(infeatures) // group).astype(np.int32)),
              "rows": rank, "cols": infeatures}
        c1 = {"qweight": t(ref["ns_c1_qweight"][kw:kw + kwords]), "qzeros": t(ref["ns_c1_qzeros"][go:go + 1]),
              "scales": t(ref["ns_c1_scales"][go:go + 1]), "g_idx": t(np.zeros(rank, np.int32)), "rows": outfeatures, "cols": rank}
        experts.append({"c1": c1, "c2": c2})
    got = tm.build_grouped_ns_compensation_payload(experts, "cpu", torch.float16)
    assert got is not None
    for key, want in ref.items():
        have = got[key]
        have = have.numpy() if isinstance(have, torch.Tensor) else np.array(int(have))
        assert np.array_equal(have, want), key
