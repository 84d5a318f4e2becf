"""Generates the golden fixtures in this directory by running the TriS-MoE reference's own
Python code on CPU.  Needs a checkout of the reference tree (TRIS_REFERENCE_ROOT points at
it); the fixtures it writes are committed so that the tests never need it.

    TRIS_REFERENCE_ROOT=<path to the TriS-MoE tree> python tests/golden/make_golden.py

Reference code exercised (paths inside the TriS-MoE tree):
  utils/pack_utils.py: build_compact3_packed_payload                      (payload tensors)
  qlinear_cuda.py: QuantLinear.pack_expert, _restore_dense_bool_matrix_from_sparse,
                   _pack_block_gr_gmap_tensor, _dequantize_compact3_matrix,
                   ExpertSharedMatrix.set_shared_sv, build_grouped_route (torch branch),
                   PackedQuantMatrix4bit.set_quantized / dequantize                 (4-bit backbone),
                   build_grouped_ns_compensation_payload, _apply_grouped_ns_compensation,
                   QuantLinear._get_ns_matrices                      (null-space compensation, ns_mode == 2)
  modeling_olmoe.py: OlmoeSparseMoeBlock.forward -> _forward_expert_loop  (fp16 CPU layer output)
  grouped_payload_sidecar.py: save_grouped_payload_sidecar, load_grouped_payload_from_sidecar
                   (a sidecar file written by the reference and what its own loader returns from it)
The `import auto_gptq` package init needs `accelerate`, which is absent, so the needed
sub-packages are registered as empty namespace modules first.
"""
import math
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.environ.get("TRIS_REFERENCE_ROOT", "")


def load_reference():
    if not REF or not os.path.isdir(REF):
        raise SystemExit("set TRIS_REFERENCE_ROOT to a checkout of the TriS-MoE reference tree")
    sys.path.insert(0, REF)
    base = os.path.join(REF, "AutoGPTQ", "auto_gptq")
    for name, sub in [("auto_gptq", ""), ("auto_gptq.nn_modules", "nn_modules"),
                      ("auto_gptq.nn_modules.qlinear", "nn_modules/qlinear"),
                      ("auto_gptq.modeling_tris_moe", "modeling_tris_moe")]:
        mod = types.ModuleType(name)
        mod.__path__ = [os.path.join(base, sub)]
        sys.modules[name] = mod
    import auto_gptq.nn_modules.qlinear.qlinear_cuda as QL
    import auto_gptq.modeling_tris_moe.modeling_olmoe as MO
    import utils.pack_utils as PU
    return QL, MO, PU


def raw_expert(rng, O, r, group, p_sal, p_g, unit_cols):
    G = math.ceil(r / group)
    c_map = rng.random(r) < p_sal
    raw = dict(
        b1=rng.random((O, r)) < 0.5, b2=rng.random((O, r)) < 0.5, c_map=c_map,
        g_map=(rng.random((O, r)) < p_g) & ~c_map[None, :],
        g_idx=(np.arange(r) // group).astype(np.int32),
    )
    sc = lambda shape, mul=1.0: (mul * np.abs(rng.normal(0, 0.02, size=shape))).astype(np.float16)
    raw.update(s_r1=sc((O, G)), s_r2=sc((O, G), 0.5), ns_d_r1=sc((O, G), 2.0), ns_nd_r1=sc((O, G)))
    for n in ("s_c1", "s_c2", "ns_d_c1", "ns_nd_c1"):
        raw[n] = np.ones(r, np.float16) if unit_cols else (1 + 0.25 * rng.standard_normal(r)).astype(np.float16)
    return raw


def ref_payload(PU, raw):
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a))
    return PU.build_compact3_packed_payload(
        device=torch.device("cpu"), mode="expert_compact3", b1=t(raw["b1"]), b2=t(raw["b2"]),
        g_map_non_salient=t(raw["g_map"]), c_map=t(raw["c_map"]), g_idx=t(raw["g_idx"]),
        scales_s_r1=t(raw["s_r1"]), scales_s_r2=t(raw["s_r2"]), scales_ns_d_r1=t(raw["ns_d_r1"]),
        scales_ns_nd_r1=t(raw["ns_nd_r1"]), scales_s_c1=t(raw["s_c1"]), scales_s_c2=t(raw["s_c2"]),
        scales_ns_d_c1=t(raw["ns_d_c1"]), scales_ns_nd_c1=t(raw["ns_nd_c1"]))


class _NoBias:
    bias = None


def ref_module(QL, payload, in_features, out_features, group):
    ql = QL.QuantLinear(1, group, in_features, out_features, False)
    ql.pack_expert(_NoBias(), payload)
    return ql


def ref_expert_outputs(QL, ql, r):
    dense = ql._restore_dense_bool_matrix_from_sparse(ql.expert_q_gmap_sparse, ql.expert_q_gmap_sparse_prefix,
                                                      ql.expert_c_map, r, torch.device("cpu"))
    words, offsets, meta = ql._pack_block_gr_gmap_tensor(dense)
    weight = ql._dequantize_compact3_matrix(ql.expert_qweight1, ql.expert_qweight2_sparse, ql.expert_q_gmap_sparse,
                                            ql.expert_c_map, ql.expert_g_idx, ql.expert_col_pack3, ql.expert_row_pack3,
                                            r, torch.device("cpu"), torch.float16)
    return dense, words, offsets, meta, weight


def save(name, arrays):
    path = os.path.join(HERE, name)
    np.savez_compressed(path, **arrays)
    print(name, os.path.getsize(path), "bytes")


def case_projection(QL, PU, name, seed, E, O, r, group, in_features, p_sal, p_g, unit_cols):
    rng = np.random.default_rng(seed)
    out = {"dims": np.array([E, O, r, group], np.int64)}
    for e in range(E):
        raw = raw_expert(rng, O, r, group, p_sal, p_g, unit_cols)
        payload = ref_payload(PU, raw)
        ql = ref_module(QL, payload, in_features, O, group)
        dense, words, offsets, meta, weight = ref_expert_outputs(QL, ql, r)
        for k, v in raw.items():
            out[f"raw{e}_{k}"] = np.packbits(v, axis=-1) if v.dtype == bool else v
        for k in ("qweight1", "qweight2_sparse", "qweight2_sparse_prefix", "q_gmap_sparse", "q_gmap_sparse_prefix",
                  "c_map_packed", "g_idx", "row_pack3", "col_pack3"):
            out[f"ref{e}_{k}"] = payload[k].numpy()
        out[f"ref{e}_dense_gmap"] = dense.numpy()
        out[f"ref{e}_gr_words"] = words.numpy()
        out[f"ref{e}_gr_offsets"] = offsets.numpy()
        out[f"ref{e}_gr_meta"] = meta.numpy()
        out[f"ref{e}_weight_f16"] = weight.numpy()
    save(name, out)


def case_gr_sweep(QL):
    """Dense maps whose blocks have different densities so that the reference encoder picks
    every k in 0..7, an empty block and a raw block; also the force_raw path."""
    rng = np.random.default_rng(7)
    ql = QL.QuantLinear(1, 128, 64, 64, False)
    out = {}
    densities = [0.0, 0.5, 0.42, 0.27, 0.15, 0.08, 0.04, 0.02, 0.01, 0.004, 0.0015, 0.0005]
    pr, O = 5, 2 * 64 + 17  # odd packed rows, ragged outputs: 3 k-blocks x 3 out-blocks
    bits = np.zeros((pr * 32, O), dtype=bool)
    blk = 0
    for kb in range(3):
        for ob in range(3):
            d = densities[blk % len(densities)]
            rows = slice(kb * 64, min(pr * 32, kb * 64 + 64))
            cols = slice(ob * 64, min(O, ob * 64 + 64))
            shape = (rows.stop - rows.start, cols.stop - cols.start)
            bits[rows, cols] = rng.random(shape) < d
            blk += 1
    bits2 = np.zeros((2 * 32, 3 * 64), dtype=bool)
    for ob, d in enumerate(densities[9:12]):
        bits2[:, ob * 64:(ob + 1) * 64] = rng.random((64, 64)) < d
    bits2[63, 191] = True  # a one in the very last position of a block
    for tag, b in (("a", bits), ("b", bits2)):
        packed = np.packbits(b.reshape(-1, 32, b.shape[1]).transpose(0, 2, 1), axis=-1, bitorder="little").view("<u4")[..., 0]
        dense = torch.from_numpy(packed.view(np.int32).copy())
        words, offsets, meta = ql._pack_block_gr_gmap_tensor(dense)
        out[f"{tag}_dense"] = dense.numpy()
        out[f"{tag}_words"] = words.numpy()
        out[f"{tag}_offsets"] = offsets.numpy()
        out[f"{tag}_meta"] = meta.numpy()
        if tag == "b":
            words, offsets, meta = ql._pack_block_gr_gmap_tensor(dense, force_raw=True)
            out["braw_words"], out["braw_offsets"], out["braw_meta"] = words.numpy(), offsets.numpy(), meta.numpy()
    ks = sorted(set(int(m) & 15 for t in ("a", "b") for m in out[f"{t}_meta"] if not (int(m) & 16)))
    print("k values covered:", ks, "raw blocks:", sum(int(m) == 16 for m in out["a_meta"]))
    save("block_gr_sweep.npz", out)


def case_layer(QL, MO, PU):
    """Small MoE block through the reference's OlmoeSparseMoeBlock on CPU (expert loop)."""
    rng = np.random.default_rng(11)
    E, k, H, I, r, group, T = 6, 2, 128, 96, 64, 32, 9
    cfg = types.SimpleNamespace(num_experts=E, num_experts_per_tok=k, norm_topk_prob=True, hidden_size=H,
                                intermediate_size=I, hidden_act="silu", _name_or_path=None)
    block = MO.OlmoeSparseMoeBlock(cfg).to(torch.float16)
    out = {"dims": np.array([E, k, H, I, r, group, T], np.int64)}
    shared = {}
    for name, (O, K) in (("gate", (I, H)), ("up", (I, H)), ("down", (H, I))):
        sv = torch.from_numpy(rng.normal(0, 0.05, size=(r, K)).astype(np.float16))
        shared[name] = QL.ExpertSharedMatrix()
        shared[name].set_shared_sv(sv)
        out[f"shared_{name}"] = sv.numpy()
    for e in range(E):
        for name, (O, K) in (("gate", (I, H)), ("up", (I, H)), ("down", (H, I))):
            raw = raw_expert(rng, O, r, group, 0.12, 0.1, False)
            # scales around 1/sqrt(r) so that activations keep a healthy fp16 range
            for key in ("s_r1", "s_r2", "ns_d_r1", "ns_nd_r1"):
                raw[key] = (raw[key].astype(np.float32) * 6.0).astype(np.float16)
            payload = ref_payload(PU, raw)
            ql = ref_module(QL, payload, K, O, group)
            ql.bind_shared_matrix(shared[name])
            setattr(block.experts[e], name + "_proj", ql)
            for kk in ("qweight1", "qweight2_sparse", "qweight2_sparse_prefix", "q_gmap_sparse", "q_gmap_sparse_prefix",
                       "c_map_packed", "g_idx", "row_pack3", "col_pack3"):
                out[f"{name}{e}_{kk}"] = payload[kk].numpy()
    router = torch.from_numpy((rng.standard_normal((E, H)) / math.sqrt(H)).astype(np.float16))
    block.gate.weight.data = router
    x = rng.standard_normal((T, H)).astype(np.float32)
    x[:, rng.choice(H, 2, replace=False)] *= 20
    x = torch.from_numpy(x.astype(np.float16))
    os.environ["TRIS_GROUPED_EXPERTS"] = "0"
    with torch.no_grad():
        y, logits = block(x.view(1, T, H))
        sel = torch.topk(torch.softmax(logits, dim=1, dtype=torch.float), k, dim=-1)[1]
        route = QL.build_grouped_route(sel, E)
    out["router_weight"] = router.numpy()
    out["x"] = x.numpy()
    out["ref_y_f16"] = y.view(T, H).numpy()
    out["ref_router_logits_f16"] = logits.numpy()
    out["ref_selected"] = sel.numpy()
    for key in ("grouped_expert_ids", "expert_ids", "segment_offsets", "problem_offsets"):
        out["ref_route_" + key] = route[key].numpy()
    out["ref_route_total_problem_tiles"] = np.array([route["total_problem_tiles_host"]], np.int64)
    # token index of each grouped row is well defined only as a multiset per segment
    out["ref_route_grouped_token_indices"] = route["grouped_token_indices"].numpy()
    save("moe_layer_small.npz", out)
    case_sidecar(block)


def case_sidecar(block):
    """The block above written to a standalone sidecar by the reference's own writer, plus what the
    reference's own loader returns from that file (python scalars and tensors per payload key)."""
    import auto_gptq.modeling_tris_moe.grouped_payload_sidecar as SC

    model = types.SimpleNamespace(layers=[types.SimpleNamespace(mlp=block)])
    path = os.path.join(HERE, "ref_sidecar.safetensors")
    SC.save_grouped_payload_sidecar(model, path)
    loaded = {}
    for key in ("gate", "up", "down", "gate_ns", "up_ns", "down_ns"):
        payload = SC.load_grouped_payload_from_sidecar(path, "model.layers.0.mlp", key, torch.device("cpu"), torch.float16)
        assert payload is not None, key
        for name, value in payload.items():
            if name.startswith("_"):
                continue
            if isinstance(value, torch.Tensor):
                loaded[f"{key}/{name}"] = value.numpy()
            elif isinstance(value, bool):
                loaded[f"{key}/{name}@bool"] = np.array([value])
            elif isinstance(value, int):
                loaded[f"{key}/{name}@int"] = np.array([value], np.int64)
            elif value is None:
                loaded[f"{key}/{name}@none"] = np.zeros(0, np.int8)
            else:
                raise TypeError((key, name, type(value)))
    save("ref_sidecar_loaded.npz", loaded)
    print(f"  ref_sidecar.safetensors: {os.path.getsize(path) / 1024:.1f} KiB")


def case_backbone4(QL):
    """4-bit packed backbones through PackedQuantMatrix4bit.dequantize (fp16, CPU)."""
    rng = np.random.default_rng(44)
    out = {}
    for tag, rows, cols, group in (("pc", 80, 200, 0), ("g64", 64, 256, 64), ("perm", 40, 96, 32)):
        groups = 1 if group == 0 else math.ceil(cols / group)
        qweight = rng.integers(-2**31, 2**31, size=(math.ceil(cols / 8), rows), dtype=np.int64).astype(np.int32)
        qzeros = rng.integers(-2**31, 2**31, size=(groups, math.ceil(rows / 8)), dtype=np.int64).astype(np.int32)
        scales = np.abs(rng.normal(0, 0.01, size=(groups, rows))).astype(np.float16)
        g_idx = np.zeros(cols, np.int32) if group == 0 else (np.arange(cols) // group).astype(np.int32)
        if tag == "perm":
            g_idx = rng.permutation(g_idx)   # act-order style: groups not contiguous in the column order
        m = QL.PackedQuantMatrix4bit(weight_dtype=torch.float16)
        m.set_quantized(torch.from_numpy(qweight), torch.from_numpy(qzeros), torch.from_numpy(scales),
                        torch.from_numpy(g_idx), rows, cols)
        w = m.dequantize(torch.device("cpu"), torch.float16)
        assert tuple(w.shape) == (rows, cols)
        out.update({f"{tag}_qweight": qweight, f"{tag}_qzeros": qzeros, f"{tag}_scales": scales, f"{tag}_g_idx": g_idx,
                    f"{tag}_dims": np.array([rows, cols, groups], np.int64), f"{tag}_weight_f16": w.numpy()})
    save("backbone4.npz", out)


def case_ns_compensation(QL):
    """Null-space compensation: QuantLinear modules with ns_mode == 2 and 4-bit C1/C2 pairs ->
    build_grouped_ns_compensation_payload (the grouped payload tensors) and the reference's
    per-segment fallback _apply_grouped_ns_compensation (F.linear(F.linear(x, c2), c1) in fp16 on
    CPU) on a grouped batch."""
    rng = np.random.default_rng(77)
    infeatures, outfeatures, group = 256, 96, 128
    ranks = [16, 0, 24, 16, 40]

    def packed(rows, cols, group_size):
        groups = max(1, math.ceil(cols / group_size))
        qweight = rng.integers(-2**31, 2**31, size=(math.ceil(cols / 8), rows), dtype=np.int64).astype(np.int32)
        qzeros = rng.integers(-2**31, 2**31, size=(groups, math.ceil(rows / 8)), dtype=np.int64).astype(np.int32)
        scales = np.abs(rng.normal(0, 0.02, size=(groups, rows))).astype(np.float16)
        g_idx = np.minimum(np.arange(cols) // group_size, groups - 1).astype(np.int32)
        return (torch.from_numpy(qweight), torch.from_numpy(qzeros), torch.from_numpy(scales), torch.from_numpy(g_idx), rows, cols)

    modules = []
    for rank in ranks:
        m = QL.QuantLinear(1, group, infeatures, outfeatures, False)
        if rank:
            m.ns_mode.fill_(2)
            m.ns_c2_quant.set_quantized(*packed(rank, infeatures, group))
            m.ns_c1_quant.set_quantized(*packed(outfeatures, rank, group))
        m._refresh_runtime_scalar_cache()
        modules.append(m)
    payload = QL.build_grouped_ns_compensation_payload(modules, torch.device("cpu"), torch.float16)
    assert payload is not None and int(payload["max_ns_rank"]) == max(ranks)
    out = {}
    for k, v in payload.items():
        out["payload_" + k] = v.numpy() if isinstance(v, torch.Tensor) else np.array(int(v), np.int64)
    expert_ids = np.array([0, 1, 2, 4], np.int32)       # expert 3 gets no rows, expert 1 has no pair
    lengths = np.array([3, 2, 9, 5], np.int64)
    seg = np.concatenate([[0], np.cumsum(lengths)]).astype(np.int32)
    x = (rng.standard_normal((int(seg[-1]), infeatures)) * 0.5).astype(np.float16)
    tiles = np.concatenate([[0], np.cumsum((lengths + 3) // 4)]).astype(np.int32)   # 4-row problem tiles per segment
    route = {"expert_ids": torch.from_numpy(expert_ids), "segment_offsets": torch.from_numpy(seg),
             "problem_offsets": torch.from_numpy(tiles), "total_problem_tiles": torch.tensor([int(tiles[-1])])}
    assert QL._coerce_grouped_route(route, torch.device("cpu")) is not None
    comp = torch.zeros((x.shape[0], outfeatures), dtype=torch.float16)
    QL._apply_grouped_ns_compensation(modules, torch.from_numpy(x), route, [comp])
    for e, rank in enumerate(ranks):
        if rank:
            c1, c2 = modules[e]._get_ns_matrices(torch.device("cpu"), torch.float16)
            out[f"c1_{e}"], out[f"c2_{e}"] = c1.numpy(), c2.numpy()
    out.update(expert_ids=expert_ids, segment_offsets=seg, x=x, compensation_f16=comp.numpy(), ranks=np.array(ranks, np.int64))
    save("ns_compensation.npz", out)


def main():
    torch.manual_seed(0)
    QL, MO, PU = load_reference()
    case_projection(QL, PU, "proj_ragged.npz", 1, E=3, O=96, r=80, group=32, in_features=160, p_sal=0.15, p_g=0.1,
                    unit_cols=False)
    case_projection(QL, PU, "proj_r256.npz", 2, E=2, O=128, r=256, group=128, in_features=512, p_sal=0.1, p_g=0.1,
                    unit_cols=True)
    case_gr_sweep(QL)
    case_layer(QL, MO, PU)
    case_backbone4(QL)
    case_ns_compensation(QL)


if __name__ == "__main__":
    main()
