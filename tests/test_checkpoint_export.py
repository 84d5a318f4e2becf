"""CPU tests of the block-GR exporter and the layer-batched loader against the sidecar the
reference wrote (tests/golden/ref_sidecar.safetensors): its payloads carry the sparse g_map planes
AND the block-GR streams the reference's own encoder made from them, so the exporter must
reproduce those streams bit for bit from the sparse planes alone."""
import os

import numpy as np
import pytest
import torch

import trismoe_oracle as orc
from helpers import GOLDEN


def _load_all(path):
    from safetensors import safe_open

    with safe_open(path, framework="pt", device="cpu") as fh:
        return {k: fh.get_tensor(k) for k in fh.keys()}, dict(fh.metadata() or {})


def test_exporter_reproduces_the_reference_streams(lib):
    from trismoe_b200 import checkpoint_export as ce

    tensors, _ = _load_all(os.path.join(GOLDEN, "ref_sidecar.safetensors"))
    want = {k: v.clone() for k, v in tensors.items() if ".q_gmap_gr_" in k}
    assert len(want) == 9
    for k in want:  # forget the streams: the exporter starts from the sparse planes
        tensors[k] = torch.empty((0,), dtype=torch.int32)
    for k in [k for k in tensors if k.endswith(".compact3_use_block_gr")]:
        tensors[k] = torch.tensor([False])
    built, words = ce.build_grouped_blockgr_payloads(tensors, "compressed")
    assert built == 3 and words == sum(int(v.numel()) for k, v in want.items() if k.endswith("q_gmap_gr_words"))
    for k, v in want.items():
        assert tensors[k].dtype == v.dtype and torch.equal(tensors[k], v), k
    assert all(bool(tensors[k][0]) for k in tensors if k.endswith(".gate.compact3_use_block_gr"))


def test_dense_restore_matches_oracle_and_k_bounds(lib):
    from trismoe_b200 import checkpoint_export as ce, synth

    shape = synth.LayerShape(96, 160, 2, 1, rank=80, group_size=16)
    p = synth.synth_layer(shape, seed=9, keep_sparse_gmap=True)["gate"]
    for e in range(2):
        dense = ce.restore_dense_packed_gmap_from_sparse(p["q_gmap_sparse"][e], p["c_map"][e], 80, 160)
        assert torch.equal(dense, p["_dense_gmap_words"][e])
    assert ce.resolve_block_gr_search_bounds() == (0, 7) and ce.resolve_block_gr_search_bounds(fixed_k=3) == (3, 3)
    with pytest.raises(ValueError):
        ce.resolve_block_gr_search_bounds(fixed_k=3, k_min=1, k_max=2)
    with pytest.raises(ValueError):
        ce.resolve_block_gr_search_bounds(k_min=5, k_max=2)


def test_export_file_round_trip_modes_and_layer_batches(lib, tmp_path):
    """compressed / fixed-k / raw exports of a two-layer sidecar: metadata as the reference exporter
    writes it, the sparse planes dropped unless asked for, streams that decode (oracle decoder)
    back to the dense maps, and the layer-batched loader returning every layer once."""
    from safetensors import safe_open

    from trismoe_b200 import checkpoint_export as ce, sidecar, synth

    shape = synth.LayerShape(64, 96, 3, 2, rank=64, group_size=32)
    layers, dense = {}, {}
    for L in range(3):
        layer = synth.synth_layer(shape, seed=20 + L, keep_sparse_gmap=True, use_block_gr=False)
        prefix = sidecar.layer_prefix(L)
        layers[prefix] = {k: layer[k] for k in ("gate", "up", "down")}
        dense[prefix] = {k: layer[k]["_dense_gmap_words"] for k in ("gate", "up", "down")}
    src = os.path.join(tmp_path, "src", sidecar.GROUPED_PAYLOAD_SIDECAR_BASENAME)
    os.makedirs(os.path.dirname(src))
    sidecar.save_grouped_payloads_to_sidecar(src, layers)
    for tag, kw in (("c", {}), ("k2", {"fixed_k": 2}), ("raw", {"mode": "raw", "keep_sparse": True})):
        out = os.path.join(tmp_path, tag, sidecar.GROUPED_PAYLOAD_SIDECAR_BASENAME)
        stats = ce.export_grouped_blockgr_checkpoint(src, out, **kw)
        assert stats["built_grouped_payloads"] == 9
        with safe_open(out, framework="pt") as fh:
            meta = fh.metadata()
            assert meta["olmoe_grouped_block_gr_export"] == "v1" and meta["olmoe_grouped_block_gr_mode"] == kw.get("mode", "compressed")
            assert meta["olmoe_grouped_block_gr_keep_sparse"] == ("1" if kw.get("keep_sparse") else "0")
            assert (meta.get("olmoe_grouped_block_gr_k") == "2") == (tag == "k2")
        seen = []
        for batch in ce.iter_layer_payload_batches(out, layers_per_batch=2):
            assert 1 <= len(batch) <= 2
            for prefix, by_key in batch.items():
                seen.append(prefix)
                for key, payload in by_key.items():
                    assert payload["compact3_use_block_gr"] is True
                    assert (payload["q_gmap_sparse"].numel() > 0) == bool(kw.get("keep_sparse"))
                    meta_words = payload["q_gmap_gr_meta"].numpy()
                    if tag == "k2":
                        assert set(int(m) & 15 for m in meta_words.reshape(-1) if not int(m) & 16) <= {2}
                    if tag == "raw":
                        assert all(int(m) & 16 for m in meta_words.reshape(-1))
                    for e in range(3):
                        got = orc.gr_decode_tensor(payload["q_gmap_gr_words"][e].numpy(), payload["q_gmap_gr_offsets"][e].numpy(),
                                                   payload["q_gmap_gr_meta"][e].numpy(), 2, int(payload["qweight1"].shape[2]))
                        assert np.array_equal(got.view(np.int32), dense[prefix][key][e].numpy()), (tag, prefix, key, e)
        assert seen == [sidecar.layer_prefix(L) for L in range(3)]


def test_packed4_group_rules_on_cpu():
    """Which 4-bit matrices the in-place GEMM takes (uniform groups of a multiple of 32 columns, or one group)
    and the group size the reference infers from g_idx (_infer_packed_group_size_from_g_idx, qlinear_cuda.py:460-483)."""
    import numpy as np
    import torch

    import trismoe_b200 as tm
    from trismoe_b200 import synth
    from trismoe_b200.ns_compensation import infer_packed_group_size

    rng = np.random.default_rng(0)
    uniform = synth.packed4_matrix(rng, 64, 256, 128)
    assert infer_packed_group_size(uniform) == 128 and tm.Packed4Linear.supports(uniform)
    one_group = synth.packed4_matrix(rng, 40, 200, 200)
    assert infer_packed_group_size(one_group) == 200 and tm.Packed4Linear.supports(one_group)
    narrow = synth.packed4_matrix(rng, 40, 96, 16)          # uniform, but 16-column groups
    assert infer_packed_group_size(narrow) == 16 and not tm.Packed4Linear.supports(narrow)
    permuted = dict(uniform)
    permuted["g_idx"] = torch.from_numpy(rng.permutation(uniform["g_idx"].numpy()))
    assert infer_packed_group_size(permuted) == 256 and not tm.Packed4Linear.supports(permuted)
    with __import__("pytest").raises(RuntimeError):
        tm.Packed4Linear(uniform, "cpu")                    # no CPU path


def test_streaming_sparse_single_file_export(lib, tmp_path):
    """The single-file streaming export: expert module tensors other than the kept state leaves are dropped (OLMoE and
    Mixtral naming), payload and non-expert tensors stay, an all-zero compact3 output scale is repaired, the metadata
    carries the embedded / deployment-only / staging-ready keys, payloads load back unchanged, and a source without
    sparse g_map planes is refused."""
    from safetensors import safe_open
    from safetensors.torch import save_file

    from trismoe_b200 import checkpoint_export as ce, sidecar, synth

    assert ce.split_moe_expert_tensor_name("model.layers.3.mlp.experts.12.up_proj.qweight1") == ("up_proj", "qweight1")
    assert ce.split_moe_expert_tensor_name("model.layers.0.block_sparse_moe.experts.1.w2.ns_vector_row") == ("down_proj", "ns_vector_row")
    assert ce.split_moe_expert_tensor_name("model.layers.0.mlp.experts.1.router.weight") is None
    assert ce.split_moe_expert_tensor_name("model.layers.0.mlp.gate.weight") is None
    assert ce.split_moe_expert_tensor_name("model.layers.0.mlp.experts.1.gate_proj") is None

    shape = synth.LayerShape(64, 96, 2, 1, rank=64, group_size=32)
    layer = synth.synth_layer(shape, seed=31, keep_sparse_gmap=True, use_block_gr=False)
    prefix = sidecar.layer_prefix(0)
    src = os.path.join(tmp_path, "src.safetensors")
    sidecar.save_grouped_payloads_to_sidecar(src, {prefix: {k: layer[k] for k in ("gate", "up", "down")}}, embedded=True)
    tensors, meta = _load_all(src)
    scale_name = sidecar.payload_tensor_name(prefix, "down", "output_scale")
    tensors[scale_name] = torch.zeros_like(tensors[scale_name])
    tensors[sidecar.payload_tensor_name(prefix, "down", "has_output_scale")] = torch.tensor([True])
    extra = {"model.embed_tokens.weight": torch.ones(4, 4, dtype=torch.float16),
             "model.layers.0.mlp.gate.weight": torch.ones(2, 4, dtype=torch.float16),
             "model.layers.0.self_attn.q_proj.qweight1": torch.ones(3, dtype=torch.int32),
             "model.layers.0.mlp.experts.0.gate_proj.qweight1": torch.ones(5, dtype=torch.int32),
             "model.layers.0.mlp.experts.0.gate_proj.ns_mode": torch.tensor([2], dtype=torch.int32),
             "model.layers.0.mlp.experts.1.down_proj.expert_input_scale": torch.ones(4, dtype=torch.float16),
             "model.layers.0.block_sparse_moe.experts.1.w3.scale_u": torch.ones(4, dtype=torch.float16),
             "model.layers.0.block_sparse_moe.experts.1.w3.mode": torch.tensor([1], dtype=torch.int32)}
    tensors.update(extra)
    save_file({k: v.contiguous() for k, v in tensors.items()}, src, metadata={**meta, "note": "kept"})

    out = os.path.join(tmp_path, "out", "model.safetensors")
    stats = ce.export_grouped_streaming_sparse_checkpoint(src, out)
    assert stats["repaired_grouped_output_scales"] == 1 and stats["dropped_tensors"] == 2 and stats["single_file"]
    got, got_meta = _load_all(out)
    assert "model.layers.0.mlp.experts.0.gate_proj.qweight1" not in got
    assert "model.layers.0.block_sparse_moe.experts.1.w3.scale_u" not in got
    for name in extra:
        if not name.endswith(("gate_proj.qweight1", "w3.scale_u")):
            assert torch.equal(got[name], extra[name]), name
    assert got_meta["format"] == "pt" and got_meta["note"] == "kept"
    assert got_meta[sidecar.GROUPED_PAYLOAD_EMBEDDED_METADATA_KEY] == "v1"
    assert got_meta[sidecar.GROUPED_PAYLOAD_DEPLOYMENT_ONLY_METADATA_KEY] == "v1"
    assert got_meta["olmoe_grouped_qgmap_cpu_staging_ready"] == "v1"
    assert got_meta["olmoe_grouped_qgmap_cpu_staging_single_file"] == "1"
    assert bool(torch.all(got[scale_name] == 1)) and not bool(got[sidecar.payload_tensor_name(prefix, "down", "has_output_scale")][0])
    for key in ("gate", "up", "down"):
        payload = sidecar.load_grouped_payload_from_sidecar(out, prefix, key)
        assert torch.equal(payload["q_gmap_sparse"], layer[key]["q_gmap_sparse"].cpu())
        assert torch.equal(payload["qweight1"], layer[key]["qweight1"].cpu())
        staged = sidecar.load_grouped_qgmap_from_sidecar(out, prefix, key, pin_memory=False)
        assert staged is not None and torch.equal(staged["q_gmap_sparse_prefix"], layer[key]["q_gmap_sparse_prefix"].cpu())

    dense_only = {k: v for k, v in got.items() if not k.endswith(("q_gmap_sparse", "q_gmap_sparse_prefix"))}
    bad = os.path.join(tmp_path, "dense.safetensors")
    save_file(dense_only, bad, metadata=got_meta)
    with pytest.raises(ValueError, match="sparse qgmap"):
        ce.export_grouped_streaming_sparse_checkpoint(bad, os.path.join(tmp_path, "out2", "model.safetensors"))
