"""CPU tests of the grouped payload sidecar (safetensors key scheme and scalar encoding)."""
import os

import torch


def test_sidecar_round_trip_and_repair(lib, tmp_path):
    from safetensors import safe_open

    from trismoe_b200 import sidecar, synth

    shape = synth.LayerShape(64, 96, 4, 2, rank=32, group_size=32)
    layers = {}
    originals = {}
    for L, family in ((0, "olmoe"), (3, "mixtral")):
        layer = synth.synth_layer(shape, seed=L, keep_sparse_gmap=True)
        prefix = sidecar.layer_prefix(L, family)
        layers[prefix] = {k: layer[k] for k in ("gate", "up", "down")}
        originals[prefix] = layer
    layers["model.layers.0.mlp"]["down"] = dict(layers["model.layers.0.mlp"]["down"])
    layers["model.layers.0.mlp"]["down"]["output_scale"] = torch.zeros((4, 64), dtype=torch.float16)
    layers["model.layers.0.mlp"]["down"]["has_output_scale"] = True
    path = os.path.join(tmp_path, sidecar.GROUPED_PAYLOAD_SIDECAR_BASENAME)
    n = sidecar.save_grouped_payloads_to_sidecar(path, layers, {"olmoe_grouped_block_gr_export": "v1"})
    assert n > 0 and sidecar.sidecar_has_grouped_payloads(path)
    with safe_open(path, framework="pt") as fh:
        keys = set(fh.keys())
        assert "model.layers.0.mlp.grouped_payload.gate.qweight1" in keys
        assert "model.layers.3.block_sparse_moe.grouped_payload.down.q_gmap_gr_words" in keys
        assert fh.metadata()["olmoe_grouped_runtime_payload"] == "v1"
        assert fh.get_tensor("model.layers.0.mlp.grouped_payload.gate.compact3_use_block_gr").dtype == torch.bool
        assert fh.get_tensor("model.layers.0.mlp.grouped_payload.gate.bias").numel() == 0
        assert not any("._" in k or k.split(".")[-1].startswith("_") for k in keys)
    assert sidecar.split_payload_tensor_name("model.layers.3.block_sparse_moe.grouped_payload.up.c_map") == \
        ("model.layers.3.block_sparse_moe", "up", "c_map")
    got = sidecar.load_grouped_payload_from_sidecar(path, "model.layers.3.block_sparse_moe", "up")
    ref = originals["model.layers.3.block_sparse_moe"]["up"]
    for key in ("qweight1", "qweight2_sparse", "q_gmap_sparse", "q_gmap_gr_words", "q_gmap_gr_offsets", "c_map",
                "col_pack3", "row_pack3", "g_idx"):
        assert torch.equal(got[key], ref[key]), key
    assert got["compact3_use_block_gr"] is True and got["has_bias"] is False and got["bias"] is None
    repaired = sidecar.load_grouped_payload_from_sidecar(path, "model.layers.0.mlp", "down")
    assert bool(torch.all(repaired["output_scale"] == 1)) and repaired["has_output_scale"] is False
    assert sidecar.load_grouped_payload_from_sidecar(path, "model.layers.9.mlp", "gate") is None
    lean = sidecar.load_grouped_payload_from_sidecar(path, "model.layers.0.mlp", "gate", skip_qgmap=True)
    assert "q_gmap_sparse" not in lean and "qweight1" in lean
    bitmap = sidecar.load_grouped_qgmap_from_sidecar(path, "model.layers.0.mlp", "gate", pin_memory=False)
    assert torch.equal(bitmap["q_gmap_sparse"], originals["model.layers.0.mlp"]["gate"]["q_gmap_sparse"])
