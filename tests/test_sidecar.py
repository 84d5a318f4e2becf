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
        assert fh.metadata()["format"] == "olmoe_grouped_runtime_payload_v1"  # standalone sidecar, as the reference writes it
        assert "olmoe_grouped_runtime_payload" not in fh.metadata()
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
    assert got["compact3_use_block_gr"] is True and got["has_bias"] is False and got["bias"].numel() == 0
    repaired = sidecar.load_grouped_payload_from_sidecar(path, "model.layers.0.mlp", "down")
    assert bool(torch.all(repaired["output_scale"] == 1)) and repaired["has_output_scale"] is False
    assert sidecar.load_grouped_payload_from_sidecar(path, "model.layers.9.mlp", "gate") is None
    lean = sidecar.load_grouped_payload_from_sidecar(path, "model.layers.0.mlp", "gate", skip_qgmap=True)
    assert "q_gmap_sparse" not in lean and "qweight1" in lean
    bitmap = sidecar.load_grouped_qgmap_from_sidecar(path, "model.layers.0.mlp", "gate", pin_memory=False)
    assert torch.equal(bitmap["q_gmap_sparse"], originals["model.layers.0.mlp"]["gate"]["q_gmap_sparse"])


def test_reads_a_sidecar_written_by_the_reference(lib):
    """tests/golden/ref_sidecar.safetensors was written by the reference's own
    save_grouped_payload_sidecar (grouped_payload_sidecar.py:532-550); ref_sidecar_loaded.npz holds
    what the reference's load_grouped_payload_from_sidecar (:628-688) returns from it.  This loader
    must recognise the file and return the same tensors and scalars, key for key."""
    import numpy as np

    from helpers import GOLDEN, load_golden
    from trismoe_b200 import sidecar

    path = os.path.join(GOLDEN, "ref_sidecar.safetensors")
    want = load_golden("ref_sidecar_loaded.npz")
    assert sidecar.sidecar_has_grouped_payloads(path)
    seen = 0
    for key in ("gate", "up", "down", "gate_ns", "up_ns", "down_ns"):
        got = sidecar.load_grouped_payload_from_sidecar(path, "model.layers.0.mlp", key)
        assert got is not None, key
        names = {k.split("/", 1)[1].split("@")[0]: k for k in want.keys() if k.startswith(key + "/")}
        assert set(names) == {n for n in got if not n.startswith("_")}, (key, sorted(set(names) ^ set(got)))
        for name, full in names.items():
            ref, mine = want[full], got[name]
            if full.endswith("@bool"):
                assert isinstance(mine, bool) and mine == bool(ref[0]), (key, name)
            elif full.endswith("@int"):
                assert isinstance(mine, int) and not isinstance(mine, bool) and mine == int(ref[0]), (key, name)
            else:
                assert isinstance(mine, torch.Tensor), (key, name)
                arr = mine.numpy()
                assert arr.dtype == ref.dtype and arr.shape == ref.shape, (key, name, arr.dtype, arr.shape, ref.dtype, ref.shape)
                assert np.array_equal(arr.view(np.uint8) if arr.size else arr, ref.view(np.uint8) if ref.size else ref), (key, name)
            seen += 1
    assert seen > 60
    # the file round-trips through this writer with the reference's standalone metadata
    bitmap = sidecar.load_grouped_qgmap_from_sidecar(path, "model.layers.0.mlp", "down", pin_memory=False)
    assert bitmap is not None and bitmap["q_gmap_sparse"].dtype == torch.int32


def test_payload_flags_follow_the_reference_when_keys_are_missing(lib):
    """A payload without has_output_scale derives it from the tensor (anything but exact ones is a
    scale), tensor-valued flags count, and a missing has_bias follows the bias tensor - the
    reference's _payload_has_output_scale / _payload_flag (qlinear_cuda.py:310-321)."""
    from trismoe_b200 import qlinear_grouped as q

    ones = torch.ones((2, 8), dtype=torch.float16)
    assert q._payload_has_output_scale({"output_scale": ones}) is False
    assert q._payload_has_output_scale({"output_scale": ones * 0.5}) is True
    assert q._payload_has_output_scale({"output_scale": ones * 0.5, "has_output_scale": False}) is False
    assert q._payload_has_output_scale({"output_scale": ones, "has_output_scale": torch.tensor([True])}) is True
    assert q._payload_has_output_scale({"output_scale": ones, "has_output_scale": torch.tensor(False)}) is False
    assert q._payload_has_bias({"bias": None}) is False
    assert q._payload_has_bias({"bias": torch.empty((0,), dtype=torch.float16)}) is False
    assert q._payload_has_bias({"bias": ones}) is True
    assert q._payload_has_bias({"bias": ones, "has_bias": torch.tensor([0], dtype=torch.int32)}) is False
    assert q._payload_flag({"compact3_use_block_gr": torch.tensor([1], dtype=torch.int32)}, "compact3_use_block_gr") is True
    assert q._payload_flag({}, "compact3_use_block_gr", True) is True
