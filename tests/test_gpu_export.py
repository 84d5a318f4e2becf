"""GPU test of the exporter's stored derived tensors: a block-GR export made with
store_derived=True carries the sub-stream index, packed-row groups and tile records; a payload
loaded from it is prepared without rebuilding them and gives bit-identical decoded bitmaps,
dequantised weights and operator outputs."""
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_export_with_derived_tensors_is_adopted(lib, tmp_path):
    import trismoe_b200 as tm
    from trismoe_b200 import checkpoint_export as ce, sidecar, synth

    shape = synth.LayerShape(256, 192, 4, 2, rank=96, group_size=32)
    layer = synth.synth_layer(shape, seed=61, keep_sparse_gmap=True, use_block_gr=False)
    prefix = sidecar.layer_prefix(0)
    src = os.path.join(tmp_path, "src.safetensors")
    out = os.path.join(tmp_path, "out.safetensors")
    sidecar.save_grouped_payloads_to_sidecar(src, {prefix: {k: layer[k] for k in ("gate", "up", "down")}})
    stats = ce.export_grouped_blockgr_checkpoint(src, out, store_derived=True, device="cuda")
    assert stats["derived_payloads"] == 3
    batch = next(ce.iter_layer_payload_batches(out, layers_per_batch=1))
    stored = batch[prefix]["down"]
    assert stored.get("_tris_derived_from_checkpoint") is True
    adopted = tm.prepare_grouped_payload(stored, "cuda")
    assert adopted.get("_tris_derived_from_checkpoint") is True  # shapes fitted: nothing was rebuilt
    plain = sidecar.load_grouped_payload_from_sidecar(out, prefix, "down")
    for name in ce.DERIVED_NAMES:
        plain.pop(name, None)
    rebuilt = tm.prepare_grouped_payload(plain, "cuda")
    assert torch.equal(adopted["_tris_tile_records"], rebuilt["_tris_tile_records"])
    assert torch.equal(tm.decode_block_gr_gmap(adopted), tm.decode_block_gr_gmap(rebuilt))
    assert torch.equal(tm.dequantize_grouped_payload(adopted), tm.dequantize_grouped_payload(rebuilt))
    hidden = torch.randn((10, 96), device="cuda").half()
    lengths = [3, 0, 5, 2]
    ya = tm.run_grouped_structured_expert_forward(adopted, hidden, None, lengths)
    yb = tm.run_grouped_structured_expert_forward(rebuilt, hidden, None, lengths)
    assert torch.equal(ya, yb) and float(ya.float().abs().mean()) > 0
    # derived tensors that do not fit the payload are dropped and rebuilt, not trusted
    broken = next(ce.iter_layer_payload_batches(out, layers_per_batch=1))[prefix]["gate"]
    broken["_tris_gr_index"] = broken["_tris_gr_index"][:, :-1]
    fixed = tm.prepare_grouped_payload(broken, "cuda")
    assert not fixed.get("_tris_derived_from_checkpoint") and fixed["_tris_tile_records"] is not None
