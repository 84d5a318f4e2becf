"""GPU test of the end-to-end decode harness on a tiny decoder: the KV-cache decode step gives the
logits a full re-computation of the sequence gives, the CUDA-graph loop produces the tokens the
eager loop produces, and the reported numbers follow the reference benchmark's definitions."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _tiny_model(tm, layers=2, max_length=32, max_batch=4):
    from trismoe_b200 import decode_harness as dh, synth

    shape = synth.LayerShape(256, 192, 8, 2, rank=96, group_size=32)
    blocks = []
    for l in range(layers):
        layer = synth.synth_layer(shape, seed=80 + l)
        for name in ("gate", "up", "down"):
            layer["shared_" + name] = (layer["shared_" + name].float() * 5.0).half()
        blk = tm.TrisSparseMoeBlock(shape.hidden_size, shape.intermediate_size, shape.num_experts, shape.top_k, True)
        blk.load_grouped_payloads(layer["gate"], layer["up"], layer["down"], layer["shared_gate"], layer["shared_up"],
                                  layer["shared_down"], layer["router_weight"], device="cuda")
        blocks.append(blk)
    dshape = dh.DecoderShape(hidden_size=256, num_heads=4, head_dim=64, num_kv_heads=2, vocab_size=512)
    return dh.TrisDecoder(blocks, dshape, max_length=max_length, max_batch=max_batch, device="cuda", seed=3), dh


def test_cached_decode_matches_recomputation_and_graph_matches_eager(lib):
    import trismoe_b200 as tm

    model, dh = _tiny_model(tm)
    B, L = 3, 7
    ids = torch.randint(0, 512, (B, L), generator=torch.Generator().manual_seed(1)).cuda()
    pos = torch.arange(L, device="cuda")[None, :].expand(B, L).contiguous()
    with torch.no_grad():
        first = model(ids, pos).argmax(-1, keepdim=True)
        cached = model(first, torch.full((B, 1), L, dtype=torch.long, device="cuda"))            # one decode step on the cache
        full_pos = torch.arange(L + 1, device="cuda")[None, :].expand(B, L + 1).contiguous()
        recomputed = model(torch.cat([ids, first], dim=1), full_pos)                              # same tokens from scratch
    scale = float(recomputed.abs().mean())
    assert scale > 1e-3 and float((cached - recomputed).abs().max()) <= 0.05 * max(1.0, scale)
    eager = dh.run_exact_generation(model, ids, output_length=6, use_graph=False)
    graph = dh.run_exact_generation(model, ids, output_length=6, use_graph=True)
    assert graph["launch_mode"] == "cuda graph" and eager["launch_mode"] == "eager"
    assert torch.equal(eager["tokens"], graph["tokens"])
    assert torch.equal(eager["tokens"][:, 0:1], first)
    assert int(graph["tokens"].min()) >= 0 and int(graph["tokens"].max()) < 512
    assert graph["decode_steps"] == 5 and graph["decode_tokens_per_s"] > 0 and graph["prefill_tokens_per_s"] > 0
    for blk in model.blocks:
        blk.raise_on_kernel_status()
    with pytest.raises(RuntimeError, match="cache too small"):
        dh.run_exact_generation(model, ids, output_length=64)
