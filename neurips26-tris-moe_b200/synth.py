"""Seeded synthetic TriS-MoE layers in the reference's payload format.

Real quantized checkpoints are not available offline, so benchmarks and tests draw the
bit planes and scales from the distributions of the headline configuration: sign bits
Bernoulli(0.5), salient columns Bernoulli(p) per column, grouping bit Bernoulli(p) per
element on non-salient columns (block Golomb-Rice coded in 4096-bit blocks), row scales
|N(0, 0.02)| fp16 per 128-column group, column scales 1.0, fp16 backbone N(0, 0.02) of
rank r, activations N(0, 1) with 1 % of the channels scaled by 20.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import numpy as np
import torch

from .formats import (
    _as_i32_tensor,
    _pack_last_axis,
    block_gr_encode,
    build_sparse_bit_prefix,
    pack_half4_words,
)


@dataclass
class LayerShape:
    hidden_size: int
    intermediate_size: int
    num_experts: int
    top_k: int
    rank: int = 256
    group_size: int = 128
    norm_topk_prob: bool = True


OLMOE = LayerShape(2048, 1024, 64, 8)
MIXTRAL = LayerShape(4096, 14336, 8, 2)
QWEN35 = LayerShape(2048, 512, 256, 8)


def raw_projection(rng: np.random.Generator, num_experts: int, out_features: int, rank: int, group_size: int = 128,
                   p_salient: float = 0.1, p_gmap: float = 0.1, col_scale_one: bool = True) -> dict:
    """Unpacked random planes and scales of one projection for all experts."""
    E, O, r = num_experts, out_features, rank
    G = math.ceil(r / group_size)
    c_map = rng.random((E, r)) < p_salient
    raw = {
        "b1": rng.random((E, O, r)) < 0.5,
        "b2": rng.random((E, O, r)) < 0.5,
        "c_map": c_map,
        "g_map": (rng.random((E, O, r)) < p_gmap) & ~c_map[:, None, :],
        "g_idx": np.broadcast_to((np.arange(r) // group_size).astype(np.int32), (E, r)).copy(),
    }
    base = lambda shape: np.abs(rng.normal(0.0, 0.02, size=shape)).astype(np.float16)
    raw["s_r1"] = base((E, O, G))
    raw["s_r2"] = (0.5 * base((E, O, G)).astype(np.float32)).astype(np.float16)
    raw["ns_d_r1"] = (2.0 * base((E, O, G)).astype(np.float32)).astype(np.float16)
    raw["ns_nd_r1"] = base((E, O, G))
    for name in ("s_c1", "s_c2", "ns_d_c1", "ns_nd_c1"):
        raw[name] = np.ones((E, r), dtype=np.float16) if col_scale_one else (
            1.0 + 0.25 * rng.standard_normal((E, r))).astype(np.float16)
    return raw


def pack_projection(raw: dict, device="cpu", use_block_gr: bool = True, keep_sparse_gmap: bool = True) -> dict:
    """E-stacked payload (keys of ``build_grouped_precomputed_payload``,
    qlinear_cuda.py:1512-1636 in the TriS-MoE tree) from :func:`raw_projection` output,
    vectorised over experts."""
    b1, b2, c_map, g_map = raw["b1"], raw["b2"], raw["c_map"], raw["g_map"]
    E, O, r = b1.shape
    pr = math.ceil(r / 32)
    dev = torch.device(device)

    def plane(bits_eok):  # bool [E, O, K] -> int32 [E, ceil(K/32), O]
        return np.ascontiguousarray(_pack_last_axis(bits_eok).transpose(0, 2, 1))

    def sparse_plane(bits, active):  # per expert: keep active columns, pack, pad rows
        per = []
        for e in range(E):
            cols = active[e]
            if cols.any():
                per.append(np.ascontiguousarray(_pack_last_axis(bits[e][:, cols]).T))
            else:
                per.append(np.zeros((0, O), dtype="<u4"))
        rows = max(p.shape[0] for p in per)
        out = np.zeros((E, rows, O), dtype="<u4")
        for e, p in enumerate(per):
            out[e, : p.shape[0]] = p
        return out

    dense_gmap = plane(g_map & ~c_map[:, None, :])
    payload = {
        "is_compact3": True,
        "qweight1": _as_i32_tensor(plane(b1), dev),
        "qweight2_sparse": _as_i32_tensor(sparse_plane(b2, c_map), dev),
        "qweight2_sparse_prefix": torch.stack([build_sparse_bit_prefix(c_map[e]) for e in range(E)]).to(dev),
        "q_gmap_sparse_prefix": torch.stack([build_sparse_bit_prefix(~c_map[e]) for e in range(E)]).to(dev),
        "c_map": _as_i32_tensor(_pack_last_axis(c_map), dev),
        "g_idx": torch.from_numpy(raw["g_idx"].astype(np.int32)).to(dev),
        "col_pack3": pack_half4_words(raw["s_c1"], raw["s_c2"], raw["ns_d_c1"], raw["ns_nd_c1"], dev),
        "row_pack3": pack_half4_words(raw["s_r1"], raw["s_r2"], raw["ns_d_r1"], raw["ns_nd_r1"], dev),
    }
    if keep_sparse_gmap:
        payload["q_gmap_sparse"] = _as_i32_tensor(sparse_plane(g_map, ~c_map), dev)
    else:
        payload["q_gmap_sparse"] = torch.zeros((E, 0, O), dtype=torch.int32, device=dev)
    if use_block_gr:
        streams = [block_gr_encode(torch.from_numpy(dense_gmap[e].view(np.int32))) for e in range(E)]
        max_words = max(int(s[0].numel()) for s in streams)
        words = torch.zeros((E, max_words), dtype=torch.int32)
        for e, s in enumerate(streams):
            words[e, : s[0].numel()] = s[0]
        payload["q_gmap_gr_words"] = words.to(dev)
        payload["q_gmap_gr_offsets"] = torch.stack([s[1] for s in streams]).to(dev)
        payload["q_gmap_gr_meta"] = torch.stack([s[2] for s in streams]).to(dev)
        payload["_gr_words_used"] = [int(s[0].numel()) for s in streams]
    else:
        for key in ("q_gmap_gr_words", "q_gmap_gr_offsets", "q_gmap_gr_meta"):
            payload[key] = torch.empty((0, 0), dtype=torch.int32, device=dev)
    payload["compact3_use_block_gr"] = bool(use_block_gr)
    payload["output_scale"] = torch.ones((E, O), dtype=torch.float16, device=dev)
    payload["has_output_scale"] = False
    payload["bias"] = None
    payload["has_bias"] = False
    payload["_dense_gmap_words"] = torch.from_numpy(dense_gmap.view(np.int32).copy())  # test aid, stays on the host
    return payload


def synth_layer(shape: LayerShape, seed: int, device="cpu", use_block_gr: bool = True, keep_sparse_gmap: bool = False,
                keep_raw: bool = False) -> dict:
    """One MoE layer: payloads for gate/up/down, three fp16 backbones and a router weight."""
    rng = np.random.default_rng(seed)
    H, I, E, r = shape.hidden_size, shape.intermediate_size, shape.num_experts, shape.rank
    layer = {"shape": shape}
    for name, (O, K) in (("gate", (I, H)), ("up", (I, H)), ("down", (H, I))):
        raw = raw_projection(rng, E, O, r, shape.group_size)
        layer[name] = pack_projection(raw, device, use_block_gr, keep_sparse_gmap)
        if keep_raw:
            layer[name + "_raw"] = raw
        layer["shared_" + name] = torch.from_numpy(rng.normal(0.0, 0.02, size=(r, K)).astype(np.float16)).to(device)
    layer["router_weight"] = torch.from_numpy((rng.standard_normal((E, H)) / math.sqrt(H)).astype(np.float16)).to(device)
    return layer


def synth_activations(num_tokens: int, hidden_size: int, seed: int, device="cpu") -> torch.Tensor:
    """fp16 N(0,1) activations with 1 % of the channels scaled by 20 (outlier channels)."""
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((num_tokens, hidden_size)).astype(np.float32)
    outliers = rng.choice(hidden_size, size=max(1, hidden_size // 100), replace=False)
    x[:, outliers] *= 20.0
    return torch.from_numpy(x.astype(np.float16)).to(device)


def synth_router_logits(num_tokens: int, num_experts: int, seed: int, device="cpu") -> torch.Tensor:
    rng = np.random.default_rng(seed)
    return torch.from_numpy(rng.standard_normal((num_tokens, num_experts)).astype(np.float32)).to(device)


def projection_algorithmic_bytes(payload: dict, experts) -> int:
    """Compressed bytes a kernel must read for the given experts of one projection:
    sign plane 1, salient sign plane rows actually occupied, GR words actually occupied,
    offsets + meta, c_map, prefix, column and row scale packs (padding not counted)."""
    E, pr, O = (int(s) for s in payload["qweight1"].shape)
    r = int(payload["g_idx"].shape[1])
    G = int(payload["row_pack3"].shape[2])
    nblk = math.ceil(pr / 2) * math.ceil(O / 64)
    pre2 = payload["qweight2_sparse_prefix"].cpu()
    total = 0
    for e in experts:
        s_e = int(pre2[e, -1])
        total += 4 * pr * O + 4 * math.ceil(s_e / 32) * O + 4 * pr + 4 * (pr + 1) + 8 * r + 8 * O * G
        if payload["compact3_use_block_gr"]:
            total += 4 * payload["_gr_words_used"][e] + 4 * (2 * nblk + 1)
        else:
            total += 4 * math.ceil((r - s_e) / 32) * O + 4 * (pr + 1)
    return total


def packed4_matrix(rng: np.random.Generator, rows: int, cols: int, group_size: int = 128, scale_std: float = 0.02) -> dict:
    """Random 4-bit packed matrix ``[rows, cols]`` in the layout of ``PackedQuantMatrix4bit``
    (qlinear_cuda.py:2637-2784): qweight ``[ceil(cols/8), rows]`` int32, qzeros
    ``[groups, ceil(rows/8)]`` int32 (zero points minus one), scales ``[groups, rows]`` fp16, g_idx
    ``[cols]`` with uniform groups."""
    groups = max(1, -(-cols // group_size))
    qweight = rng.integers(-2**31, 2**31, size=(-(-cols // 8), rows), dtype=np.int64).astype(np.int32)
    qzeros = rng.integers(-2**31, 2**31, size=(groups, -(-rows // 8)), dtype=np.int64).astype(np.int32)
    scales = np.abs(rng.normal(0, scale_std, size=(groups, rows))).astype(np.float16)
    g_idx = np.minimum(np.arange(cols) // group_size, groups - 1).astype(np.int32)
    return {"qweight": torch.from_numpy(qweight), "qzeros": torch.from_numpy(qzeros), "scales": torch.from_numpy(scales),
            "g_idx": torch.from_numpy(g_idx), "rows": rows, "cols": cols}
