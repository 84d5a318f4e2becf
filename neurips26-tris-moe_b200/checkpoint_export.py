"""Checkpoint tooling for the grouped payload sidecar: the block Golomb-Rice exporter and a
layer-batched loader (TriS-MoE tree: ``tools/export_grouped_blockgr_checkpoint.py:140-233``,
``build_grouped_blockgr_payloads`` in ``tools/rewrite_runtime_min_checkpoint.py:363-444``,
``restore_dense_packed_gmap_from_sparse`` :147-159, ``drop_blockgr_sparse_payloads``; the
layer-batched loader of ``auto_gptq/modeling/_base.py:708-781``; the single-file streaming export of
``tools/export_grouped_streaming_sparse_checkpoint.py``).

``export_grouped_blockgr_checkpoint`` turns a sidecar (or embedded checkpoint) whose grouped
payloads carry the sparse g_map planes into one that carries the block-GR streams, tensor names,
dtypes, shapes and metadata as the reference exporter writes them.  With ``store_derived=True`` and a
CUDA device it also stores what this runtime derives at load time - the sub-stream index, the
packed-row groups and the tile-major records the kernels read - under ``tris_*`` names next to
each payload, so that loading a checkpoint does not rebuild them; ``attach_derived`` puts them
back into a loaded payload dict and ``prepare_grouped_payload`` then skips the rebuild.
"""
from __future__ import annotations

import math
import os
from typing import Dict, Iterator, List, Optional, Tuple

import numpy as np
import torch

from .formats import block_gr_encode
from .sidecar import (
    GROUPED_PAYLOAD_DEPLOYMENT_ONLY_METADATA_KEY,
    GROUPED_PAYLOAD_EMBEDDED_METADATA_KEY,
    GROUPED_PAYLOAD_METADATA,
    GROUPED_PRECOMPUTED_KEYS,
    GROUPED_QGMAP_PAYLOAD_NAMES,
    load_grouped_payload_from_sidecar,
    payload_tensor_name,
    split_payload_tensor_name,
)

BLOCK_GR_EXPORT_METADATA_KEY = "olmoe_grouped_block_gr_export"
DERIVED_NAMES = ("tris_gr_index", "tris_packed_row_group", "tris_tile_records", "tris_tile_desc", "tris_col_records",
                 "tris_tile_meta")


def collect_grouped_payloads(tensors: Dict[str, torch.Tensor]) -> Dict[Tuple[str, str], Dict[str, torch.Tensor]]:
    """``{(layer_prefix, cache_key): {payload_name: tensor}}`` of every grouped payload tensor."""
    out: Dict[Tuple[str, str], Dict[str, torch.Tensor]] = {}
    for name, tensor in tensors.items():
        split = split_payload_tensor_name(name)
        if split is None:
            continue
        prefix, cache_key, payload_name = split
        out.setdefault((prefix, cache_key), {})[payload_name] = tensor
    return out


def restore_dense_packed_gmap_from_sparse(q_gmap_sparse: torch.Tensor, c_map: torch.Tensor, ncols: int,
                                          out_features: int) -> torch.Tensor:
    """Dense packed g_map ``[ceil(ncols/32), O]`` int32 of one expert from its sparse plane (grouping
    bits of the non-salient columns only, ascending, packed 32 per word; salient columns read 0)."""
    pr = math.ceil(ncols / 32)
    cm = np.unpackbits(c_map.detach().cpu().numpy().astype("<i4").view(np.uint8), bitorder="little")[:ncols].astype(bool)
    sparse = q_gmap_sparse.detach().cpu().numpy().astype("<i4").view(np.uint32)              # [rows, O]
    active = np.flatnonzero(~cm)
    bits = np.zeros((pr * 32, out_features), dtype=np.uint8)
    if active.size and sparse.size:
        unpacked = np.unpackbits(sparse.T.copy().view(np.uint8), axis=-1, bitorder="little")  # [O, rows*32]
        bits[active, :] = unpacked[:, : active.size].T
    words = np.packbits(bits.reshape(pr, 32, out_features).transpose(0, 2, 1), axis=-1, bitorder="little")
    return torch.from_numpy(words.view("<u4").reshape(pr, out_features).view(np.int32).copy())


def _flag(payload: dict, name: str) -> bool:
    t = payload.get(name)
    return isinstance(t, torch.Tensor) and t.numel() > 0 and bool(t.reshape(-1)[0].item())


def build_grouped_blockgr_payloads(tensors: Dict[str, torch.Tensor], mode: str = "compressed", fixed_k: Optional[int] = None,
                                   k_min: Optional[int] = None, k_max: Optional[int] = None) -> Tuple[int, int]:
    """Adds ``q_gmap_gr_words / _offsets / _meta`` and ``compact3_use_block_gr = True`` to every compact3
    grouped payload in ``tensors`` (in place), encoded from the sparse planes; returns (payloads
    updated, words written).  ``mode`` is ``"compressed"`` or ``"raw"`` (every block stored verbatim)."""
    lo, hi = resolve_block_gr_search_bounds(fixed_k, k_min, k_max)
    updated = total_words = 0
    for (prefix, cache_key), payload in sorted(collect_grouped_payloads(tensors).items()):
        if cache_key not in GROUPED_PRECOMPUTED_KEYS or not _flag(payload, "is_compact3"):
            continue
        need = ("q_gmap_sparse", "c_map", "qweight1", "g_idx")
        if not all(isinstance(payload.get(n), torch.Tensor) for n in need) or payload["q_gmap_sparse"].dim() != 3:
            raise RuntimeError(f"missing compact3 payload tensors for {prefix}:{cache_key}")
        E = int(payload["qweight1"].shape[0])
        O = int(payload["qweight1"].shape[2])
        ncols = int(payload["g_idx"].shape[1])
        streams = []
        for e in range(E):
            dense = restore_dense_packed_gmap_from_sparse(payload["q_gmap_sparse"][e], payload["c_map"][e], ncols, O)
            streams.append(block_gr_encode(dense, force_raw=(mode == "raw"), k_min=lo, k_max=hi))
        max_words = max(int(s[0].numel()) for s in streams)
        words = torch.zeros((E, max_words), dtype=torch.int32)
        for e, s in enumerate(streams):
            words[e, : s[0].numel()] = s[0]
        tensors[payload_tensor_name(prefix, cache_key, "compact3_use_block_gr")] = torch.tensor([True], dtype=torch.bool)
        tensors[payload_tensor_name(prefix, cache_key, "q_gmap_gr_words")] = words.contiguous()
        tensors[payload_tensor_name(prefix, cache_key, "q_gmap_gr_offsets")] = torch.stack([s[1] for s in streams]).contiguous()
        tensors[payload_tensor_name(prefix, cache_key, "q_gmap_gr_meta")] = torch.stack([s[2] for s in streams]).contiguous()
        updated += 1
        total_words += int(words.numel())
    return updated, total_words


def resolve_block_gr_search_bounds(fixed_k: Optional[int] = None, k_min: Optional[int] = None,
                                   k_max: Optional[int] = None) -> Tuple[int, int]:
    """Bounds of the per-block Rice parameter search (rewrite_runtime_min_checkpoint.py:227-250)."""
    if fixed_k is not None:
        if k_min is not None or k_max is not None:
            raise ValueError("a fixed k cannot be combined with k_min / k_max")
        if not 0 <= fixed_k <= 7:
            raise ValueError(f"k must be in [0, 7], got {fixed_k}")
        return fixed_k, fixed_k
    if k_min is None and k_max is None:
        return 0, 7
    if k_min is None or k_max is None:
        raise ValueError("k_min and k_max must be given together")
    if not 0 <= k_min <= k_max <= 7:
        raise ValueError(f"k_min / k_max must satisfy 0 <= min <= max <= 7, got {k_min}, {k_max}")
    return k_min, k_max


def drop_blockgr_sparse_payloads(tensors: Dict[str, torch.Tensor]) -> Tuple[int, int]:
    """Removes the sparse g_map planes of payloads that now carry block-GR streams (the exporter's
    default, ``--keep-sparse`` off); returns (payloads with streams, keys removed)."""
    with_streams = removed = 0
    for (prefix, cache_key), payload in collect_grouped_payloads(tensors).items():
        if cache_key not in GROUPED_PRECOMPUTED_KEYS or not _flag(payload, "compact3_use_block_gr"):
            continue
        with_streams += 1
        for name in GROUPED_QGMAP_PAYLOAD_NAMES:
            key = payload_tensor_name(prefix, cache_key, name)
            if key in tensors:
                ref = tensors.pop(key)
                # an empty tensor of the same rank keeps the key set the loaders expect
                tensors[key] = torch.empty((ref.shape[0],) + (0,) * (ref.dim() - 1), dtype=ref.dtype) if name == "q_gmap_sparse" else ref
                removed += int(name == "q_gmap_sparse")
    return with_streams, removed


def build_derived_tensors(tensors: Dict[str, torch.Tensor], device) -> int:
    """Builds, on a CUDA device, what ``prepare_grouped_payload`` derives for every block-GR payload
    (sub-stream index, packed-row groups, tile records) and stores it under ``tris_*`` names."""
    from .qlinear_grouped import prepare_grouped_payload
    from .sidecar import _decode_payload

    built = 0
    for (prefix, cache_key), raw in sorted(collect_grouped_payloads(tensors).items()):
        if cache_key not in GROUPED_PRECOMPUTED_KEYS or not _flag(raw, "compact3_use_block_gr"):
            continue
        payload = prepare_grouped_payload(_decode_payload({k: v.clone() for k, v in raw.items() if not k.startswith("tris_")}), device)
        derived = {
            "tris_gr_index": payload["_tris_gr_index"],
            "tris_packed_row_group": payload["_tris_packed_row_group"],
            "tris_tile_records": payload["_tris_tile_records"],
            "tris_tile_desc": payload["_tris_tile_desc"],
            "tris_col_records": payload["_tris_col_records"],
            "tris_tile_meta": torch.tensor(list(payload["_tris_tile_meta"]), dtype=torch.int32),
        }
        for name, t in derived.items():
            if isinstance(t, torch.Tensor):
                tensors[payload_tensor_name(prefix, cache_key, name)] = t.detach().cpu().contiguous()
        built += 1
    return built


def attach_derived(payload: dict) -> dict:
    """Moves the stored ``tris_*`` tensors of a loaded payload to the private keys
    ``prepare_grouped_payload`` reads, so that it uses them instead of rebuilding."""
    names = {"tris_gr_index": "_tris_gr_index", "tris_packed_row_group": "_tris_packed_row_group",
             "tris_tile_records": "_tris_tile_records", "tris_tile_desc": "_tris_tile_desc",
             "tris_col_records": "_tris_col_records"}
    if all(isinstance(payload.get(n), torch.Tensor) and payload[n].numel() > 0 for n in names) and \
            isinstance(payload.get("tris_tile_meta"), torch.Tensor) and payload["tris_tile_meta"].numel() == 3:
        for stored, private in names.items():
            payload[private] = payload.pop(stored)
        payload["_tris_tile_meta"] = tuple(int(v) for v in payload.pop("tris_tile_meta").tolist())
        payload["_tris_derived_from_checkpoint"] = True
    else:
        for n in DERIVED_NAMES:
            payload.pop(n, None)
    return payload


def export_grouped_blockgr_checkpoint(source_path: str, output_path: str, mode: str = "compressed", fixed_k: Optional[int] = None,
                                      k_min: Optional[int] = None, k_max: Optional[int] = None, keep_sparse: bool = False,
                                      store_derived: bool = False, device=None) -> dict:
    """Reads ``source_path`` (a safetensors file with grouped payload tensors), writes ``output_path``
    with block-GR streams; returns the counters the reference exporter prints."""
    from safetensors import safe_open
    from safetensors.torch import save_file

    if mode not in ("compressed", "raw"):
        raise ValueError("mode must be 'compressed' or 'raw'")
    lo, hi = resolve_block_gr_search_bounds(fixed_k, k_min, k_max)
    with safe_open(source_path, framework="pt", device="cpu") as fh:
        metadata = {str(k): str(v) for k, v in (fh.metadata() or {}).items()}
        tensors = {k: fh.get_tensor(k).contiguous() for k in fh.keys()}
    built, words = build_grouped_blockgr_payloads(tensors, mode, fixed_k, k_min, k_max)
    with_streams = removed = 0
    if not keep_sparse:
        with_streams, removed = drop_blockgr_sparse_payloads(tensors)
    derived = 0
    if store_derived:
        dev = torch.device(device) if device is not None else torch.device("cuda")
        if dev.type != "cuda":
            raise RuntimeError("trismoe_b200 export: the derived tensors are built by CUDA kernels (there is no CPU path)")
        derived = build_derived_tensors(tensors, dev)
    embedded = metadata.get(GROUPED_PAYLOAD_EMBEDDED_METADATA_KEY) == "v1" or metadata.get("format") == "pt"
    if embedded:  # the reference marks its exports deployment-only (export_grouped_blockgr_checkpoint.py:207)
        metadata["format"] = "pt"
        metadata[GROUPED_PAYLOAD_EMBEDDED_METADATA_KEY] = "v1"
        metadata[GROUPED_PAYLOAD_DEPLOYMENT_ONLY_METADATA_KEY] = "v1"
    else:
        metadata.update(GROUPED_PAYLOAD_METADATA)
    metadata[BLOCK_GR_EXPORT_METADATA_KEY] = "v1"
    metadata["olmoe_grouped_block_gr_mode"] = mode
    metadata["olmoe_grouped_block_gr_keep_sparse"] = "1" if keep_sparse else "0"
    if fixed_k is not None:
        metadata["olmoe_grouped_block_gr_k"] = str(fixed_k)
    else:
        metadata["olmoe_grouped_block_gr_k_min"] = str(lo)
        metadata["olmoe_grouped_block_gr_k_max"] = str(hi)
    if derived:
        metadata["tris_b200_derived"] = "v1"
    os.makedirs(os.path.dirname(os.path.abspath(output_path)), exist_ok=True)
    save_file(tensors, output_path, metadata=metadata)
    return {"built_grouped_payloads": built, "built_grouped_words": words, "grouped_blockgr_payload_count": with_streams,
            "removed_grouped_sparse_keys": removed, "derived_payloads": derived, "blockgr_k_search_min": lo,
            "blockgr_k_search_max": hi, "keep_sparse": bool(keep_sparse)}


STREAMING_READY_METADATA_KEY = "olmoe_grouped_qgmap_cpu_staging_ready"
STREAMING_SINGLE_FILE_METADATA_KEY = "olmoe_grouped_qgmap_cpu_staging_single_file"
# per-expert module state a deployment-only checkpoint keeps (grouped_payload_sidecar.py:38-46)
DEPLOYMENT_ONLY_EXPERT_LEAVES = frozenset({"mode", "ns_mode", "ns_vector_row", "ns_vector_col", "expert_input_scale"})
_EXPERT_MODULES = {"gate_proj": "gate_proj", "up_proj": "up_proj", "down_proj": "down_proj",  # OLMoE / Qwen naming
                   "w1": "gate_proj", "w3": "up_proj", "w2": "down_proj"}  # Mixtral naming


def split_moe_expert_tensor_name(name: str) -> Optional[Tuple[str, str]]:
    """``model.layers.<i>.mlp.experts.<e>.<proj>.<leaf>`` (or Mixtral's ``block_sparse_moe.experts.<e>.w1|w2|w3``)
    -> (logical projection, leaf); None for every other tensor (grouped_payload_sidecar.py:467-497)."""
    parts = name.split(".")
    if len(parts) < 8 or parts[0] != "model" or parts[1] != "layers" or not parts[2].isdigit():
        return None
    if parts[4] != "experts" or not parts[5].isdigit():
        return None
    if parts[3] == "mlp":
        allowed = ("gate_proj", "up_proj", "down_proj")
    elif parts[3] == "block_sparse_moe":
        allowed = ("w1", "w2", "w3")
    else:
        return None
    if parts[6] not in allowed:
        return None
    return _EXPERT_MODULES[parts[6]], ".".join(parts[7:])


def build_deployment_only_checkpoint_tensors(tensors: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    """Drops what a grouped runtime never reads: per-expert module tensors other than the few state
    leaves, keeping grouped payload tensors and everything outside the expert modules
    (``build_deployment_only_checkpoint_tensors``, grouped_payload_sidecar.py:508-517)."""
    kept = {}
    for name, t in tensors.items():
        if split_payload_tensor_name(name) is None:
            expert = split_moe_expert_tensor_name(name)
            if expert is not None and expert[1] not in DEPLOYMENT_ONLY_EXPERT_LEAVES:
                continue
        kept[name] = t
    return kept


def repair_grouped_payload_tensors(tensors: Dict[str, torch.Tensor]) -> int:
    """An all-zero ``output_scale`` of a compact3 payload (written by an exporter that had none) becomes ones with
    ``has_output_scale`` cleared; returns how many payloads were repaired (grouped_payload_sidecar.py:306-337)."""
    repaired = 0
    for (prefix, key), payload in collect_grouped_payloads(tensors).items():
        if key not in GROUPED_PRECOMPUTED_KEYS or not _flag(payload, "is_compact3"):
            continue
        scale = payload.get("output_scale")
        if not isinstance(scale, torch.Tensor) or scale.numel() == 0 or bool(torch.any(scale != 0)):
            continue
        tensors[payload_tensor_name(prefix, key, "output_scale")] = torch.ones_like(scale).contiguous()
        flag_name = payload_tensor_name(prefix, key, "has_output_scale")
        if flag_name in tensors:
            tensors[flag_name] = torch.zeros_like(tensors[flag_name], dtype=torch.bool).contiguous()
        repaired += 1
    return repaired


def has_sparse_qgmap_payloads(tensors: Dict[str, torch.Tensor]) -> bool:
    """True when a grouped projection or an attention linear carries the sparse g_map planes the
    bitmap streaming manager pages (export_grouped_streaming_sparse_checkpoint.py:55-66)."""
    for name in tensors:
        split = split_payload_tensor_name(name)
        if split is not None:
            if split[1] in GROUPED_PRECOMPUTED_KEYS and split[2] == "q_gmap_sparse":
                return True
        elif ".self_attn." in name and name.endswith(".q_gmap_sparse"):
            return True
    return False


def export_grouped_streaming_sparse_checkpoint(source_path: str, output_path: str) -> dict:
    """A single-file checkpoint ready for host-staged bitmap streaming out of a sparse grouped checkpoint
    (tools/export_grouped_streaming_sparse_checkpoint.py:37-86): deployment-only tensor filter, output-scale repair,
    a source without sparse g_map planes refused, embedded + deployment-only metadata and the two staging-ready keys."""
    from safetensors import safe_open
    from safetensors.torch import save_file

    with safe_open(source_path, framework="pt", device="cpu") as fh:
        metadata = {str(k): str(v) for k, v in (fh.metadata() or {}).items()}
        tensors = {k: fh.get_tensor(k).contiguous() for k in fh.keys()}
    total = len(tensors)
    tensors = build_deployment_only_checkpoint_tensors(tensors)
    repaired = repair_grouped_payload_tensors(tensors)
    if not has_sparse_qgmap_payloads(tensors):
        raise ValueError("source checkpoint does not contain sparse qgmap payloads; "
                         "the streaming export expects a sparse source checkpoint")
    metadata["format"] = "pt"
    metadata[GROUPED_PAYLOAD_EMBEDDED_METADATA_KEY] = "v1"
    metadata[GROUPED_PAYLOAD_DEPLOYMENT_ONLY_METADATA_KEY] = "v1"
    metadata[STREAMING_READY_METADATA_KEY] = "v1"
    metadata[STREAMING_SINGLE_FILE_METADATA_KEY] = "1"
    os.makedirs(os.path.dirname(os.path.abspath(output_path)), exist_ok=True)
    save_file(tensors, output_path, metadata=metadata)
    return {"streaming_sparse": True, "single_file": True, "repaired_grouped_output_scales": repaired,
            "kept_tensors": len(tensors), "dropped_tensors": total - len(tensors)}


def layer_prefixes_in(path: str) -> List[str]:
    from safetensors import safe_open

    with safe_open(path, framework="pt", device="cpu") as fh:
        found = {split[0] for split in (split_payload_tensor_name(k) for k in fh.keys()) if split is not None}

    def order(prefix: str):
        parts = prefix.split(".")
        nums = [int(p) for p in parts if p.isdigit()]
        return (nums[0] if nums else 0, prefix)

    return sorted(found, key=order)


def iter_layer_payload_batches(path: str, layers_per_batch: int = 4, device="cpu",
                               cache_keys=GROUPED_PRECOMPUTED_KEYS) -> Iterator[Dict[str, Dict[str, dict]]]:
    """Yields ``{layer_prefix: {cache_key: payload}}`` for ``layers_per_batch`` layers at a time, so
    that a whole model's payloads never sit in host memory together (the layer-batched load of
    ``_base.py:708-781``); stored derived tensors are attached."""
    prefixes = layer_prefixes_in(path)
    for i in range(0, len(prefixes), max(1, int(layers_per_batch))):
        batch = {}
        for prefix in prefixes[i: i + layers_per_batch]:
            batch[prefix] = {}
            for key in cache_keys:
                payload = load_grouped_payload_from_sidecar(path, prefix, key, device=device)
                if payload is not None:
                    batch[prefix][key] = attach_derived(payload)
        yield batch
