"""Grouped payload sidecar: the single safetensors file the reference's deployment runtime
loads its E-stacked expert payloads from (``grouped_payload_sidecar.py`` in the TriS-MoE
tree: names :18-46 and :109-127, encoding :168-180, decoding :282-303, zero output_scale
repair :264-279, loader :628-688).

Key scheme: ``{layer_prefix}.grouped_payload.{cache_key}.{name}`` with ``layer_prefix`` =
``model.layers.{L}.mlp`` (OLMoE/Qwen) or ``model.layers.{L}.block_sparse_moe`` (Mixtral) and
``cache_key`` in gate/up/down (+ ``*_ns``).  Python scalars are stored as one-element tensors,
``None`` as an empty tensor.
"""
from __future__ import annotations

import os
from typing import Dict, Optional

import torch

GROUPED_PAYLOAD_SIDECAR_BASENAME = "grouped_runtime_payload.safetensors"
GROUPED_PAYLOAD_METADATA = {"format": "olmoe_grouped_runtime_payload_v1"}  # standalone sidecar (grouped_payload_sidecar.py:20)
GROUPED_PAYLOAD_EMBEDDED_METADATA_KEY = "olmoe_grouped_runtime_payload"
GROUPED_PAYLOAD_DEPLOYMENT_ONLY_METADATA_KEY = "olmoe_deployment_only"
GROUPED_PRECOMPUTED_KEYS = ("gate", "up", "down")
GROUPED_NS_KEYS = ("gate_ns", "up_ns", "down_ns")
GROUPED_QGMAP_PAYLOAD_NAMES = frozenset({"q_gmap_sparse", "q_gmap_sparse_prefix"})
_BOOL_SCALARS = {"is_compact3", "compact3_use_block_gr", "has_output_scale", "has_bias"}
_INT_SCALARS = {"max_ns_rank", "infeatures", "outfeatures", "group_size"}


def default_grouped_payload_sidecar_path(model_dir: str) -> str:
    return os.path.join(model_dir, GROUPED_PAYLOAD_SIDECAR_BASENAME)


def layer_prefix(layer_index: int, family: str = "olmoe") -> str:
    """``model.layers.{L}.mlp`` or, for Mixtral, ``model.layers.{L}.block_sparse_moe``
    (grouped_payload_sidecar.py:57-82)."""
    leaf = "block_sparse_moe" if family.lower() == "mixtral" else "mlp"
    return f"model.layers.{layer_index}.{leaf}"


def payload_tensor_name(prefix: str, cache_key: str, name: str) -> str:
    return f"{prefix}.grouped_payload.{cache_key}.{name}"


def split_payload_tensor_name(name: str):
    marker = ".grouped_payload."
    if marker not in name:
        return None
    prefix, rest = name.split(marker, 1)
    if "." not in rest:
        return None
    cache_key, payload_name = rest.split(".", 1)
    return (prefix, cache_key, payload_name) if cache_key and payload_name else None


def _encode(name: str, value) -> Optional[torch.Tensor]:
    if isinstance(value, torch.Tensor):
        t = value.detach().to("cpu").contiguous()
        return t.reshape(1) if t.ndim == 0 else t
    if value is None:
        return torch.empty((0,), dtype=torch.float16)
    if isinstance(value, bool):
        return torch.tensor([value], dtype=torch.bool)
    if isinstance(value, int):
        return torch.tensor([value], dtype=torch.int32)
    return None  # not part of the on-disk format (derived indexes, python lists)


def save_grouped_payloads_to_sidecar(path: str, layers: Dict[str, Dict[str, dict]], metadata: Optional[dict] = None,
                                     embedded: bool = False, deployment_only: bool = False) -> int:
    """Writes ``{layer_prefix: {cache_key: payload}}``; returns the number of tensors.  Metadata as
    the reference writes it (grouped_payload_sidecar.py:438-446, 532-550): a standalone sidecar
    carries ``format = olmoe_grouped_runtime_payload_v1``; a file that also holds the model state
    (``embedded``) carries ``format = pt`` plus the embedded / deployment-only markers."""
    from safetensors.torch import save_file

    tensors = {}
    for prefix, by_key in layers.items():
        for cache_key, payload in by_key.items():
            for name, value in payload.items():
                if name.startswith("_"):
                    continue
                t = _encode(name, value)
                if t is not None:
                    tensors[payload_tensor_name(prefix, cache_key, name)] = t
    meta = {str(k): str(v) for k, v in (metadata or {}).items()}
    if embedded:
        meta["format"] = "pt"
        meta[GROUPED_PAYLOAD_EMBEDDED_METADATA_KEY] = "v1"
        if deployment_only:
            meta[GROUPED_PAYLOAD_DEPLOYMENT_ONLY_METADATA_KEY] = "v1"
    else:
        meta.update(GROUPED_PAYLOAD_METADATA)
    save_file(tensors, path, metadata=meta)
    return len(tensors)


def sidecar_has_grouped_payloads(path: str) -> bool:
    from safetensors import safe_open

    if not path or not os.path.exists(path):
        return False
    with safe_open(path, framework="pt", device="cpu") as fh:
        meta = fh.metadata() or {}
        if meta.get(GROUPED_PAYLOAD_EMBEDDED_METADATA_KEY) == "v1" or meta.get("format") == GROUPED_PAYLOAD_METADATA["format"]:
            return True
        # the reference loader does not look at metadata at all: any payload tensor name counts
        return any(split_payload_tensor_name(key) is not None for key in fh.keys())


def load_grouped_payload_from_sidecar(path: str, prefix: str, cache_key: str, device="cpu",
                                      dtype: torch.dtype = torch.float16, skip_qgmap: bool = False) -> Optional[dict]:
    """One projection's payload, scalars decoded to python values, an all-zero
    ``output_scale`` repaired to ones; ``None`` when the file has no such payload.
    ``skip_qgmap`` leaves the streamed bitmap tensors out (they are loaded to pinned memory by
    :func:`load_grouped_qgmap_from_sidecar`)."""
    from safetensors import safe_open

    if not path or not os.path.exists(path):
        return None
    stem = payload_tensor_name(prefix, cache_key, "")
    payload = {}
    with safe_open(path, framework="pt", device="cpu") as fh:
        for key in fh.keys():
            if not key.startswith(stem):
                continue
            name = key[len(stem):]
            if skip_qgmap and name in GROUPED_QGMAP_PAYLOAD_NAMES:
                continue
            payload[name] = fh.get_tensor(key)
    if not payload:
        return None
    return _decode_payload(payload, device=device, dtype=dtype)


def _decode_payload(payload: Dict[str, torch.Tensor], device="cpu", dtype: torch.dtype = torch.float16) -> dict:
    """Stored tensors of one payload -> the runtime dict: one-element scalars become python values
    (grouped_payload_sidecar.py:282-303), floating tensors get ``dtype``, an all-zero compact3
    ``output_scale`` is repaired to ones (:264-279)."""
    out = {}
    for name, t in payload.items():
        if name in _BOOL_SCALARS and t.numel() == 1:
            out[name] = bool(t.reshape(-1)[0].item())
        elif name in _INT_SCALARS and t.numel() == 1:
            out[name] = int(t.reshape(-1)[0].item())
        else:  # an absent tensor (None when written) comes back empty, as the reference loader returns it
            out[name] = (t.to(device=device, dtype=dtype) if t.is_floating_point() else t.to(device=device)).contiguous()
    scale = out.get("output_scale")
    if out.get("is_compact3") and isinstance(scale, torch.Tensor) and scale.numel() and bool(torch.all(scale == 0)):
        out["output_scale"] = torch.ones_like(scale)
        out["has_output_scale"] = False
    return out


def load_grouped_qgmap_from_sidecar(path: str, prefix: str, cache_key: str, pin_memory: bool = True) -> Optional[dict]:
    """The streamed bitmap tensors of one projection on the host
    (``load_grouped_qgmap_from_sidecar`` of the reference)."""
    from safetensors import safe_open

    if not path or not os.path.exists(path):
        return None
    out = {}
    with safe_open(path, framework="pt", device="cpu") as fh:
        for name in GROUPED_QGMAP_PAYLOAD_NAMES:
            key = payload_tensor_name(prefix, cache_key, name)
            if key in fh.keys():
                t = fh.get_tensor(key).contiguous()
                out[name] = t.pin_memory() if pin_memory and torch.cuda.is_available() else t
    return out if len(out) == len(GROUPED_QGMAP_PAYLOAD_NAMES) else None
