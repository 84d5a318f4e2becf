"""Shared helpers for the tests: golden fixture loading and payload conversion."""
import os

import numpy as np
import torch

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")

PAYLOAD_KEYS = ("qweight1", "qweight2_sparse", "qweight2_sparse_prefix", "q_gmap_sparse", "q_gmap_sparse_prefix",
                "c_map_packed", "g_idx", "row_pack3", "col_pack3")
RAW_BOOL = ("b1", "b2", "c_map", "g_map")


def load_golden(name):
    return np.load(os.path.join(GOLDEN, name))


def golden_raw_expert(z, e, O, r):
    raw = {}
    for k in RAW_BOOL:
        packed = z[f"raw{e}_{k}"]
        raw[k] = np.unpackbits(packed, axis=-1)[..., :r].astype(bool)
    for k in ("g_idx", "s_r1", "s_r2", "ns_d_r1", "ns_nd_r1", "s_c1", "s_c2", "ns_d_c1", "ns_nd_c1"):
        raw[k] = z[f"raw{e}_{k}"]
    return raw


def golden_expert_payload(z, prefix):
    """Per-expert payload dict of CPU tensors from fixture arrays named ``{prefix}_{key}``."""
    p = {k: torch.from_numpy(z[f"{prefix}_{k}"].copy()) for k in PAYLOAD_KEYS}
    p["mode"] = "expert_compact3"
    return p


def to_numpy_payload(payload):
    return {k: (v.detach().cpu().numpy() if isinstance(v, torch.Tensor) else v) for k, v in payload.items()}
