"""Bit packers, compact3 payload builder and block Golomb-Rice encoder.

These produce, bit for bit, the tensors the TriS-MoE reference stores for one quantized
expert projection (``utils/pack_utils.py:6-125`` and
``QuantLinear._pack_block_gr_gmap_tensor``, ``qlinear_cuda.py:3793-3859``) and the
E-stacked dictionaries its grouped runtime consumes
(``build_grouped_precomputed_payload``, ``qlinear_cuda.py:1512-1636``).  They are host-side
data preparation (numpy); the GR bit stream itself is written by the C encoder in
``csrc/abi.cpp``.

Layout reminders: a packed word holds 32 consecutive K positions of one output, LSB =
lowest K; sparse planes keep only the active columns, in ascending order; ``*_prefix[p]``
counts the active columns below column ``32*p``.
"""
from __future__ import annotations

import ctypes as C
import math
from typing import Iterable, Sequence

import numpy as np
import torch

from . import _native

BLOCK_GR_PACKED_ROWS = 2
BLOCK_GR_TILE_OUT = 64
BLOCK_GR_WORDS_PER_BLOCK = 128
BLOCK_GR_META_RAW_FLAG = 16
BLOCK_GR_META_ONE_COUNT_SHIFT = 8
BLOCK_GR_MAX_K = 7


def _np_bool(x) -> np.ndarray:
    if isinstance(x, torch.Tensor):
        x = x.detach().cpu().numpy()
    return np.ascontiguousarray(np.asarray(x).astype(bool))


def _pack_last_axis(bits: np.ndarray) -> np.ndarray:
    """bool [..., n] -> uint32 [..., ceil(n/32)], bit j of word w = bits[..., 32*w + j]."""
    n = bits.shape[-1]
    pad = (-n) % 32
    if pad:
        bits = np.concatenate([bits, np.zeros(bits.shape[:-1] + (pad,), dtype=bool)], axis=-1)
    packed = np.packbits(bits, axis=-1, bitorder="little")
    return np.ascontiguousarray(packed).view("<u4")


def _as_i32_tensor(words: np.ndarray, device) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(words).view(np.int32).copy()).to(device)


def pack_bool_vector(values, device="cpu") -> torch.Tensor:
    """``pack_bool_vector`` (utils/pack_utils.py:6-16): bool [n] -> int32 [ceil(n/32)]."""
    bits = _np_bool(values).reshape(-1)
    if bits.size == 0:
        return torch.zeros((0,), dtype=torch.int32, device=device)
    return _as_i32_tensor(_pack_last_axis(bits), device)


def pack_bool_matrix(matrix, device="cpu") -> torch.Tensor:
    """``pack_bool_matrix`` (utils/pack_utils.py:19-29): bool [O, K] -> int32 [ceil(K/32), O]."""
    bits = _np_bool(matrix)
    if bits.ndim != 2:
        raise ValueError("pack_bool_matrix expects a 2-D matrix")
    if bits.shape[1] == 0:
        return torch.zeros((0, bits.shape[0]), dtype=torch.int32, device=device)
    return _as_i32_tensor(_pack_last_axis(bits).T, device)


def pack_sparse_bool_matrix(matrix, active_cols, device="cpu") -> torch.Tensor:
    """Packs only the columns flagged in ``active_cols`` (utils/pack_utils.py:32-36)."""
    bits = _np_bool(matrix)
    active = _np_bool(active_cols).reshape(-1)
    if active.size == 0 or not active.any():
        return torch.zeros((0, bits.shape[0]), dtype=torch.int32, device=device)
    return pack_bool_matrix(bits[:, active], device)


def build_sparse_bit_prefix(active_cols, device="cpu") -> torch.Tensor:
    """prefix[p] = active columns below 32*p, length ceil(n/32)+1 (utils/pack_utils.py:39-52)."""
    active = _np_bool(active_cols).reshape(-1)
    rows = math.ceil(active.size / 32)
    prefix = np.zeros((rows + 1,), dtype=np.int32)
    if rows:
        pad = (-active.size) % 32
        padded = np.concatenate([active, np.zeros((pad,), dtype=bool)]) if pad else active
        prefix[1:] = np.cumsum(padded.reshape(rows, 32).sum(axis=1))
    return torch.from_numpy(prefix).to(device)


def _half_bits(x) -> np.ndarray:
    if isinstance(x, torch.Tensor):
        x = x.detach().cpu().to(torch.float16).numpy()
    return np.ascontiguousarray(np.asarray(x, dtype=np.float16)).view(np.uint16).astype(np.uint64)


def pack_half4_words(first, second, third, fourth, device="cpu") -> torch.Tensor:
    """fp16 bit patterns at bits 0/16/32/48 of an int64 (utils/pack_utils.py:55-64)."""
    w = _half_bits(first) | (_half_bits(second) << np.uint64(16)) | (_half_bits(third) << np.uint64(32)) | (
        _half_bits(fourth) << np.uint64(48)
    )
    return torch.from_numpy(w.view(np.int64).copy()).to(device)


def dense_gmap_words(g_map_non_salient, c_map, device="cpu") -> torch.Tensor:
    """Dense packed g_map [ceil(K/32), O] with salient columns cleared: the block-GR input
    (``_restore_dense_bool_matrix_from_sparse``, qlinear_cuda.py:3682-3700)."""
    g = _np_bool(g_map_non_salient)
    c = _np_bool(c_map).reshape(-1)
    return pack_bool_matrix(g & ~c[None, :], device)


def build_compact3_packed_payload(
    *,
    device="cpu",
    mode="expert_compact3",
    b1,
    b2,
    g_map_non_salient,
    c_map,
    g_idx,
    scales_s_r1,
    scales_s_r2,
    scales_ns_d_r1,
    scales_ns_nd_r1,
    scales_s_c1,
    scales_s_c2,
    scales_ns_d_c1,
    scales_ns_nd_c1,
) -> dict:
    """Per-expert payload with the keys and dtypes of ``build_compact3_packed_payload``
    (utils/pack_utils.py:67-125, without null-space vector folding)."""
    c = _np_bool(c_map).reshape(-1)
    return {
        "mode": mode,
        "qweight1": pack_bool_matrix(b1, device),
        "qweight2_sparse": pack_sparse_bool_matrix(b2, c, device),
        "qweight2_sparse_prefix": build_sparse_bit_prefix(c, device),
        "q_gmap_sparse": pack_sparse_bool_matrix(g_map_non_salient, ~c, device),
        "q_gmap_sparse_prefix": build_sparse_bit_prefix(~c, device),
        "c_map_packed": pack_bool_vector(c, device),
        "g_idx": torch.as_tensor(np.asarray(g_idx), dtype=torch.int32).to(device).contiguous(),
        "row_pack3": pack_half4_words(scales_s_r1, scales_s_r2, scales_ns_d_r1, scales_ns_nd_r1, device),
        "col_pack3": pack_half4_words(scales_s_c1, scales_s_c2, scales_ns_d_c1, scales_ns_nd_c1, device),
    }


def block_gr_encode(dense_words: torch.Tensor, force_raw: bool = False, k_min: int = 0, k_max: int = 7):
    """Block Golomb-Rice code of a dense packed g_map ``[pr, O]`` int32.

    Returns ``(words, offsets, meta)`` int32 CPU tensors exactly as
    ``QuantLinear._pack_block_gr_gmap_tensor`` (qlinear_cuda.py:3793-3859) would; ``k_min`` /
    ``k_max`` bound the per-block search of the Rice parameter as the reference exporter's
    ``pack_block_gr_gmap_tensor(fixed_k, k_min, k_max)`` does (tools/rewrite_runtime_min_checkpoint.py:252-347).
    """
    dense = dense_words.detach().to("cpu", torch.int32).contiguous()
    if dense.numel() == 0:
        empty = torch.zeros((0,), dtype=torch.int32)
        return empty, empty.clone(), empty.clone()
    pr, out = int(dense.shape[0]), int(dense.shape[1])
    nblk = math.ceil(pr / BLOCK_GR_PACKED_ROWS) * math.ceil(out / BLOCK_GR_TILE_OUT)
    words = torch.empty((nblk * BLOCK_GR_WORDS_PER_BLOCK,), dtype=torch.int32)
    offsets = torch.empty((nblk + 1,), dtype=torch.int32)
    meta = torch.empty((nblk,), dtype=torch.int32)
    count = C.c_int64(0)
    lib = _native.load()
    st = lib.tris_block_gr_encode_host_k(
        dense.data_ptr(), pr, out, int(bool(force_raw)), int(k_min), int(k_max), words.data_ptr(), words.numel(),
        offsets.data_ptr(), meta.data_ptr(), C.byref(count),
    )
    _native.check(st, "block_gr_encode")
    return words[: count.value].clone(), offsets, meta


def _pad_rows(t: torch.Tensor, rows: int) -> torch.Tensor:
    if t.shape[0] == rows:
        return t
    pad = torch.zeros((rows - t.shape[0],) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
    return torch.cat([t, pad], dim=0)


def stack_expert_payloads(
    payloads: Sequence[dict],
    device="cpu",
    *,
    use_block_gr: bool = True,
    keep_sparse_gmap: bool = True,
    output_scale: torch.Tensor | None = None,
    bias: torch.Tensor | None = None,
) -> dict:
    """E-stacked grouped payload with the keys of ``build_grouped_precomputed_payload``
    (qlinear_cuda.py:1512-1636): sparse planes zero-padded on the row dim to the max over
    experts, GR word streams zero-padded to the longest stream."""
    if len(payloads) == 0:
        raise ValueError("need at least one expert payload")
    dev = torch.device(device)
    out_features = int(payloads[0]["qweight1"].shape[1])
    rows2 = max(int(p["qweight2_sparse"].shape[0]) for p in payloads)
    rowsg = max(int(p["q_gmap_sparse"].shape[0]) for p in payloads)

    def cat(key, rows=None):
        ts = [p[key].to("cpu") for p in payloads]
        if rows is not None:
            ts = [_pad_rows(t.reshape(t.shape[0], out_features) if t.numel() else t.reshape(0, out_features), rows) for t in ts]
        return torch.stack(ts, dim=0).contiguous().to(dev)

    stacked = {
        "is_compact3": True,
        "qweight1": cat("qweight1"),
        "qweight2_sparse": cat("qweight2_sparse", rows2),
        "qweight2_sparse_prefix": cat("qweight2_sparse_prefix"),
        "q_gmap_sparse_prefix": cat("q_gmap_sparse_prefix"),
        "c_map": torch.stack([p["c_map_packed"].to("cpu") for p in payloads]).contiguous().to(dev),
        "g_idx": cat("g_idx"),
        "col_pack3": cat("col_pack3"),
        "row_pack3": cat("row_pack3"),
    }
    if keep_sparse_gmap:
        stacked["q_gmap_sparse"] = cat("q_gmap_sparse", rowsg)
    else:
        stacked["q_gmap_sparse"] = torch.zeros((len(payloads), 0, out_features), dtype=torch.int32, device=dev)
    if use_block_gr:
        streams = []
        for p in payloads:
            if "q_gmap_gr_words" in p:
                streams.append((p["q_gmap_gr_words"], p["q_gmap_gr_offsets"], p["q_gmap_gr_meta"]))
            else:
                rank = int(p["g_idx"].shape[0])
                streams.append(block_gr_encode(restore_dense_gmap_words(p, rank)))
        max_words = max(int(s[0].numel()) for s in streams)
        words = torch.zeros((len(streams), max_words), dtype=torch.int32)
        for i, s in enumerate(streams):
            words[i, : s[0].numel()] = s[0].to("cpu")
        stacked["q_gmap_gr_words"] = words.to(dev)
        stacked["q_gmap_gr_offsets"] = torch.stack([s[1].to("cpu") for s in streams]).contiguous().to(dev)
        stacked["q_gmap_gr_meta"] = torch.stack([s[2].to("cpu") for s in streams]).contiguous().to(dev)
    else:
        for key in ("q_gmap_gr_words", "q_gmap_gr_offsets", "q_gmap_gr_meta"):
            stacked[key] = torch.empty((0, 0), dtype=torch.int32, device=dev)
    stacked["compact3_use_block_gr"] = bool(use_block_gr)
    if output_scale is None:
        output_scale = torch.ones((len(payloads), out_features), dtype=torch.float16)
    stacked["output_scale"] = output_scale.to(dev, torch.float16).contiguous()
    stacked["has_output_scale"] = not bool(torch.all(stacked["output_scale"] == 1).item())
    stacked["bias"] = None if bias is None else bias.to(dev, torch.float16).contiguous()
    stacked["has_bias"] = bias is not None
    return stacked


def unpack_bool_matrix(packed: torch.Tensor, ncols: int) -> np.ndarray:
    """int32 [rows, O] -> bool [O, ncols] (inverse of :func:`pack_bool_matrix`)."""
    words = packed.detach().cpu().contiguous().numpy().view("<u4")
    if words.size == 0:
        return np.zeros((words.shape[1] if words.ndim == 2 else 0, ncols), dtype=bool)
    bits = np.unpackbits(np.ascontiguousarray(words.T).view(np.uint8), axis=-1, bitorder="little")
    return bits[:, :ncols].astype(bool)


def restore_dense_gmap_words(payload: dict, rank: int) -> torch.Tensor:
    """Dense packed g_map of one expert rebuilt from its sparse plane
    (``_restore_dense_bool_matrix_from_sparse``, qlinear_cuda.py:3682-3700)."""
    c_words = payload["c_map_packed"] if "c_map_packed" in payload else payload["c_map"]
    c = np.unpackbits(c_words.detach().cpu().contiguous().numpy().view(np.uint8), bitorder="little")[:rank].astype(bool)
    out_features = int(payload["qweight1"].shape[1])
    dense = np.zeros((out_features, rank), dtype=bool)
    n_inactive = int((~c).sum())
    if n_inactive and payload["q_gmap_sparse"].numel():
        dense[:, ~c] = unpack_bool_matrix(payload["q_gmap_sparse"], n_inactive)
    return pack_bool_matrix(dense)


def payload_nbytes(payload: dict) -> int:
    """Bytes of every tensor in a payload dict (for reporting)."""
    return sum(v.numel() * v.element_size() for v in payload.values() if isinstance(v, torch.Tensor))
