"""Grouped compact3 operators with the names and argument order of the reference module
``auto_gptq/nn_modules/qlinear/qlinear_cuda.py`` (TriS-MoE tree), running on the
trismoe_b200 CUDA library.

Covered surface: ``build_grouped_precomputed_payload`` (qlinear_cuda.py:1512),
``build_grouped_route`` (:1301), ``run_grouped_structured_expert_forward`` (:2131),
``run_grouped_structured_expert_pair_forward`` (:2338), ``compute_shared_hidden`` (:4454,
fp16 backbone branch) and ``ExpertSharedMatrix`` (:2787, fp16 ``shared_sv`` only).

Error behaviour follows the reference wrappers: shape/dtype mismatches return ``None``
(the reference's "kernel unavailable" signal); anything the library itself rejects, a
missing library, or tensors that are not on a CUDA device raise ``RuntimeError`` - there
is no CPU or PyTorch fallback to fall back to.
"""
from __future__ import annotations

import ctypes as C
import math
from typing import Optional, Sequence

import torch

from . import _native, envflags
from ._native import TrisProjView, TrisRouteView
from .formats import stack_expert_payloads

TRIS_COMPACT3_KERNEL_ABI_VERSION = 2
GROUPED_SEGMENT_M_TILE = 4
DEFAULT_GR_SUBSTREAMS = 32
# column orders of activation rows (TRIS_OUT_F16 / _PAIR_INTERLEAVED / _LANE_ORDER of the C header)
HIDDEN_ROW_MAJOR, HIDDEN_PAIR_INTERLEAVED, HIDDEN_LANE_ORDER = 0, 2, 3


def _stream_ptr(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    if t is None or t.numel() == 0:
        return None
    return t.data_ptr()


def _payload_flag(payload: dict, key: str, default: bool = False) -> bool:
    """Boolean payload entry that may be a Python bool or a 0-dim / 1-element tensor, as sidecars
    store scalars (``_payload_flag``, qlinear_cuda.py:310-316)."""
    value = payload.get(key, default)
    if isinstance(value, torch.Tensor):
        if value.numel() == 0:
            return default
        return bool(value.reshape(-1)[0].item())
    return bool(value)


def _payload_has_output_scale(payload: dict) -> bool:
    """``_payload_has_output_scale`` (qlinear_cuda.py:318-321): the flag when the payload carries one,
    otherwise derived from the tensor (anything but exact ones is a real scale)."""
    if "has_output_scale" in payload:
        return _payload_flag(payload, "has_output_scale", False)
    scale = payload.get("output_scale")
    if not isinstance(scale, torch.Tensor) or scale.numel() == 0:
        return False
    return not bool(torch.all(scale == 1).item())


def _payload_has_bias(payload: dict) -> bool:
    """The ``has_bias`` flag when present; a payload without the key has a bias exactly when it
    carries a non-empty bias tensor (build_grouped_precomputed_payload, qlinear_cuda.py:1543-1553)."""
    if "has_bias" in payload:
        return _payload_flag(payload, "has_bias", False)
    bias = payload.get("bias")
    return isinstance(bias, torch.Tensor) and bias.numel() > 0


def _use_block_gr(payload: dict) -> bool:
    """Which g_map encoding the kernels read: the block-GR streams when the payload has them and
    ``TRIS_COMPACT3_BLOCK_GR`` is not switched off (``_compact3_block_gr_enabled``,
    qlinear_cuda.py:235-240); with the switch off, the sparse planes if the payload still has them."""
    offsets = payload.get("q_gmap_gr_offsets")
    has_gr = _payload_flag(payload, "compact3_use_block_gr", False) and isinstance(offsets, torch.Tensor) and offsets.numel() > 0
    if has_gr and not envflags.compact3_block_gr_enabled():
        sparse = payload.get("q_gmap_sparse")
        if isinstance(sparse, torch.Tensor) and sparse.numel() > 0:
            return False
    return has_gr


def _ensure(t: torch.Tensor, dtype, device) -> torch.Tensor:
    if t.dtype != dtype or t.device != device or not t.is_contiguous():
        t = t.to(device=device, dtype=dtype).contiguous()
    return t


# ---------------------------------------------------------------------------------------
# payloads
# ---------------------------------------------------------------------------------------
def prepare_grouped_payload(payload: dict, device=None, gr_substreams: int = DEFAULT_GR_SUBSTREAMS,
                            tile_records: bool = True) -> dict:
    """Moves an E-stacked payload to ``device`` and derives what the kernels need beyond the
    reference tensors: the per-packed-row group table (validating ``g_idx`` as
    ``prepare_compact3_k64_groups`` does, qlinear_cuda.py:364-407) and, for block-GR
    payloads, the sub-stream index (validating offsets/meta) and the tile-major records the
    grouped kernels read (one contiguous piece per expert, 64 outputs and 256 columns, so a
    tile arrives with one bulk copy; ``tile_records=False`` skips them and the kernels gather
    the tile from the E-stacked tensors).  Runs once at load time and synchronises to read the
    validation status.  Idempotent."""
    if payload.get("_tris_prepared") and (device is None or payload["qweight1"].device == torch.device(device)):
        return payload
    lib = _native.load()
    dev = torch.device(device) if device is not None else payload["qweight1"].device
    if dev.type != "cuda":
        raise RuntimeError("trismoe_b200 prepare_grouped_payload: payloads must live on a CUDA device")
    i32 = torch.int32
    for key in ("qweight1", "qweight2_sparse", "qweight2_sparse_prefix", "q_gmap_sparse", "q_gmap_sparse_prefix",
                "q_gmap_gr_words", "q_gmap_gr_offsets", "q_gmap_gr_meta", "c_map", "g_idx"):
        if isinstance(payload.get(key), torch.Tensor):
            payload[key] = _ensure(payload[key], i32, dev)
    for key in ("col_pack3", "row_pack3"):
        payload[key] = _ensure(payload[key], torch.int64, dev)
    for key in ("output_scale", "bias"):
        if isinstance(payload.get(key), torch.Tensor):
            payload[key] = _ensure(payload[key], torch.float16, dev)
    qw1 = payload["qweight1"]
    if qw1.dim() != 3:
        raise RuntimeError("trismoe_b200: qweight1 must be [experts, packed_rows, out_features]")
    E, pr, O = (int(s) for s in qw1.shape)
    rank = int(payload["g_idx"].shape[-1])
    row_pack = payload["row_pack3"]
    G = int(row_pack.shape[2]) if row_pack.dim() == 3 else 1
    if pr != math.ceil(rank / 32) or tuple(payload["col_pack3"].shape) != (E, rank) or tuple(row_pack.shape[:2]) != (E, O):
        raise RuntimeError("trismoe_b200: inconsistent compact3 payload shapes")
    if payload.get("_tris_derived_from_checkpoint") and _adopt_stored_derived(payload, dev, E, pr, O, rank, G):
        payload["_tris_prepared"] = True
        payload["_tris_view"] = _build_view(payload, need_index=True)
        return payload
    status = torch.zeros((2,), dtype=i32, device=dev)
    stream = _stream_ptr(dev)
    with torch.cuda.device(dev):
        groups = torch.empty((E, pr), dtype=i32, device=dev)
        _native.check(
            lib.tris_build_row_groups(payload["g_idx"].data_ptr(), E, rank, G, groups.data_ptr(), status[0:].data_ptr(), stream),
            "build_row_groups",
        )
        payload["_tris_packed_row_group"] = groups
        payload["_tris_dims"] = (E, O, rank, G)
        use_gr = _use_block_gr(payload)
        payload["_tris_gr_index"] = None
        payload["_tris_gr_substreams"] = 0
        if use_gr:
            nblk = math.ceil(pr / 2) * math.ceil(O / 64)
            if tuple(payload["q_gmap_gr_offsets"].shape) != (E, nblk + 1) or tuple(payload["q_gmap_gr_meta"].shape) != (E, nblk):
                raise RuntimeError("trismoe_b200: block-GR offsets/meta have the wrong shape")
            index = torch.empty((E, nblk, gr_substreams), dtype=i32, device=dev)
            payload["_tris_gr_substreams"] = int(gr_substreams)
            view = _build_view(payload, need_index=False)
            _native.check(
                lib.tris_block_gr_build_index(C.byref(view), index.data_ptr(), gr_substreams, status[1:].data_ptr(), stream),
                "block_gr_build_index",
            )
            payload["_tris_gr_index"] = index
    st = status.cpu().tolist()
    for key in ("_tris_tile_records", "_tris_tile_desc", "_tris_col_records"):
        payload[key] = None
    payload["_tris_tile_meta"] = (0, 0, 0)
    if st[0] != 0:
        raise RuntimeError("trismoe_b200: g_idx is not constant inside every 32-column word (unsupported layout)")
    if st[1] != 0:
        raise RuntimeError("trismoe_b200: corrupt block-GR stream (offsets/meta/bit stream failed validation)")
    if use_gr and tile_records and int(gr_substreams) == 32:
        _build_tile_records(payload, lib, dev)
    payload["_tris_prepared"] = True
    payload["_tris_view"] = _build_view(payload, need_index=True)
    return payload


def _adopt_stored_derived(payload: dict, dev, E: int, pr: int, O: int, rank: int, G: int) -> bool:
    """Uses the derived tensors a checkpoint exporter stored next to the payload (sub-stream index,
    packed-row groups, tile records) instead of rebuilding them; False when their shapes do not fit
    this payload (then they are dropped and everything is rebuilt and re-validated)."""
    nblk = math.ceil(pr / 2) * math.ceil(O / 64)
    count = E * math.ceil(O / 64) * math.ceil(pr / 8)
    idx, grp, rec, desc, col = (payload.get(k) for k in ("_tris_gr_index", "_tris_packed_row_group", "_tris_tile_records",
                                                        "_tris_tile_desc", "_tris_col_records"))
    meta = payload.get("_tris_tile_meta")
    ok = all(isinstance(t, torch.Tensor) for t in (idx, grp, rec, desc, col)) and isinstance(meta, tuple) and len(meta) == 3
    ok = ok and tuple(idx.shape) == (E, nblk, 32) and tuple(grp.shape) == (E, pr) and tuple(desc.shape) == (count + 1, 2)
    ok = ok and col.numel() == E * math.ceil(pr / 8) * int(meta[0]) and rec.dtype == torch.uint8 and col.dtype == torch.uint8
    if ok:
        last = desc[count - 1].to(torch.int64)
        ok = int((last[0] & 0xFFFFFFFF) * 16 + (last[1] & 0xFFFFFFFF)) <= rec.numel()
    if not ok:
        for k in ("_tris_gr_index", "_tris_packed_row_group", "_tris_tile_records", "_tris_tile_desc", "_tris_col_records",
                  "_tris_tile_meta", "_tris_derived_from_checkpoint"):
            payload.pop(k, None)
        return False
    payload["_tris_gr_index"] = idx.to(dev, torch.int32).contiguous()
    payload["_tris_packed_row_group"] = grp.to(dev, torch.int32).contiguous()
    payload["_tris_tile_records"] = rec.to(dev).contiguous()
    payload["_tris_tile_desc"] = desc.to(dev, torch.int32).contiguous()
    payload["_tris_col_records"] = col.to(dev).contiguous()
    payload["_tris_gr_substreams"] = 32
    payload["_tris_dims"] = (E, O, rank, G)
    return True


def _build_tile_records(payload: dict, lib, dev) -> None:
    """Plans and fills the tile-major records of a block-GR payload (``tris_tile_records_plan`` /
    ``tris_tile_records_build``) into tensors kept in the payload dict."""
    view = _build_view(payload, need_index=True)
    stream = _stream_ptr(dev)
    with torch.cuda.device(dev):
        count = int(lib.tris_tile_record_count(C.byref(view)))
        desc = torch.empty((count + 1, 2), dtype=torch.int32, device=dev)
        info = torch.zeros((4,), dtype=torch.int64, device=dev)
        _native.check(lib.tris_tile_records_plan(C.byref(view), desc.data_ptr(), info.data_ptr(), stream), "tile_records_plan")
        total, max_rec, max_sal, _ = (int(v) for v in info.cpu().tolist())
        col_total = int(lib.tris_col_record_bytes(C.byref(view), max_sal))
        records = torch.empty((max(total, 16),), dtype=torch.uint8, device=dev)
        cols = torch.empty((max(col_total, 16),), dtype=torch.uint8, device=dev)
        _native.check(lib.tris_tile_records_build(C.byref(view), desc.data_ptr(), records.data_ptr(), cols.data_ptr(),
                                                  max_sal, stream), "tile_records_build")
    payload["_tris_tile_records"] = records
    payload["_tris_tile_desc"] = desc
    payload["_tris_col_records"] = cols
    payload["_tris_tile_meta"] = (64 + 1024 + 256 * max_sal, max_rec, max_sal)


def _build_view(payload: dict, need_index: bool) -> TrisProjView:
    E, O, rank, G = payload["_tris_dims"]
    use_gr = _use_block_gr(payload)
    v = TrisProjView()
    v.num_experts, v.out_features, v.rank, v.num_groups = E, O, rank, G
    v.sign2_rows = int(payload["qweight2_sparse"].shape[1]) if payload["qweight2_sparse"].dim() == 3 else 0
    gsp = payload.get("q_gmap_sparse")
    v.gmap_sparse_rows = int(gsp.shape[1]) if isinstance(gsp, torch.Tensor) and gsp.dim() == 3 else 0
    v.gr_max_words = int(payload["q_gmap_gr_words"].shape[1]) if use_gr else 0
    v.use_block_gr = int(use_gr)
    v.qweight1 = _ptr(payload["qweight1"])
    v.qweight2_sparse = _ptr(payload["qweight2_sparse"])
    v.qweight2_sparse_prefix = _ptr(payload["qweight2_sparse_prefix"])
    v.q_gmap_sparse = _ptr(gsp) if isinstance(gsp, torch.Tensor) else None
    v.q_gmap_sparse_prefix = _ptr(payload["q_gmap_sparse_prefix"])
    v.q_gmap_gr_words = _ptr(payload["q_gmap_gr_words"]) if use_gr else None
    v.q_gmap_gr_offsets = _ptr(payload["q_gmap_gr_offsets"]) if use_gr else None
    v.q_gmap_gr_meta = _ptr(payload["q_gmap_gr_meta"]) if use_gr else None
    v.c_map = _ptr(payload["c_map"])
    v.g_idx = _ptr(payload["g_idx"])
    v.col_pack3 = _ptr(payload["col_pack3"])
    v.row_pack3 = _ptr(payload["row_pack3"])
    v.output_scale = _ptr(payload.get("output_scale")) if _payload_has_output_scale(payload) else None
    v.bias = _ptr(payload.get("bias")) if _payload_has_bias(payload) else None
    v.gr_index = _ptr(payload.get("_tris_gr_index")) if need_index else None
    v.gr_substreams = int(payload.get("_tris_gr_substreams", 0))
    v.packed_row_group = _ptr(payload["_tris_packed_row_group"])
    slot = payload.get("_tris_gmap_slot")
    v.gmap_slot = _ptr(slot) if isinstance(slot, torch.Tensor) else None
    if need_index and isinstance(payload.get("_tris_tile_records"), torch.Tensor):
        v.tile_records = payload["_tris_tile_records"].data_ptr()
        v.tile_desc = payload["_tris_tile_desc"].data_ptr()
        v.col_records = payload["_tris_col_records"].data_ptr()
        v.col_record_bytes, v.max_record_bytes, v.max_sal_words = payload["_tris_tile_meta"]
    return v


def grouped_hidden_layout(payload_a: dict, payload_b: Optional[dict], num_rows: int, num_segments: int,
                          max_rows_per_segment: int) -> int:
    """Column order (``HIDDEN_*``) in which the grouped operators read activation rows fastest for
    these payloads and a route of that size (``tris_grouped_hidden_layout``): pass it to
    ``compute_shared_hidden(..., layout=...)`` and as ``route["_hidden_layout"]``."""
    lib = _native.load()
    va = proj_view(payload_a)
    vb = proj_view(payload_b) if payload_b is not None else None
    return int(lib.tris_grouped_hidden_layout(C.byref(va), None if vb is None else C.byref(vb), int(num_rows),
                                              int(num_segments), int(max_rows_per_segment)))


HIDDEN_LAYOUT_ROUTE_FLAG = {0: 0, 2: 1, 3: 2}  # HIDDEN_* -> TRIS_ROUTE_HIDDEN_* bit


def proj_view(payload: dict) -> TrisProjView:
    """ctypes view of a prepared payload (rebuilt when staging swaps the bitmap buffer)."""
    if not payload.get("_tris_prepared"):
        prepare_grouped_payload(payload)
    if payload.get("_tris_view_dirty"):
        payload["_tris_view"] = _build_view(payload, need_index=True)
        payload["_tris_view_dirty"] = False
    return payload["_tris_view"]


def build_grouped_precomputed_payload(modules, device, dtype=torch.float16):
    """``build_grouped_precomputed_payload`` (qlinear_cuda.py:1512-1636).  ``modules`` is a
    sequence of per-expert payload dicts (the output of ``build_compact3_packed_payload``)
    or of objects carrying one as ``.compact3_payload``.  Returns ``None`` for an empty
    list, like the reference."""
    if len(modules) == 0:
        return None
    if dtype != torch.float16:
        return None
    dicts = [m if isinstance(m, dict) else getattr(m, "compact3_payload") for m in modules]
    stacked = stack_expert_payloads(dicts, device="cpu", use_block_gr=True)
    return prepare_grouped_payload(stacked, device)


def decode_block_gr_gmap(payload: dict) -> torch.Tensor:
    """Dense packed g_map ``[E, pr, O]`` int32 decoded on the GPU from the block-GR stream
    (the shared-memory image of ``decode_block_gr_block``, TriSMoE_cuda_kernel.cu:426-479)."""
    lib = _native.load()
    view = proj_view(payload)
    dev = payload["qweight1"].device
    E, O, rank, _ = payload["_tris_dims"]
    out = torch.empty((E, math.ceil(rank / 32), O), dtype=torch.int32, device=dev)
    with torch.cuda.device(dev):
        _native.check(lib.tris_block_gr_decode(C.byref(view), out.data_ptr(), _stream_ptr(dev)), "block_gr_decode")
    return out


def dequantize_grouped_payload(payload: dict) -> torch.Tensor:
    """fp16 weights ``[E, O, r]`` from the kernels' own unpack path
    (``_dequantize_compact3_matrix``, qlinear_cuda.py:4200-4236)."""
    lib = _native.load()
    view = proj_view(payload)
    dev = payload["qweight1"].device
    E, O, rank, _ = payload["_tris_dims"]
    out = torch.empty((E, O, rank), dtype=torch.float16, device=dev)
    with torch.cuda.device(dev):
        _native.check(lib.tris_compact3_dequantize(C.byref(view), out.data_ptr(), _stream_ptr(dev)), "compact3_dequantize")
    return out


# ---------------------------------------------------------------------------------------
# route
# ---------------------------------------------------------------------------------------
def _empty_grouped_route(device):
    z_long = torch.empty((0,), device=device, dtype=torch.long)
    z_i32 = torch.empty((0,), device=device, dtype=torch.int32)
    zero = torch.zeros((1,), device=device, dtype=torch.int32)
    return {
        "perm": z_long, "grouped_token_indices": z_long, "grouped_slots": z_long,
        "grouped_expert_ids": z_i32, "expert_ids": z_i32, "segment_offsets": zero, "problem_offsets": zero.clone(),
        "total_problem_tiles": torch.zeros((1,), dtype=torch.int64), "total_problem_tiles_host": 0,
        "_row_of_flat": z_i32.clone(), "_max_rows_per_segment": 0,
    }


def build_grouped_route(selected_experts: torch.Tensor, num_experts: int, m_tile: int = GROUPED_SEGMENT_M_TILE):
    """``build_grouped_route`` (qlinear_cuda.py:1301-1378): same keys, dtypes and sizes.
    Rows inside a segment are in ascending (token, slot) order.  Reads the number of active
    experts back to size the tensors (the reference does the same, TriSMoE_cuda.cpp:781)."""
    if selected_experts.dim() != 2:
        return None
    device = selected_experts.device
    if m_tile <= 0:
        return _empty_grouped_route(device)
    _native.require_cuda(selected_experts, "build_grouped_route")
    T, k = (int(s) for s in selected_experts.shape)
    R = T * k
    if R == 0:
        return _empty_grouped_route(device)
    lib = _native.load()
    sel = selected_experts.to(torch.int32).contiguous()
    E = int(num_experts)
    scratch_n = ((R + 2047) // 2048) * E  # scratch that lets the sort of >= 8192 rows run on several CTAs
    buf = torch.empty((4 * R + 3 * E + 2 + 2 + scratch_n,), dtype=torch.int32, device=device)
    perm, tok, slot, rof = (buf[i * R:(i + 1) * R] for i in range(4))
    base = 4 * R
    expert_ids = buf[base: base + E]
    seg = buf[base + E: base + 2 * E + 1]
    prob = buf[base + 2 * E + 1: base + 3 * E + 2]
    counts = buf[base + 3 * E + 2: base + 3 * E + 4]
    with torch.cuda.device(device):
        _native.check(
            lib.tris_build_grouped_route_ex(sel.data_ptr(), 1, 0, T, k, E, int(m_tile), perm.data_ptr(), tok.data_ptr(),
                                            slot.data_ptr(), rof.data_ptr(), expert_ids.data_ptr(), seg.data_ptr(),
                                            prob.data_ptr(), counts.data_ptr(), buf[base + 3 * E + 4:].data_ptr(),
                                            4 * scratch_n, _stream_ptr(device)),
            "build_grouped_route",
        )
    nseg, tiles = (int(v) for v in counts.cpu().tolist())
    expert_ids = expert_ids[:nseg].contiguous()
    seg = seg[: nseg + 1].contiguous()
    lengths = (seg[1:] - seg[:-1])
    return {
        "perm": perm.to(torch.long),
        "grouped_token_indices": tok.to(torch.long),
        "grouped_slots": slot.to(torch.long),
        "grouped_expert_ids": torch.repeat_interleave(expert_ids, lengths, output_size=R).contiguous(),
        "expert_ids": expert_ids,
        "segment_offsets": seg,
        "problem_offsets": prob[: nseg + 1].contiguous(),
        "total_problem_tiles": torch.tensor([tiles], dtype=torch.int64),
        "total_problem_tiles_host": tiles,
        "_row_of_flat": rof,
        "_max_rows_per_segment": T,
    }


def _coerce_grouped_route(route_or_lengths, device, expert_ids=None):
    if isinstance(route_or_lengths, dict):
        return route_or_lengths
    lengths = torch.as_tensor(route_or_lengths, dtype=torch.long).reshape(-1)
    if lengths.numel() == 0 or bool((lengths < 0).any()):
        return None
    ids = torch.arange(lengths.numel(), dtype=torch.int32) if expert_ids is None else torch.as_tensor(expert_ids, dtype=torch.int32).reshape(-1)
    if ids.numel() != lengths.numel():
        return None
    keep = lengths > 0
    lengths, ids = lengths[keep], ids[keep]
    seg = torch.cat([torch.zeros(1, dtype=torch.long), torch.cumsum(lengths, 0)]).to(torch.int32)
    return {
        "expert_ids": ids.to(device), "segment_offsets": seg.to(device),
        "_max_rows_per_segment": int(lengths.max().item()) if lengths.numel() else 0,
    }


def _route_view(route: dict, num_rows: int, keep: list) -> TrisRouteView:
    rv = TrisRouteView()
    ids = route["expert_ids"]
    seg = route["segment_offsets"]
    if ids.dtype != torch.int32 or not ids.is_contiguous():
        ids = ids.to(torch.int32).contiguous()
    if seg.dtype != torch.int32 or not seg.is_contiguous():
        seg = seg.to(torch.int32).contiguous()
    keep += [ids, seg]
    rv.expert_ids = ids.data_ptr() if ids.numel() else None
    rv.segment_offsets = seg.data_ptr()
    rv.num_segments_dev = None
    rv.num_segments = int(ids.numel())
    rv.num_rows = int(num_rows)
    rv.max_rows_per_segment = int(route.get("_max_rows_per_segment", 0) or 0)
    rv.row_gather = None
    rv.status_dev = None
    rv.flags = 0
    # extensions of the route dict (no reference counterpart): "_row_gather" [R] int32 makes grouped
    # row i read activation row gather[i] (so the caller need not index_select the backbone output),
    # "_hidden_layout" names the column order of the activation rows (HIDDEN_ROW_MAJOR by default;
    # HIDDEN_LANE_ORDER / HIDDEN_PAIR_INTERLEAVED = what compute_shared_hidden(..., layout=...) wrote)
    gather = route.get("_row_gather")
    if isinstance(gather, torch.Tensor):
        if gather.dtype != torch.int32 or not gather.is_contiguous():
            gather = gather.to(torch.int32).contiguous()
        keep.append(gather)
        rv.row_gather = gather.data_ptr()
    rv.flags = HIDDEN_LAYOUT_ROUTE_FLAG[int(route.get("_hidden_layout", HIDDEN_ROW_MAJOR))]
    scale = route.get("_hidden_col_scale")  # fp16 [rank]: the input scale vector of an ordinary compact3 linear
    if isinstance(scale, torch.Tensor):
        if scale.dtype != torch.float16 or not scale.is_contiguous():
            scale = scale.to(torch.float16).contiguous()
        keep.append(scale)
        rv.hidden_col_scale = scale.data_ptr()
    # extension of the route dict (no reference counterpart): "_out_row_scatter" [R] int32 sends the
    # result of grouped row i to output row scatter[i] (a negative entry drops it)
    scatter = route.get("_out_row_scatter")
    if isinstance(scatter, torch.Tensor):
        if scatter.dtype != torch.int32 or not scatter.is_contiguous():
            scatter = scatter.to(torch.int32).contiguous()
        keep.append(scatter)
        rv.out_row_scatter = scatter.data_ptr()
    return rv


def _ns_payload_is_noop(ns_payload) -> bool:
    if ns_payload is None:
        return True
    if isinstance(ns_payload, dict):
        for key in ("max_ns_rank", "rank", "ns_rank"):
            if key in ns_payload:
                v = ns_payload[key]
                try:
                    return int(v.item() if isinstance(v, torch.Tensor) else v) == 0
                except (TypeError, ValueError):
                    return False
        return True
    return False


# ---------------------------------------------------------------------------------------
# grouped operators
# ---------------------------------------------------------------------------------------
def run_grouped_structured_expert_forward(
    payload_or_modules,
    hidden_grouped: torch.Tensor,
    x_grouped: torch.Tensor,
    grouped_route_or_segment_lengths,
    expert_modules=None,
    expert_ids=None,
    ns_payload=None,
    prefer_ns_fused_decode: bool = False,
):
    """``run_grouped_structured_expert_forward`` (qlinear_cuda.py:2131-2335): ``[R, O]`` fp16 =
    per-segment ``dequant(U_e) @ hidden_grouped`` rows.  ``x_grouped`` is only read by
    null-space compensation, which must be rank 0 here."""
    _native.require_cuda(hidden_grouped, "run_grouped_structured_expert_forward")
    if hidden_grouped.dtype != torch.float16:
        return envflags.return_or_raise_none("run_grouped_structured_expert_forward", "hidden_grouped must be float16")
    if x_grouped is not None and (x_grouped.device != hidden_grouped.device or x_grouped.dtype != hidden_grouped.dtype):
        return envflags.return_or_raise_none("run_grouped_structured_expert_forward", "x_grouped device/dtype mismatch")
    if hidden_grouped.dim() != 2 or (x_grouped is not None and (x_grouped.dim() != 2 or x_grouped.size(0) != hidden_grouped.size(0))):
        return envflags.return_or_raise_none("run_grouped_structured_expert_forward", "hidden_grouped / x_grouped shape mismatch")
    route = _coerce_grouped_route(grouped_route_or_segment_lengths, hidden_grouped.device, expert_ids=expert_ids)
    if route is None:
        return envflags.return_or_raise_none("run_grouped_structured_expert_forward", "invalid route or segment lengths")
    tok = route.get("grouped_token_indices")
    if tok is not None and tok.numel() not in (0, hidden_grouped.size(0)) and route.get("_row_gather") is None:
        return envflags.return_or_raise_none("run_grouped_structured_expert_forward", "route size does not match hidden_grouped")
    payload = payload_or_modules if isinstance(payload_or_modules, dict) else build_grouped_precomputed_payload(
        payload_or_modules, hidden_grouped.device, hidden_grouped.dtype)
    if payload is None:
        return envflags.return_or_raise_none("run_grouped_structured_expert_forward", "no grouped payload")
    with_ns = not _ns_payload_is_noop(ns_payload)
    if with_ns and (x_grouped is None or isinstance(route.get("_out_row_scatter"), torch.Tensor)):
        return envflags.return_or_raise_none("run_grouped_structured_expert_forward",
                                             "null-space compensation needs x_grouped and outputs in grouped row order")
    lib = _native.load()
    view = proj_view(payload)
    E, O, rank, _ = payload["_tris_dims"]
    if hidden_grouped.size(1) != rank:
        return envflags.return_or_raise_none("run_grouped_structured_expert_forward", "hidden width does not match the payload rank")
    hidden = hidden_grouped.contiguous()
    R = int(route["_row_gather"].numel()) if isinstance(route.get("_row_gather"), torch.Tensor) else int(hidden.size(0))
    out = torch.empty((R, O), dtype=torch.float16, device=hidden.device)
    if R == 0:
        return out
    keep: list = []
    rv = _route_view(route, R, keep)
    with torch.cuda.device(hidden.device):
        _native.check(
            lib.tris_grouped_forward(C.byref(view), C.byref(rv), hidden.data_ptr(), out.data_ptr(), _stream_ptr(hidden.device)),
            "grouped_forward",
        )
    if with_ns:  # out += (x . C2^T) . C1^T of each row's expert (qlinear_cuda.py:2318-2333)
        from .ns_compensation import run_grouped_ns_compensation_forward

        run_grouped_ns_compensation_forward(ns_payload, x_grouped, route, out=out, accumulate=True)
    return out


def run_grouped_structured_expert_pair_forward(
    payload_or_modules_a,
    payload_or_modules_b,
    hidden_grouped_a: torch.Tensor,
    hidden_grouped_b: torch.Tensor,
    x_grouped: torch.Tensor,
    grouped_route_or_segment_lengths,
    expert_modules_a=None,
    expert_modules_b=None,
    expert_ids=None,
    ns_payload_a=None,
    ns_payload_b=None,
    fuse_silu_mul: bool = False,
):
    """``run_grouped_structured_expert_pair_forward`` (qlinear_cuda.py:2338-2634): gate and up
    in one launch, returning ``(out_a, out_b)``.  With ``fuse_silu_mul=True`` (an addition)
    returns ``(silu(out_a) * out_b, None)`` computed in fp32 inside the kernel."""
    _native.require_cuda(hidden_grouped_a, "run_grouped_structured_expert_pair_forward")
    if hidden_grouped_a.dtype != torch.float16 or hidden_grouped_b.dtype != torch.float16:
        return envflags.return_or_raise_none("run_grouped_structured_expert_pair_forward", "hidden states must be float16"), None
    if hidden_grouped_a.dim() != 2 or hidden_grouped_b.shape != hidden_grouped_a.shape:
        return envflags.return_or_raise_none("run_grouped_structured_expert_pair_forward", "hidden_grouped_a / hidden_grouped_b shape mismatch"), None
    if hidden_grouped_b.device != hidden_grouped_a.device:
        return envflags.return_or_raise_none("run_grouped_structured_expert_pair_forward", "hidden states on different devices"), None
    route = _coerce_grouped_route(grouped_route_or_segment_lengths, hidden_grouped_a.device, expert_ids=expert_ids)
    if route is None:
        return envflags.return_or_raise_none("run_grouped_structured_expert_pair_forward", "invalid route or segment lengths"), None
    dev, dt = hidden_grouped_a.device, hidden_grouped_a.dtype
    pa = payload_or_modules_a if isinstance(payload_or_modules_a, dict) else build_grouped_precomputed_payload(payload_or_modules_a, dev, dt)
    pb = payload_or_modules_b if isinstance(payload_or_modules_b, dict) else build_grouped_precomputed_payload(payload_or_modules_b, dev, dt)
    if pa is None or pb is None:
        return envflags.return_or_raise_none("run_grouped_structured_expert_pair_forward", "no grouped payload"), None
    ns_a, ns_b = not _ns_payload_is_noop(ns_payload_a), not _ns_payload_is_noop(ns_payload_b)
    if (ns_a or ns_b) and (x_grouped is None or isinstance(route.get("_out_row_scatter"), torch.Tensor)):
        return envflags.return_or_raise_none("run_grouped_structured_expert_pair_forward",
                                             "null-space compensation needs x_grouped and outputs in grouped row order"), None
    # the compensation is added to gate and up before the activation: with it the pair runs unfused
    fuse_requested, fuse_silu_mul = fuse_silu_mul, bool(fuse_silu_mul) and not (ns_a or ns_b)
    lib = _native.load()
    va, vb = proj_view(pa), proj_view(pb)
    _, O, rank, _ = pa["_tris_dims"]
    if hidden_grouped_a.size(1) != rank:
        return envflags.return_or_raise_none("run_grouped_structured_expert_pair_forward", "hidden width does not match the payload rank"), None
    ha, hb = hidden_grouped_a.contiguous(), hidden_grouped_b.contiguous()
    R = int(route["_row_gather"].numel()) if isinstance(route.get("_row_gather"), torch.Tensor) else int(ha.size(0))
    out_a = torch.empty((R, O), dtype=torch.float16, device=dev)
    out_b = None if fuse_silu_mul else torch.empty((R, O), dtype=torch.float16, device=dev)
    if R == 0:
        return out_a, out_b
    keep: list = []
    rv = _route_view(route, R, keep)
    with torch.cuda.device(dev):
        _native.check(
            lib.tris_grouped_pair_forward(C.byref(va), C.byref(vb), C.byref(rv), ha.data_ptr(), hb.data_ptr(),
                                          out_a.data_ptr(), None if out_b is None else out_b.data_ptr(),
                                          int(bool(fuse_silu_mul)), _stream_ptr(dev)),
            "grouped_pair_forward",
        )
    if ns_a or ns_b:  # qlinear_cuda.py:2611-2633
        from .ns_compensation import run_grouped_ns_compensation_forward

        if ns_a:
            run_grouped_ns_compensation_forward(ns_payload_a, x_grouped, route, out=out_a, accumulate=True)
        if ns_b:
            run_grouped_ns_compensation_forward(ns_payload_b, x_grouped, route, out=out_b, accumulate=True)
        if fuse_requested:
            return (torch.nn.functional.silu(out_a.float()) * out_b.float()).to(torch.float16), None
    return out_a, out_b


# ---------------------------------------------------------------------------------------
# backbone
# ---------------------------------------------------------------------------------------
def compute_shared_hidden(x: torch.Tensor, shared_sv: torch.Tensor, layout: int = HIDDEN_ROW_MAJOR) -> torch.Tensor:
    """``hidden = x @ shared_sv.T`` in fp16 with fp32 accumulation
    (``QuantLinear.compute_shared_hidden`` fp16 branch, qlinear_cuda.py:4454-4502).  ``layout``
    (an addition) picks the column order of the result: row-major like the reference, or one of
    the permuted orders the grouped kernels consume without re-ordering (pass the same value as
    ``route["_hidden_layout"]``)."""
    _native.require_cuda(x, "compute_shared_hidden")
    if x.dtype != torch.float16 or shared_sv.dtype != torch.float16:
        raise RuntimeError("trismoe_b200 compute_shared_hidden: fp16 activations and backbone required")
    lib = _native.load()
    x2 = x.reshape(-1, x.shape[-1]).contiguous()
    sv = shared_sv.contiguous()
    rank, in_features = (int(s) for s in sv.shape)
    if x2.shape[1] != in_features:
        raise RuntimeError("trismoe_b200 compute_shared_hidden: x and shared_sv disagree on in_features")
    out = torch.empty((x2.shape[0], rank), dtype=torch.float16, device=x.device)
    if x2.shape[0]:
        with torch.cuda.device(x.device):
            _native.check(
                lib.tris_shared_hidden_forward(x2.data_ptr(), None, int(x2.shape[0]), None, in_features, sv.data_ptr(), rank,
                                               out.data_ptr(), int(layout), _stream_ptr(x.device)),
                "shared_hidden_forward",
            )
    return out.reshape(x.shape[:-1] + (rank,))


def dequantize_packed_4bit(payload: dict, device) -> torch.Tensor:
    """fp16 matrix ``[rows, cols]`` of a 4-bit packed matrix payload (keys ``qweight``, ``qzeros``,
    ``scales``, ``g_idx`` and optionally ``rows``/``cols``), bit for bit what
    ``PackedQuantMatrix4bit.dequantize`` (qlinear_cuda.py:2756-2784) computes in fp16; built by
    a CUDA kernel on ``device``."""
    dev = torch.device(device)
    if dev.type != "cuda":
        raise RuntimeError("trismoe_b200: the 4-bit backbone is expanded on a CUDA device (there is no CPU fallback)")
    lib = _native.load()
    as_int = lambda v: int(v.item()) if isinstance(v, torch.Tensor) else (None if v is None else int(v))
    qweight = payload["qweight"].to(dev, torch.int32).contiguous()
    qzeros = payload["qzeros"].to(dev, torch.int32).contiguous()
    scales = payload["scales"].to(dev, torch.float16).contiguous()
    g_idx = payload["g_idx"].to(dev, torch.int32).contiguous()
    rows, cols = as_int(payload.get("rows")), as_int(payload.get("cols"))
    rows = int(scales.shape[1]) if rows is None else rows
    cols = int(g_idx.numel()) if cols is None else cols
    groups = int(scales.shape[0])
    if qweight.shape != ((cols + 7) // 8, rows) or qzeros.shape != (groups, (rows + 7) // 8) or g_idx.numel() != cols:
        raise RuntimeError(f"trismoe_b200: inconsistent 4-bit matrix payload: qweight {tuple(qweight.shape)}, qzeros "
                           f"{tuple(qzeros.shape)}, scales {tuple(scales.shape)}, g_idx {g_idx.numel()}, rows {rows}, cols {cols}")
    out = torch.empty((rows, cols), dtype=torch.float16, device=dev)
    with torch.cuda.device(dev):
        _native.check(lib.tris_packed4_dequantize(qweight.data_ptr(), qzeros.data_ptr(), scales.data_ptr(), g_idx.data_ptr(),
                                                  rows, cols, groups, out.data_ptr(),
                                                  torch.cuda.current_stream(dev).cuda_stream), "packed4_dequantize")
    return out


class ExpertSharedMatrix(torch.nn.Module):
    """Holder of one shared input-side backbone ``shared_sv [r, in]`` fp16
    (``ExpertSharedMatrix``, qlinear_cuda.py:2787-2968).  ``set_shared_sv`` takes the fp16 matrix
    or, as real checkpoints store it, the 4-bit packed payload dict (``qweight``, ``qzeros``,
    ``scales``, ``g_idx``, ``rows``, ``cols``; qlinear_cuda.py:2937-2945), which is expanded to
    fp16 once on the GPU (the fp16 copy is what every forward uses)."""

    def __init__(self, weight_dtype=torch.float16):
        super().__init__()
        self.register_buffer("shared_sv", torch.zeros((0, 0), dtype=weight_dtype))
        self.shared_sv_quant = None  # the packed payload, when the matrix was given in 4 bits

    def set_shared_sv(self, payload, device=None):
        if isinstance(payload, dict) and "qweight" in payload:
            dev = torch.device(device) if device is not None else payload["qweight"].device
            self.shared_sv_quant = {k: v for k, v in payload.items()}
            self.shared_sv = dequantize_packed_4bit(payload, dev)
            return self
        tensor = payload if isinstance(payload, torch.Tensor) else payload["shared_sv"]
        self.shared_sv_quant = None
        self.shared_sv = tensor.to(dtype=torch.float16).contiguous()
        return self

    def get_shared_sv(self, device, dtype=torch.float16):
        return self.shared_sv.to(device=device, dtype=dtype)

    def compute_shared_hidden(self, x: torch.Tensor) -> torch.Tensor:
        return compute_shared_hidden(x, self.shared_sv)
