"""Null-space compensation of ``ns_mode == 2`` experts and the 4-bit packed linear it is built
on (``build_grouped_ns_compensation_payload``, qlinear_cuda.py:1734-1882;
``run_grouped_ns_compensation_forward``, qlinear_cuda.py:2024-2128; ``run_grouped_ns_c1_forward``,
qlinear_cuda.py:1963-2021; ``_run_packed_4bit_linear_cuda``, qlinear_cuda.py:1148-1168).

An expert with a null-space pair adds ``F.linear(F.linear(x, C2), C1)`` to its output
(``QuantLinear.forward``, qlinear_cuda.py:4737-4747): ``C2 [ns_rank, in]`` and ``C1 [out, ns_rank]``
are GPTQ-style 4-bit matrices (``PackedQuantMatrix4bit``, qlinear_cuda.py:2637-2784).  The grouped
payload concatenates every expert's C2 along the output axis and every C1 along the input axis,
with per-expert offset tables; the kernels read the nibbles where they lie (no fp16 copy).
There is no CPU path: tensors must live on a CUDA device.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence

import torch

from . import _native, envflags
from ._native import TrisPacked4View

_TENSOR_KEYS = ("ns_rank_per_expert", "ns_c2_rank_offsets", "ns_c2_rank_word_offsets", "ns_c1_rank_word_offsets",
                "ns_c1_group_offsets", "ns_c2_qweight", "ns_c2_qzeros", "ns_c2_scales", "ns_c1_qweight", "ns_c1_qzeros",
                "ns_c1_scales")


def _as_int(v) -> Optional[int]:
    if v is None:
        return None
    return int(v.item()) if isinstance(v, torch.Tensor) else int(v)


def _matrix_dims(m: dict):
    """(rows, cols, groups) of one packed matrix dict (keys qweight, qzeros, scales, g_idx, rows, cols)."""
    rows, cols = _as_int(m.get("rows")), _as_int(m.get("cols"))
    rows = int(m["scales"].shape[1]) if rows is None else rows
    cols = int(m["g_idx"].numel()) if cols is None else cols
    return rows, cols, int(m["scales"].shape[0])


def infer_packed_group_size(m: dict) -> int:
    """Uniform group size of a packed matrix, or its column count when the groups are not uniform
    (``_infer_packed_group_size_from_g_idx``, qlinear_cuda.py:460-483)."""
    _, cols, _ = _matrix_dims(m)
    g_idx = m.get("g_idx")
    if cols <= 0:
        return 1
    if not isinstance(g_idx, torch.Tensor) or g_idx.numel() == 0:
        return cols
    g = g_idx.detach().to("cpu", torch.int64).flatten()
    groups = int(g.max().item()) + 1
    if groups <= 1 or cols % groups:
        return cols
    size = cols // groups
    return size if torch.equal(torch.arange(cols, dtype=torch.int64) // size, g) else cols


def build_grouped_ns_compensation_payload(experts: Sequence, device, dtype=torch.float16, infeatures: Optional[int] = None,
                                          outfeatures: Optional[int] = None):
    """The grouped compensation payload of a layer's experts, with the reference's keys and layout
    (qlinear_cuda.py:1734-1882).  ``experts[e]`` is ``None`` (no compensation) or a dict
    ``{"c1": matrix, "c2": matrix}`` of packed-matrix dicts; two experts that hold the *same* ``c2``
    object share one copy, as experts bound to one shared C2 do in the reference.  Returns ``None``
    for an empty list or inconsistent shapes, like the reference."""
    if len(experts) == 0 or dtype != torch.float16:
        return None
    dev = torch.device(device)
    ranks, group_size = [], None
    for ex in experts:
        if ex is None:
            ranks.append(0)
            continue
        c1, c2 = ex["c1"], ex["c2"]
        r2, k2, _ = _matrix_dims(c2)
        o1, k1, _ = _matrix_dims(c1)
        if k1 != r2:
            return None
        if infeatures is None:
            infeatures = k2
        if outfeatures is None:
            outfeatures = o1
        if k2 != infeatures or o1 != outfeatures:
            return None
        gs = infer_packed_group_size(c2)
        if group_size is None:
            group_size = gs
        elif group_size != gs:
            return None
        ranks.append(r2)
    if infeatures is None or outfeatures is None:
        return None
    if group_size is None:
        group_size = infeatures
    in_groups = (infeatures + group_size - 1) // group_size if infeatures > 0 else 0
    c2_off, c2_woff, c1_woff, c1_goff = [], [], [], []
    tot_rank = tot_rank_words = tot_c1_words = tot_c1_groups = 0
    c2_chunks, c1_chunks, shared = ([], [], []), ([], [], []), {}
    for ex, rank in zip(experts, ranks):
        c1_woff.append(tot_c1_words)
        c1_goff.append(tot_c1_groups)
        if rank <= 0:
            c2_off.append(tot_rank)
            c2_woff.append(tot_rank_words)
            continue
        c1, c2 = ex["c1"], ex["c2"]
        entry = shared.get(id(c2))
        if entry is None:
            entry = (tot_rank, tot_rank_words, rank)
            shared[id(c2)] = entry
            for dst, key, dt in zip(c2_chunks, ("qweight", "qzeros", "scales"), (torch.int32, torch.int32, dtype)):
                dst.append(c2[key].to(dev, dt))
            tot_rank += rank
            tot_rank_words += int(c2["qzeros"].shape[1])
        elif entry[2] != rank:
            return None
        c2_off.append(entry[0])
        c2_woff.append(entry[1])
        for dst, key, dt in zip(c1_chunks, ("qweight", "qzeros", "scales"), (torch.int32, torch.int32, dtype)):
            dst.append(c1[key].to(dev, dt))
        tot_c1_words += int(c1["qweight"].shape[0])
        tot_c1_groups += int(c1["qzeros"].shape[0])
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    empty = lambda shape, dt: torch.zeros(shape, dtype=dt, device=dev)
    cat = lambda chunks, dim, shape, dt: torch.cat(chunks, dim=dim).contiguous() if chunks else empty(shape, dt)
    return {
        "ns_rank_per_expert": i32(ranks), "ns_c2_rank_offsets": i32(c2_off), "ns_c2_rank_word_offsets": i32(c2_woff),
        "ns_c1_rank_word_offsets": i32(c1_woff), "ns_c1_group_offsets": i32(c1_goff),
        "max_ns_rank": max(ranks) if ranks else 0, "infeatures": int(infeatures), "outfeatures": int(outfeatures),
        "group_size": int(group_size),
        "ns_c2_qweight": cat(c2_chunks[0], 1, ((infeatures + 7) // 8, 0), torch.int32),
        "ns_c2_qzeros": cat(c2_chunks[1], 1, (in_groups, 0), torch.int32),
        "ns_c2_scales": cat(c2_chunks[2], 1, (in_groups, 0), dtype),
        "ns_c1_qweight": cat(c1_chunks[0], 0, (0, outfeatures), torch.int32),
        "ns_c1_qzeros": cat(c1_chunks[1], 0, (0, (outfeatures + 7) // 8), torch.int32),
        "ns_c1_scales": cat(c1_chunks[2], 0, (0, outfeatures), dtype),
    }


def ns_payload_max_rank(ns_payload) -> int:
    """Largest null-space rank a compensation payload holds (0: nothing to add)."""
    if not isinstance(ns_payload, dict):
        return 0
    for key in ("max_ns_rank", "rank", "ns_rank"):
        if key in ns_payload:
            return _as_int(ns_payload[key]) or 0
    return 0


def prepare_ns_payload(payload: dict, device) -> dict:
    """Moves a compensation payload (reference keys) to ``device`` and builds the two matrix views
    the kernels take; cached in the dict."""
    dev = torch.device(device)
    if payload.get("_tris_ns_prepared") == str(dev):
        return payload
    if dev.type != "cuda":
        raise RuntimeError("trismoe_b200: null-space compensation runs on a CUDA device (there is no CPU fallback)")
    for key in _TENSOR_KEYS:
        t = payload[key]
        want = torch.float16 if key.endswith("scales") else torch.int32
        payload[key] = t.to(dev, want).contiguous()
    ranks = payload["ns_rank_per_expert"]
    E = int(ranks.numel())
    infeatures, outfeatures = _as_int(payload["infeatures"]), _as_int(payload["outfeatures"])
    group_size, max_rank = _as_int(payload["group_size"]), _as_int(payload["max_ns_rank"])
    goff = payload["ns_c1_group_offsets"].to("cpu", torch.int64)
    total_groups = int(payload["ns_c1_qzeros"].shape[0])
    ends = torch.cat([goff[1:], torch.tensor([total_groups], dtype=torch.int64)])
    payload["_tris_c1_groups"] = (ends - goff).clamp_(min=0).to(dev, torch.int32).contiguous()
    c2, c1 = TrisPacked4View(), TrisPacked4View()
    c2.qweight, c2.qzeros, c2.scales = (payload[k].data_ptr() for k in ("ns_c2_qweight", "ns_c2_qzeros", "ns_c2_scales"))
    c2.n_off, c2.z_off = payload["ns_c2_rank_offsets"].data_ptr(), payload["ns_c2_rank_word_offsets"].data_ptr()
    c2.n_count = ranks.data_ptr()
    c2.q_ld, c2.z_ld, c2.s_ld = (max(1, int(payload[k].shape[1])) for k in ("ns_c2_qweight", "ns_c2_qzeros", "ns_c2_scales"))
    c2.n, c2.k, c2.num_groups = max(1, max_rank), infeatures, int(payload["ns_c2_scales"].shape[0])
    c2.group_size, c2.num_experts = group_size, E
    c1.qweight, c1.qzeros, c1.scales = (payload[k].data_ptr() for k in ("ns_c1_qweight", "ns_c1_qzeros", "ns_c1_scales"))
    c1.kw_off, c1.g_off = payload["ns_c1_rank_word_offsets"].data_ptr(), payload["ns_c1_group_offsets"].data_ptr()
    c1.k_count, c1.g_count = ranks.data_ptr(), payload["_tris_c1_groups"].data_ptr()
    c1.q_ld, c1.z_ld, c1.s_ld = outfeatures, (outfeatures + 7) // 8, outfeatures
    c1.n, c1.k, c1.num_groups = outfeatures, max_rank, max(1, int(payload["_tris_c1_groups"].max().item()) if E else 1)
    c1.group_size, c1.num_experts = group_size, E
    payload["_tris_c2_view"], payload["_tris_c1_view"] = c2, c1
    payload["_tris_hidden_ld"] = (max(1, max_rank) + 7) // 8 * 8
    payload["_tris_ns_prepared"] = str(dev)
    return payload


def _route_rows(route: dict, x: torch.Tensor) -> int:
    gather = route.get("_row_gather")
    return int(gather.numel()) if isinstance(gather, torch.Tensor) else int(x.size(0))


def _launch(view, route, x, x_ld, rows, out, out_ld, accumulate, gather: bool):
    from .qlinear_grouped import _route_view, _stream_ptr

    keep: list = []
    rv = _route_view(route, rows, keep)
    if not gather:
        rv.row_gather = None
    lib = _native.load()
    with torch.cuda.device(x.device):
        _native.check(lib.tris_packed4_grouped_forward(C.byref(view), C.byref(rv), x.data_ptr(), int(x_ld), int(rows), out.data_ptr(),
                                                       int(out_ld), 0, int(bool(accumulate)), _stream_ptr(x.device)),
                      "packed4_grouped_forward")


def run_grouped_ns_c1_forward(payload: dict, hidden_grouped: torch.Tensor, grouped_route_or_segment_lengths, expert_modules=None,
                              expert_ids=None, out: Optional[torch.Tensor] = None, accumulate: bool = False):
    """Second half of the compensation: ``hidden_grouped [R, >= max_ns_rank]`` (the C2 product of
    every grouped row) times each segment's C1 (``run_grouped_ns_c1_forward``,
    qlinear_cuda.py:1963-2021).  Returns ``[R, outfeatures]`` fp16, or adds into ``out`` when
    ``accumulate`` is set."""
    from .qlinear_grouped import _coerce_grouped_route

    _native.require_cuda(hidden_grouped, "run_grouped_ns_c1_forward")
    route = _coerce_grouped_route(grouped_route_or_segment_lengths, hidden_grouped.device, expert_ids=expert_ids)
    if route is None or hidden_grouped.dtype != torch.float16 or hidden_grouped.dim() != 2:
        return envflags.return_or_raise_none("run_grouped_ns_c1_forward", "fp16 [R, rank] hidden states and a route required")
    payload = prepare_ns_payload(payload, hidden_grouped.device)
    R, O = int(hidden_grouped.size(0)), _as_int(payload["outfeatures"])
    if hidden_grouped.size(1) < _as_int(payload["max_ns_rank"]) or hidden_grouped.stride(1) != 1:
        return envflags.return_or_raise_none("run_grouped_ns_c1_forward", "hidden states narrower than max_ns_rank")
    if out is None:
        out, accumulate = torch.empty((R, O), dtype=torch.float16, device=hidden_grouped.device), False
    if R and _as_int(payload["max_ns_rank"]) <= 0:
        return out if accumulate else out.zero_()
    if R:
        _launch(payload["_tris_c1_view"], route, hidden_grouped, hidden_grouped.stride(0), R, out, out.stride(0), accumulate, gather=False)
    return out


def run_grouped_ns_compensation_forward(payload_or_modules, x_grouped: torch.Tensor, grouped_route_or_segment_lengths,
                                        expert_modules=None, expert_ids=None, prefer_fused_decode: bool = False,
                                        out: Optional[torch.Tensor] = None, accumulate: bool = False):
    """``[R, outfeatures]`` fp16 compensation of every grouped row: ``(x . C2_e^T) . C1_e^T`` with the
    matrices of the row's expert; rows of experts without a null-space pair get zeros
    (``run_grouped_ns_compensation_forward``, qlinear_cuda.py:2024-2128).  The intermediate
    ``[R, max_ns_rank]`` is rounded to fp16 like the reference's (CU:1305).  With ``out`` and
    ``accumulate=True`` the result is added to ``out`` in fp16 instead (what the grouped expert
    operators do with it, qlinear_cuda.py:2620-2633).  ``prefer_fused_decode`` is accepted for
    signature parity; both halves always run as two launches of one kernel."""
    from .qlinear_grouped import _coerce_grouped_route

    _native.require_cuda(x_grouped, "run_grouped_ns_compensation_forward")
    if not isinstance(payload_or_modules, dict):
        return envflags.return_or_raise_none("run_grouped_ns_compensation_forward", "a compensation payload dict is required")
    route = _coerce_grouped_route(grouped_route_or_segment_lengths, x_grouped.device, expert_ids=expert_ids)
    if route is None or x_grouped.dtype != torch.float16 or x_grouped.dim() != 2:
        return envflags.return_or_raise_none("run_grouped_ns_compensation_forward", "fp16 [R, in] activations and a route required")
    payload = prepare_ns_payload(payload_or_modules, x_grouped.device)
    if x_grouped.size(1) != _as_int(payload["infeatures"]):
        return envflags.return_or_raise_none("run_grouped_ns_compensation_forward", "x_grouped width does not match infeatures")
    x = x_grouped if x_grouped.stride(1) == 1 else x_grouped.contiguous()
    R, O = _route_rows(route, x), _as_int(payload["outfeatures"])
    if out is None:
        out, accumulate = torch.empty((R, O), dtype=torch.float16, device=x.device), False
    if R == 0:
        return out
    if _as_int(payload["max_ns_rank"]) <= 0:  # no expert of this layer has a null-space pair
        return out if accumulate else out.zero_()
    hidden = torch.empty((R, payload["_tris_hidden_ld"]), dtype=torch.float16, device=x.device)
    _launch(payload["_tris_c2_view"], route, x, x.stride(0), R, hidden, hidden.stride(0), False, gather=True)
    _launch(payload["_tris_c1_view"], route, hidden, hidden.stride(0), R, out, out.stride(0), accumulate, gather=False)
    return out


class Packed4Linear(torch.nn.Module):
    """One 4-bit packed matrix ``[rows, cols]`` kept in its nibbles, applied as ``y = x @ W.T``
    (``_run_packed_4bit_linear_cuda``, qlinear_cuda.py:1148-1168).  Needs uniform groups whose size is a
    multiple of 32 (or one group); other matrices go through ``dequantize_packed_4bit``."""

    def __init__(self, payload: dict, device=None):
        super().__init__()
        dev = torch.device(device) if device is not None else payload["qweight"].device
        if dev.type != "cuda":
            raise RuntimeError("trismoe_b200 Packed4Linear: a CUDA device is required (there is no CPU fallback)")
        self.rows, self.cols, self.groups = _matrix_dims(payload)
        self.group_size = infer_packed_group_size(payload)
        if not self.supports(payload):
            raise RuntimeError("trismoe_b200 Packed4Linear: groups must be uniform, of a size that is a multiple of 32")
        self.qweight = payload["qweight"].to(dev, torch.int32).contiguous()
        self.qzeros = payload["qzeros"].to(dev, torch.int32).contiguous()
        self.scales = payload["scales"].to(dev, torch.float16).contiguous()
        v = TrisPacked4View()
        v.qweight, v.qzeros, v.scales = self.qweight.data_ptr(), self.qzeros.data_ptr(), self.scales.data_ptr()
        v.q_ld, v.z_ld, v.s_ld = self.rows, int(self.qzeros.shape[1]), self.rows
        v.n, v.k, v.num_groups, v.group_size, v.num_experts = self.rows, self.cols, self.groups, self.group_size, 1
        self._view = v

    @staticmethod
    def supports(payload: dict) -> bool:
        _, cols, groups = _matrix_dims(payload)
        size = infer_packed_group_size(payload)
        return groups == 1 or (size * groups == cols and size % 32 == 0)

    @property
    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.qweight, self.qzeros, self.scales))

    def forward(self, x: torch.Tensor, layout: int = 0) -> torch.Tensor:
        """``layout``: column order of the result (``HIDDEN_*`` of qlinear_grouped; 0 = row major)."""
        from .qlinear_grouped import _stream_ptr

        _native.require_cuda(x, "Packed4Linear.forward")
        if x.dtype != torch.float16 or x.shape[-1] != self.cols:
            return envflags.return_or_raise_none("Packed4Linear.forward", "fp16 input of the matrix's column count required")
        x2 = x.reshape(-1, self.cols)
        x2 = x2 if x2.stride(1) == 1 else x2.contiguous()
        out = torch.empty((x2.shape[0], self.rows), dtype=torch.float16, device=x.device)
        if x2.shape[0]:
            lib = _native.load()
            with torch.cuda.device(x.device):
                _native.check(lib.tris_packed4_grouped_forward(C.byref(self._view), None, x2.data_ptr(), int(x2.stride(0)),
                                                               int(x2.shape[0]), out.data_ptr(), self.rows, int(layout), 0,
                                                               _stream_ptr(x.device)), "packed4_grouped_forward")
        return out.reshape(x.shape[:-1] + (self.rows,))
