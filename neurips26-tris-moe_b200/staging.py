"""Streaming loader: expert payloads held in pinned host memory and paged to the GPU on a
side stream, overlapped with compute.

Role of ``GroupedQGmapCPUStagingManager`` (``grouped_payload_sidecar.py:764-1146`` in the
TriS-MoE tree), with two modes:

``mode="bitmap"``   what the reference streams: only the sparse grouping bitmap
                    ``q_gmap_sparse`` of every projection leaves the GPU (README:281-283);
                    signs and scales stay resident.  Payloads must use the sparse bitmap
                    format (``compact3_use_block_gr = False``).
``mode="payload"``  every bulky per-expert tensor (sign planes, bitmap or block-GR stream and
                    its index, scale packs) lives in pinned host memory; only the small
                    tables (c_map, prefixes, offsets/meta, group table) stay resident.

Mechanism (differs from the reference on purpose).  The reference learns the active experts on
the host (a ``.cpu().tolist()`` of the route), then issues one ``copy_`` per expert range and
one kernel per chunk.  Here the copy is itself a kernel (``tris_page_experts``) that reads the
pinned buffers through their device mapping and is driven by the device-side route: it is
enqueued on a side stream right after the route kernel, copies exactly the active experts'
blocks into staging slot ``s`` = segment index, and writes the expert -> slot table the
grouped kernels index with.  Nothing is read back to the host.  Ordering is by events:
compute waits on "paged", the pager of the next use of a slot waits on "consumed".

Statistics: ``pipeline_stats`` counts calls and bytes as the reference's does (exact bytes
need the active expert count, which only the device knows, so ``bytes`` is an upper bound
from the slot count); :meth:`overlap_report` turns CUDA-event timings into the overlapped
fraction ``1 - stall / copy``.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from . import _native
from ._native import TrisPageJob
from .qlinear_grouped import proj_view

BITMAP_KEYS = ("q_gmap_sparse",)
PAYLOAD_KEYS = ("qweight1", "qweight2_sparse", "q_gmap_sparse", "q_gmap_gr_words", "_tris_gr_index", "col_pack3", "row_pack3")
PROJECTIONS = ("gate", "up", "down")
MAX_PAGE_JOBS = 16  # TRIS_MAX_PAGE_JOBS of the C header


class _Entry:
    """One projection of one layer: pinned host tensors and their per-expert block sizes."""

    def __init__(self, payload: dict, keys):
        self.payload = payload
        self.host = {}
        self.block_bytes = {}
        E = int(payload["qweight1"].shape[0])
        for key in keys:
            t = payload.get(key)
            if not isinstance(t, torch.Tensor) or t.numel() == 0:
                continue
            per = t.numel() // E * t.element_size()
            if per == 0:
                continue
            shape = list(t.shape)
            if per % 16:
                # only a 2-D stream (block-GR words) can be ragged: pad each expert's row with zeros
                if t.dim() != 2 or (16 % t.element_size()):
                    raise RuntimeError(f"trismoe_b200 staging: {key} has {per} bytes per expert, not a multiple of 16")
                step = 16 // t.element_size()
                shape[1] = (shape[1] + step - 1) // step * step
                per = shape[1] * t.element_size()
            host = torch.zeros(shape, dtype=t.dtype, pin_memory=True)
            host[tuple(slice(0, d) for d in t.shape)].copy_(t)
            self.host[key] = host
            self.block_bytes[key] = per


def staging_requested() -> bool:
    """True when the host asks for the streaming mode through ``TRIS_GROUPED_QGMAP_CPU_STAGING`` (or
    the reference's per-family names; ``_grouped_qgmap_cpu_staging_enabled``,
    grouped_payload_sidecar.py:147-152)."""
    from . import envflags

    return envflags.grouped_qgmap_cpu_staging_enabled()


class GroupedQGmapCPUStagingManager:
    """Pages expert payloads of the registered MoE blocks from pinned host memory."""

    def __init__(self, moe_blocks, mode: str = "bitmap", max_active_experts: Optional[int] = None, slots: int = 2):
        if mode not in ("bitmap", "payload"):
            raise ValueError("mode must be 'bitmap' or 'payload'")
        self.blocks = list(moe_blocks)
        self.mode = mode
        self.ring = int(slots)
        self.max_active = max_active_experts
        self.device = None
        self.entries = {}          # (block index, projection) -> _Entry
        self.buffers = {}          # (ring slot, projection, key) -> device staging tensor
        self.slot_tables = []      # per ring slot: {"gate" (shared with up), "down"}: int32 [E] expert -> staging
                                   # slot; down has its own because each pager call resets its table and down is
                                   # paged while the gate/up kernel is still reading the table of gate and up
        self._paged = []           # per ring slot: event "pager done" (all three projections)
        self._paged_gu = []        # per ring slot: event "gate and up paged" (down may still be in flight)
        self._consumed = []        # per ring slot: event "compute done with this slot"
        self._used = []
        self._copy_stream = None
        self._next = 0
        self._initialized = False
        self.pipeline_stats = {"calls": 0, "chunks": 0, "bytes": 0, "slot_reuses": 0}
        self._timings = []         # (copy_start, copy_end, wait_start, wait_end) events
        self.collect_timings = True  # set False while capturing the forward into a CUDA graph
        # A stream that is being captured may not wait for an event recorded outside the
        # capture.  Slot uses are therefore stamped with an epoch that changes whenever a
        # capture starts or ends; a pager only waits for "consumed" events of its own epoch
        # (work of an earlier epoch is ordered before it by the stream itself: the caller
        # captures, and replays, on the stream the earlier work ran on or has synchronised).
        self._epoch = 0
        self._capturing = False
        self._consumed_epoch = []

    @property
    def buffer_nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.buffers.values())

    def initialize(self) -> bool:
        if self._initialized:
            return True
        if not self.blocks:
            return False
        keys = BITMAP_KEYS if self.mode == "bitmap" else PAYLOAD_KEYS
        first = self.blocks[0]._get_grouped_payload("gate")
        self.device = first["qweight1"].device
        if self.device.type != "cuda":
            raise RuntimeError("trismoe_b200 staging: payloads must be on a CUDA device before staging starts")
        E = int(first["qweight1"].shape[0])
        cap = E if self.max_active is None else max(1, min(E, int(self.max_active)))
        sizes = {}
        for bi, blk in enumerate(self.blocks):
            for proj in PROJECTIONS:
                payload = blk._get_grouped_payload(proj)
                if payload["qweight1"].device != self.device:
                    raise RuntimeError("trismoe_b200 staging: all layers must live on one CUDA device")
                if self.mode == "bitmap" and bool(payload.get("compact3_use_block_gr", False)):
                    raise RuntimeError("trismoe_b200 staging: bitmap streaming needs the sparse bitmap format "
                                       "(block-GR payloads stay resident, as in the reference)")
                entry = _Entry(payload, keys)
                self.entries[(bi, proj)] = entry
                for key, per in entry.block_bytes.items():
                    sizes[(proj, key)] = max(sizes.get((proj, key), 0), per)
        for ring in range(self.ring):
            for (proj, key), per in sizes.items():
                # a few bytes of slack: the GR span copy may round its end up to 16 bytes
                self.buffers[(ring, proj, key)] = torch.zeros((cap * per + 64,), dtype=torch.uint8, device=self.device)
            self.slot_tables.append({proj: torch.full((E,), -1, dtype=torch.int32, device=self.device) for proj in ("gate", "down")})
            self._paged.append(torch.cuda.Event())
            self._paged_gu.append(torch.cuda.Event())
            self._consumed.append(torch.cuda.Event())
            self._used.append(False)
            self._consumed_epoch.append(-1)
        self._copy_stream = torch.cuda.Stream(device=self.device)
        self.capacity = cap
        # drop the device copies: from here on the tensors exist only in pinned host memory
        for entry in self.entries.values():
            for key in entry.host:
                entry.payload[key] = torch.empty((0,), dtype=entry.host[key].dtype, device=self.device)
            if self.mode == "payload":
                # the resident tile-major copy of the same planes would defeat the point of paging them
                for key in ("_tris_tile_records", "_tris_tile_desc", "_tris_col_records", "_tris_tile_meta"):
                    entry.payload.pop(key, None)
                view = proj_view(entry.payload)
                view.tile_records = view.tile_desc = view.col_records = None
            entry.payload["_qgmap_staging"] = (self, entry)
        self._initialized = True
        return True

    # -- one layer ---------------------------------------------------------------------------
    def page_layer(self, block_index: int, route: dict):
        """Enqueues, on the side stream, the paging of gate/up/down of one layer for the
        experts of ``route`` (device arrays from ``tris_build_grouped_route``), and returns a
        handle whose views the grouped kernels of this layer must use."""
        self.initialize()
        lib = _native.load()
        ring = self._next
        self._next = (self._next + 1) % self.ring
        compute = torch.cuda.current_stream(self.device)
        copy = self._copy_stream
        copy.wait_stream(compute)  # the route must be final before the pager reads it
        capturing = bool(torch.cuda.is_current_stream_capturing())
        if capturing != self._capturing:
            self._capturing = capturing
            self._epoch += 1
        if self._used[ring] and self._consumed_epoch[ring] == self._epoch:
            copy.wait_event(self._consumed[ring])
            self.pipeline_stats["slot_reuses"] += 1
        nseg_bound = min(int(route["experts"]), int(route["rows"]), self.capacity)
        tables = self.slot_tables[ring]
        timed = self.collect_timings
        start = end = None
        if timed:
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        views = {}
        with torch.cuda.stream(copy):
            if timed:
                start.record(copy)
            # gate and up go in one launch (they are needed together and share a slot table), down in a second one
            # that runs while the gate/up kernel computes
            for group in (("gate", "up"), ("down",)):
                pairs = [(proj, key) for proj in group for key in self.entries[(block_index, proj)].host]
                table = tables[group[0]]
                for lo in range(0, len(pairs), MAX_PAGE_JOBS):
                    part = pairs[lo: lo + MAX_PAGE_JOBS]
                    jobs = (TrisPageJob * len(part))()
                    for j, (proj, key) in enumerate(part):
                        entry = self.entries[(block_index, proj)]
                        jobs[j].host_src = entry.host[key].data_ptr()
                        jobs[j].dst = self.buffers[(ring, proj, key)].data_ptr()
                        jobs[j].bytes_per_expert = entry.block_bytes[key]
                        self.pipeline_stats["bytes"] += nseg_bound * entry.block_bytes[key]
                    _native.check(lib.tris_page_experts(jobs, len(part), route["expert_ids"].data_ptr(),
                                                        route["counts"].data_ptr(), nseg_bound, int(route["experts"]),
                                                        table.data_ptr(), copy.cuda_stream), "page_experts")
                    self.pipeline_stats["chunks"] += 1
                for proj in group:
                    views[proj] = self._staged_view(self.entries[(block_index, proj)], ring, proj, table)
                if group[0] == "gate":  # the gate/up kernel may start while down is still paged
                    self._paged_gu[ring].record(copy)
            if timed:
                end.record(copy)
            self._paged[ring].record(copy)
        self.pipeline_stats["calls"] += 1
        self._used[ring] = True
        return _PagedLayer(self, ring, views, start, end)

    def _staged_view(self, entry: _Entry, ring: int, proj: str, table: torch.Tensor):
        """Copy of the projection's ctypes view whose paged tensors point at the staging slots."""
        base = proj_view(entry.payload)
        view = type(base)()
        C.pointer(view)[0] = base
        field = {"qweight1": "qweight1", "qweight2_sparse": "qweight2_sparse", "q_gmap_sparse": "q_gmap_sparse",
                 "q_gmap_gr_words": "q_gmap_gr_words", "_tris_gr_index": "gr_index", "col_pack3": "col_pack3",
                 "row_pack3": "row_pack3"}
        for key in entry.host:
            setattr(view, field[key], self.buffers[(ring, proj, key)].data_ptr())
        if self.mode == "bitmap":
            view.gmap_slot = table.data_ptr()
            view.gmap_sparse_rows = int(entry.host["q_gmap_sparse"].shape[1])
        else:
            view.expert_slot = table.data_ptr()
            if "q_gmap_sparse" in entry.host:
                view.gmap_sparse_rows = int(entry.host["q_gmap_sparse"].shape[1])
            if "q_gmap_gr_words" in entry.host:
                view.gr_max_words = int(entry.host["q_gmap_gr_words"].shape[1])
        return view

    # -- reporting -----------------------------------------------------------------------------
    def overlap_report(self) -> dict:
        """Overlapped fraction of the transfer time: 1 - (time compute stalled on a pager) /
        (pager time), from CUDA events; call after a synchronize."""
        copy_ms = stall_ms = 0.0
        n = 0
        for c0, c1, w0, w1 in self._timings:
            if c0 is not c1:  # a layer's second wait carries no copy interval of its own
                copy_ms += c0.elapsed_time(c1)
                n += 1
            stall_ms += w0.elapsed_time(w1)
        self._timings = []
        frac = 1.0 - stall_ms / copy_ms if copy_ms > 0 else None
        return {"layers": n, "copy_ms": copy_ms, "stall_ms": stall_ms, "overlapped_fraction": frac}

    def finalize_forward(self) -> None:
        """Kept for interface parity (grouped_payload_sidecar.py:1143): nothing to unbind."""


class _PagedLayer:
    def __init__(self, manager: GroupedQGmapCPUStagingManager, ring: int, views: dict, start, end):
        self.manager, self.ring, self.views = manager, ring, views
        self._copy_start, self._copy_end = start, end
        self._waited = False
        self._waited_gu = False

    def wait(self, which: str = "all") -> None:
        """Makes the current (compute) stream wait for this layer's pager, timing the stall.
        ``which="gate_up"`` waits only until gate and up are in (the pager goes on with down, which
        then pages under the gate/up kernel and the down backbone); ``"all"`` waits for everything."""
        if self._waited or (which == "gate_up" and self._waited_gu):
            return
        compute = torch.cuda.current_stream(self.manager.device)
        event = self.manager._paged_gu[self.ring] if which == "gate_up" else self.manager._paged[self.ring]
        if self._copy_start is None:
            compute.wait_event(event)
        else:
            w0, w1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            w0.record(compute)
            compute.wait_event(event)
            w1.record(compute)
            # the copy interval is counted once (with the first wait), every wait adds its stall
            zero = (w0, w0) if (self._waited_gu and which != "gate_up") else (self._copy_start, self._copy_end)
            self.manager._timings.append((zero[0], zero[1], w0, w1))
        if which == "gate_up":
            self._waited_gu = True
        else:
            self._waited = True

    def release(self) -> None:
        """Marks the staging slots free once the kernels enqueued so far have consumed them."""
        self.manager._consumed[self.ring].record(torch.cuda.current_stream(self.manager.device))
        self.manager._consumed_epoch[self.ring] = self.manager._epoch


def maybe_create_grouped_qgmap_cpu_staging_manager(moe_blocks, mode: str = "bitmap", **kw):
    """``maybe_create_grouped_qgmap_cpu_staging_manager`` (grouped_payload_sidecar.py:1149-1153)."""
    manager = GroupedQGmapCPUStagingManager(moe_blocks, mode=mode, **kw)
    return manager if manager.initialize() else None
