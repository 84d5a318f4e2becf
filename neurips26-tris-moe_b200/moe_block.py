"""MoE block on the trismoe_b200 runtime, mirroring ``OlmoeSparseMoeBlock``
(``auto_gptq/modeling_tris_moe/modeling_olmoe.py:621-1105`` in the TriS-MoE tree; the
Mixtral and Qwen2-MoE blocks call the same operators with other shapes).

``forward`` runs the whole block through one C-ABI call (``tris_moe_layer_forward``):
router, route, both input-side backbones, grouped gate/up with SiLU*mul, down backbone,
grouped down and the weighted combine, stream-ordered with no host synchronisation.
``forward_grouped_ops`` composes the same result from the individual reference-named
operators, the way ``_forward_grouped`` (modeling_olmoe.py:916-1044) does.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch
from torch import nn

from . import _native, envflags
from ._native import TrisMoeLayerView
from .ns_compensation import Packed4Linear
from .qlinear_grouped import (
    build_grouped_route,
    compute_shared_hidden,
    dequantize_packed_4bit,
    prepare_grouped_payload,
    proj_view,
    run_grouped_structured_expert_forward,
    run_grouped_structured_expert_pair_forward,
)


class TrisSparseMoeBlock(nn.Module):
    """Quantized grouped-expert MoE layer.

    Args mirror the HF config fields the reference block reads: ``hidden_size``,
    ``intermediate_size``, ``num_experts``, ``num_experts_per_tok``, ``norm_topk_prob``.
    Weights are attached with :meth:`load_grouped_payloads`.
    """

    def __init__(self, hidden_size: int, intermediate_size: int, num_experts: int, num_experts_per_tok: int,
                 norm_topk_prob: bool = False):
        super().__init__()
        self.hidden_size = int(hidden_size)
        self.intermediate_size = int(intermediate_size)
        self.num_experts = int(num_experts)
        self.top_k = int(num_experts_per_tok)
        self.norm_topk_prob = bool(norm_topk_prob)
        self.gate = nn.Linear(self.hidden_size, self.num_experts, bias=False, dtype=torch.float16)
        self.register_buffer("shared_gate", torch.zeros((0, 0), dtype=torch.float16))
        self.register_buffer("shared_up", torch.zeros((0, 0), dtype=torch.float16))
        self.register_buffer("shared_down", torch.zeros((0, 0), dtype=torch.float16))
        self.packed_backbones: dict = {}  # name -> Packed4Linear: backbones kept in their 4-bit nibbles
        self.input_scales: dict = {}      # name -> fp16 [in]: vector null-space input scale (ns_mode == 1)
        self.ns_payloads: dict = {}       # name -> grouped null-space compensation payload (ns_mode == 2)
        self._grouped_payload_cache: dict = {}
        self._layer_view: Optional[TrisMoeLayerView] = None
        self._expanded_view: Optional[dict] = None  # expanded backbone names -> layer view
        self._workspace: Optional[torch.Tensor] = None
        self._status_word: Optional[torch.Tensor] = None  # status of the kernels forward_streaming launches

    # -- loading ---------------------------------------------------------------------------
    # activation rows above which a 4-bit backbone is expanded to fp16 scratch and run on the dense GEMM
    # (measured on B200, 2048 x 2048: the 4-bit GEMM takes 7 / 8 / 16 / 23 us at 1 / 16 / 64 / 128 rows, the
    # expansion 4 us plus 7 / 8 / 14 / 15 us of fp16 GEMM)
    PACKED_BACKBONE_MAX_ROWS = 64
    _expand_scratch: dict = {}  # (device, name, shape) -> fp16 scratch shared by every block of a model

    def load_grouped_payloads(self, gate: dict, up: dict, down: dict, shared_gate, shared_up, shared_down,
                              router_weight: Optional[torch.Tensor] = None, device=None,
                              packed_backbone: Optional[str] = None, input_scales: Optional[dict] = None) -> "TrisSparseMoeBlock":
        """Attaches the E-stacked payloads (``enable_grouped_deployment_only``,
        modeling_olmoe.py:732-804) and the three backbones, moving everything to ``device`` and
        deriving the decode index once.  A backbone is an fp16 matrix ``[r, in]`` or, as real
        checkpoints store it, a 4-bit packed payload dict (``shared_sv_quant``: ``qweight``, ``qzeros``,
        ``scales``, ``g_idx``, ``rows``, ``cols``).  ``packed_backbone`` (default: the environment
        variable ``TRIS_PACKED4_BACKBONE``, else ``"nibbles"``) says how packed backbones are kept:
        ``"nibbles"`` - in place, read by the 4-bit GEMM (a quarter of the bytes; gate and up switch
        together, matrices with non-uniform groups are expanded), ``"fp16"`` - expanded once at load.
        ``input_scales`` (``{"gate" | "up" | "down": fp16 [in]}``): the vector null-space input scale of
        ``ns_mode == 1`` checkpoints (``expert_input_scale`` of expert 0, qlinear_cuda.py:3918-3923): the
        backbone of that projection sees ``x * scale`` rounded to fp16 (qlinear_cuda.py:4477-4480); the
        matching output scale travels in the payload (``output_scale``).  With input scales the block
        runs operator by operator (gate and up no longer share their input rows)."""
        import os

        dev = torch.device(device) if device is not None else gate["qweight1"].device
        self._grouped_payload_cache = {
            "gate": prepare_grouped_payload(gate, dev),
            "up": prepare_grouped_payload(up, dev),
            "down": prepare_grouped_payload(down, dev),
        }
        mode = (packed_backbone or os.environ.get("TRIS_PACKED4_BACKBONE", "nibbles")).lower()
        if mode not in ("nibbles", "fp16"):
            raise ValueError("packed_backbone must be 'nibbles' or 'fp16'")
        given = {"gate": shared_gate, "up": shared_up, "down": shared_down}
        is_packed = {n: isinstance(m, dict) and "qweight" in m for n, m in given.items()}
        keep = {n: mode == "nibbles" and is_packed[n] and Packed4Linear.supports(m) for n, m in given.items()}
        keep["gate"] = keep["up"] = keep["gate"] and keep["up"]
        self.packed_backbones = {}
        for name, m in given.items():
            if keep[name]:
                self.packed_backbones[name] = Packed4Linear(m, dev)
                dense = torch.zeros((0, 0), dtype=torch.float16, device=dev)
            elif is_packed[name]:
                dense = dequantize_packed_4bit(m, dev)
            else:
                dense = m.to(dev, torch.float16).contiguous()
            setattr(self, "shared_" + name, dense)
        if router_weight is not None:
            self.gate.weight = nn.Parameter(router_weight.to(dev, torch.float16).contiguous(), requires_grad=False)
        else:
            self.gate.to(dev)
        self.input_scales = {n: v.reshape(-1).to(dev, torch.float16).contiguous() for n, v in (input_scales or {}).items()}
        if set(self.input_scales) - set(given):
            raise ValueError("input_scales keys must be among 'gate', 'up', 'down'")
        self._layer_view = self._expanded_view = None
        return self

    def load_ns_compensation_payloads(self, gate_ns: Optional[dict] = None, up_ns: Optional[dict] = None,
                                      down_ns: Optional[dict] = None) -> "TrisSparseMoeBlock":
        """Attaches the grouped null-space compensation payloads of ``ns_mode == 2`` checkpoints (the
        ``gate_ns`` / ``up_ns`` / ``down_ns`` entries of the reference's payload cache,
        modeling_olmoe.py:950-975; built by ``build_grouped_ns_compensation_payload``).  With any of
        them the block runs operator by operator and each grouped operator adds its compensation."""
        from .ns_compensation import ns_payload_max_rank

        self.ns_payloads = {n: p for n, p in (("gate", gate_ns), ("up", up_ns), ("down", down_ns))
                            if p is not None and ns_payload_max_rank(p) > 0}
        return self

    def backbone_rank(self, name: str) -> int:
        p = self.packed_backbones.get(name)
        return p.rows if p is not None else int(getattr(self, "shared_" + name).shape[0])

    def backbone_hidden(self, name: str, x: torch.Tensor, layout: int = 0) -> torch.Tensor:
        """``x . backbone^T`` (``compute_shared_hidden``) for the fp16 or the 4-bit form of a backbone."""
        scale = self.input_scales.get(name)
        if scale is not None:
            x = x * scale
        p = self.packed_backbones.get(name)
        if p is not None:
            return p(x, layout)
        return compute_shared_hidden(x, getattr(self, "shared_" + name), layout=layout)

    def _get_grouped_payload(self, cache_key: str) -> dict:
        if cache_key not in self._grouped_payload_cache:
            raise RuntimeError(f"trismoe_b200: grouped payload '{cache_key}' was not loaded")
        return self._grouped_payload_cache[cache_key]

    def layer_view(self) -> TrisMoeLayerView:
        views = [proj_view(self._get_grouped_payload(k)) for k in ("gate", "up", "down")]
        if self._layer_view is None or any(self._get_grouped_payload(k).get("_tris_layer_dirty") for k in ("gate", "up", "down")):
            v = TrisMoeLayerView()
            v.hidden_size, v.intermediate_size = self.hidden_size, self.intermediate_size
            v.num_experts, v.top_k, v.norm_topk_prob = self.num_experts, self.top_k, int(self.norm_topk_prob)
            v.router_weight = self.gate.weight.data_ptr()
            for name in ("gate", "up", "down"):
                p = self.packed_backbones.get(name)
                setattr(v, "shared_" + name, None if p is not None else getattr(self, "shared_" + name).data_ptr())
                setattr(v, "packed_" + name, None if p is None else C.addressof(p._view))
            v.gate, v.up, v.down = views
            for k in ("gate", "up", "down"):
                self._get_grouped_payload(k)["_tris_layer_dirty"] = False
            self._layer_view, self._expanded_view = v, None
        return self._layer_view

    def _expanded_layer_view(self, dev, names) -> TrisMoeLayerView:
        """The layer view with the 4-bit backbones in ``names`` expanded into fp16 scratch (enqueued on
        the current stream): what large batches use, where the dense GEMM beats re-expanding nibbles for
        every pass over the rows.  The scratch is shared by all blocks of a model."""
        base = self.layer_view()
        if self._expanded_view is None:
            self._expanded_view = {}
        key = tuple(sorted(names))
        v = self._expanded_view.get(key)
        if v is None:
            v = TrisMoeLayerView()
            C.pointer(v)[0] = base
            self._expanded_view[key] = v
        lib = _native.load()
        for name in key:
            p = self.packed_backbones[name]
            skey = (str(dev), name, p.rows, p.cols)
            scratch = TrisSparseMoeBlock._expand_scratch.get(skey)
            if scratch is None:
                scratch = torch.empty((p.rows, p.cols), dtype=torch.float16, device=dev)
                TrisSparseMoeBlock._expand_scratch[skey] = scratch
            if getattr(p, "_g_idx", None) is None:
                g_idx = (torch.arange(p.cols, device=dev, dtype=torch.int32) // max(1, p.group_size)).clamp_(max=p.groups - 1)
                p._g_idx = g_idx.to(torch.int32).contiguous()
            with torch.cuda.device(dev):
                _native.check(lib.tris_packed4_dequantize(p.qweight.data_ptr(), p.qzeros.data_ptr(), p.scales.data_ptr(),
                                                          p._g_idx.data_ptr(), p.rows, p.cols, p.groups, scratch.data_ptr(),
                                                          torch.cuda.current_stream(dev).cuda_stream), "packed4_dequantize")
            setattr(v, "shared_" + name, scratch.data_ptr())
            setattr(v, "packed_" + name, None)
        return v

    def workspace(self, num_tokens: int, device) -> torch.Tensor:
        lib = _native.load()
        need = int(lib.tris_moe_layer_workspace_bytes(C.byref(self.layer_view()), int(num_tokens)))
        if need == 0 and num_tokens > 0:
            raise RuntimeError("trismoe_b200: invalid layer view (workspace size query failed)")
        if self._workspace is None or self._workspace.numel() < need or self._workspace.device != device:
            if self._workspace is not None:
                self.raise_on_kernel_status()  # do not lose a report with the old buffer
            self._workspace = torch.empty((need,), dtype=torch.uint8, device=device)
            self._workspace[:16].zero_()  # count words and the sticky status word
        return self._workspace

    def last_kernel_status(self, clear: bool = True) -> int:
        """Status word of every kernel :meth:`forward` launched since the last clear: 0, or 6
        (``TRIS_ERR_TIMEOUT``) when a bounded device-side wait ran out and a CTA skipped its stores.
        Synchronises the current stream; call it where the host waits for the GPU anyway (end of a
        decode step, before results are handed on)."""
        streamed = 0
        if self._status_word is not None:
            streamed = int(self._status_word.item())
            if clear and streamed:
                self._status_word.zero_()
        if self._workspace is None:
            return streamed
        lib = _native.load()
        dev = self._workspace.device
        word = C.c_int32(0)
        with torch.cuda.device(dev):
            _native.check(lib.tris_moe_layer_last_status(self._workspace.data_ptr(), int(bool(clear)),
                                                         torch.cuda.current_stream(dev).cuda_stream, C.byref(word)),
                          "moe_layer_last_status")
        return int(word.value) or streamed

    def raise_on_kernel_status(self) -> None:
        """Raises ``RuntimeError`` if a kernel reported a time-out since the last check (the outputs
        of those calls are not trustworthy); the reference surfaces kernel failures as exceptions too."""
        status = self.last_kernel_status(clear=True)
        if status != 0:
            raise RuntimeError(f"trismoe_b200: a grouped kernel reported {_native.STATUS_NAMES.get(status, status)} "
                               "(TRIS_ERR_TIMEOUT: a bounded wait on a copy ran out; TRIS_ERR_WORKSPACE: a streamed batch activated "
                               "more experts than the staging manager has slots for; output rows of that launch are stale)")

    # -- forward ---------------------------------------------------------------------------
    def forward(self, hidden_states: torch.Tensor, router_logits: Optional[torch.Tensor] = None):
        """Returns ``(final_hidden_states [B, S, H], router_logits [T, E])`` like
        ``OlmoeSparseMoeBlock.forward`` (modeling_olmoe.py:1046-1105).  ``router_logits``
        (fp32 ``[T, E]``) may be passed in to skip the router linear."""
        _native.require_cuda(hidden_states, "TrisSparseMoeBlock.forward")
        if not envflags.grouped_experts_enabled() or self.input_scales or self.ns_payloads:
            # TRIS_GROUPED_EXPERTS=0, per-projection input scales or null-space pairs: operator by operator
            return self.forward_grouped_ops(hidden_states, router_logits)
        if hidden_states.dtype != torch.float16:
            raise RuntimeError(f"trismoe_b200: grouped expert kernels require float16 hidden states, got {hidden_states.dtype}")
        lib = _native.load()
        shape = hidden_states.shape
        x = hidden_states.reshape(-1, shape[-1]).contiguous()
        T = int(x.shape[0])
        dev = x.device
        y = torch.empty_like(x)
        if router_logits is not None:
            logits = router_logits.reshape(T, self.num_experts).to(torch.float32).contiguous()
            logits_in, logits_out = logits.data_ptr(), None
        else:
            logits = torch.empty((T, self.num_experts), dtype=torch.float32, device=dev)
            logits_in, logits_out = None, logits.data_ptr()
        if T:
            ws = self.workspace(T, dev)
            view = self.layer_view()
            if self.packed_backbones:  # gate and up see T rows, down T * top_k
                big = [n for n in self.packed_backbones
                       if (T * self.top_k if n == "down" else T) > self.PACKED_BACKBONE_MAX_ROWS]
                if "gate" in big or "up" in big:
                    big = sorted(set(big) | ({"gate", "up"} & set(self.packed_backbones)))
                if big:
                    view = self._expanded_layer_view(dev, big)
            with torch.cuda.device(dev):
                _native.check(
                    lib.tris_moe_layer_forward(C.byref(view), x.data_ptr(), logits_in, T, y.data_ptr(),
                                               logits_out, ws.data_ptr(), ws.numel(),
                                               torch.cuda.current_stream(dev).cuda_stream),
                    "moe_layer_forward",
                )
        return y.reshape(shape), logits

    def forward_streaming(self, hidden_states: torch.Tensor, manager, block_index: int,
                          router_logits: Optional[torch.Tensor] = None):
        """Forward with the expert payloads paged in by a
        :class:`~.staging.GroupedQGmapCPUStagingManager` (the streaming mode of
        ``OlmoeModel.forward``, modeling_olmoe.py:1305-1339): the route is built first, the
        pager for gate/up/down starts on the side stream and overlaps the input-side backbone
        GEMM; the grouped kernels wait on its event.  Nothing synchronises with the host."""
        _native.require_cuda(hidden_states, "TrisSparseMoeBlock.forward_streaming")
        lib = _native.load()
        shape = hidden_states.shape
        x = hidden_states.reshape(-1, shape[-1]).contiguous()
        T, dev = int(x.shape[0]), x.device
        E, k, H, I = self.num_experts, self.top_k, self.hidden_size, self.intermediate_size
        R = T * k
        y = torch.empty_like(x)
        if T == 0:
            return y.reshape(shape), x.new_zeros((0, E), dtype=torch.float32)
        stream = lambda: torch.cuda.current_stream(dev).cuda_stream
        f16 = torch.float16
        with torch.cuda.device(dev):
            if router_logits is None:
                logits = torch.empty((T, E), dtype=torch.float32, device=dev)
                _native.check(lib.tris_shared_hidden_forward(x.data_ptr(), None, T, None, H, self.gate.weight.data_ptr(), E,
                                                             logits.data_ptr(), 1, stream()), "router")
            else:
                logits = router_logits.reshape(T, E).to(torch.float32).contiguous()
            sel = torch.empty((T, k), dtype=torch.int32, device=dev)
            wts = torch.empty((T, k), dtype=torch.float32, device=dev)
            _native.check(lib.tris_router_topk(logits.data_ptr(), T, E, k, int(self.norm_topk_prob), sel.data_ptr(),
                                               wts.data_ptr(), stream()), "router_topk")
            buf = torch.empty((4 * R + 3 * E + 6,), dtype=torch.int32, device=dev)
            perm, tok, slot, rof = (buf[i * R:(i + 1) * R] for i in range(4))
            ids, seg = buf[4 * R: 4 * R + E], buf[4 * R + E: 4 * R + 2 * E + 1]
            prob, counts = buf[4 * R + 2 * E + 1: 4 * R + 3 * E + 2], buf[4 * R + 3 * E + 2: 4 * R + 3 * E + 6]
            _native.check(lib.tris_build_grouped_route(sel.data_ptr(), T, k, E, 4, perm.data_ptr(), tok.data_ptr(),
                                                       slot.data_ptr(), rof.data_ptr(), ids.data_ptr(), seg.data_ptr(),
                                                       prob.data_ptr(), counts.data_ptr(), stream()), "route")
            route = {"expert_ids": ids, "segment_offsets": seg, "counts": counts, "experts": E, "rows": R}
            paged = manager.page_layer(block_index, route)  # side stream, starts now

            r_gu, r_d = self.backbone_rank("gate"), self.backbone_rank("down")
            mode_gu, mode_d = (2 if r_gu % 32 == 0 else 0), (2 if r_d % 32 == 0 else 0)
            hg = self.backbone_hidden("gate", x, mode_gu)
            hu = self.backbone_hidden("up", x, mode_gu)
            rv = _native.TrisRouteView()
            rv.expert_ids, rv.segment_offsets, rv.num_segments_dev = ids.data_ptr(), seg.data_ptr(), counts.data_ptr()
            rv.num_segments, rv.num_rows, rv.max_rows_per_segment = min(E, R), R, T
            if self._status_word is None or self._status_word.device != dev:
                self._status_word = torch.zeros((1,), dtype=torch.int32, device=dev)
            rv.row_gather, rv.status_dev, rv.flags = tok.data_ptr(), self._status_word.data_ptr(), (1 if mode_gu else 0)
            paged.wait("gate_up")  # down keeps paging under the gate/up kernel and the down backbone
            mlp = torch.empty((R, I), dtype=f16, device=dev)
            _native.check(lib.tris_grouped_pair_forward(C.byref(paged.views["gate"]), C.byref(paged.views["up"]), C.byref(rv),
                                                        hg.data_ptr(), hu.data_ptr(), mlp.data_ptr(), None, 1, stream()),
                          "grouped_pair_forward")
            hd = self.backbone_hidden("down", mlp, mode_d)
            rv.row_gather, rv.flags = None, (1 if mode_d else 0)
            paged.wait("all")
            down = torch.empty((R, H), dtype=f16, device=dev)
            _native.check(lib.tris_grouped_forward(C.byref(paged.views["down"]), C.byref(rv), hd.data_ptr(), down.data_ptr(),
                                                   stream()), "grouped_forward")
            paged.release()
            _native.check(lib.tris_combine_routed(down.data_ptr(), rof.data_ptr(), wts.data_ptr(), T, k, H, y.data_ptr(),
                                                  stream()), "combine")
        return y.reshape(shape), logits

    def forward_grouped_ops(self, hidden_states: torch.Tensor, router_logits: Optional[torch.Tensor] = None):
        """Same result as :meth:`forward`, composed from the reference-named operators in
        the order of ``_forward_grouped`` (modeling_olmoe.py:916-1044); torch is used only
        for the glue the reference also does in torch (softmax/top-k, gathers, act*mul,
        index_add_)."""
        shape = hidden_states.shape
        x = hidden_states.reshape(-1, shape[-1])
        if router_logits is None:
            router_logits = torch.nn.functional.linear(x, self.gate.weight)
        if x.shape[0] == 0:
            return x.new_zeros(shape), router_logits
        routing = torch.softmax(router_logits, dim=1, dtype=torch.float)
        routing, selected = torch.topk(routing, self.top_k, dim=-1)
        if self.norm_topk_prob:
            routing = routing / routing.sum(dim=-1, keepdim=True)
        routing = routing.to(x.dtype)
        route = build_grouped_route(selected, self.num_experts)
        tok, slots = route["grouped_token_indices"], route["grouped_slots"]
        x_grouped = x.index_select(0, tok)
        grouped_routing = routing[tok, slots].unsqueeze(-1)
        gate_hidden = self.backbone_hidden("gate", x).index_select(0, tok)
        up_hidden = self.backbone_hidden("up", x).index_select(0, tok)
        gate_out, up_out = run_grouped_structured_expert_pair_forward(
            self._get_grouped_payload("gate"), self._get_grouped_payload("up"), gate_hidden, up_hidden, x_grouped, route,
            ns_payload_a=self.ns_payloads.get("gate"), ns_payload_b=self.ns_payloads.get("up"))
        mlp = torch.nn.functional.silu(gate_out) * up_out
        down_hidden = self.backbone_hidden("down", mlp)
        down_out = run_grouped_structured_expert_forward(self._get_grouped_payload("down"), down_hidden, mlp, route,
                                                         ns_payload=self.ns_payloads.get("down"))
        # weighted sum of every token's k expert rows, taken in slot order (the reference scatters them with
        # index_add_, whose atomic order varies from run to run; this is the same sum, reproducible)
        weighted = (down_out * grouped_routing).to(x.dtype)
        rows_of_token = route["_row_of_flat"].to(torch.long)
        final = weighted.index_select(0, rows_of_token).view(x.shape[0], self.top_k, x.shape[1]).float().sum(dim=1).to(x.dtype)
        return final.reshape(shape), router_logits


class TrisQwen2SparseMoeBlock(TrisSparseMoeBlock):
    """``Qwen2MoeSparseMoeBlock`` of the reference (modeling_qwen2_moe.py:249-822): the routed experts
    of :class:`TrisSparseMoeBlock` plus one always-on shared expert - a dense gate/up/down MLP of
    ordinary compact3 linears whose output is scaled by ``sigmoid(shared_expert_gate(x))`` and added
    (modeling_qwen2_moe.py:815-818).  The shared expert's gate and up run as one dual launch with
    SiLU*mul fused (``run_compact3_shared_expert_gate_up_forward``, modeling_qwen2_moe.py:117-123)."""

    def __init__(self, hidden_size: int, intermediate_size: int, num_experts: int, num_experts_per_tok: int,
                 norm_topk_prob: bool = False):
        super().__init__(hidden_size, intermediate_size, num_experts, num_experts_per_tok, norm_topk_prob)
        self.shared_expert_gate = nn.Linear(self.hidden_size, 1, bias=False, dtype=torch.float16)
        self.shared_expert = None  # (gate, up, down) Compact3Linear

    def load_shared_expert(self, gate_proj, up_proj, down_proj, shared_expert_gate_weight: torch.Tensor, device=None):
        """``gate_proj`` / ``up_proj`` / ``down_proj``: :class:`~.compact3_linear.Compact3Linear` modules or the
        per-module compact3 payload dicts they are built from; ``shared_expert_gate_weight``: ``[1, hidden]``."""
        from .compact3_linear import Compact3Linear

        dev = torch.device(device) if device is not None else self.gate.weight.device
        mods = [m if isinstance(m, Compact3Linear) else Compact3Linear(m, device=dev) for m in (gate_proj, up_proj, down_proj)]
        self.shared_expert = tuple(mods)
        self.shared_expert_gate.weight = nn.Parameter(shared_expert_gate_weight.reshape(1, self.hidden_size).to(dev, torch.float16).contiguous(),
                                                      requires_grad=False)
        return self

    def forward(self, hidden_states: torch.Tensor, router_logits: Optional[torch.Tensor] = None):
        from .compact3_linear import run_compact3_gate_up_forward

        if self.shared_expert is None:
            raise RuntimeError("trismoe_b200: the shared expert was not loaded (load_shared_expert)")
        routed, logits = super().forward(hidden_states, router_logits)
        gate_proj, up_proj, down_proj = self.shared_expert
        mlp = run_compact3_gate_up_forward(gate_proj, up_proj, hidden_states, fuse_silu_mul=True)
        shared = down_proj(mlp)
        if shared is None:
            raise RuntimeError("trismoe_b200: shared expert kernels returned no result")
        scale = torch.sigmoid(torch.nn.functional.linear(hidden_states, self.shared_expert_gate.weight))
        return routed + scale * shared, logits
