"""Ordinary (non-expert) compact3 linears on the grouped kernels: the attention q/k/v/o
projections and the Qwen shared expert of a TriS-MoE checkpoint (``QuantLinear`` mode 4 of the
reference: ``_run_compact3_cuda``, qlinear_cuda.py:4238-4361 -> ``compact3_linear_forward``,
TriSMoE_cuda_kernel.cu:2146-3743; fused QKV ``run_compact3_qkv_block_gr_forward``,
qlinear_cuda.py:915-1022; dual gate/up of the shared expert, qlinear_cuda.py:1025-1099).

An ordinary linear is the grouped operator with one expert and one segment that holds every row,
so it runs on the same tile-record kernels: ``y = x @ dequant(W).T`` with ``W`` the compact3
matrix ``[out_features, in_features]`` (the columns are the layer's input features, several
256-column chunks), optionally ``x`` scaled per input column and ``y`` per output row
(``ns_mode == 1``: ``ns_vector_col`` / ``ns_vector_row``) and a bias.  Null-space matrices of rank
> 0 are not supported.  There is no CPU path: tensors must live on a CUDA device.
"""
from __future__ import annotations

from typing import Optional

import torch
from torch import nn

from . import _native, envflags
from .formats import stack_expert_payloads
from .qlinear_grouped import (
    prepare_grouped_payload,
    run_grouped_structured_expert_forward,
    run_grouped_structured_expert_pair_forward,
)


class Compact3Linear(nn.Module):
    """One compact3 linear.  ``payload`` is the per-module dict of ``build_compact3_packed_payload``
    (utils/pack_utils.py:67-125) or an already stacked single-expert payload."""

    def __init__(self, payload: dict, bias: Optional[torch.Tensor] = None, ns_vector_row: Optional[torch.Tensor] = None,
                 ns_vector_col: Optional[torch.Tensor] = None, device=None):
        super().__init__()
        stacked = payload if payload["qweight1"].dim() == 3 else stack_expert_payloads([payload], use_block_gr=True)
        if int(stacked["qweight1"].shape[0]) != 1:
            raise RuntimeError("trismoe_b200 Compact3Linear: the payload must hold exactly one matrix")
        dev = torch.device(device) if device is not None else stacked["qweight1"].device
        out_features = int(stacked["qweight1"].shape[2])
        if ns_vector_row is not None:  # output scale of ns_mode == 1 (has_output_scale, qlinear_cuda.py:4254-4258)
            stacked["output_scale"] = ns_vector_row.reshape(1, out_features).to(torch.float16)
            stacked["has_output_scale"] = True
        if bias is not None:
            stacked["bias"] = bias.reshape(1, out_features).to(torch.float16)
            stacked["has_bias"] = True
        self.payload = prepare_grouped_payload(stacked, dev)
        self.in_features = int(self.payload["g_idx"].shape[-1])
        self.out_features = out_features
        self.input_scale = None if ns_vector_col is None else ns_vector_col.reshape(self.in_features).to(dev, torch.float16).contiguous()

    def _route(self, rows: int, device) -> dict:
        zero = torch.zeros((1,), dtype=torch.int32, device=device)
        route = {"expert_ids": zero, "segment_offsets": torch.tensor([0, rows], dtype=torch.int32, device=device),
                 "_max_rows_per_segment": rows}
        if self.input_scale is not None:
            route["_hidden_col_scale"] = self.input_scale
        return route

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        _native.require_cuda(x, "Compact3Linear.forward")
        if x.dtype != torch.float16 or x.shape[-1] != self.in_features:
            return envflags.return_or_raise_none("Compact3Linear.forward", "fp16 input of the layer's in_features required")
        x2 = x.reshape(-1, self.in_features).contiguous()
        y = run_grouped_structured_expert_forward(self.payload, x2, None, self._route(int(x2.shape[0]), x.device))
        return None if y is None else y.reshape(x.shape[:-1] + (self.out_features,))


def _same_shape(*mods: Compact3Linear) -> bool:
    return all(m.in_features == mods[0].in_features and m.out_features == mods[0].out_features for m in mods)


def run_compact3_qkv_forward(q_proj: Compact3Linear, k_proj: Compact3Linear, v_proj: Compact3Linear, hidden_states: torch.Tensor):
    """``(q, k, v)`` of one attention block (``run_compact3_qkv_block_gr_forward``,
    qlinear_cuda.py:915-1022).  k and v share the activation staging of one launch when they
    have the same shape (the gate/up dual kernel, two projections per CTA); q runs in its own
    launch (with grouped-query attention its width differs from k/v's)."""
    _native.require_cuda(hidden_states, "run_compact3_qkv_forward")
    if any(m.input_scale is not None for m in (q_proj, k_proj, v_proj)):
        return envflags.return_or_raise_none("run_compact3_qkv_forward", "input scales are not supported by the fused form")
    if hidden_states.dtype != torch.float16 or hidden_states.shape[-1] != q_proj.in_features:
        return envflags.return_or_raise_none("run_compact3_qkv_forward", "fp16 input of the layer's in_features required")
    x2 = hidden_states.reshape(-1, q_proj.in_features).contiguous()
    rows = int(x2.shape[0])
    lead = hidden_states.shape[:-1]
    q = run_grouped_structured_expert_forward(q_proj.payload, x2, None, q_proj._route(rows, x2.device))
    if _same_shape(k_proj, v_proj):
        k, v = run_grouped_structured_expert_pair_forward(k_proj.payload, v_proj.payload, x2, x2, None, k_proj._route(rows, x2.device))
    else:
        k = run_grouped_structured_expert_forward(k_proj.payload, x2, None, k_proj._route(rows, x2.device))
        v = run_grouped_structured_expert_forward(v_proj.payload, x2, None, v_proj._route(rows, x2.device))
    if q is None or k is None or v is None:
        return None
    return (q.reshape(lead + (q_proj.out_features,)), k.reshape(lead + (k_proj.out_features,)),
            v.reshape(lead + (v_proj.out_features,)))


def run_compact3_gate_up_forward(gate_proj: Compact3Linear, up_proj: Compact3Linear, hidden_states: torch.Tensor,
                                 fuse_silu_mul: bool = True):
    """Gate and up of a dense MLP (the Qwen shared expert) in one launch
    (``run_compact3_dual_gate_up_block_gr_forward``, qlinear_cuda.py:1025-1099); with
    ``fuse_silu_mul`` returns ``silu(gate) * up`` computed in fp32 inside the kernel, else
    ``(gate, up)``."""
    _native.require_cuda(hidden_states, "run_compact3_gate_up_forward")
    if not _same_shape(gate_proj, up_proj) or gate_proj.input_scale is not None or up_proj.input_scale is not None:
        return envflags.return_or_raise_none("run_compact3_gate_up_forward", "gate and up must share their shape and have no input scale")
    x2 = hidden_states.reshape(-1, gate_proj.in_features).contiguous()
    a, b = run_grouped_structured_expert_pair_forward(gate_proj.payload, up_proj.payload, x2, x2, None,
                                                      gate_proj._route(int(x2.shape[0]), x2.device), fuse_silu_mul=fuse_silu_mul)
    lead = hidden_states.shape[:-1]
    if a is None:
        return None
    if fuse_silu_mul:
        return a.reshape(lead + (gate_proj.out_features,))
    return a.reshape(lead + (gate_proj.out_features,)), b.reshape(lead + (up_proj.out_features,))
