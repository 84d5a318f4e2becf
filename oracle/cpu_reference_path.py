"""CPU port of the reference's expert-loop MoE path, used ONLY as the timed CPU baseline of
the benchmark and as a checker in tests (test infrastructure, never on the product path).

It mirrors what the TriS-MoE reference executes on CPU when its CUDA extension is absent
(paths inside the TriS-MoE tree): OlmoeSparseMoeBlock.forward -> _forward_expert_loop
(modeling_olmoe.py:1046-1105, 854-914): fp16 router linear, fp32 softmax, top-k,
renormalisation; compute_shared_hidden = F.linear with the fp16 backbone
(qlinear_cuda.py:4454-4502); per active expert forward_from_precomputed_hidden
(qlinear_cuda.py:4504-4566) = _dequantize_compact3_matrix (qlinear_cuda.py:4200-4236, torch
fp16 tensor ops on the unpacked bit planes, redone on every call) followed by F.linear;
deferred down projection over the concatenated rows; index_add_ of the weighted outputs.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F


def _unpack_rows(packed: torch.Tensor, ncols: int) -> torch.Tensor:
    """int32 [rows, O] -> bool [O, ncols] (qlinear_cuda.py:3651-3656)."""
    shifts = torch.arange(32, dtype=torch.int64).view(1, 1, 32)
    bits = ((packed.to(torch.int64).unsqueeze(-1) >> shifts) & 1).permute(0, 2, 1).reshape(-1, packed.shape[1])
    return bits[:ncols].t().contiguous().bool()


def _unpack_vector(packed: torch.Tensor, n: int) -> torch.Tensor:
    shifts = torch.arange(32, dtype=torch.int64).view(1, 32)
    return ((packed.to(torch.int64).unsqueeze(-1) >> shifts) & 1).reshape(-1)[:n].bool()


def _unpack_half4(packed: torch.Tensor):
    p = packed.to(torch.int64)
    return tuple(((p >> s) & 0xFFFF).to(torch.int16).view(torch.float16) for s in (0, 16, 32, 48))


def dequantize_expert(payload: dict, e: int) -> torch.Tensor:
    """fp16 [O, r] with the tensor-op sequence of _dequantize_compact3_matrix."""
    qw1 = payload["qweight1"][e]
    O = qw1.shape[1]
    r = payload["g_idx"].shape[1]
    dt = torch.float16
    b1 = _unpack_rows(qw1, r).to(dt).mul_(2).sub_(1)
    sal = _unpack_vector(payload["c_map"][e], r)
    nsal = ~sal
    b2 = torch.zeros((O, r), dtype=torch.bool)
    ns = int(sal.sum())
    if ns:
        b2[:, sal] = _unpack_rows(payload["qweight2_sparse"][e], ns)
    b2 = b2.to(dt).mul_(2).sub_(1)
    g = torch.zeros((O, r), dtype=torch.bool)
    nn_ = int(nsal.sum())
    if nn_:
        g[:, nsal] = _unpack_rows(payload["q_gmap_sparse"][e], nn_)
    s_c1, s_c2, d_c, nd_c = _unpack_half4(payload["col_pack3"][e])
    gi = payload["g_idx"][e].long()
    s_r1, s_r2, d_r, nd_r = (t[:, gi] for t in _unpack_half4(payload["row_pack3"][e]))
    sal_m = sal.unsqueeze(0).expand(O, -1)
    d_m = nsal.unsqueeze(0).expand(O, -1) & g
    nd_m = nsal.unsqueeze(0).expand(O, -1) & ~g
    w = torch.zeros((O, r), dtype=dt)
    w += b1 * (s_r1 * s_c1.unsqueeze(0)) * sal_m.to(dt)
    w += b2 * (s_r2 * s_c2.unsqueeze(0)) * sal_m.to(dt)
    w += b1 * (d_r * d_c.unsqueeze(0)) * d_m.to(dt)
    w += b1 * (nd_r * nd_c.unsqueeze(0)) * nd_m.to(dt)
    return w


def moe_block_forward(x: torch.Tensor, layer: dict, top_k: int, norm_topk_prob: bool,
                      router_logits: torch.Tensor | None = None) -> torch.Tensor:
    """x [T, H] fp16 on CPU -> [T, H] fp16; ``layer`` holds CPU payloads with the sparse
    g_map plane (``keep_sparse_gmap=True``), the three backbones and the router weight."""
    T, H = x.shape
    E = layer["gate"]["qweight1"].shape[0]
    if router_logits is None:
        router_logits = F.linear(x, layer["router_weight"])
    routing = F.softmax(router_logits, dim=1, dtype=torch.float)
    routing, selected = torch.topk(routing, top_k, dim=-1)
    if norm_topk_prob:
        routing = routing / routing.sum(dim=-1, keepdim=True)
    routing = routing.to(x.dtype)
    final = torch.zeros((T, H), dtype=x.dtype)
    mask = F.one_hot(selected, num_classes=E).permute(2, 1, 0)
    gate_all = F.linear(x, layer["shared_gate"])
    up_all = F.linear(x, layer["shared_up"])
    deferred = []
    for e in range(E):
        idx, top_x = torch.where(mask[e])
        if top_x.numel() == 0:
            continue
        gate_out = F.linear(gate_all.index_select(0, top_x), dequantize_expert(layer["gate"], e))
        up_out = F.linear(up_all.index_select(0, top_x), dequantize_expert(layer["up"], e))
        deferred.append((e, top_x, idx, F.silu(gate_out) * up_out))
    if deferred:
        down_all = F.linear(torch.cat([m for *_, m in deferred], dim=0), layer["shared_down"])
        start = 0
        for e, top_x, idx, mlp in deferred:
            end = start + mlp.shape[0]
            out = F.linear(down_all[start:end], dequantize_expert(layer["down"], e))
            final.index_add_(0, top_x, (out * routing[top_x, idx, None]).to(x.dtype))
            start = end
    return final
