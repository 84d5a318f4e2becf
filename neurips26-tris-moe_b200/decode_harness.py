"""End-to-end decode harness: a decoder stack whose MoE layers run on the trismoe_b200 kernels,
with fp16 attention and a KV cache around them, and the generation loop of the reference's
latency benchmark (``tools/benchmark_e2e_grid.py:325-420``, ``run_exact_generation``: exactly
``output_length`` tokens, greedy argmax inside the loop, synchronisation at phase boundaries only,
``decode_tokens_per_s = batch * decode_steps / decode_time``).

The attention half is plain PyTorch (``scaled_dot_product_attention`` over a preallocated cache):
it is the fixed fp16 context the MoE path is measured in, not part of the product.  The decode step
has static shapes - the cache has its full length from the start and a position tensor masks the
unwritten tail - so one step is captured into a CUDA graph and replayed ``output_length - 1`` times
with no host work between steps.
"""
from __future__ import annotations

import math
import time
from dataclasses import dataclass
from typing import List, Optional

import torch
import torch.nn.functional as F

from .moe_block import TrisSparseMoeBlock


@dataclass
class DecoderShape:
    hidden_size: int = 2048
    num_heads: int = 16
    head_dim: int = 128
    num_kv_heads: int = 16
    vocab_size: int = 50304
    rope_theta: float = 10000.0
    rms_eps: float = 1e-5


def _rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    return F.rms_norm(x, (x.shape[-1],), weight, eps)  # one kernel; statistics in fp32


def _rope_tables(max_length: int, head_dim: int, theta: float, device):
    """cos / sin of every (position, frequency), fp32 [max_length, head_dim / 2]."""
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, device=device, dtype=torch.float32) / head_dim))
    ang = torch.arange(max_length, device=device, dtype=torch.float32)[:, None] * inv
    return ang.cos().contiguous(), ang.sin().contiguous()


def _rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x [B, heads, S, D]; cos / sin [B, 1, S, D/2] (fp32, already gathered at the tokens' positions)."""
    d = x.shape[-1]
    x1, x2 = x[..., : d // 2].float(), x[..., d // 2:].float()
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1).to(x.dtype)


class TrisDecoder(torch.nn.Module):
    """``len(moe_blocks)`` decoder layers: RMSNorm -> attention (fp16, KV cache) -> RMSNorm -> MoE."""

    def __init__(self, moe_blocks: List[TrisSparseMoeBlock], shape: DecoderShape, max_length: int, max_batch: int,
                 device, seed: int = 0):
        super().__init__()
        self.shape, self.blocks = shape, list(moe_blocks)
        self.max_length, self.max_batch = int(max_length), int(max_batch)
        dev = torch.device(device)
        g = torch.Generator(device="cpu").manual_seed(seed)
        H, hd, nh, nkv = shape.hidden_size, shape.head_dim, shape.num_heads, shape.num_kv_heads
        rnd = lambda *s, std: (torch.randn(*s, generator=g) * std).to(dev, torch.float16)
        self.embed = rnd(shape.vocab_size, H, std=1.0)
        self.lm_head = rnd(shape.vocab_size, H, std=1.0 / math.sqrt(H))
        self.final_norm = torch.ones(H, dtype=torch.float16, device=dev)
        self.rope_cos, self.rope_sin = _rope_tables(self.max_length, hd, shape.rope_theta, dev)
        self.key_index = torch.arange(self.max_length, device=dev)[None, None, None, :]
        self.layers = []
        for _ in self.blocks:
            self.layers.append({
                "ln1": torch.ones(H, dtype=torch.float16, device=dev), "ln2": torch.ones(H, dtype=torch.float16, device=dev),
                "wqkv": rnd((nh + 2 * nkv) * hd, H, std=1.0 / math.sqrt(H)), "wo": rnd(H, nh * hd, std=1.0 / math.sqrt(nh * hd)),
                "k": torch.zeros((max_batch, nkv, max_length, hd), dtype=torch.float16, device=dev),
                "v": torch.zeros((max_batch, nkv, max_length, hd), dtype=torch.float16, device=dev),
            })

    def _attention(self, layer: dict, x: torch.Tensor, positions: torch.Tensor, batch: int, rope, mask) -> torch.Tensor:
        """x [B, S, H]; positions [B, S] absolute positions of these tokens.  Writes K/V at the
        positions and attends over cache entries <= the token's own position.  ``rope`` (cos, sin at the
        positions) and ``mask`` are the same for every layer of a step and are built once per step."""
        s = self.shape
        B, S, _ = x.shape
        nq, nkv = s.num_heads, s.num_kv_heads
        qkv = F.linear(x, layer["wqkv"]).view(B, S, nq + 2 * nkv, s.head_dim).transpose(1, 2)
        qk = _rope(qkv[:, : nq + nkv], *rope)  # queries and keys rotate together
        q, k, v = qk[:, :nq], qk[:, nq:], qkv[:, nq + nkv:]
        idx = positions[:, None, :, None].expand(B, nkv, S, s.head_dim)
        layer["k"][:batch].scatter_(2, idx, k)
        layer["v"][:batch].scatter_(2, idx, v)
        keys, vals = layer["k"][:batch], layer["v"][:batch]
        if nkv != nq:
            rep = nq // nkv
            keys, vals = keys.repeat_interleave(rep, dim=1), vals.repeat_interleave(rep, dim=1)
        out = F.scaled_dot_product_attention(q, keys, vals, attn_mask=mask)
        return F.linear(out.transpose(1, 2).reshape(B, S, nq * s.head_dim), layer["wo"])

    def forward(self, token_ids: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
        """token_ids, positions [B, S] -> logits of the last position [B, vocab] (fp32)."""
        B, S = token_ids.shape
        h = F.embedding(token_ids, self.embed)
        rope = (self.rope_cos[positions][:, None], self.rope_sin[positions][:, None])  # [B, 1, S, D/2]
        mask = self.key_index <= positions[:, None, :, None]
        for layer, blk in zip(self.layers, self.blocks):
            h = h + self._attention(layer, _rms_norm(h, layer["ln1"], self.shape.rms_eps), positions, B, rope, mask)
            y, _ = blk(_rms_norm(h, layer["ln2"], self.shape.rms_eps))
            h = h + y
        last = _rms_norm(h[:, -1], self.final_norm, self.shape.rms_eps)
        return F.linear(last, self.lm_head).float()


def run_exact_generation(model: TrisDecoder, input_ids: torch.Tensor, output_length: int, use_graph: bool = True,
                         measure_latency: bool = True) -> dict:
    """Prefill ``input_ids`` [B, L], then generate exactly ``output_length`` tokens greedily.  Returns the
    reference benchmark's fields (prefill_ms, decode_ms, decode_tokens_per_s, ...) and the tokens."""
    dev = input_ids.device
    B, L = (int(v) for v in input_ids.shape)
    if L + output_length > model.max_length or B > model.max_batch:
        raise RuntimeError("trismoe_b200 decode harness: cache too small for this prompt / output length / batch")
    decode_steps = max(output_length - 1, 0)
    sync = lambda: torch.cuda.synchronize(dev)
    positions = torch.arange(L, device=dev)[None, :].expand(B, L).contiguous()
    sync()
    t0 = time.perf_counter()
    with torch.no_grad():
        logits = model(input_ids, positions)
    sync()
    t1 = time.perf_counter()
    tokens = torch.empty((B, output_length), dtype=torch.long, device=dev)
    cur = logits.argmax(dim=-1, keepdim=True)  # [B, 1]
    pos = torch.full((B, 1), L, dtype=torch.long, device=dev)
    tokens[:, 0:1] = cur
    step_index = torch.ones((1,), dtype=torch.long, device=dev)

    def step():
        with torch.no_grad():
            nxt = model(cur, pos).argmax(dim=-1, keepdim=True)
            cur.copy_(nxt)
            tokens.index_copy_(1, step_index, nxt)
            pos.add_(1)
            step_index.add_(1)

    graph = None
    if use_graph and decode_steps > 1:
        # warm up on a side stream with the state restored afterwards, then capture one step
        saved = (cur.clone(), pos.clone(), step_index.clone(), tokens.clone())
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            step()
        torch.cuda.current_stream(dev).wait_stream(side)
        sync()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            step()
        for dst, src in zip((cur, pos, step_index, tokens), saved):
            dst.copy_(src)
    sync()
    t2 = time.perf_counter()
    for _ in range(decode_steps):
        if graph is not None:
            graph.replay()
        else:
            step()
    sync()
    t3 = time.perf_counter()
    prefill_ms, decode_ms = (t1 - t0) * 1e3, (t3 - t2) * 1e3
    out = {"batch_size": B, "input_length": L, "output_length": output_length, "decode_steps": decode_steps, "tokens": tokens,
           "launch_mode": "cuda graph" if graph is not None else "eager"}
    if measure_latency:
        out.update({
            "prefill_ms": prefill_ms, "decode_ms": decode_ms,
            "avg_decode_step_ms": decode_ms / decode_steps if decode_steps else 0.0,
            "prefill_tokens_per_s": B * L * 1e3 / prefill_ms,
            "decode_tokens_per_s": B * decode_steps * 1e3 / decode_ms if decode_steps and decode_ms > 0 else 0.0,
        })
    return out
