"""CPU oracle for the grouped-expert dequant-GEMM path of TriS-MoE.  TEST INFRASTRUCTURE:
only the tests, the smoke check and the CPU-baseline leg of the benchmark may import it;
nothing the library ships routes through it.

It restates, in numpy, the reference algorithm (paths inside the TriS-MoE tree):
  * block Golomb-Rice decode      - decode_block_gr_block,
                                    AutoGPTQ/autogptq_extension/TriSMoE/TriSMoE_cuda_kernel.cu:426-479
                                    (the reference has no CPU decoder; the encoder it inverts is
                                    QuantLinear._pack_block_gr_gmap_tensor, qlinear_cuda.py:3793-3859)
  * compact3 dequantisation       - QuantLinear._dequantize_compact3_matrix, qlinear_cuda.py:4200-4236
  * MoE block, expert loop        - OlmoeSparseMoeBlock.forward / _forward_expert_loop,
                                    modeling_olmoe.py:1046-1105 / 854-914
  * grouped route                 - build_grouped_route, qlinear_cuda.py:1301-1378

Pinning: tests/test_oracle_golden.py checks every function here against fixtures produced
by running the reference's own Python code (tests/golden/make_golden.py).
"""
from __future__ import annotations

import math

import numpy as np

GR_BLOCK_OUT = 64
GR_BLOCK_ROWS = 2
GR_BLOCK_WORDS = 128
GR_META_K_MASK = 0xF
GR_META_RAW = 16
GR_META_ONES_SHIFT = 8


def _u32(a) -> np.ndarray:
    return np.ascontiguousarray(np.asarray(a)).astype(np.int64).astype(np.uint32) if np.asarray(a).dtype != np.uint32 else np.asarray(a)


def _to_u32(a) -> np.ndarray:
    a = np.ascontiguousarray(np.asarray(a))
    if a.dtype == np.int32:
        return a.view(np.uint32)
    return (a.astype(np.int64) & 0xFFFFFFFF).astype(np.uint32)


# ---------------------------------------------------------------------------------------
# block Golomb-Rice
# ---------------------------------------------------------------------------------------
def gr_decode_block(words: np.ndarray, meta: int) -> np.ndarray:
    """One block -> 128 uint32 words.  Follows TriSMoE_cuda_kernel.cu:426-479: zero the
    block; raw blocks are copied; otherwise ``one_count`` times read a unary quotient up to
    the terminating one, then k remainder bits LSB first, advance, set the bit, advance by
    one; stop when the position leaves the 4096-bit block or the stream ends."""
    out = np.zeros(GR_BLOCK_WORDS, dtype=np.uint32)
    n = len(words)
    if n <= 0:
        return out
    if meta & GR_META_RAW:
        m = min(n, GR_BLOCK_WORDS)
        out[:m] = words[:m]
        return out
    k = meta & GR_META_K_MASK
    ones = meta >> GR_META_ONES_SHIFT
    bits = np.unpackbits(np.ascontiguousarray(words).view(np.uint8), bitorder="little")
    total = bits.size
    one_pos = np.flatnonzero(bits)
    bp = 0
    fp = 0
    for _ in range(ones):
        # quotient: zeros up to the next one (or to the end of the stream)
        j = np.searchsorted(one_pos, bp)
        if j < one_pos.size:
            q = int(one_pos[j]) - bp
            bp = int(one_pos[j]) + 1
        else:
            q = total - bp
            bp = total
        rem = 0
        for s in range(k):
            if bp < total:
                rem |= int(bits[bp]) << s
                bp += 1
        fp += (q << k) | rem
        if fp >= GR_BLOCK_WORDS * 32:
            break
        out[fp >> 5] |= np.uint32(1 << (fp & 31))
        fp += 1
    return out


def gr_decode_tensor(words, offsets, meta, packed_rows: int, out_features: int) -> np.ndarray:
    """Whole stream of one expert -> dense packed g_map uint32 [packed_rows, out_features].
    Block order: k_block outer, out_block inner (qlinear_cuda.py:3809-3811); block word
    layout [local packed row][local out]."""
    words, offsets, meta = _to_u32(words), np.asarray(offsets).astype(np.int64), np.asarray(meta).astype(np.int64)
    nkb = math.ceil(packed_rows / GR_BLOCK_ROWS)
    nob = math.ceil(out_features / GR_BLOCK_OUT)
    dense = np.zeros((nkb * GR_BLOCK_ROWS, nob * GR_BLOCK_OUT), dtype=np.uint32)
    b = 0
    for kb in range(nkb):
        for ob in range(nob):
            blk = gr_decode_block(words[offsets[b]: offsets[b + 1]], int(meta[b]))
            dense[kb * 2: kb * 2 + 2, ob * 64: ob * 64 + 64] = blk.reshape(2, 64)
            b += 1
    return dense[:packed_rows, :out_features]


# ---------------------------------------------------------------------------------------
# compact3
# ---------------------------------------------------------------------------------------
def unpack_rows(packed, ncols: int) -> np.ndarray:
    """uint32 [rows, O] -> bool [O, ncols]; bit j of word [p, o] is column 32p+j of output o
    (utils/pack_utils.py:19-29)."""
    w = _to_u32(packed)
    if w.size == 0:
        return np.zeros((w.shape[1] if w.ndim == 2 else 0, ncols), dtype=bool)
    bits = np.unpackbits(np.ascontiguousarray(w.T).view(np.uint8), axis=-1, bitorder="little")
    return bits[:, :ncols].astype(bool)


def unpack_vector(packed, n: int) -> np.ndarray:
    return np.unpackbits(_to_u32(packed).view(np.uint8), bitorder="little")[:n].astype(bool)


def unpack_half4(packed) -> tuple:
    """int64 -> four fp16 arrays from bits 0/16/32/48 (utils/pack_utils.py:55-64)."""
    w = np.ascontiguousarray(np.asarray(packed)).astype(np.int64).view(np.uint64)
    return tuple(((w >> np.uint64(s)) & np.uint64(0xFFFF)).astype(np.uint16).view(np.float16) for s in (0, 16, 32, 48))


def restore_sparse(packed_sparse, active_cols: np.ndarray, out_features: int) -> np.ndarray:
    """Sparse plane (only the active columns, ascending) -> dense bool [O, ncols]
    (_restore_dense_sparse_bool_matrix, qlinear_cuda.py:3748-3754)."""
    dense = np.zeros((out_features, active_cols.size), dtype=bool)
    n = int(active_cols.sum())
    if n and np.asarray(packed_sparse).size:
        dense[:, active_cols] = unpack_rows(packed_sparse, n)
    return dense


def dequantize_compact3(qweight1, qweight2_sparse, gmap_dense_bits, c_map, g_idx, col_pack3, row_pack3,
                        ncols: int) -> np.ndarray:
    """fp16 [O, ncols].  Arithmetic of qlinear_cuda.py:4200-4236 evaluated in fp16: every
    scale product is rounded to fp16, the salient weight is fp16(+-p1 +- p2); sign bit 1
    means +.  ``gmap_dense_bits`` is bool [O, ncols] (already expanded)."""
    O = int(np.asarray(qweight1).shape[1])
    f16 = np.float16
    b1 = unpack_rows(qweight1, ncols).astype(f16) * f16(2) - f16(1)
    sal = unpack_vector(c_map, ncols)
    b2 = restore_sparse(qweight2_sparse, sal, O).astype(f16) * f16(2) - f16(1)
    g = np.asarray(gmap_dense_bits, dtype=bool) & ~sal[None, :]
    s_c1, s_c2, d_c, nd_c = unpack_half4(col_pack3)
    s_r1, s_r2, d_r, nd_r = (t.reshape(O, -1)[:, np.asarray(g_idx).astype(np.int64)] for t in unpack_half4(row_pack3))
    p1 = (s_r1 * s_c1[None, :]).astype(f16)
    p2 = (s_r2 * s_c2[None, :]).astype(f16)
    pd = (d_r * d_c[None, :]).astype(f16)
    pn = (nd_r * nd_c[None, :]).astype(f16)
    w_sal = ((b1 * p1).astype(f16) + (b2 * p2).astype(f16)).astype(f16)
    w_ns = np.where(g, (b1 * pd).astype(f16), (b1 * pn).astype(f16))
    return np.where(sal[None, :], w_sal, w_ns).astype(f16)


def expert_dense_gmap_bits(payload: dict, e: int) -> np.ndarray:
    """bool [O, r] grouping bits of expert e from whichever encoding the payload holds."""
    O = int(payload["qweight1"].shape[2])
    r = int(payload["g_idx"].shape[1])
    pr = math.ceil(r / 32)
    if payload.get("compact3_use_block_gr") and np.asarray(payload["q_gmap_gr_offsets"]).size:
        dense = gr_decode_tensor(np.asarray(payload["q_gmap_gr_words"][e]), np.asarray(payload["q_gmap_gr_offsets"][e]),
                                 np.asarray(payload["q_gmap_gr_meta"][e]), pr, O)
        return unpack_rows(dense, r)
    sal = unpack_vector(np.asarray(payload["c_map"][e]), r)
    return restore_sparse(np.asarray(payload["q_gmap_sparse"][e]), ~sal, O)


def dequantize_expert(payload: dict, e: int) -> np.ndarray:
    """fp16 [O, r] weight of expert e of an E-stacked payload (numpy arrays or CPU tensors)."""
    r = int(payload["g_idx"].shape[1])
    a = lambda k: np.asarray(payload[k][e])
    w = dequantize_compact3(a("qweight1"), a("qweight2_sparse"), expert_dense_gmap_bits(payload, e), a("c_map"),
                            a("g_idx"), a("col_pack3"), a("row_pack3"), r)
    return w


# ---------------------------------------------------------------------------------------
# route and MoE block
# ---------------------------------------------------------------------------------------
def build_route(selected: np.ndarray, num_experts: int, m_tile: int = 4) -> dict:
    """Grouped route of qlinear_cuda.py:1301-1378 with a stable sort (rows of an expert in
    ascending flat (token, slot) order)."""
    T, k = selected.shape
    flat = selected.reshape(-1).astype(np.int64)
    perm = np.argsort(flat, kind="stable")
    counts = np.bincount(flat, minlength=num_experts)
    active = np.flatnonzero(counts > 0)
    lengths = counts[active]
    return {
        "perm": perm,
        "grouped_token_indices": perm // k,
        "grouped_slots": perm % k,
        "grouped_expert_ids": flat[perm].astype(np.int32),
        "expert_ids": active.astype(np.int32),
        "segment_offsets": np.concatenate([[0], np.cumsum(lengths)]).astype(np.int32),
        "problem_offsets": np.concatenate([[0], np.cumsum((lengths + m_tile - 1) // m_tile)]).astype(np.int32),
        "total_problem_tiles_host": int(((lengths + m_tile - 1) // m_tile).sum()),
    }


def router_topk(logits: np.ndarray, top_k: int, norm: bool):
    """softmax (fp32) -> top-k -> optional renormalisation (modeling_olmoe.py:1052-1057).
    Ties go to the lower expert index."""
    z = logits.astype(np.float32)
    z = z - z.max(axis=1, keepdims=True)
    p = np.exp(z)
    p = p / p.sum(axis=1, keepdims=True)
    order = np.argsort(-p, axis=1, kind="stable")[:, :top_k]
    w = np.take_along_axis(p, order, axis=1)
    if norm:
        w = w / w.sum(axis=1, keepdims=True)
    return order.astype(np.int32), w.astype(np.float32)


def moe_layer_fp32(x: np.ndarray, logits: np.ndarray, weights: dict, shared: dict, top_k: int, norm: bool) -> np.ndarray:
    """fp32 oracle of the MoE block: dequantised fp16 expert weights and fp16 backbones
    upcast to fp32, every intermediate kept in fp32 (no rounding), expert loop of
    modeling_olmoe.py:854-914.  ``weights[name][e]`` is the fp16 [O, r] matrix of expert e,
    ``shared[name]`` the fp16 backbone [r, in]."""
    x32 = x.astype(np.float32)
    sel, w = router_topk(logits, top_k, norm)
    hg = x32 @ shared["gate"].astype(np.float32).T
    hu = x32 @ shared["up"].astype(np.float32).T
    sd = shared["down"].astype(np.float32)
    out = np.zeros_like(x32)
    for e in np.unique(sel):
        tok, slot = np.nonzero(sel == e)
        g = hg[tok] @ weights["gate"][e].astype(np.float32).T
        u = hu[tok] @ weights["up"][e].astype(np.float32).T
        mlp = g / (1.0 + np.exp(-g)) * u
        dh = mlp @ sd.T
        y = dh @ weights["down"][e].astype(np.float32).T
        np.add.at(out, tok, y * w[tok, slot][:, None])
    return out


def error_metrics(y: np.ndarray, ref: np.ndarray) -> tuple:
    """(max-abs error, mean-relative error = mean|y - ref| / mean|ref|)."""
    y = y.astype(np.float64)
    ref = ref.astype(np.float64)
    return float(np.abs(y - ref).max()), float(np.abs(y - ref).mean() / max(np.abs(ref).mean(), 1e-30))


def canonical_half_bits(a: np.ndarray) -> np.ndarray:
    """uint16 bit patterns with -0 folded onto +0 (the reference's accumulation into a zero
    matrix never yields -0, a product that underflows with a minus sign does)."""
    return (np.asarray(a, dtype=np.float16) + np.float16(0)).view(np.uint16)


def dequantize_packed4(qweight: np.ndarray, qzeros: np.ndarray, scales: np.ndarray, g_idx: np.ndarray,
                       rows: int, cols: int) -> np.ndarray:
    """fp16 matrix [rows, cols] of a 4-bit packed backbone, as PackedQuantMatrix4bit.dequantize
    computes it in fp16 (qlinear_cuda.py:2756-2784): qweight [ceil(cols/8), rows] int32 holds the
    nibbles of input columns 8i..8i+7 of output row r (nibble j at bits 4j); qzeros
    [groups, ceil(rows/8)] int32 holds zero points minus one, packed the same way along rows;
    scales [groups, rows] fp16; g_idx [cols] the group of every input column.
    weight[r, c] = fp16((q - zero) * scale), q - zero exact, one rounding in the product."""
    shifts = (np.arange(8, dtype=np.int64) * 4).reshape(1, 1, 8)
    qz = qzeros.astype(np.int64) & 0xFFFFFFFF
    zeros = ((qz[:, :, None] >> shifts) & 0xF).reshape(qz.shape[0], -1)[:, :rows] + 1          # [groups, rows]
    qw = qweight.astype(np.int64) & 0xFFFFFFFF
    intweight = ((qw[:, :, None] >> shifts) & 0xF).transpose(0, 2, 1).reshape(-1, qw.shape[1])[:cols]  # [cols, rows]
    g = g_idx.astype(np.int64)
    diff = (intweight - zeros[g]).astype(np.float16)                                           # exact: |q - z| <= 16
    weight = (diff.astype(np.float32) * scales.astype(np.float16)[g].astype(np.float32)).astype(np.float16)
    return np.ascontiguousarray(weight.T)


def ns_expert_matrices(payload: dict, e: int) -> tuple:
    """(C1 [out, rank], C2 [rank, in]) fp16 of expert e from a grouped compensation payload with
    the reference's keys and layout (build_grouped_ns_compensation_payload,
    qlinear_cuda.py:1734-1882): C2 matrices are concatenated along the output axis of
    ns_c2_qweight / _scales (offset ns_c2_rank_offsets[e]) and of ns_c2_qzeros (word offset
    ns_c2_rank_word_offsets[e]); C1 matrices along the input axis of ns_c1_qweight (word-row offset
    ns_c1_rank_word_offsets[e]) and of ns_c1_qzeros / _scales (group-row offset
    ns_c1_group_offsets[e]).  Groups are uniform: group = min(col // group_size, groups - 1), as the
    reference kernels index them (dot8_packed4_uniform_shared_stride, TriSMoE_cuda_kernel.cu:1119-1174).
    Returns (None, None) for an expert of rank 0."""
    rank = int(payload["ns_rank_per_expert"][e])
    if rank <= 0:
        return None, None
    infeatures, outfeatures = int(payload["infeatures"]), int(payload["outfeatures"])
    group_size = int(payload["group_size"])
    off, woff = int(payload["ns_c2_rank_offsets"][e]), int(payload["ns_c2_rank_word_offsets"][e])
    zwords = (rank + 7) // 8
    groups2 = int(payload["ns_c2_scales"].shape[0])
    g2 = np.minimum(np.arange(infeatures) // max(1, group_size), groups2 - 1)
    c2 = dequantize_packed4(payload["ns_c2_qweight"][:, off:off + rank], payload["ns_c2_qzeros"][:, woff:woff + zwords],
                            payload["ns_c2_scales"][:, off:off + rank], g2, rank, infeatures)
    kw, go = int(payload["ns_c1_rank_word_offsets"][e]), int(payload["ns_c1_group_offsets"][e])
    goffs = [int(v) for v in payload["ns_c1_group_offsets"]] + [int(payload["ns_c1_qzeros"].shape[0])]
    groups1 = max(1, goffs[e + 1] - go)
    kwords = (rank + 7) // 8
    g1 = np.minimum(np.arange(rank) // max(1, group_size), groups1 - 1)
    c1 = dequantize_packed4(payload["ns_c1_qweight"][kw:kw + kwords], payload["ns_c1_qzeros"][go:go + groups1],
                            payload["ns_c1_scales"][go:go + groups1], g1, outfeatures, rank)
    return c1, c2


def ns_compensation_fp32(payload: dict, x_grouped: np.ndarray, expert_ids, segment_offsets) -> np.ndarray:
    """[R, outfeatures] fp32 compensation of grouped rows: for the rows of each segment,
    F.linear(F.linear(x, C2), C1) with the fp16 matrices of the segment's expert
    (QuantLinear.forward, qlinear_cuda.py:4737-4747; _apply_grouped_ns_compensation,
    qlinear_cuda.py:1917-1948), sums in fp32, the intermediate rounded to fp16 as both the
    reference's fallback and its kernels do (TriSMoE_cuda_kernel.cu:1305); rows of experts
    without a pair get zeros."""
    out = np.zeros((x_grouped.shape[0], int(payload["outfeatures"])), np.float32)
    for s, e in enumerate(expert_ids):
        a, b = int(segment_offsets[s]), int(segment_offsets[s + 1])
        c1, c2 = ns_expert_matrices(payload, int(e))
        if c1 is None or b <= a:
            continue
        hidden = (x_grouped[a:b].astype(np.float32) @ c2.astype(np.float32).T).astype(np.float16)
        out[a:b] = hidden.astype(np.float32) @ c1.astype(np.float32).T
    return out
