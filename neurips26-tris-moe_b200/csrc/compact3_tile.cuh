// Per-CTA staging of one compact3 weight tile and the register-level unpack that feeds
// the tensor-core fragments.  Shared by the grouped kernels and by the two dump kernels
// (decoded g_map words, dequantized fp16 weights) so that what the tests compare bit for
// bit is exactly what the matmul consumes.
//
// Geometry.  A CTA of 256 threads (8 warps) owns, per projection, OW consecutive outputs
// of one expert and walks K in chunks of KC = 8 packed rows (256 columns).  With NPROJ = 2
// (gate + up in one launch) OW = 64, with NPROJ = 1 OW = 128; either way a chunk is 1024
// 32-bit words per bit plane and 8 block-GR blocks (block = 2 packed rows x 64 outputs,
// QL:486-494 / CU:63-68 of the TriS-MoE tree).
//
// Column order inside a packed row.  Dot products do not care about the order of K, so a
// lane never moves bits sideways: lane (g = lane/4, t = lane%4) of a warp owns outputs
// g and g+8 of its 16-output sub-tile and, in every 32-column word, the eight columns
// {t+4i, t+4i+16 : i = 0..3}.  Columns j and j+16 sit 16 bits apart in the word, i.e. in
// the same position of the two halves of a half2, so one shift lines a bit pair up with
// the sign bits (15, 31) or with the byte MSBs that PRMT can replicate into a 16-bit
// select mask.  The activation rows are staged in shared memory in the same order.
#pragma once
#include "common.cuh"

namespace tris {

constexpr int kThreads = 256;
constexpr int kWarps = 8;
constexpr int KC = 8;            // packed rows per K chunk
constexpr int kTileWords = 1024; // words per bit plane per chunk (all projections)
constexpr int kBlocksPerChunk = 8;

template <int NPROJ>
struct Geom {
  static constexpr int OW = 128 / NPROJ;  // outputs per projection per CTA
  static constexpr int NOB = OW / 64;     // block-GR out blocks per projection per CTA
};

// Shared-memory image of one chunk.  NT = number of 8-row activation tiles staged.
template <int NPROJ, int NT>
struct alignas(16) TileSmem {
  uint4 coltab[NPROJ * KC * 16];            // [proj][p][i][t] -> {cd2, cnd2, c1_2, c2_2}
  uint4 htab[NPROJ * NT * KC * 32];         // [proj][nt][p][n][t] -> 8 halves (B fragments)
  uint2 rowtab[kTileWords];                 // [proj][p][o] -> row_pack3 word of the row's group
  uint32_t s1[kTileWords];                  // sign plane 1
  uint32_t g[kTileWords];                   // decoded g_map, then the select plane
  uint32_t grw[kBlocksPerChunk * 128 + 8];  // staged block-GR words
  uint32_t gridx[kBlocksPerChunk * 32];     // staged sub-stream index
  int32_t binfo[kBlocksPerChunk * 4];       // {begin, count, meta, block index}
  uint32_t cw[NPROJ * KC];                  // c_map word of each packed row
};

__device__ __forceinline__ int proj_packed_rows(const TrisProjView& v) { return (v.rank + 31) >> 5; }
__device__ __forceinline__ int proj_num_blocks(const TrisProjView& v) {
  return ((proj_packed_rows(v) + 1) >> 1) * ((v.out_features + 63) >> 6);
}

// ---- block Golomb-Rice ----------------------------------------------------------------
// Stream of one block (QL:3763-3791): for every one-bit, the zero run before it as
// (run >> k) zeros, a one, then the low k bits of run LSB first; bits fill 32-bit words
// LSB first.  Decoder semantics follow decode_block_gr_block (CU:426-479).

__device__ __forceinline__ uint32_t gr_peek32(const uint32_t* w, int nwords, int bitpos) {
  const int wi = bitpos >> 5;
  const uint32_t lo = (wi < nwords) ? w[wi] : 0u;
  const uint32_t hi = (wi + 1 < nwords) ? w[wi + 1] : 0u;
  return __funnelshift_r(lo, hi, bitpos & 31);
}

// Decodes `n_ones` codewords starting at (bitpos, flatpos) and calls set(flat) for each.
template <typename SetBit>
__device__ __forceinline__ void gr_decode_run(const uint32_t* w, int nwords, int k, int n_ones,
                                              int bitpos, int flatpos, SetBit set) {
  const int total_bits = nwords << 5;
  const uint32_t kmask = (1u << k) - 1u;
  for (int n = 0; n < n_ones; ++n) {
    int q = 0;
    uint32_t v = gr_peek32(w, nwords, bitpos);
    while (v == 0u) {
      q += 32;
      bitpos += 32;
      if (bitpos >= total_bits) return;  // stream ran out: malformed, stop
      v = gr_peek32(w, nwords, bitpos);
    }
    const int t = __ffs(v) - 1;
    q += t;
    bitpos += t + 1;
    uint32_t rem;
    if (t + 1 + k <= 32) {
      rem = (t == 31) ? 0u : ((v >> (t + 1)) & kmask);
    } else {
      rem = gr_peek32(w, nwords, bitpos) & kmask;
    }
    bitpos += k;
    flatpos += (q << k) | static_cast<int>(rem);
    if (flatpos >= TRIS_GR_BLOCK_WORDS * 32) return;
    set(flatpos);
    ++flatpos;
  }
}

// Word index inside the chunk planes of flat word `wl` (0..127) of chunk-local block b.
template <int NPROJ>
__device__ __forceinline__ int block_word_to_tile(int b, int wl) {
  constexpr int OW = Geom<NPROJ>::OW;
  constexpr int NOB = Geom<NPROJ>::NOB;
  const int obl = b % NOB;
  const int kbl = (b / NOB) & 3;
  const int proj = b / (NOB * 4);
  return (proj * KC + 2 * kbl + (wl >> 6)) * OW + obl * 64 + (wl & 63);
}

// Fills sm.g with the dense g_map words of the chunk (zeros where a projection has no
// block-GR stream).  All 256 threads must call; ends with a barrier.
template <int NPROJ, int NT>
__device__ __forceinline__ void stage_gmap_block_gr(TileSmem<NPROJ, NT>& sm, const TrisProjView* views,
                                                    int e, int o0, int p0) {
  constexpr int NOB = Geom<NPROJ>::NOB;
  const int tid = threadIdx.x;
  if (tid < kBlocksPerChunk) {
    const int b = tid;
    const int obl = b % NOB;
    const int kbl = (b / NOB) & 3;
    const TrisProjView& v = views[b / (NOB * 4)];
    const int pr = proj_packed_rows(v);
    const int nkb = (pr + 1) >> 1;
    const int nob = (v.out_features + 63) >> 6;
    const int kb = (p0 >> 1) + kbl;
    const int ob = (o0 >> 6) + obl;
    int begin = 0, count = 0, meta = 0, bi = 0;
    if (v.use_block_gr && v.q_gmap_gr_words != nullptr && kb < nkb && ob < nob) {
      const int nblk = nkb * nob;
      bi = kb * nob + ob;
      const int32_t* off = v.q_gmap_gr_offsets + static_cast<size_t>(e) * (nblk + 1);
      begin = off[bi];
      const int end = off[bi + 1];
      meta = v.q_gmap_gr_meta[static_cast<size_t>(e) * nblk + bi];
      count = end - begin;
      if (count > TRIS_GR_BLOCK_WORDS) count = TRIS_GR_BLOCK_WORDS;
      if (begin < 0 || count < 0 || begin + count > v.gr_max_words) count = 0;
    }
    sm.binfo[b * 4 + 0] = begin;
    sm.binfo[b * 4 + 1] = count;
    sm.binfo[b * 4 + 2] = meta;
    sm.binfo[b * 4 + 3] = bi;
  }
  __syncthreads();
  for (int i = tid; i < kBlocksPerChunk * 128; i += kThreads) {
    const int b = i >> 7, wl = i & 127;
    const int count = sm.binfo[b * 4 + 1];
    uint32_t word = 0u;
    if (wl < count) {
      const TrisProjView& v = views[b / (NOB * 4)];
      word = static_cast<uint32_t>(
          v.q_gmap_gr_words[static_cast<size_t>(e) * v.gr_max_words + sm.binfo[b * 4 + 0] + wl]);
    }
    sm.grw[i] = word;
    const bool raw = (sm.binfo[b * 4 + 2] & TRIS_GR_META_RAW_FLAG) != 0;
    sm.g[block_word_to_tile<NPROJ>(b, wl)] = raw ? word : 0u;
  }
  const int sub = views[0].gr_substreams;
  for (int i = tid; i < kBlocksPerChunk * sub; i += kThreads) {
    const int b = i / sub, j = i - b * sub;
    const TrisProjView& v = views[b / (NOB * 4)];
    uint32_t packed = 0u;
    if (sm.binfo[b * 4 + 1] > 0 && v.gr_index != nullptr) {
      const size_t nblk = static_cast<size_t>(proj_num_blocks(v));
      packed = v.gr_index[(static_cast<size_t>(e) * nblk + sm.binfo[b * 4 + 3]) * sub + j];
    }
    sm.gridx[b * 32 + j] = packed;
  }
  __syncthreads();
  for (int i = tid; i < kBlocksPerChunk * sub; i += kThreads) {
    const int b = i / sub, j = i - b * sub;
    const int count = sm.binfo[b * 4 + 1];
    const int meta = sm.binfo[b * 4 + 2];
    if (count <= 0 || (meta & TRIS_GR_META_RAW_FLAG)) continue;
    const int k = meta & TRIS_GR_META_K_MASK;
    const int one_count = meta >> TRIS_GR_META_ONE_COUNT_SHIFT;
    const int per = (one_count + sub - 1) / sub;
    const int first = j * per;
    if (per == 0 || first >= one_count) continue;
    const int n_ones = min(per, one_count - first);
    const uint32_t packed = sm.gridx[b * 32 + j];
    uint32_t* gbase = sm.g;
    gr_decode_run(sm.grw + b * 128, count, k, n_ones, static_cast<int>(packed & 0xFFFFu),
                  static_cast<int>(packed >> 16), [&](int flat) {
                    atomicOr(gbase + block_word_to_tile<NPROJ>(b, flat >> 5), 1u << (flat & 31));
                  });
  }
  __syncthreads();
}

// ---- bit-plane helpers ----------------------------------------------------------------
// 32 bits of the column-bit stream of one output, starting at `rank` (sparse planes pack
// only the active columns, 32 per row; utils/pack_utils.py:19-52).
__device__ __forceinline__ uint32_t sparse_bits_at(const int32_t* plane, int rows, int o_stride, int rank,
                                                   int need) {
  const int q = rank >> 5, sh = rank & 31;
  const uint32_t lo = (q < rows) ? static_cast<uint32_t>(plane[static_cast<size_t>(q) * o_stride]) : 0u;
  uint32_t hi = 0u;
  if (sh + need > 32 && q + 1 < rows) hi = static_cast<uint32_t>(plane[static_cast<size_t>(q + 1) * o_stride]);
  return __funnelshift_r(lo, hi, sh);
}

// Places the low popc(mask) bits of `bits` at the set positions of `mask`, ascending.
__device__ __forceinline__ uint32_t deposit_bits(uint32_t bits, uint32_t mask) {
  uint32_t out = 0u;
  while (mask) {
    const int pos = __ffs(mask) - 1;
    out |= (bits & 1u) << pos;
    bits >>= 1;
    mask &= mask - 1;
  }
  return out;
}

// Opens a zero gap at every set position of `holes` (ascending), shifting higher bits up.
__device__ __forceinline__ uint32_t spread_around(uint32_t bits, uint32_t holes) {
  while (holes) {
    const int pos = __ffs(holes) - 1;
    const uint32_t low = (1u << pos) - 1u;
    bits = (bits & low) | ((bits & ~low) << 1);
    holes &= holes - 1;
  }
  return bits;
}

// ---- chunk staging --------------------------------------------------------------------
// Builds sign plane, select plane and the scale tables of the chunk from global memory.
// Preconditions: sm.g holds the dense g_map words for projections stored as block-GR.
// Select plane: for a non-salient column the g_map bit (1 -> "d" scale pair, CU:736-737);
// for a salient column XNOR(sign1, sign2), because
//   fp16(+-a +- b) = sign1 * fp16(a + (sign1*sign2) b)
// so a salient weight is again "pick one of two magnitudes, then apply sign1" with
// magnitudes fp16(a+b) and fp16(a-b).
template <int NPROJ, int NT>
__device__ __forceinline__ void stage_planes_and_scales(TileSmem<NPROJ, NT>& sm, const TrisProjView* views,
                                                        int e, int o0, int p0, uint32_t* gmap_dump) {
  constexpr int OW = Geom<NPROJ>::OW;
  const int tid = threadIdx.x;
  for (int i = tid; i < kTileWords; i += kThreads) {
    const int proj = i / (KC * OW);
    const int p = (i / OW) % KC;
    const int o = i % OW;
    const TrisProjView& v = views[proj];
    const int pr = proj_packed_rows(v);
    const int pg = p0 + p, og = o0 + o;
    uint32_t s1 = 0u, sel = 0u;
    uint2 rp = make_uint2(0u, 0u);
    if (pg < pr && og < v.out_features) {
      const int O = v.out_features;
      s1 = static_cast<uint32_t>(v.qweight1[(static_cast<size_t>(e) * pr + pg) * O + og]);
      const uint32_t cwv = static_cast<uint32_t>(v.c_map[static_cast<size_t>(e) * pr + pg]);
      uint32_t s2 = 0u;
      const int cnt = __popc(cwv);
      if (cnt > 0 && v.qweight2_sparse != nullptr) {
        const int rank0 = v.qweight2_sparse_prefix[static_cast<size_t>(e) * (pr + 1) + pg];
        const uint32_t bits = sparse_bits_at(
            v.qweight2_sparse + static_cast<size_t>(e) * v.sign2_rows * O + og, v.sign2_rows, O, rank0, cnt);
        s2 = deposit_bits(bits, cwv);
      }
      uint32_t gm;
      if (v.use_block_gr) {
        gm = sm.g[i];
      } else {
        const int ncols = min(32, v.rank - 32 * pg);
        const uint32_t colmask = (ncols >= 32) ? 0xFFFFFFFFu : ((1u << ncols) - 1u);
        const uint32_t nsmask = ~cwv & colmask;
        gm = 0u;
        if (nsmask != 0u && v.q_gmap_sparse != nullptr) {
          const int rank0 = v.q_gmap_sparse_prefix[static_cast<size_t>(e) * (pr + 1) + pg];
          const int slot = v.gmap_slot ? v.gmap_slot[e] : e;
          const uint32_t bits = sparse_bits_at(
              v.q_gmap_sparse + static_cast<size_t>(slot) * v.gmap_sparse_rows * O + og,
              v.gmap_sparse_rows, O, rank0, __popc(nsmask));
          gm = spread_around(bits, cwv & colmask) & nsmask;
        }
      }
      if (gmap_dump) gmap_dump[i] = gm;
      sel = (gm & ~cwv) | (cwv & ~(s1 ^ s2));
      const int grp = v.packed_row_group ? v.packed_row_group[static_cast<size_t>(e) * pr + pg] : 0;
      if (grp >= 0 && grp < v.num_groups) {
        const unsigned long long w = static_cast<unsigned long long>(
            v.row_pack3[(static_cast<size_t>(e) * O + og) * v.num_groups + grp]);
        rp = make_uint2(static_cast<uint32_t>(w), static_cast<uint32_t>(w >> 32));
      }
    } else if (gmap_dump) {
      gmap_dump[i] = 0u;
    }
    sm.s1[i] = s1;
    sm.g[i] = sel;
    sm.rowtab[i] = rp;
  }
  for (int i = tid; i < NPROJ * KC * 16; i += kThreads) {
    const int proj = i / (KC * 16);
    const int p = (i >> 4) % KC;
    const int ii = (i >> 2) & 3;
    const int t = i & 3;
    const TrisProjView& v = views[proj];
    const int pr = proj_packed_rows(v);
    const int pg = p0 + p;
    uint4 entry = make_uint4(0u, 0u, 0u, 0u);
    uint32_t cwv = 0u;
    if (pg < pr) {
      cwv = static_cast<uint32_t>(v.c_map[static_cast<size_t>(e) * pr + pg]);
      const int ja = t + 4 * ii, jb = ja + 16;
      unsigned long long pa = 0ull, pb = 0ull;
      if (32 * pg + ja < v.rank) pa = static_cast<unsigned long long>(v.col_pack3[static_cast<size_t>(e) * v.rank + 32 * pg + ja]);
      if (32 * pg + jb < v.rank) pb = static_cast<unsigned long long>(v.col_pack3[static_cast<size_t>(e) * v.rank + 32 * pg + jb]);
      const bool sa = (cwv >> ja) & 1u, sb = (cwv >> jb) & 1u;
      // col_pack3 halves: (s_c1, s_c2, ns_d_c1, ns_nd_c1) at bits 0/16/32/48 (utils/pack_utils.py:55-64)
      const uint32_t c1a = pa & 0xFFFFu, c2a = (pa >> 16) & 0xFFFFu, cda = (pa >> 32) & 0xFFFFu, cna = (pa >> 48) & 0xFFFFu;
      const uint32_t c1b = pb & 0xFFFFu, c2b = (pb >> 16) & 0xFFFFu, cdb = (pb >> 32) & 0xFFFFu, cnb = (pb >> 48) & 0xFFFFu;
      entry.x = (sa ? 0u : cda) | ((sb ? 0u : cdb) << 16);
      entry.y = (sa ? 0u : cna) | ((sb ? 0u : cnb) << 16);
      entry.z = (sa ? c1a : 0u) | ((sb ? c1b : 0u) << 16);
      entry.w = (sa ? c2a : 0u) | ((sb ? c2b : 0u) << 16);
    }
    sm.coltab[i] = entry;
    if ((i & 15) == 0) sm.cw[proj * KC + p] = cwv;
  }
}

// Stages NT*8 activation rows of the chunk's 256 columns in fragment order.
// row_src(n) returns the hidden row of local row n, or -1 for padding.
template <int NPROJ, int NT, typename RowSrc>
__device__ __forceinline__ void stage_hidden(TileSmem<NPROJ, NT>& sm, const __half* const* hidden,
                                             const TrisProjView* views, int p0, int nt_count, RowSrc row_src) {
  const int tid = threadIdx.x;
  __half* dst = reinterpret_cast<__half*>(sm.htab);
  const int items = NPROJ * nt_count * 8 * KC * 4;
  for (int i = tid; i < items; i += kThreads) {
    const int j0 = (i & 3) * 8;
    const int p = (i >> 2) % KC;
    const int n_local = (i / (4 * KC)) % (nt_count * 8);
    const int proj = i / (4 * KC * nt_count * 8);
    const int rank = views[proj].rank;
    const int col = 32 * (p0 + p) + j0;
    const int src = row_src(n_local);
    __half vals[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) vals[u] = __ushort_as_half(0);
    if (src >= 0 && col < rank) {
      const __half* rowp = hidden[proj] + static_cast<size_t>(src) * rank + col;
      if ((rank & 7) == 0 && col + 8 <= rank) {
        *reinterpret_cast<uint4*>(vals) = *reinterpret_cast<const uint4*>(rowp);
      } else {
        for (int u = 0; u < 8 && col + u < rank; ++u) vals[u] = rowp[u];
      }
    }
    const int nt = n_local >> 3, n = n_local & 7;
    const size_t base = ((static_cast<size_t>(proj) * NT + nt) * KC + p) * 8 + n;
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int j = j0 + u;
      const int t = j & 3, ii = (j >> 2) & 3, hi = j >> 4;
      dst[(base * 4 + t) * 8 + 2 * ii + hi] = vals[u];
    }
  }
}

// ---- register unpack ------------------------------------------------------------------
// Weights of packed row p for the lane's two outputs (h = 0: out g, h = 1: out g+8) and
// four column pairs (t+4i, t+4i+16) as half2 bit patterns a[h][i].
// Exact arithmetic of _dequantize_compact3_matrix (QL:4200-4236): each product rounded to
// fp16 once, salient weight = fp16(+-p1 +- p2).
template <int NPROJ, int NT>
__device__ __forceinline__ void unpack_fragments(const TileSmem<NPROJ, NT>& sm, int proj, int p, int out_local,
                                                 int lane, uint32_t (&a)[2][4]) {
  constexpr int OW = Geom<NPROJ>::OW;
  const int g = lane >> 2, t = lane & 3;
  const uint32_t cwv = sm.cw[proj * KC + p];
  uint4 ct[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) ct[i] = sm.coltab[((proj * KC + p) * 4 + i) * 4 + t];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int idx = (proj * KC + p) * OW + out_local + g + 8 * h;
    const uint32_t s1 = sm.s1[idx];
    const uint32_t se = sm.g[idx];
    const uint2 rp = sm.rowtab[idx];
    // row_pack3 halves: (s_r1, s_r2, ns_d_r1, ns_nd_r1)
    const __half2 r1 = u32_as_h2(prmt(rp.x, 0u, 0x1010u));
    const __half2 r2 = u32_as_h2(prmt(rp.x, 0u, 0x3232u));
    const __half2 rd = u32_as_h2(prmt(rp.y, 0u, 0x1010u));
    const __half2 rn = u32_as_h2(prmt(rp.y, 0u, 0x3232u));
    const uint32_t st = s1 << (3 - t);   // column t+4i at bit 3+4i, column t+4i+16 at bit 19+4i
    const uint32_t gt = se << (3 - t);
    const uint32_t gt4 = gt << 4;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __half2 ca, cb;
      const uint32_t pairmask = 0x000F000Fu << (4 * i);  // columns of pair i over all four t
      if (cwv & pairmask) {
        const __half2 p1 = __hmul2_rn(u32_as_h2(ct[i].z), r1);
        const __half2 p2 = __hmul2_rn(u32_as_h2(ct[i].w), r2);
        const __half2 ssum = __hadd2_rn(p1, p2);
        const __half2 sdif = __hsub2_rn(p1, p2);
        // the non-salient half has p1 = p2 = 0, the salient half has cd = cnd = 0
        ca = __hfma2(u32_as_h2(ct[i].x), rd, ssum);
        cb = __hfma2(u32_as_h2(ct[i].y), rn, sdif);
      } else {
        ca = __hmul2_rn(u32_as_h2(ct[i].x), rd);
        cb = __hmul2_rn(u32_as_h2(ct[i].y), rn);
      }
      // select mask: replicate the select bit of each half over its 16 bits
      const uint32_t src = (i & 1) ? gt : gt4;               // i=1,3 use gt; i=0,2 use gt<<4
      const uint32_t m = prmt(src, 0u, (i >= 2) ? 0xBB99u : 0xAA88u);
      const uint32_t mag = (h2_as_u32(ca) & m) | (h2_as_u32(cb) & ~m);
      // sign: plane bit 1 -> +, 0 -> -   (QL:4213)
      const uint32_t sbits = st << (12 - 4 * i);             // pair i at bits 15 and 31
      a[h][i] = mag ^ (~sbits & 0x80008000u);
    }
  }
}

}  // namespace tris
