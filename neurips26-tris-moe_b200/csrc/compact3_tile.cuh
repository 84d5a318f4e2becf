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
// Staging.  Everything bulky comes in through untiled TMA copies (cp.async.bulk) that
// complete on mbarriers: warp 0 issues the copies whose addresses need no table lookup
// (sign plane rows, column and row scale packs, the block-GR sub-stream index), warp 1
// reads offsets/prefixes and issues the dependent ones (block-GR word spans or sparse
// g_map rows, salient sign rows), warp 2 issues one copy per activation row.  A copy whose
// source or size is not 16-byte aligned (odd shapes) is done with plain loads by the lane
// that would have issued it.  Waits on the mbarriers are bounded; a time-out is reported
// through a status word and the CTA leaves without storing results.
//
// Column order inside a packed row.  Dot products do not care about the order of K, so a
// lane never moves bits sideways: lane (g = lane/4, t = lane%4) of a warp owns outputs
// g and g+8 of its 16-output sub-tile and, in every 32-column word, the four column pairs
// (4t+i, 4t+i+16), i = 0..3.  Columns j and j+16 sit 16 bits apart in the word, i.e. in
// the same position of the two halves of a half2, so one shift lines a bit pair up with
// the sign bits (15, 31), which are also the byte MSBs that PRMT can replicate into a
// 16-bit select mask.  Activation rows are consumed "pair-interleaved": inside every group
// of 32 columns, column j sits at position 2*(j%16) + j/16, so a lane's B fragment for a
// packed row is one 16-byte shared-memory load.  The backbone GEMM writes that order
// directly; row-major activations handed in through the operator API are re-ordered while
// they are staged.
#pragma once
#include "common.cuh"

namespace tris {

constexpr int kThreads = 256;
constexpr int kWarps = 8;
constexpr int KC = 8;             // packed rows per K chunk
constexpr int kTileWords = 1024;  // words per bit plane per chunk (all projections)
constexpr int kBlocksPerChunk = 8;
constexpr int kSparseRows = 9;    // sparse plane rows a 256-column chunk can touch
constexpr int kRawWords = 1152;   // kSparseRows * 128
constexpr int kHiddenRowBytes = 576;  // 512 B of activations + 64 B so that 8 rows hit 8 bank groups
constexpr int kRowTabEntries = 1024;

template <int NPROJ>
struct Geom {
  static constexpr int OW = 128 / NPROJ;  // outputs per projection per CTA
  static constexpr int NOB = OW / 64;     // block-GR out blocks per projection per CTA
  static constexpr int SPAN = NOB * 128 + 8;  // words reserved per block-GR span
};

struct PackedRowInfo {
  uint32_t cw;      // c_map word (bit = salient column)
  int32_t rank2;    // salient columns below this packed row, relative to the staged sign2 rows
  int32_t rankg;    // non-salient columns below it, relative to the staged sparse g_map rows
  int32_t gslot;    // row scale slot of this packed row
};

// Shared-memory image of one chunk.  NT = number of 8-row activation tiles staged.
template <int NPROJ, int NT>
struct alignas(128) TileSmem {
  uint8_t hrows[NPROJ * NT * 8 * kHiddenRowBytes];  // [proj][row] pair-interleaved activations
  uint32_t s1[kTileWords];                           // sign plane 1, [proj][p][o]
  uint2 colraw[NPROJ * 256];                         // col_pack3 of the chunk's columns
  uint2 rowtab[kRowTabEntries];                      // [proj][o][slot] row_pack3 words
  uint32_t s2raw[kRawWords];                         // [proj][row][o] salient sign rows
  uint32_t gmraw[kRawWords + 8];                     // block-GR spans or sparse g_map rows
  uint32_t gridx[kBlocksPerChunk * 32];              // block-GR sub-stream index
  uint4 coltab[NPROJ * KC * 16];                     // [proj][p][i][t] -> {cd2, cnd2, c1_2, c2_2}
  uint32_t g[kTileWords];                            // decoded g_map, then the select plane
  PackedRowInfo ptab[NPROJ * (KC + 1)];
  int32_t binfo[kBlocksPerChunk * 4];                // {word offset in gmraw, count, meta, -}
  uint64_t mbar[3];                                  // W0: all a chunk needs but the sign plane, W1: sign plane + row scales, H: activations
  int32_t row_stride;
};

__device__ __forceinline__ int proj_packed_rows(const TrisProjView& v) { return (v.rank + 31) >> 5; }
__device__ __forceinline__ int proj_num_blocks(const TrisProjView& v) {
  return ((proj_packed_rows(v) + 1) >> 1) * ((v.out_features + 63) >> 6);
}

// ---- copies ---------------------------------------------------------------------------
// One lane moves nwords 32-bit words global -> shared: a TMA bulk copy when both ends are
// 16-byte aligned and the size is a multiple of 16 bytes, plain loads otherwise.  Returns
// the bytes the mbarrier must expect.
__device__ __forceinline__ uint32_t lane_copy(uint32_t* dst, const uint32_t* src, int nwords, uint64_t* bar) {
  if (nwords <= 0) return 0;
  const bool aligned = ((reinterpret_cast<uintptr_t>(src) | smem_u32(dst)) & 15u) == 0 && (nwords & 3) == 0;
  if (aligned) {
    bulk_g2s(dst, src, static_cast<uint32_t>(nwords) * 4u, bar);
    return static_cast<uint32_t>(nwords) * 4u;
  }
  for (int w = 0; w < nwords; ++w) dst[w] = src[w];
  return 0;
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

__device__ __forceinline__ uint32_t lds_u32(uint32_t smem_addr) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(smem_addr));
  return v;
}

// Decodes `n_ones` codewords of a block staged in shared memory, starting at (bitpos,
// flatpos), and calls set(flat) for each one.  The loop is a serial dependency chain (the
// next codeword starts where this one ends).  The common case runs in a branch-light inner
// loop: the stream is read through a three-word register window (the 64 bits being parsed
// plus one word fetched ahead, so no load sits on the chain), a codeword costs a funnel
// shift, a count of trailing zeros and a few adds, and positions past the block are dropped
// by predication.  A zero run of 32 or more, or a remainder that straddles the 32-bit view,
// leaves the inner loop for a general step that also bounds malformed streams.  Reads stay
// inside the block's words plus three words behind them; every staged span has that much
// slack (its neighbour's words or the tail of the buffer).
template <typename SetBit>
__device__ __forceinline__ void gr_decode_run(const uint32_t* w, int nwords, int k, int n_ones, int bitpos,
                                              int flatpos, SetBit set) {
  const int total_bits = nwords << 5;
  const uint32_t kmask = (1u << k) - 1u;
  const int k1 = k + 1;
  const uint32_t base = smem_u32(w);
  const uint32_t last = base + (static_cast<uint32_t>(nwords) << 2);
  uint32_t addr = base + (static_cast<uint32_t>(min(bitpos >> 5, nwords)) << 2);
  uint32_t lo = lds_u32(addr), hi = lds_u32(addr + 4), nx = lds_u32(addr + 8);
  int sh = bitpos & 31;
  int n = 0;
  for (;;) {
    int t = 0;
#pragma unroll 2
    for (; n < n_ones; ++n) {
      const uint32_t v = __funnelshift_r(lo, hi, sh);
      t = __clz(__brev(v));  // zero run length; 32 when the view holds no one
      if (t + k1 > 32) break;
      const uint32_t rem = __funnelshift_r(v, 0u, t + 1) & kmask;
      const int pos = flatpos + (t << k) + static_cast<int>(rem);
      if (pos < TRIS_GR_BLOCK_WORDS * 32) set(pos);
      flatpos = pos + 1;
      sh += t + k1;
      if (sh >= 32) {
        sh -= 32;
        lo = hi;
        hi = nx;
        addr = min(addr + 4, last);
        nx = lds_u32(addr + 8);  // needed two words from now: its latency is off the chain
      }
    }
    if (n >= n_ones) return;
    // general step: long zero run or remainder beyond the 32-bit view
    bitpos = (static_cast<int>(addr - base) << 3) + sh;
    int q = 0;
    uint32_t v = gr_peek32(w, nwords, bitpos);
    while (v == 0u) {
      q += 32;
      bitpos += 32;
      if (bitpos >= total_bits) return;  // stream ran out: malformed, stop
      v = gr_peek32(w, nwords, bitpos);
    }
    t = __ffs(v) - 1;
    const uint32_t rem = gr_peek32(w, nwords, bitpos + t + 1) & kmask;
    bitpos += t + k1;
    const int pos = flatpos + ((q + t) << k) + static_cast<int>(rem);
    if (pos >= TRIS_GR_BLOCK_WORDS * 32 || bitpos > total_bits) return;
    set(pos);
    flatpos = pos + 1;
    ++n;
    addr = base + (static_cast<uint32_t>(min(bitpos >> 5, nwords)) << 2);
    lo = lds_u32(addr), hi = lds_u32(addr + 4), nx = lds_u32(addr + 8);
    sh = bitpos & 31;
  }
}

// The bit planes of a chunk (sign plane, g_map / select plane) are stored block by block, in
// the block-GR order: chunk-local block b = (proj * 4 + k block) * NOB + out block holds its
// 128 words [packed row parity][64 outputs] contiguously, so a decoded block needs no index
// arithmetic and a raw block is a straight copy.
template <int NPROJ>
__device__ __forceinline__ int plane_index(int proj, int p, int o) {
  constexpr int NOB = Geom<NPROJ>::NOB;
  return ((proj * 4 + (p >> 1)) * NOB + (o >> 6)) * 128 + (p & 1) * 64 + (o & 63);
}

// ---- bit-plane helpers ----------------------------------------------------------------
// Places the low popc(mask) bits of `bits` at the set positions of `mask`, ascending.
__device__ __forceinline__ uint32_t deposit_bits(uint32_t bits, uint32_t mask) {
  uint32_t out = 0u;
  while (mask) {
    const uint32_t low = mask & (0u - mask);
    out |= (0u - (bits & 1u)) & low;
    bits >>= 1;
    mask ^= low;
  }
  return out;
}

// Opens a zero gap at every set position of `holes` (ascending), shifting higher bits up.
__device__ __forceinline__ uint32_t spread_around(uint32_t bits, uint32_t holes) {
  while (holes) {
    const uint32_t low = (holes & (0u - holes)) - 1u;
    bits = (bits & low) | ((bits & ~low) << 1);
    holes &= holes - 1;
  }
  return bits;
}

// 32 bits starting at bit `rank` of the column-bit stream of output o stored as rows of
// 32 bits in shared memory ([row][o], row stride OW words).
__device__ __forceinline__ uint32_t staged_bits_at(const uint32_t* rows, int ow, int o, int rank) {
  const int q = rank >> 5, sh = rank & 31;
  const uint32_t lo = (q < kSparseRows) ? rows[q * ow + o] : 0u;
  const uint32_t hi = (sh != 0 && q + 1 < kSparseRows) ? rows[(q + 1) * ow + o] : 0u;
  return __funnelshift_r(lo, hi, sh);
}

// ---- stage 1: issue -------------------------------------------------------------------
// Called by all threads after a barrier that ended every earlier use of the buffers it
// fills.  The copies of chunk (e, o0, p0) form two sets with a barrier each:
//   W0 (mbar[0])  column scale packs, block-GR sub-stream index and spans, salient sign rows,
//                 sparse g_map rows, and the table ptab: all that decode needs
//   W1 (mbar[1])  sign plane and row scale packs: needed for the select plane and the main loop
// `parts` selects the sets to issue (bit 0: W0, bit 1: W1).
// A warp issues its bulk copies one lane after the other (60-70 cycles each), warps issue
// side by side, and a warp that waits for a table entry stalls with all its lanes.  So every
// warp gets one kind of work and at most ten copies:
//   warp 0  sign-plane pieces 0-7 (W1), column scale packs (W0)
//   warp 4  sign-plane pieces 8-15, row scale packs (W1)
//   warp 5  block-GR sub-stream index blocks (W0); lanes 16+: ptab of projection 0
//   warp 6  lanes 16+: ptab of projection 1
//   warp 1  block-GR spans, after reading the block offsets (W0)
//   warps 2, 3  salient sign rows / sparse g_map rows of projection 0, 1, after the prefixes (W0)
// Lane 0 of every warp arrives on the barriers of the issued sets with its warp's byte counts.
// `e` indexes the bulky E-stacked tensors (sign planes, bitmap data, scale packs: a staging
// slot when the payload is paged in), `ex` is the expert id and indexes the small tables
// (c_map, prefixes, packed-row groups, block-GR offsets and meta), which stay resident.
// Only packed rows [p_lo, p_hi) of the chunk (multiples of 2) are staged: a cluster may split a
// chunk's K range over its CTAs.
enum { STAGE_W0 = 1, STAGE_W1 = 2, STAGE_ALL = 3 };
template <int NPROJ, int NT>
__device__ __forceinline__ void stage_issue_weights(TileSmem<NPROJ, NT>& sm, const TrisProjView* views, int e,
                                                    int ex, int o0, int p0, int p_lo = 0, int p_hi = KC,
                                                    int parts = STAGE_ALL) {
  constexpr int OW = Geom<NPROJ>::OW;
  constexpr int NOB = Geom<NPROJ>::NOB;
  constexpr int SPAN = Geom<NPROJ>::SPAN;
  const bool w0 = (parts & STAGE_W0) != 0, w1 = (parts & STAGE_W1) != 0;
  static_assert(NPROJ * KC * NOB == 16 && kBlocksPerChunk == 8 && kWarps == 8 && kSparseRows <= 16, "copy roles");
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint64_t* bar_0 = &sm.mbar[0];
  uint64_t* bar_1 = &sm.mbar[1];
  uint32_t bytes_0 = 0, bytes_1 = 0;
  if (lane < 16) fence_proxy_async();
  if (warp == 0 || warp == 4) {
    if (lane < 8 && w1) {  // sign plane: 16 pieces of one packed row x 64 outputs
      const int piece = 2 * warp + lane;  // warp 0: 0-7, warp 4: 8-15
      const int obl = piece % NOB, p = (piece / NOB) % KC, proj = piece / (NOB * KC);
      const TrisProjView& v = views[proj];
      const int pr = proj_packed_rows(v);
      const int wv = min(64, v.out_features - (o0 + 64 * obl));
      if (p0 + p < pr && wv > 0 && p >= p_lo && p < p_hi)
        bytes_1 += lane_copy(sm.s1 + plane_index<NPROJ>(proj, p, 64 * obl),
                             reinterpret_cast<const uint32_t*>(v.qweight1) +
                                 (static_cast<size_t>(e) * pr + p0 + p) * v.out_features + o0 + 64 * obl,
                             wv, bar_1);
    } else if (lane >= 8 && lane < 8 + NPROJ) {
      const int proj = lane - 8;
      const TrisProjView& v = views[proj];
      if (warp == 0) {  // column scale packs
        const int c0 = 32 * p0, c1 = min(v.rank, 32 * (p0 + KC));
        if (c1 > c0 && w0)
          bytes_0 += lane_copy(reinterpret_cast<uint32_t*>(sm.colraw + proj * 256),
                               reinterpret_cast<const uint32_t*>(v.col_pack3 + static_cast<size_t>(e) * v.rank + c0),
                               2 * (c1 - c0), bar_0);
      } else if (w1) {  // row scale packs, all groups, when they fit
        const int G = v.num_groups;
        const int wv = min(OW, v.out_features - o0);
        if (G * NPROJ * OW <= kRowTabEntries && wv > 0)
          bytes_1 += lane_copy(reinterpret_cast<uint32_t*>(sm.rowtab + proj * OW * G),
                               reinterpret_cast<const uint32_t*>(v.row_pack3 + (static_cast<size_t>(e) * v.out_features + o0) * G),
                               2 * wv * G, bar_1);
      }
    }
  } else if (warp == 5 && lane < kBlocksPerChunk && w0) {  // block-GR sub-stream index
    const int b = lane;
    const TrisProjView& v = views[b / (NOB * 4)];
    if (v.use_block_gr && v.gr_index != nullptr) {
      const int pr = proj_packed_rows(v);
      const int nkb = (pr + 1) >> 1, nob = (v.out_features + 63) >> 6;
      const int kbl = (b / NOB) & 3;
      const int kb = (p0 >> 1) + kbl, ob = (o0 >> 6) + (b % NOB);
      if (kb < nkb && ob < nob && 2 * kbl >= p_lo && 2 * kbl < p_hi) {
        const size_t bi = static_cast<size_t>(e) * nkb * nob + static_cast<size_t>(kb) * nob + ob;
        bytes_0 += lane_copy(sm.gridx + b * 32, v.gr_index + bi * v.gr_substreams, v.gr_substreams, bar_0);
      }
    }
  } else if (warp == 1) {
    if (lane < NPROJ * 4 && w0) {  // one block-GR span = the NOB blocks of (proj, k block)
      const int proj = lane >> 2, kbl = lane & 3;
      const TrisProjView& v = views[proj];
      const int pr = proj_packed_rows(v);
      const int nkb = (pr + 1) >> 1, nob = (v.out_features + 63) >> 6;
      const int kb = (p0 >> 1) + kbl, ob0 = o0 >> 6;
      int begins[NOB + 1];
      int metas[NOB];
      bool ok = v.use_block_gr && v.q_gmap_gr_words != nullptr && kb < nkb && 2 * kbl >= p_lo && 2 * kbl < p_hi;
#pragma unroll
      for (int j = 0; j < NOB; ++j) metas[j] = 0;
#pragma unroll
      for (int j = 0; j <= NOB; ++j) begins[j] = 0;
      int nvalid = 0;
      if (ok) {
        nvalid = min(NOB, nob - ob0);
        const int nblk = nkb * nob;
        const int32_t* off = v.q_gmap_gr_offsets + static_cast<size_t>(ex) * (nblk + 1) + kb * nob + ob0;
        const int32_t* met = v.q_gmap_gr_meta + static_cast<size_t>(ex) * nblk + kb * nob + ob0;
#pragma unroll
        for (int j = 0; j <= NOB; ++j)
          if (j <= nvalid) begins[j] = off[j];
#pragma unroll
        for (int j = 0; j < NOB; ++j)
          if (j < nvalid) metas[j] = met[j];
      }
      const int first = begins[0];
      int last = first;
#pragma unroll
      for (int j = 0; j < NOB; ++j) {
        const int b = lane * NOB + j;
        int count = (j < nvalid) ? begins[j + 1] - begins[j] : 0;
        if (count < 0 || count > TRIS_GR_BLOCK_WORDS || begins[j] < 0 || begins[j] + count > v.gr_max_words ||
            begins[j] < last)
          count = 0;  // corrupt offsets were already rejected at load time; stay in bounds regardless
        if (count > 0) last = begins[j] + count;
        sm.binfo[b * 4 + 1] = count;
        sm.binfo[b * 4 + 2] = metas[j];
        sm.binfo[b * 4 + 0] = begins[j];  // made relative below
      }
      int nwords = last - first;
      if (nwords < 0 || nwords > NOB * TRIS_GR_BLOCK_WORDS) {
        nwords = 0;
#pragma unroll
        for (int j = 0; j < NOB; ++j) sm.binfo[(lane * NOB + j) * 4 + 1] = 0;
      }
      uint32_t* region = sm.gmraw + lane * SPAN;
      int shift = 0;
      if (nwords > 0) {
        const size_t abs0 = static_cast<size_t>(e) * v.gr_max_words + first;
        const size_t total = static_cast<size_t>(v.num_experts) * v.gr_max_words;
        const uint32_t* base = reinterpret_cast<const uint32_t*>(v.q_gmap_gr_words);
        const bool base_aligned = (reinterpret_cast<uintptr_t>(base) & 15u) == 0;
        shift = base_aligned ? static_cast<int>(abs0 & 3) : 0;  // words above a 16-byte boundary
        const size_t a0 = abs0 - shift;
        size_t a1 = base_aligned ? ((abs0 + nwords + 3) & ~static_cast<size_t>(3)) : (abs0 + nwords);
        if (a1 > total) a1 = abs0 + nwords;
        const int n_al = static_cast<int>(a1 - a0);
        if ((n_al & 3) == 0 && a0 + n_al <= total) {
          bytes_0 += lane_copy(region, base + a0, n_al, bar_0);
        } else {
          const int bulk = (n_al >> 2) << 2;
          bytes_0 += lane_copy(region, base + a0, bulk, bar_0);
          for (int w = bulk; w < n_al; ++w) region[w] = base[a0 + w];
        }
      }
#pragma unroll
      for (int j = 0; j < NOB; ++j) {
        const int b = lane * NOB + j;
        sm.binfo[b * 4 + 0] = lane * SPAN + shift + (sm.binfo[b * 4 + 0] - first);
      }
    }
  } else if ((warp == 2 || warp == 3) && warp - 2 < NPROJ && lane < kSparseRows && w0) {
    // salient sign rows and (streaming format) sparse g_map rows of one projection
    const int proj = warp - 2, rq = lane;
    const TrisProjView& v = views[proj];
    const int pr = proj_packed_rows(v);
    const int wv = min(OW, v.out_features - o0);
    if (p0 < pr && wv > 0) {
      if (v.sign2_rows > 0 && v.qweight2_sparse != nullptr) {
        const int32_t* pre = v.qweight2_sparse_prefix + static_cast<size_t>(ex) * (pr + 1);
        const int r0 = pre[p0], r1 = pre[min(pr, p0 + KC)];
        const int q0 = max(0, r0 >> 5);
        const int q1 = min(min(v.sign2_rows, (r1 + 31) >> 5), q0 + kSparseRows);
        if (q0 + rq < q1)
          bytes_0 += lane_copy(sm.s2raw + (proj * kSparseRows + rq) * OW,
                               reinterpret_cast<const uint32_t*>(v.qweight2_sparse) +
                                   (static_cast<size_t>(e) * v.sign2_rows + q0 + rq) * v.out_features + o0,
                               wv, bar_0);
      }
      if (!v.use_block_gr && v.gmap_sparse_rows > 0 && v.q_gmap_sparse != nullptr) {
        const int32_t* pre = v.q_gmap_sparse_prefix + static_cast<size_t>(ex) * (pr + 1);
        const int r0 = pre[p0], r1 = pre[min(pr, p0 + KC)];
        const int slot = v.gmap_slot ? v.gmap_slot[ex] : e;
        const int q0 = max(0, r0 >> 5);
        const int q1 = min(min(v.gmap_sparse_rows, (r1 + 31) >> 5), q0 + kSparseRows);
        if (q0 + rq < q1)
          bytes_0 += lane_copy(sm.gmraw + (proj * kSparseRows + rq) * OW,
                               reinterpret_cast<const uint32_t*>(v.q_gmap_sparse) +
                                   (static_cast<size_t>(slot) * v.gmap_sparse_rows + q0 + rq) * v.out_features + o0,
                               wv, bar_0);
      }
    }
  }
  if (warp >= 5 && warp < 5 + NPROJ && lane >= 16 && lane <= 16 + KC && w0) {
    // ---- per packed row table -----------------------------------------------------------
    {
      const int proj = warp - 5, p = lane - 16;
      if (p <= KC) {
        const TrisProjView& v = views[proj];
        const int pr = proj_packed_rows(v);
        const int pg = p0 + p;
        PackedRowInfo info{0u, 0, 0, 0};
        if (p0 < pr) {
          const int pc = min(pg, pr);
          int base2 = 0, baseg = 0;
          if (v.qweight2_sparse_prefix) {
            const int32_t* pre = v.qweight2_sparse_prefix + static_cast<size_t>(ex) * (pr + 1);
            base2 = max(0, pre[p0] >> 5) << 5;
            info.rank2 = pre[pc] - base2;
          }
          if (!v.use_block_gr && v.q_gmap_sparse_prefix) {
            const int32_t* pre = v.q_gmap_sparse_prefix + static_cast<size_t>(ex) * (pr + 1);
            baseg = max(0, pre[p0] >> 5) << 5;
            info.rankg = pre[pc] - baseg;
          }
          if (pg < pr) {
            info.cw = static_cast<uint32_t>(v.c_map[static_cast<size_t>(ex) * pr + pg]);
            const int grp = v.packed_row_group ? v.packed_row_group[static_cast<size_t>(ex) * pr + pg] : 0;
            const bool all_groups = v.num_groups * NPROJ * OW <= kRowTabEntries;
            info.gslot = all_groups ? min(max(grp, 0), v.num_groups - 1) : (p < KC ? p : 0);
          }
        }
        sm.ptab[proj * (KC + 1) + p] = info;
      }
    }
  }
  if (threadIdx.x == 0 && w0) {
    const int G = views[0].num_groups;
    sm.row_stride = (G * NPROJ * OW <= kRowTabEntries) ? G : KC;
  }
  bytes_0 = __reduce_add_sync(0xFFFFFFFFu, bytes_0);
  bytes_1 = __reduce_add_sync(0xFFFFFFFFu, bytes_1);
  if (lane == 0) {
    if (w0) {
      if (bytes_0) mbar_arrive_expect_tx(bar_0, bytes_0);
      else mbar_arrive(bar_0);
    }
    if (w1) {
      if (bytes_1) mbar_arrive_expect_tx(bar_1, bytes_1);
      else mbar_arrive(bar_1);
    }
  }
}

// Activation rows.  row_src(n) returns the source row of local row n or -1 for padding.
// `interleaved` activations are copied as they are, one bulk copy per row; lanes 24-31 of
// every warp take eight rows per round, so that no warp issues more than a few copies in a
// row.  Row-major activations are re-ordered by all threads.  Lane 0 of every warp arrives
// on mbar[2].  All threads must call.
template <int NPROJ, int NT, typename RowSrc>
__device__ __forceinline__ void stage_issue_hidden(TileSmem<NPROJ, NT>& sm, const __half* const* hidden,
                                                   const TrisProjView* views, int p0, int nrows, bool interleaved,
                                                   int row_stride, RowSrc row_src) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rank = views[0].rank;
  const int c0 = 32 * p0;
  const int ncols = min(256, rank - c0);
  uint32_t bytes = 0;
  if (interleaved && lane >= 24) {  // callers pass interleaved only when rank % 32 == 0
    fence_proxy_async();
    for (int i = warp * 8 + (lane - 24); i < NPROJ * nrows; i += kWarps * 8) {
      const int proj = i / nrows, n = i - proj * nrows;
      const int src = row_src(n);
      if (src >= 0)
        bytes += lane_copy(reinterpret_cast<uint32_t*>(sm.hrows + (proj * NT * 8 + n) * kHiddenRowBytes),
                           reinterpret_cast<const uint32_t*>(hidden[proj] + static_cast<size_t>(src) * row_stride + c0),
                           ncols >> 1, &sm.mbar[2]);
    }
  }
  bytes = __reduce_add_sync(0xFFFFFFFFu, bytes);
  if (lane == 0) {
    if (bytes) mbar_arrive_expect_tx(&sm.mbar[2], bytes);
    else mbar_arrive(&sm.mbar[2]);
  }
  if (interleaved) return;
  // row-major activations: 8 columns per item, scattered to their pair-interleaved positions
  const int items = NPROJ * nrows * 32;
  for (int i = threadIdx.x; i < items; i += kThreads) {
    const int j8 = i & 31;  // 8-column group inside the chunk
    const int n = (i >> 5) % nrows;
    const int proj = i / (32 * nrows);
    const int col = c0 + 8 * j8;
    const int src = row_src(n);
    __half vals[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) vals[u] = __ushort_as_half(0);
    if (src >= 0 && col < rank) {
      const __half* rowp = hidden[proj] + static_cast<size_t>(src) * row_stride + col;
      if ((rank & 7) == 0 && col + 8 <= rank && (reinterpret_cast<uintptr_t>(rowp) & 15u) == 0) {
        *reinterpret_cast<uint4*>(vals) = *reinterpret_cast<const uint4*>(rowp);
      } else {
        for (int u = 0; u < 8 && col + u < rank; ++u) vals[u] = rowp[u];
      }
    }
    __half* dst = reinterpret_cast<__half*>(sm.hrows + (proj * NT * 8 + n) * kHiddenRowBytes);
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int j = (8 * j8 + u) & 31;
      dst[((8 * j8) & ~31) + 2 * (j & 15) + (j >> 4)] = vals[u];
    }
  }
}

// ---- stage 2: decode + tables ---------------------------------------------------------
// All threads.  Waits for copy set W0 (phase parity0 of mbar[0]), builds the column table
// and expands the block-GR blocks into sm.g; then waits for W1 (parity1 of
// mbar[1]) and builds the select plane (optionally handing the dense g_map words to
// `gmap_dump`).  Returns false when a wait timed out.
template <int NPROJ, int NT>
__device__ __forceinline__ bool stage_finish_weights(TileSmem<NPROJ, NT>& sm, const TrisProjView* views, int e,
                                                     int ex, int o0, int p0, uint32_t parity0, uint32_t parity1,
                                                     uint32_t* gmap_dump, int p_lo = 0, int p_hi = KC) {
  constexpr int OW = Geom<NPROJ>::OW;
  const int tid = threadIdx.x;
  bool ok = mbar_wait_bounded(&sm.mbar[0], parity0);

  // column table: pairs (4t+i, 4t+i+16); scales a column does not use are zeroed so that
  // one fused multiply-add serves salient and non-salient halves alike
  for (int i = tid; i < NPROJ * KC * 16; i += kThreads) {
    const int proj = i / (KC * 16);
    const int p = (i >> 4) % KC;
    const int ii = (i >> 2) & 3;
    const int t = i & 3;
    const TrisProjView& v = views[proj];
    const uint32_t cwv = sm.ptab[proj * (KC + 1) + p].cw;
    const int ja = 4 * t + ii, jb = ja + 16;
    const int ca = 32 * (p0 + p) + ja, cb = ca + 16;
    uint2 pa = make_uint2(0u, 0u), pb = make_uint2(0u, 0u);
    if (ca < v.rank) pa = sm.colraw[proj * 256 + 32 * p + ja];
    if (cb < v.rank) pb = sm.colraw[proj * 256 + 32 * p + jb];
    const bool sa = (cwv >> ja) & 1u, sb = (cwv >> jb) & 1u;
    // col_pack3 halves: (s_c1, s_c2, ns_d_c1, ns_nd_c1) at bits 0/16/32/48 (utils/pack_utils.py:55-64)
    uint4 entry;
    entry.x = (sa ? 0u : (pa.y & 0xFFFFu)) | ((sb ? 0u : (pb.y & 0xFFFFu)) << 16);
    entry.y = (sa ? 0u : (pa.y >> 16)) | ((sb ? 0u : (pb.y >> 16)) << 16);
    entry.z = (sa ? (pa.x & 0xFFFFu) : 0u) | ((sb ? (pb.x & 0xFFFFu) : 0u) << 16);
    entry.w = (sa ? (pa.x >> 16) : 0u) | ((sb ? (pb.x >> 16) : 0u) << 16);
    sm.coltab[((proj * KC + p) * 4 + ii) * 4 + t] = entry;
  }
  // row scale packs when the projection has too many groups to stage them all
  if (sm.row_stride == KC && views[0].num_groups * NPROJ * OW > kRowTabEntries) {
    for (int i = tid; i < kRowTabEntries; i += kThreads) {
      const int p = i % KC;
      const int o = (i / KC) % OW;
      const int proj = i / (KC * OW);
      const TrisProjView& v = views[proj];
      const int pr = proj_packed_rows(v);
      uint2 rp = make_uint2(0u, 0u);
      if (p0 + p < pr && o0 + o < v.out_features) {
        const int grp = v.packed_row_group ? v.packed_row_group[static_cast<size_t>(ex) * pr + p0 + p] : 0;
        if (grp >= 0 && grp < v.num_groups) {
          const unsigned long long w = static_cast<unsigned long long>(
              v.row_pack3[(static_cast<size_t>(e) * v.out_features + o0 + o) * v.num_groups + grp]);
          rp = make_uint2(static_cast<uint32_t>(w), static_cast<uint32_t>(w >> 32));
        }
      }
      sm.rowtab[i] = rp;
    }
  }

  const bool gr = views[0].use_block_gr != 0;
  if (gr) {
    // zero the blocks (raw blocks are copied verbatim)
    for (int i = tid; i < kBlocksPerChunk * 128; i += kThreads) {
      const int b = i >> 7, wl = i & 127;
      const bool raw = (sm.binfo[b * 4 + 2] & TRIS_GR_META_RAW_FLAG) != 0;
      uint32_t word = 0u;
      if (raw && wl < sm.binfo[b * 4 + 1]) word = sm.gmraw[sm.binfo[b * 4 + 0] + wl];
      sm.g[i] = word;
    }
    __syncthreads();
    const int sub = views[0].gr_substreams;  // a power of two
    const int sub_log2 = 31 - __clz(sub);
    for (int i = tid; i < kBlocksPerChunk * sub; i += kThreads) {
      const int b = i >> sub_log2, j = i & (sub - 1);
      const int count = sm.binfo[b * 4 + 1];
      const int meta = sm.binfo[b * 4 + 2];
      if (count <= 0 || (meta & TRIS_GR_META_RAW_FLAG)) continue;
      const int k = meta & TRIS_GR_META_K_MASK;
      const int one_count = min(meta >> TRIS_GR_META_ONE_COUNT_SHIFT, TRIS_GR_BLOCK_WORDS * 32);  // a block has 4096 bits
      const int per = (one_count + sub - 1) >> sub_log2;
      const int first = j * per;
      if (per == 0 || first >= one_count) continue;
      const int n_ones = min(per, one_count - first);
      const uint32_t packed = sm.gridx[b * 32 + j];
      uint32_t* gblock = sm.g + b * 128;
      gr_decode_run(sm.gmraw + sm.binfo[b * 4 + 0], count, k, n_ones, static_cast<int>(packed & 0xFFFFu),
                    static_cast<int>(packed >> 16),
                    [&](int flat) { atomicOr(gblock + (flat >> 5), 1u << (flat & 31)); });
    }
    __syncthreads();
  }

  ok = mbar_wait_bounded(&sm.mbar[1], parity1) && ok;  // the sign plane
  // select plane: for a non-salient column the g_map bit (1 -> "d" scale pair, CU:736-737);
  // for a salient column XNOR(sign1, sign2), because
  //   fp16(+-a +- b) = sign1 * fp16(a + (sign1*sign2) b)
  // so a salient weight is again "pick one of two magnitudes, then apply sign1" with
  // magnitudes fp16(a+b) and fp16(a-b).
  constexpr int NOB = Geom<NPROJ>::NOB;
  for (int i = tid; i < kTileWords; i += kThreads) {  // i is a plane index (block-major)
    const int b = i >> 7, wl = i & 127;
    const int proj = b / (NOB * 4);
    const int p = 2 * ((b / NOB) & 3) + (wl >> 6);
    const int o = (b % NOB) * 64 + (wl & 63);
    if (p < p_lo || p >= p_hi) continue;
    const TrisProjView& v = views[proj];
    const PackedRowInfo info = sm.ptab[proj * (KC + 1) + p];
    const uint32_t cwv = info.cw;
    const uint32_t s1 = sm.s1[i];
    uint32_t s2 = 0u;
    if (cwv) s2 = deposit_bits(staged_bits_at(sm.s2raw + proj * kSparseRows * OW, OW, o, info.rank2), cwv);
    uint32_t gm;
    if (gr) {
      gm = sm.g[i];
    } else {
      const int ncols = min(32, v.rank - 32 * (p0 + p));
      const uint32_t colmask = (ncols >= 32) ? 0xFFFFFFFFu : (ncols <= 0 ? 0u : ((1u << ncols) - 1u));
      const uint32_t nsmask = ~cwv & colmask;
      gm = 0u;
      if (nsmask) gm = spread_around(staged_bits_at(sm.gmraw + proj * kSparseRows * OW, OW, o, info.rankg), cwv & colmask) & nsmask;
    }
    if (gmap_dump) gmap_dump[i] = gm;
    sm.g[i] = (gm & ~cwv) | (cwv & ~(s1 ^ s2));
  }
  return ok;
}

// ---- register unpack ------------------------------------------------------------------
// Row scale pairs of one output for the current group, broadcast to both halves.
struct RowScales {
  __half2 r1, r2, rd, rn;  // row_pack3 halves: (s_r1, s_r2, ns_d_r1, ns_nd_r1)
};
__device__ __forceinline__ RowScales broadcast_row_scales(uint2 rp) {
  RowScales r;
  r.r1 = u32_as_h2(prmt(rp.x, 0u, 0x1010u));
  r.r2 = u32_as_h2(prmt(rp.x, 0u, 0x3232u));
  r.rd = u32_as_h2(prmt(rp.y, 0u, 0x1010u));
  r.rn = u32_as_h2(prmt(rp.y, 0u, 0x3232u));
  return r;
}

// Weights of one packed row for one output and the lane's four column pairs (4t+i, 4t+i+16)
// as half2 bit patterns.  Exact arithmetic of _dequantize_compact3_matrix (QL:4200-4236):
// each product rounded to fp16 once, salient weight = fp16(+-p1 +- p2).  `any_salient` is
// warp-uniform (a property of the packed row), so the branch does not diverge.
__device__ __forceinline__ void unpack_row(uint32_t s1, uint32_t se, const RowScales& rs, const uint4 (&ct)[4],
                                           bool any_salient, int t, uint32_t (&a)[4]) {
  const uint32_t st = s1 << (12 - 4 * t);  // column 4t+i at bit 12+i, column 4t+i+16 at bit 28+i
  const uint32_t gt = se << (12 - 4 * t);
  __half2 ca[4], cb[4];
  if (any_salient) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const __half2 p1 = __hmul2_rn(u32_as_h2(ct[i].z), rs.r1);
      const __half2 p2 = __hmul2_rn(u32_as_h2(ct[i].w), rs.r2);
      // the non-salient half has p1 = p2 = 0, the salient half has cd = cnd = 0
      ca[i] = __hfma2(u32_as_h2(ct[i].x), rs.rd, __hadd2_rn(p1, p2));
      cb[i] = __hfma2(u32_as_h2(ct[i].y), rs.rn, __hsub2_rn(p1, p2));
    }
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      ca[i] = __hmul2_rn(u32_as_h2(ct[i].x), rs.rd);
      cb[i] = __hmul2_rn(u32_as_h2(ct[i].y), rs.rn);
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    // select mask: replicate bits 15 and 31 over their halves
    const uint32_t m = prmt(gt << (3 - i), 0u, 0xBB99u);
    const uint32_t mag = (h2_as_u32(ca[i]) & m) | (h2_as_u32(cb[i]) & ~m);
    // sign: plane bit 1 -> +, 0 -> -   (QL:4213)
    a[i] = mag ^ (~(st << (3 - i)) & 0x80008000u);
  }
}

// Fragments of packed row p for the lane's two outputs (h = 0: out g, h = 1: out g+8).
// `rs` caches the row scales of the group slot `rs_slot` across packed rows.
template <int NPROJ, int NT>
__device__ __forceinline__ void unpack_fragments(const TileSmem<NPROJ, NT>& sm, int proj, int p, int out_local,
                                                 int lane, RowScales (&rs)[2], int& rs_slot, uint32_t (&a)[2][4]) {
  constexpr int OW = Geom<NPROJ>::OW;
  const int g = lane >> 2, t = lane & 3;
  const PackedRowInfo info = sm.ptab[proj * (KC + 1) + p];
  if (info.gslot != rs_slot) {  // warp-uniform; groups span several packed rows
    rs_slot = info.gslot;
    const int stride = sm.row_stride;
#pragma unroll
    for (int h = 0; h < 2; ++h)
      rs[h] = broadcast_row_scales(sm.rowtab[(proj * OW + out_local + g + 8 * h) * stride + rs_slot]);
  }
  uint4 ct[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) ct[i] = sm.coltab[((proj * KC + p) * 4 + i) * 4 + t];
  const int idx = plane_index<NPROJ>(proj, p, out_local + g);
  const uint32_t s1a = sm.s1[idx], s1b = sm.s1[idx + 8];
  const uint32_t sea = sm.g[idx], seb = sm.g[idx + 8];
  const bool any_salient = info.cw != 0u;
  unpack_row(s1a, sea, rs[0], ct, any_salient, t, a[0]);
  unpack_row(s1b, seb, rs[1], ct, any_salient, t, a[1]);
}

// B fragments of packed row p, local activation row `n`: 8 halves in pair order.
template <int NPROJ, int NT>
__device__ __forceinline__ uint4 load_b_fragments(const TileSmem<NPROJ, NT>& sm, int proj, int n, int p, int t) {
  return *reinterpret_cast<const uint4*>(sm.hrows + (proj * NT * 8 + n) * kHiddenRowBytes + p * 64 + t * 16);
}

// ---- launch arguments shared by the grouped kernels ---------------------------------------
struct GroupedArgs {
  TrisProjView proj[2];
  const __half* hidden[2];
  __half* out[2];
  const int32_t* expert_ids;
  const int32_t* segment_offsets;
  const int32_t* num_segments_dev;
  const int32_t* row_gather;
  const int32_t* out_scatter;  // output row of each grouped row, or null
  int32_t* status;
  int32_t num_segments;
  int32_t num_rows;
  int32_t hidden_interleaved;
  int32_t hidden_stride;        // halves between consecutive activation rows (>= rank)
  int32_t weights_before_wait;  // route arrays were final before the predecessor kernel started
  int32_t ksplit;               // CTAs per cluster sharing one tile: each takes 8/ksplit packed rows of a chunk
  // tile-record form of the tcgen05 kernel (grouped_umma.cu): activation rows in lane order, slot sizes of the
  // staged records
  int32_t hidden_lane_order;
  int32_t rec_slot_bytes;
  int32_t col_slot_bytes;
};

enum { EPI_STORE = 0, EPI_SILU_MUL = 1 };

__device__ __forceinline__ void init_stage_barriers(uint64_t* mbar) {
  if (threadIdx.x == 0) {
    mbar_init(&mbar[0], kWarps);  // lane 0 of every warp arrives, with its warp's byte count
    mbar_init(&mbar[1], kWarps);
    mbar_init(&mbar[2], kWarps);
    fence_mbar_init();
  }
  __syncthreads();
}

}  // namespace tris
