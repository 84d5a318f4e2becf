// Tile records: the load-time, tile-major image of a block-GR compact3 projection, and the
// device code that consumes it (Golomb-Rice decode into shared memory, register unpack into
// tensor-core fragments).  Shared by the record builder, the grouped kernels and the two
// dump kernels, so that the bit-exact parity checks run the code of the hot path.
//
// Why records.  The E-stacked payload tensors of build_grouped_precomputed_payload
// (QL:1512-1636 of the TriS-MoE tree) are laid out plane by plane; a CTA that wants one
// (expert, 64 outputs, 256 columns) tile has to look up prefixes and block offsets and then
// fetch ~30 short strided rows.  A record is the same data gathered once, at load time, into
// ONE contiguous 16-byte aligned piece, so the tile arrives with a single bulk copy:
//
//   tile record (expert e, outputs 64*tile .. +63, packed rows 8*chunk .. +7)
//     header   64 B   block-GR block table, section offsets
//     s1     2048 B   sign plane qweight1, [packed row][out]
//     rowtab   512 B per row-scale slot: row_pack3 of the 64 outputs, [slot][out]
//     gridx    512 B  block-GR sub-stream index of the 4 blocks, [block][32]
//     ss1,ss2  256 B per salient word each: sign1 / sign2 of the salient columns, [word][out]
//     gr       the 4 blocks' Golomb-Rice words, verbatim (QL:3763-3859), padded to 16 B
//
//   column record (expert e, packed rows 8*chunk .. +7), shared by all output tiles
//     header   64 B   row-scale slot of each packed row, salient word count
//     coltab 1024 B   per packed row and lane: the four (d, nd) column-scale pairs a lane needs
//     salient  256 B per salient word: activation positions, (c1, c2) scale pairs, true columns
//
// A "row-scale slot" is a run of packed rows of the chunk that share one quantisation group
// (g_idx is constant inside a packed word; tris_build_row_groups checks that), so one
// row_pack3 word per (output, slot) serves the whole run.
//
// Salient columns (c_map bit set) carry two signed terms instead of one; they are ~10 % of
// the columns.  The main loop treats every column as non-salient with column scales of zero
// at the salient positions (the weight there is +-0), and a short second pass multiplies the
// salient columns, compacted into "salient words" of 32 slots: slots 0-15 hold salient columns
// of one row-scale slot, slots 16-31 of one (possibly another) slot, so that the row scales of
// a half2 (slot j, slot j+16) are two broadcast values.  ss1 is a derived copy of the sign1
// bits at the salient columns; ss2 re-aligns qweight2_sparse to the same slots.
//
// Lane order.  Lane (g = lane / 4, t = lane % 4) of a warp owns outputs g and g+8 of its 16
// outputs and, in every 32-column word, the column pairs (t+8, t+24), (t, t+16), (t+12, t+28),
// (t+4, t+20).  Two shifts per word (by 7-t and 3-t) bring those bits to the byte MSBs 15/31
// and 7/23, where PRMT's sign-replicate mode turns each pair into a half2-wide mask.  The
// activation rows are consumed in the matching order ("lane order": column j of a 32-column
// group sits at 8*(j%4) + 2*slot(j/4%4) + j/16 with slot = {1,3,0,2}), so a lane's B fragments
// for a packed row are one 16-byte shared-memory load.
#pragma once
#include "common.cuh"

namespace tris {
namespace tr {

constexpr int kTileOut = 64;       // outputs per tile record
constexpr int kChunkRows = 8;      // packed rows per record (256 columns)
constexpr int kHdrBytes = 64;
constexpr int kS1Bytes = kChunkRows * kTileOut * 4;
constexpr int kSlotBytes = kTileOut * 8;      // one row-scale slot
constexpr int kGridxBytes = 4 * 32 * 4;
constexpr int kSalPlaneBytes = kTileOut * 4;  // one salient word, one sign plane
constexpr int kColHdrBytes = 64;
constexpr int kColTabBytes = kChunkRows * 4 * 32;
constexpr int kSalEntryBytes = 256;
constexpr int kMaxSalWords = 8;    // 256 salient columns, worst case
constexpr int kHiddenRowBytes = 576;  // 512 B of activations + 64 B: 8 rows hit 8 bank groups

struct RecHeader {                 // 64 bytes
  uint32_t blk[4][2];              // per block: word offset | word count << 16 (inside gr), meta
  uint16_t off_rowtab, off_gridx, off_ss1, off_ss2, off_gr;  // byte offsets inside the record
  uint8_t num_slots, sal_words;
  uint32_t gr_words;
  uint32_t pad[4];
};
static_assert(sizeof(RecHeader) == kHdrBytes, "record header");

struct ColHeader {                 // 64 bytes
  uint8_t slot_of_row[kChunkRows];
  uint8_t sal_slot[kMaxSalWords][2];  // row-scale slot of slots 0-15 / 16-31 of each salient word
  uint16_t num_salient;
  uint8_t sal_words, num_slots;
  uint8_t slot_end[kChunkRows];       // packed rows [slot_end[s-1], slot_end[s]) of the chunk use slot s
  uint32_t pad[7];
};
static_assert(sizeof(ColHeader) == kColHdrBytes, "column record header");

__host__ __device__ inline int tiles_per_expert(int out_features) { return (out_features + kTileOut - 1) / kTileOut; }
__host__ __device__ inline int num_chunks(int rank) { return ((rank + 31) / 32 + kChunkRows - 1) / kChunkRows; }
__host__ __device__ inline int col_record_bytes(int max_sal_words) {
  return kColHdrBytes + kColTabBytes + max_sal_words * kSalEntryBytes;
}
__host__ __device__ inline int record_bytes(int num_slots, int sal_words, int gr_words) {
  return kHdrBytes + kS1Bytes + num_slots * kSlotBytes + kGridxBytes + 2 * sal_words * kSalPlaneBytes +
         ((gr_words + 3) & ~3) * 4;
}

// The two columns (inside the 32-column group) of half2 i (0..3) of lane t.
__host__ __device__ inline int lane_pair_col(int t, int i) {
  const int q = (0x1302 >> (4 * i)) & 3;  // i = 0,1,2,3 -> q = 2,0,3,1
  return t + 4 * q;                        // low half; the high half is this + 16
}

// ---- salient slot assignment ----------------------------------------------------------------
// One thread walks the chunk's packed rows.  slot_of_row[p] = index of the run of equal group
// ids that packed row p belongs to.  Salient columns of a run fill "steps" of 16 slots; a new
// run starts a new step; step s is half (s & 1) of salient word (s >> 1).  col_of_slot gets
// the chunk-relative column of every slot or 0xFFFF.  Returns the number of steps.
struct ChunkPlan {
  uint8_t slot_of_row[kChunkRows];
  uint8_t step_slot[2 * kMaxSalWords];
  int num_slots, num_steps, num_salient;
};
__device__ inline void plan_chunk(const int32_t* c_map_e, const int32_t* row_group_e, int pr, int p0, int rank,
                                  ChunkPlan& plan, uint16_t* col_of_slot /* [kMaxSalWords * 32] or null */) {
  plan.num_slots = 0;
  plan.num_steps = 0;
  plan.num_salient = 0;
  if (col_of_slot)
    for (int i = 0; i < kMaxSalWords * 32; ++i) col_of_slot[i] = 0xFFFFu;
  for (int i = 0; i < 2 * kMaxSalWords; ++i) plan.step_slot[i] = 0;
  int prev_group = -0x7fffffff, fill = 16;
  for (int p = 0; p < kChunkRows; ++p) {
    const int pg = p0 + p;
    if (pg >= pr) {
      plan.slot_of_row[p] = 0;
      continue;
    }
    const int grp = row_group_e ? row_group_e[pg] : 0;
    if (grp != prev_group) {
      prev_group = grp;
      ++plan.num_slots;
      fill = 16;  // the next salient column opens a new step
    }
    const int slot = plan.num_slots - 1;
    plan.slot_of_row[p] = static_cast<uint8_t>(slot);
    uint32_t cw = static_cast<uint32_t>(c_map_e[pg]);
    const int ncols = rank - 32 * pg;
    if (ncols < 32) cw &= (ncols <= 0) ? 0u : ((1u << ncols) - 1u);
    while (cw) {
      const int j = __ffs(cw) - 1;
      cw &= cw - 1;
      if (fill == 16) {
        fill = 0;
        plan.step_slot[plan.num_steps] = static_cast<uint8_t>(slot);
        ++plan.num_steps;
      }
      const int s = plan.num_steps - 1;
      if (col_of_slot) col_of_slot[(s >> 1) * 32 + (s & 1) * 16 + fill] = static_cast<uint16_t>(32 * p + j);
      ++fill;
      ++plan.num_salient;
    }
  }
  if (plan.num_slots == 0) plan.num_slots = 1;
}

// ---- shared-memory loads by 32-bit shared address ---------------------------------------------
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ void red_or_shared(uint32_t addr, uint32_t bits) {
  asm volatile("red.shared.or.b32 [%0], %1;" ::"r"(addr), "r"(bits) : "memory");
}
__device__ __forceinline__ uint32_t shf_r_clamp(uint32_t lo, uint32_t hi, int n) {
  uint32_t d;
  asm("shf.r.clamp.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(lo), "r"(hi), "r"(n));
  return d;
}
__device__ __forceinline__ uint32_t shf_r_wrap(uint32_t lo, uint32_t hi, int n) {
  uint32_t d;
  asm("shf.r.wrap.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(lo), "r"(hi), "r"(n));
  return d;
}
__device__ __forceinline__ uint32_t shl_wrap(uint32_t v, int n) {
  uint32_t d;
  asm("shf.l.wrap.b32 %0, %1, %1, %2;" : "=r"(d) : "r"(v), "r"(n));  // rotate; callers pass a single set bit
  return d;
}

// ---- block Golomb-Rice ------------------------------------------------------------------------
// One sub-stream of a block (QL:3763-3791: for every one-bit the zero run before it as run >> k
// zeros, a one, then the low k bits of the run LSB first; decode semantics of
// decode_block_gr_block, CU:426-479).  `words` is the shared address of the block's first word,
// (bitpos, flat) where this sub-stream starts, `plane` the shared address of the block's 128
// decoded words.  The stream is read through a three-word register window, so no load sits on
// the codeword-to-codeword dependency chain.  Reads run up to three words past the block's
// last word; callers keep that much slack behind every staged stream.
//
// Fast form: every codeword of the block fits a 32-bit view (zero run + 1 + k <= 32) and every
// decoded position lies inside the block; the record builder checks both when it parses the
// stream at load time and marks blocks that fail with kBlockSlowFlag.
constexpr int kBlockSlowFlag = 0x20;  // in the record's copy of the block meta word (not a reference bit)

__device__ __forceinline__ uint32_t ctz_nonzero(uint32_t v) {
  uint32_t r, t;
  asm("brev.b32 %0, %1;" : "=r"(r) : "r"(v));
  asm("bfind.shiftamt.u32 %0, %1;" : "=r"(t) : "r"(r));
  return t;
}

// `trips` is the warp-uniform iteration count (the longest sub-stream of the block), `n_ones`
// this lane's count: a lane past its last codeword keeps decoding whatever follows (the next
// sub-stream, then slack) with its stores switched off, so the loop has no divergent branch.
__device__ __forceinline__ void gr_decode_substream_fast(uint32_t words, int k, int n_ones, int trips, int bitpos, int flat,
                                                         uint32_t plane) {
  const int k1 = k + 1;
  const uint32_t kmask = (1u << k) - 1u;
  uint32_t addr = words + (static_cast<uint32_t>(bitpos >> 5) << 2);
  uint32_t lo = lds32(addr), hi = lds32(addr + 4), nx = lds32(addr + 8);
  int sh = bitpos & 31;
#pragma unroll 2
  for (int n = 0; n < trips; ++n) {
    const uint32_t v = shf_r_wrap(lo, hi, sh) | 0x80000000u;  // the guard bit only matters past the lane's last codeword
    const int t = static_cast<int>(ctz_nonzero(v));             // zero run
    const uint32_t rem = shf_r_clamp(v, 0u, t + 1) & kmask;
    const int pos = flat + (t << k) + static_cast<int>(rem);
    if (n < n_ones) red_or_shared(plane + ((static_cast<uint32_t>(pos) >> 3) & 0x1FCu), shl_wrap(1u, pos));
    flat = pos + 1;
    sh += t + k1;
    const bool refill = sh >= 32;
    if (refill) {
      sh -= 32;
      lo = hi;
      hi = nx;
      addr += 4;
    }
    if (refill) nx = lds32(addr + 8);  // needed two words from now: its latency is off the chain
  }
}

// General form: zero runs of any length, remainders that straddle a word, malformed streams.
static __device__ __noinline__ void gr_decode_substream_slow(uint32_t words, int nwords, int k, int n_ones, int bitpos, int flat,
                                                     uint32_t plane) {
  const uint32_t kmask = (1u << k) - 1u;
  const int total_bits = nwords << 5;
  auto peek = [&](int bp) {
    const int wi = bp >> 5;
    const uint32_t lo = (wi < nwords) ? lds32(words + (static_cast<uint32_t>(wi) << 2)) : 0u;
    const uint32_t hi = (wi + 1 < nwords) ? lds32(words + (static_cast<uint32_t>(wi + 1) << 2)) : 0u;
    return shf_r_wrap(lo, hi, bp & 31);
  };
  for (int n = 0; n < n_ones; ++n) {
    int q = 0;
    uint32_t w = peek(bitpos);
    while (w == 0u) {
      q += 32;
      bitpos += 32;
      if (bitpos >= total_bits) return;  // the stream ran out: malformed, stop
      w = peek(bitpos);
    }
    const int t = __ffs(w) - 1;
    bitpos += t + 1;
    const uint32_t rem = peek(bitpos) & kmask;
    bitpos += k;
    const int pos = flat + ((q + t) << k) + static_cast<int>(rem);
    if (pos >= TRIS_GR_BLOCK_WORDS * 32 || bitpos > total_bits) return;
    red_or_shared(plane + ((static_cast<uint32_t>(pos) >> 3) & ~3u), shl_wrap(1u, pos));
    flat = pos + 1;
  }
}

// Decodes block `b` (0..3) of a staged record with one warp: lane j takes sub-stream j.  The
// 128 decoded words [packed row parity][out] land at plane + b * 512 bytes, which the caller
// zeroed beforehand (raw blocks are copied).
__device__ __forceinline__ void gr_decode_block(const uint8_t* rec, int b, uint32_t* plane, int lane) {
  const RecHeader* hdr = reinterpret_cast<const RecHeader*>(rec);
  const uint32_t oc = hdr->blk[b][0];
  const int meta = static_cast<int>(hdr->blk[b][1]);
  const int off = static_cast<int>(oc & 0xFFFFu), count = static_cast<int>(oc >> 16);
  if (count == 0) return;
  const uint32_t* words = reinterpret_cast<const uint32_t*>(rec + hdr->off_gr) + off;
  uint32_t* out = plane + b * TRIS_GR_BLOCK_WORDS;
  if (meta & TRIS_GR_META_RAW_FLAG) {
    for (int i = lane; i < TRIS_GR_BLOCK_WORDS && i < count; i += 32) out[i] = words[i];
    return;
  }
  const int one_count = min(meta >> TRIS_GR_META_ONE_COUNT_SHIFT, TRIS_GR_BLOCK_WORDS * 32);
  const int per = (one_count + 31) >> 5;
  const int first = lane * per;
  if (per == 0 || first >= one_count) return;
  const uint32_t packed = reinterpret_cast<const uint32_t*>(rec + hdr->off_gridx)[b * 32 + lane];
  const int k = meta & TRIS_GR_META_K_MASK, n = min(per, one_count - first);
  if (meta & kBlockSlowFlag)
    gr_decode_substream_slow(smem_u32(words), count, k, n, static_cast<int>(packed & 0xFFFFu), static_cast<int>(packed >> 16),
                             smem_u32(out));
  else
    gr_decode_substream_fast(smem_u32(words), k, n, per, static_cast<int>(packed & 0xFFFFu), static_cast<int>(packed >> 16),
                             smem_u32(out));
}

// ---- register unpack --------------------------------------------------------------------------
// The integer ALU pipe (PRMT, LOP3, shifts) issues at half the rate of the FMA pipe (IMAD, HMUL2),
// and the unpack is almost all bit work, so it is written to spread over both:
//   * the two per-word shifts are multiplications by a per-lane power of two (IMAD);
//   * the sign needs only bits 15 / 31 of a half2, which the shifted word already holds for the
//     (t+8, t+24) and (t+12, t+28) pairs; for the other two pairs one more multiplication by 256
//     moves bits 7 / 23 up.  No mask is built for the sign;
//   * the g_map select does need half-wide masks: PRMT in sign-replicate mode spreads bit 15 over
//     the low half and bit 31 over the high half (selector 0xBB99), or bits 7 / 23 (0xAA88).
struct LaneShifts {
  uint32_t mul_a, mul_b;  // 1 << (7 - t), 1 << (3 - t)
  uint32_t mul_8;         // 256: moves bits 7 / 23 up to 15 / 31
};
__device__ __forceinline__ LaneShifts lane_shifts(int t) {
  LaneShifts ls;
  ls.mul_a = 1u << (7 - t);
  ls.mul_b = 1u << (3 - t);
  // keep the compiler from turning the multiplications back into (ALU pipe) shifts
  ls.mul_8 = 256u;
  asm("" : "+r"(ls.mul_a));
  asm("" : "+r"(ls.mul_b));
  asm("" : "+r"(ls.mul_8));
  return ls;
}
__device__ __forceinline__ uint32_t mask_hi(uint32_t w) { return prmt(w, 0u, 0xBB99u); }
__device__ __forceinline__ uint32_t mask_lo(uint32_t w) { return prmt(w, 0u, 0xAA88u); }

__device__ __forceinline__ uint32_t lop3_select(uint32_t a, uint32_t b, uint32_t m) {
  uint32_t d;
  asm("lop3.b32 %0, %1, %2, %3, 0xCA;" : "=r"(d) : "r"(m), "r"(a), "r"(b));  // m ? a : b
  return d;
}
// v ^ (~w & 0x80008000): sign-plane bit (at 15 / 31 of w) 1 -> +, 0 -> - (QL:4213)
__device__ __forceinline__ uint32_t flip_by_bits(uint32_t v, uint32_t w) { return v ^ (~w & 0x80008000u); }

// Non-salient weights of one packed row for one output: the lane's four column pairs as half2
// bit patterns a[0..3] (pair order of lane_pair_col).  Exact arithmetic of
// _dequantize_compact3_matrix (QL:4200-4236): one product per weight, rounded to fp16 once.
// ct = {cd(0), cn(0), cd(1), cn(1)}, {cd(2), cn(2), cd(3), cn(3)}: column scales of the d / nd
// kinds per pair, zero at salient columns.
__device__ __forceinline__ void unpack_row_ns(uint32_t s1, uint32_t gm, __half2 rd, __half2 rn, const uint4& c01,
                                              const uint4& c23, const LaneShifts& ls, uint32_t (&a)[4]) {
  const uint32_t sA = s1 * ls.mul_a, sB = s1 * ls.mul_b;
  const uint32_t gA = gm * ls.mul_a, gB = gm * ls.mul_b;
  const uint32_t cd[4] = {c01.x, c01.z, c23.x, c23.z};
  const uint32_t cn[4] = {c01.y, c01.w, c23.y, c23.w};
  const uint32_t up8 = ls.mul_8;
  const uint32_t sg[4] = {sA, sA * up8, sB, sB * up8};
  const uint32_t mg[4] = {mask_hi(gA), mask_lo(gA), mask_hi(gB), mask_lo(gB)};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t vd = h2_as_u32(__hmul2_rn(u32_as_h2(cd[i]), rd));
    const uint32_t vn = h2_as_u32(__hmul2_rn(u32_as_h2(cn[i]), rn));
    a[i] = flip_by_bits(lop3_select(vd, vn, mg[i]), sg[i]);  // g_map bit 1 -> "d" pair (CU:736-737)
  }
}

// Salient weights of one salient word for one output: fp16(+-fp16(c1 r1) +- fp16(c2 r2)).
// sc = {c1(0), c2(0), c1(1), c2(1)}, {c1(2), c2(2), c1(3), c2(3)}; r1 / r2 hold the row scales
// of the word's two halves (slots 0-15 in the low half, 16-31 in the high half).
__device__ __forceinline__ void unpack_row_sal(uint32_t w1, uint32_t w2, __half2 r1, __half2 r2, const uint4& c01,
                                               const uint4& c23, const LaneShifts& ls, uint32_t (&a)[4]) {
  const uint32_t s1A = w1 * ls.mul_a, s1B = w1 * ls.mul_b;
  const uint32_t s2A = w2 * ls.mul_a, s2B = w2 * ls.mul_b;
  const uint32_t c1[4] = {c01.x, c01.z, c23.x, c23.z};
  const uint32_t c2[4] = {c01.y, c01.w, c23.y, c23.w};
  const uint32_t up8 = ls.mul_8;
  const uint32_t g1[4] = {s1A, s1A * up8, s1B, s1B * up8};
  const uint32_t g2[4] = {s2A, s2A * up8, s2B, s2B * up8};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t p1 = flip_by_bits(h2_as_u32(__hmul2_rn(u32_as_h2(c1[i]), r1)), g1[i]);
    const uint32_t p2 = flip_by_bits(h2_as_u32(__hmul2_rn(u32_as_h2(c2[i]), r2)), g2[i]);
    a[i] = h2_as_u32(__hadd2_rn(u32_as_h2(p1), u32_as_h2(p2)));
  }
}

// Row scales of one output for one slot, broadcast to both halves: row_pack3 halves are
// (s_r1, s_r2, ns_d_r1, ns_nd_r1) (utils/pack_utils.py:55-64).
__device__ __forceinline__ void row_scales_ns(uint2 rp, __half2& rd, __half2& rn) {
  rd = u32_as_h2(prmt(rp.y, 0u, 0x1010u));
  rn = u32_as_h2(prmt(rp.y, 0u, 0x3232u));
}
__device__ __forceinline__ void row_scales_sal(uint2 rp_lo, uint2 rp_hi, __half2& r1, __half2& r2) {
  r1 = u32_as_h2(prmt(rp_lo.x, rp_hi.x, 0x5410u));
  r2 = u32_as_h2(prmt(rp_lo.x, rp_hi.x, 0x7632u));
}

// ---- fetching records ----------------------------------------------------------------------------
__device__ __forceinline__ uint2 load_desc(const TrisProjView& v, int expert, int tile, int chunk) {
  const int idx = (expert * tiles_per_expert(v.out_features) + tile) * num_chunks(v.rank) + chunk;
  return reinterpret_cast<const uint2*>(v.tile_desc)[idx];
}

// Starts the copies of one tile record (descriptor d) and, optionally, of the column record of
// (expert, chunk); arrives on `bar` with the byte count.  One thread.
__device__ __forceinline__ void issue_record(const TrisProjView& v, int expert, int chunk, uint2 d, uint8_t* rec_dst,
                                             uint8_t* col_dst, bool valid, uint64_t* bar) {
  fence_proxy_async();
  uint32_t bytes = 0;
  if (valid) {
    bulk_g2s(rec_dst, static_cast<const uint8_t*>(v.tile_records) + static_cast<size_t>(d.x) * 16, d.y, bar);
    bytes = d.y;
    if (col_dst) {
      bulk_g2s(col_dst,
               static_cast<const uint8_t*>(v.col_records) + (static_cast<size_t>(expert) * num_chunks(v.rank) + chunk) * v.col_record_bytes,
               static_cast<uint32_t>(v.col_record_bytes), bar);
      bytes += static_cast<uint32_t>(v.col_record_bytes);
    }
  }
  if (bytes) mbar_arrive_expect_tx(bar, bytes);
  else mbar_arrive(bar);
}

// ---- a staged tile: pointers into shared memory ----------------------------------------------
struct StagedTile {
  const uint8_t* rec;    // tile record
  const uint8_t* col;    // column record
  const uint32_t* gmap;  // decoded g_map plane, [packed row][out], 512 words
};

// Row scales of the lane's two outputs (o = out_local + g and o + 8) for one row-scale slot.
struct RowScalesNs {
  __half2 rd[2], rn[2];
};
__device__ __forceinline__ RowScalesNs load_row_scales_ns(const StagedTile& st, int slot, int out_local, int lane) {
  const RecHeader* hdr = reinterpret_cast<const RecHeader*>(st.rec);
  const uint2* rowtab = reinterpret_cast<const uint2*>(st.rec + hdr->off_rowtab) + slot * kTileOut + out_local + (lane >> 2);
  RowScalesNs rs;
  row_scales_ns(rowtab[0], rs.rd[0], rs.rn[0]);
  row_scales_ns(rowtab[8], rs.rd[1], rs.rn[1]);
  return rs;
}

// A fragments of packed row p for the lane's outputs o and o + 8 (o = out_local + g).
__device__ __forceinline__ void unpack_fragments_ns(const StagedTile& st, int p, int out_local, int lane,
                                                    const RowScalesNs& rs, const LaneShifts& ls, uint32_t (&a)[2][4]) {
  const int g = lane >> 2, t = lane & 3;
  const uint4* ct = reinterpret_cast<const uint4*>(st.col + kColHdrBytes) + (p * 4 + t) * 2;
  const uint4 c01 = ct[0], c23 = ct[1];
  const uint32_t* s1 = reinterpret_cast<const uint32_t*>(st.rec + kHdrBytes) + p * kTileOut + out_local + g;
  const uint32_t* gm = st.gmap + p * kTileOut + out_local + g;
  unpack_row_ns(s1[0], gm[0], rs.rd[0], rs.rn[0], c01, c23, ls, a[0]);
  unpack_row_ns(s1[8], gm[8], rs.rd[1], rs.rn[1], c01, c23, ls, a[1]);
}

__device__ __forceinline__ void unpack_fragments_sal(const StagedTile& st, int q, int out_local, int lane,
                                                     const LaneShifts& ls, uint32_t (&a)[2][4]) {
  const int g = lane >> 2, t = lane & 3;
  const RecHeader* hdr = reinterpret_cast<const RecHeader*>(st.rec);
  const ColHeader* ch = reinterpret_cast<const ColHeader*>(st.col);
  const uint2* rowtab = reinterpret_cast<const uint2*>(st.rec + hdr->off_rowtab) + out_local + g;
  const int sl = ch->sal_slot[q][0], sh = ch->sal_slot[q][1];
  __half2 r1[2], r2[2];
  row_scales_sal(rowtab[sl * kTileOut], rowtab[sh * kTileOut], r1[0], r2[0]);
  row_scales_sal(rowtab[sl * kTileOut + 8], rowtab[sh * kTileOut + 8], r1[1], r2[1]);
  const uint4* sc = reinterpret_cast<const uint4*>(st.col + kColHdrBytes + kColTabBytes + q * kSalEntryBytes + 64) + t * 2;
  const uint4 c01 = sc[0], c23 = sc[1];
  const uint32_t* w1 = reinterpret_cast<const uint32_t*>(st.rec + hdr->off_ss1) + q * kTileOut + out_local + g;
  const uint32_t* w2 = reinterpret_cast<const uint32_t*>(st.rec + hdr->off_ss2) + q * kTileOut + out_local + g;
  unpack_row_sal(w1[0], w2[0], r1[0], r2[0], c01, c23, ls, a[0]);
  unpack_row_sal(w1[8], w2[8], r1[1], r2[1], c01, c23, ls, a[1]);
}

}  // namespace tr
}  // namespace tris
