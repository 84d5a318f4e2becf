// Grouped compact3 dequant-matmul over tile records (decode / skinny regime), and the dump
// kernel the parity tests use.  See tile_records.cuh for the record layout and the unpack.
//
// Work unit = one expert segment x two tile records: the gate and the up tile of the same 64
// outputs (dual launch), or two neighbouring 64-output tiles of one projection.  A CTA has 8
// warps; warp w works on record w / 4, outputs 16 * (w % 4) .. +15.  Per unit:
//   1. two threads fetch the two tile records and their column records, one bulk copy each
//      (cp.async.bulk completing on an mbarrier);
//   2. every warp Golomb-Rice decodes one block-GR block (32 lanes = 32 indexed sub-streams)
//      into the g_map plane in shared memory;
//   3. activation rows arrive by bulk copies (one per row, issued by eight lanes of every warp);
//      the activations of the salient columns are gathered into rows of their own;
//   4. every warp unpacks its weights straight into m16n8k16 A fragments and multiplies them
//      with the staged rows, fp32 accumulation; then the short salient pass;
//   5. results go through shared memory and leave as 16-byte stores.
// No dequantised weight leaves registers.
//
// Two kernels share this code.  grouped_tiled_persistent_kernel (projections of at most 256
// columns: one chunk) runs a fixed number of CTAs per SM, each walking units blockIdx.x,
// blockIdx.x + gridDim.x, ...; the records of the next unit are fetched into the other half of
// a two-stage ring while the current unit is decoded and multiplied, so the fetch latency
// (route entry -> descriptor -> DRAM) is paid once per CTA instead of once per unit.
// grouped_tiled_kernel (any number of chunks) runs one CTA per unit and loops over the chunks.
// Waits on mbarriers are bounded; a time-out is reported through the route's status word and
// the CTA leaves without storing results.
#include <math.h>

#include <algorithm>
#include <atomic>

#include "tile_records.cuh"

namespace tris {
namespace tr {

constexpr int kThreads = 256;
constexpr int kWarps = 8;
constexpr int kOutTileRowBytes = 144;  // 64 halves + 16 bytes: rows 2t of the four t land in four bank groups
enum { MODE_SINGLE = 0, MODE_DUAL_STORE = 1, MODE_DUAL_SILU = 2 };

struct TiledArgs {
  TrisProjView proj[2];
  const __half* hidden[2];
  __half* out[2];
  const int32_t* expert_ids;
  const int32_t* segment_offsets;
  const int32_t* num_segments_dev;
  const int32_t* row_gather;
  const int32_t* out_scatter;
  int32_t* status;
  int32_t num_segments;
  int32_t num_rows;
  int32_t hidden_lane_order;    // activation rows already in lane order (else row-major)
  int32_t hidden_stride;        // halves between activation rows
  int32_t weights_before_wait;  // route arrays were final before the predecessor kernel started
  int32_t rec_slot_bytes;       // shared-memory bytes reserved per tile record (16 bytes of slack included)
  int32_t col_slot_bytes;
  int32_t sal_slots;            // salient words reserved per activation set
  const __half* col_scale;      // optional [rank]: activation rows are multiplied by it while staged (row-major rows only)
};

// Shared-memory carve-up: [mbarriers 64][stages x (2 records + NH column records)][2 g_map planes]
// [salient rows NH x sal_slots x NT*8 x 64][activation rows NH x NT*8 x 576]
struct SmemLayout {
  int stage_bytes, gmap_off, hsal_off, hrows_off, total;
};
__host__ __device__ inline SmemLayout smem_layout(int rec_slot, int col_slot, int sal_slots, int nh, int nt, int stages) {
  SmemLayout l;
  l.stage_bytes = 2 * rec_slot + nh * col_slot;
  l.gmap_off = 64 + stages * l.stage_bytes;
  l.hsal_off = l.gmap_off + 2 * 2048;
  l.hrows_off = l.hsal_off + nh * sal_slots * nt * 8 * 64;
  l.total = l.hrows_off + nh * nt * 8 * kHiddenRowBytes;
  return l;
}

// One lane moves nbytes global -> shared: a bulk copy when both ends are 16-byte aligned and the
// size is a multiple of 16, plain loads otherwise.  Returns the bytes the mbarrier must expect.
__device__ __forceinline__ uint32_t lane_copy_bytes(void* dst, const void* src, int nbytes, uint64_t* bar) {
  if (nbytes <= 0) return 0;
  if (((reinterpret_cast<uintptr_t>(src) | smem_u32(dst) | static_cast<uint32_t>(nbytes)) & 15u) == 0) {
    bulk_g2s(dst, src, static_cast<uint32_t>(nbytes), bar);
    return static_cast<uint32_t>(nbytes);
  }
  for (int i = 0; i < nbytes; i += 2)
    *reinterpret_cast<uint16_t*>(static_cast<uint8_t*>(dst) + i) = *reinterpret_cast<const uint16_t*>(static_cast<const uint8_t*>(src) + i);
  return 0;
}

// Activation rows of a pass into hrows[set][row]; row_src(n) = source row or -1.  Lane-order
// rows are copied as they are (lanes 0-7 of every warp issue one bulk copy per round); row-major
// rows are re-ordered by all threads.  Lane 0 of every warp arrives on `bar`.
template <int NT, int NH, typename RowSrc>
__device__ __forceinline__ void issue_hidden(uint8_t* hrows, const __half* const* hidden, int rank, int p0, int nrows,
                                             bool lane_order, int row_stride, uint64_t* bar, RowSrc row_src,
                                             const __half* col_scale = nullptr) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int c0 = 32 * p0;
  const int ncols = min(256, rank - c0);
  uint32_t bytes = 0;
  if (lane_order && lane < 8) {
    fence_proxy_async();
    for (int i = warp * 8 + lane; i < NH * nrows; i += kWarps * 8) {
      const int set = (NH == 2 && i >= nrows) ? 1 : 0;
      const int n = i - set * nrows;
      const int src = row_src(n);
      if (src >= 0)
        bytes += lane_copy_bytes(hrows + (set * NT * 8 + n) * kHiddenRowBytes,
                                 hidden[set] + static_cast<size_t>(src) * row_stride + c0, 2 * ncols, bar);
    }
  }
  bytes = __reduce_add_sync(0xFFFFFFFFu, bytes);
  if (lane == 0) {
    if (bytes) mbar_arrive_expect_tx(bar, bytes);
    else mbar_arrive(bar);
  }
  if (lane_order) return;
  const int items = NH * nrows * 32;  // 8 columns per item
  for (int i = threadIdx.x; i < items; i += kThreads) {
    const int j8 = i & 31, n = (i >> 5) % nrows, set = i / (32 * nrows);
    const int col = c0 + 8 * j8;
    const int src = row_src(n);
    __half vals[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) vals[u] = __ushort_as_half(0);
    if (src >= 0 && col < rank) {
      const __half* rowp = hidden[set] + static_cast<size_t>(src) * row_stride + col;
      if (col + 8 <= rank && (reinterpret_cast<uintptr_t>(rowp) & 15u) == 0) {
        *reinterpret_cast<uint4*>(vals) = *reinterpret_cast<const uint4*>(rowp);
      } else {
        for (int u = 0; u < 8 && col + u < rank; ++u) vals[u] = rowp[u];
      }
    }
    if (col_scale && src >= 0) {
#pragma unroll
      for (int u = 0; u < 8; ++u)
        if (col + u < rank) vals[u] = __hmul(vals[u], col_scale[col + u]);
    }
    __half* dst = reinterpret_cast<__half*>(hrows + (set * NT * 8 + n) * kHiddenRowBytes);
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int j = 8 * j8 + u;
      dst[(j & ~31) + lane_order_pos(j & 31)] = vals[u];
    }
  }
}

// Gathers the activations of the salient columns into rows of their own, hsal[set][word][row]
// (64 bytes: the word's 32 slots in lane order), so that the salient pass loads its B fragments
// like the main loop does.  All threads; col(set) = the staged column record of that set.
template <int NT, int NH, typename ColOf>
__device__ __forceinline__ void gather_salient(uint8_t* hsal, const uint8_t* hrows, int nrows, int sal_slots, ColOf col_of) {
#pragma unroll
  for (int set = 0; set < NH; ++set) {
    const uint8_t* col = col_of(set);
    const int words = min(static_cast<int>(reinterpret_cast<const ColHeader*>(col)->sal_words), sal_slots);
    for (int q = 0; q < words; ++q) {
      for (int i = threadIdx.x; i < nrows * 4; i += kThreads) {
        const int t = i & 3, n = i >> 2;
        const uint4 pos = *reinterpret_cast<const uint4*>(col + kColHdrBytes + kColTabBytes + q * kSalEntryBytes + t * 16);
        const uint8_t* rp = hrows + (set * NT * 8 + n) * kHiddenRowBytes;
        auto ld = [&](uint32_t off) { return static_cast<uint32_t>(*reinterpret_cast<const uint16_t*>(rp + off)); };
        uint4 v;
        v.x = ld(pos.x & 0xFFFFu) | (ld(pos.x >> 16) << 16);
        v.y = ld(pos.y & 0xFFFFu) | (ld(pos.y >> 16) << 16);
        v.z = ld(pos.z & 0xFFFFu) | (ld(pos.z >> 16) << 16);
        v.w = ld(pos.w & 0xFFFFu) | (ld(pos.w >> 16) << 16);
        *reinterpret_cast<uint4*>(hsal + (((set * sal_slots + q) * NT * 8 + n) * 4 + t) * 16) = v;
      }
    }
  }
}

// ---- main loop of one 256-column chunk ----------------------------------------------------------
// NTC (compile time) = live 8-row tiles of this pass.  The packed rows are walked slot by slot
// (runs of rows that share their row scales), so the inner loop has no branch but its own.
// Second pass of a chunk: the salient columns, compacted into 32-slot "salient words" whose
// activations gather_salient put into hsal.
template <int NT, int NTC>
__device__ __forceinline__ void sal_chunk_n(const StagedTile& st, const uint8_t* hsal_set, int out_local, int lane,
                                            float (&acc)[NT][4]) {
  const int g = lane >> 2, t = lane & 3;
  const ColHeader* ch = reinterpret_cast<const ColHeader*>(st.col);
  const int sal_words = ch->sal_words;
  const uint8_t* s_base = hsal_set + g * 64 + t * 16;
  const LaneShifts ls = lane_shifts(t);
  for (int q = 0; q < sal_words; ++q) {
    uint32_t a[2][4];
    unpack_fragments_sal(st, q, out_local, lane, ls, a);
#pragma unroll
    for (int nt = 0; nt < NTC; ++nt) {
      const uint4 hv = *reinterpret_cast<const uint4*>(s_base + (q * NT + nt) * 8 * 64);
      mma_m16n8k16(acc[nt], a[0][0], a[1][0], a[0][1], a[1][1], hv.x, hv.y);
      mma_m16n8k16(acc[nt], a[0][2], a[1][2], a[0][3], a[1][3], hv.z, hv.w);
    }
  }
}

template <int NT, int NTC>
__device__ __forceinline__ void main_chunk_n(const StagedTile& st, const uint8_t* hrows_set, const uint8_t* hsal_set,
                                             int out_local, int lane, float (&acc)[NT][4]) {
  const int g = lane >> 2, t = lane & 3;
  const uint8_t* h_base = hrows_set + g * kHiddenRowBytes + t * 16;
  const ColHeader* ch = reinterpret_cast<const ColHeader*>(st.col);
  const int num_slots = ch->num_slots;
  const LaneShifts ls = lane_shifts(t);
  int p = 0;
  for (int slot = 0; slot < num_slots; ++slot) {
    const int p_end = ch->slot_end[slot];
    const RowScalesNs rs = load_row_scales_ns(st, slot, out_local, lane);
#pragma unroll 2
    for (; p < p_end; ++p) {
      uint32_t a[2][4];
      unpack_fragments_ns(st, p, out_local, lane, rs, ls, a);
#pragma unroll
      for (int nt = 0; nt < NTC; ++nt) {
        const uint4 hv = *reinterpret_cast<const uint4*>(h_base + nt * 8 * kHiddenRowBytes + p * 64);
        mma_m16n8k16(acc[nt], a[0][0], a[1][0], a[0][1], a[1][1], hv.x, hv.y);
        mma_m16n8k16(acc[nt], a[0][2], a[1][2], a[0][3], a[1][3], hv.z, hv.w);
      }
    }
  }
  sal_chunk_n<NT, NTC>(st, hsal_set, out_local, lane, acc);
}

template <int NT>
__device__ __forceinline__ void main_chunk(const StagedTile& st, const uint8_t* hrows_set, const uint8_t* hsal_set,
                                           int out_local, int lane, int nt_count, float (&acc)[NT][4]) {
  if (NT == 1 || nt_count == 1) main_chunk_n<NT, 1>(st, hrows_set, hsal_set, out_local, lane, acc);
  else if (NT == 2 || nt_count == 2) main_chunk_n<NT, (NT >= 2 ? 2 : NT)>(st, hrows_set, hsal_set, out_local, lane, acc);
  else if (NT == 3 || nt_count == 3) main_chunk_n<NT, (NT >= 3 ? 3 : NT)>(st, hrows_set, hsal_set, out_local, lane, acc);
  else main_chunk_n<NT, NT>(st, hrows_set, hsal_set, out_local, lane, acc);
}

// ---- weights of a chunk kept in registers across row passes (segments of many rows) ------------------
// A warp owns 16 outputs x 256 columns = 64 half2 per lane: unpacked once per unit, after which a
// row pass costs only the activation loads and the MMAs.  Returns the packed rows of the chunk.
__device__ __forceinline__ int unpack_chunk_ns(const StagedTile& st, int out_local, int lane, uint32_t (&a)[kChunkRows][2][4]) {
  const ColHeader* ch = reinterpret_cast<const ColHeader*>(st.col);
  const int num_slots = ch->num_slots;
  const int p_total = num_slots > 0 ? min(static_cast<int>(ch->slot_end[num_slots - 1]), kChunkRows) : 0;
  int slot = 0;
  RowScalesNs rs = load_row_scales_ns(st, 0, out_local, lane);
  const LaneShifts ls = lane_shifts(lane & 3);
#pragma unroll
  for (int p = 0; p < kChunkRows; ++p) {
    if (p < p_total) {
      while (slot + 1 < num_slots && p >= ch->slot_end[slot]) {
        ++slot;
        rs = load_row_scales_ns(st, slot, out_local, lane);
      }
      unpack_fragments_ns(st, p, out_local, lane, rs, ls, a[p]);
    } else {
#pragma unroll
      for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int i = 0; i < 4; ++i) a[p][h][i] = 0u;
    }
  }
  return p_total;
}

template <int NT, int NTC>
__device__ __forceinline__ void main_chunk_cached_n(const StagedTile& st, const uint32_t (&a)[kChunkRows][2][4], int p_total,
                                                    const uint8_t* hrows_set, const uint8_t* hsal_set, int out_local, int lane,
                                                    float (&acc)[NT][4]) {
  const int g = lane >> 2, t = lane & 3;
  const uint8_t* h_base = hrows_set + g * kHiddenRowBytes + t * 16;
#pragma unroll
  for (int p = 0; p < kChunkRows; ++p) {
    if (p < p_total) {
#pragma unroll
      for (int nt = 0; nt < NTC; ++nt) {
        const uint4 hv = *reinterpret_cast<const uint4*>(h_base + nt * 8 * kHiddenRowBytes + p * 64);
        mma_m16n8k16(acc[nt], a[p][0][0], a[p][1][0], a[p][0][1], a[p][1][1], hv.x, hv.y);
        mma_m16n8k16(acc[nt], a[p][0][2], a[p][1][2], a[p][0][3], a[p][1][3], hv.z, hv.w);
      }
    }
  }
  sal_chunk_n<NT, NTC>(st, hsal_set, out_local, lane, acc);
}

template <int NT>
__device__ __forceinline__ void main_chunk_cached(const StagedTile& st, const uint32_t (&a)[kChunkRows][2][4], int p_total,
                                                  const uint8_t* hrows_set, const uint8_t* hsal_set, int out_local, int lane,
                                                  int nt_count, float (&acc)[NT][4]) {
  if (NT == 1 || nt_count == 1) main_chunk_cached_n<NT, 1>(st, a, p_total, hrows_set, hsal_set, out_local, lane, acc);
  else if (NT == 2 || nt_count == 2) main_chunk_cached_n<NT, (NT >= 2 ? 2 : NT)>(st, a, p_total, hrows_set, hsal_set, out_local, lane, acc);
  else if (NT == 3 || nt_count == 3) main_chunk_cached_n<NT, (NT >= 3 ? 3 : NT)>(st, a, p_total, hrows_set, hsal_set, out_local, lane, acc);
  else main_chunk_cached_n<NT, NT>(st, a, p_total, hrows_set, hsal_set, out_local, lane, acc);
}

// ---- epilogue of one row pass --------------------------------------------------------------------
// acc[nt] = {(out g, row 2t), (out g, row 2t+1), (out g+8, row 2t), (out g+8, row 2t+1)}.
// Output scale and bias; for MODE_DUAL_SILU the up warp (w + 4) hands its values to the gate warp
// (w) through `xbuf` and the gate warp computes SiLU(gate) * up.  The fp16 results are laid out as
// tiles [row][64 outputs] in `otile` and leave as 16-byte stores issued by all threads.  `scratch`
// is shared memory nobody else uses until the next barrier (the activation rows of the finished
// pass).  All threads must call; contains CTA-wide barriers.
template <int NT, int MODE>
__device__ __forceinline__ void finish_rows(const TiledArgs& args, uint8_t* scratch, int r, int og, bool tile_valid, int expert,
                                            int tile0, int r0, int rows, int nt_count, float (&acc)[NT][4]) {
  const int tid = threadIdx.x, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const TrisProjView& v = args.proj[MODE == MODE_SINGLE ? 0 : r];
  const int o_first = (tile0 + (MODE == MODE_SINGLE ? r : 0)) * kTileOut + og * 16;
  float* xbuf = reinterpret_cast<float*>(scratch);                       // [4 og][NT][32 lanes] float4
  uint8_t* otile = scratch + 4 * NT * 32 * 16;                           // [tile][row][144 B]
  if (v.output_scale || v.bias) {
    float scale[2] = {1.f, 1.f}, bias[2] = {0.f, 0.f};
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int o = o_first + g + 8 * h;
      if (o < v.out_features) {
        if (v.output_scale) scale[h] = __half2float(static_cast<const __half*>(v.output_scale)[static_cast<size_t>(expert) * v.out_features + o]);
        if (v.bias) bias[h] = __half2float(static_cast<const __half*>(v.bias)[static_cast<size_t>(expert) * v.out_features + o]);
      }
    }
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[nt][c] = acc[nt][c] * scale[c >> 1] + bias[c >> 1];
  }
  __syncthreads();  // every warp is done with the activation rows: they become scratch
  if (MODE == MODE_DUAL_SILU) {
    if (r == 1) {
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
        if (nt < nt_count)
          *reinterpret_cast<float4*>(xbuf + ((og * NT + nt) * 32 + lane) * 4) = make_float4(acc[nt][0], acc[nt][1], acc[nt][2], acc[nt][3]);
    }
    named_barrier_sync(1 + og, 64);
    if (r == 0) {
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        if (nt >= nt_count) continue;
        const float4 u = *reinterpret_cast<const float4*>(xbuf + ((og * NT + nt) * 32 + lane) * 4);
        const float up[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[nt][c] = __fdividef(acc[nt][c], 1.f + __expf(-acc[nt][c])) * up[c];
      }
    }
  }
  const bool writes = tile_valid && (MODE != MODE_DUAL_SILU || r == 0);
  if (writes) {
    uint8_t* tile = otile + (MODE == MODE_DUAL_SILU ? 0 : r) * (NT * 8 * kOutTileRowBytes);
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      if (nt >= nt_count) continue;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int n = nt * 8 + 2 * t + (c & 1);
        const int ol = og * 16 + g + 8 * (c >> 1);
        *reinterpret_cast<__half*>(tile + n * kOutTileRowBytes + ol * 2) = __float2half_rn(acc[nt][c]);
      }
    }
  }
  __syncthreads();
  // 16-byte stores: item = (tile, row, 8-output piece)
  constexpr int kTiles = (MODE == MODE_DUAL_SILU) ? 1 : 2;
  const int items = kTiles * rows * 8;
  for (int i = tid; i < items; i += kThreads) {
    const int piece = i & 7;
    const int n = (i >> 3) % rows;
    const int tl = (kTiles == 2 && (i >> 3) >= rows) ? 1 : 0;
    const TrisProjView& vo = args.proj[MODE == MODE_DUAL_STORE ? tl : 0];
    const int o = (tile0 + (MODE == MODE_SINGLE ? tl : 0)) * kTileOut + piece * 8;
    if (o >= vo.out_features) continue;
    const int orow = args.out_scatter ? args.out_scatter[r0 + n] : r0 + n;
    if (orow < 0) continue;
    __half* dst = args.out[MODE == MODE_DUAL_STORE ? tl : 0] + static_cast<size_t>(orow) * vo.out_features + o;
    const uint8_t* src = otile + tl * (NT * 8 * kOutTileRowBytes) + n * kOutTileRowBytes + piece * 16;
    if (o + 8 <= vo.out_features && (reinterpret_cast<uintptr_t>(dst) & 15u) == 0) {
      *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(src);
    } else {
      for (int u = 0; u < 8 && o + u < vo.out_features; ++u) dst[u] = reinterpret_cast<const __half*>(src)[u];
    }
  }
}

struct UnitRoute {
  int expert, row_begin, row_end;
};
__device__ __forceinline__ UnitRoute load_unit_route(const TiledArgs& args, int seg) {
  UnitRoute u;
  u.expert = args.expert_ids[seg];
  u.row_begin = args.segment_offsets[seg];
  u.row_end = min(args.segment_offsets[seg + 1], args.num_rows);
  return u;
}
__device__ __forceinline__ bool unit_live(const TiledArgs& args, const UnitRoute& u) {
  return u.expert >= 0 && u.expert < args.proj[0].num_experts && u.row_end > u.row_begin;
}

// ---- one CTA per unit, any number of chunks ---------------------------------------------------------
// grid (tiles (dual) or ceil(tiles / 2) (single), segment bound)
// One CTA per unit, four CTAs per SM (64 registers, a single record stage): measured on B200 at the OLMoE
// shape this beats the persistent kernel below (three CTAs per SM, 80 registers, records of the next unit
// prefetched) by 16 % per launch at batch 128 - the kernel is bound by instruction issue, and a fourth
// resident CTA hides more latency than the prefetch does; five CTAs (48 registers, spills) are slower.
// CACHE: single-chunk projections keep their unpacked weights in registers across the row passes of a
// segment (64 more registers: two CTAs per SM) - the variant for prefill-sized segments.
template <int NT, int MODE, bool CACHE>
__global__ void __launch_bounds__(kThreads, CACHE ? 2 : 4) grouped_tiled_kernel(const __grid_constant__ TiledArgs args) {
  constexpr bool DUAL = MODE != MODE_SINGLE;
  constexpr int NH = DUAL ? 2 : 1;
  extern __shared__ uint4 smem_raw[];
  uint8_t* sm = reinterpret_cast<uint8_t*>(smem_raw);
  const SmemLayout L = smem_layout(args.rec_slot_bytes, args.col_slot_bytes, args.sal_slots, NH, NT, 1);
  uint64_t* mbar = reinterpret_cast<uint64_t*>(sm);  // [0] records, [1] activation rows
  uint8_t* rec_base = sm + 64;
  uint8_t* col_base = rec_base + 2 * args.rec_slot_bytes;
  uint32_t* gmap_base = reinterpret_cast<uint32_t*>(sm + L.gmap_off);
  uint8_t* hsal = sm + L.hsal_off;
  uint8_t* hrows = sm + L.hrows_off;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    mbar_init(&mbar[0], 2);
    mbar_init(&mbar[1], kWarps);
    fence_mbar_init();
  }
  reinterpret_cast<uint4*>(gmap_base)[tid] = make_uint4(0u, 0u, 0u, 0u);  // both g_map planes, for the first chunk
  __syncthreads();
  // Activations come from the predecessor kernel; the route arrays too, unless the caller says
  // they are older, in which case the weight staging below overlaps the predecessor.
  bool waited = false;
  if (!args.weights_before_wait) {
    pdl_wait();
    pdl_launch_dependents();
    waited = true;
  }
  const int seg = blockIdx.y;
  const UnitRoute unit = load_unit_route(args, seg);
  const int nseg = args.num_segments_dev ? min(*args.num_segments_dev, args.num_segments) : args.num_segments;
  // Row split: CTA z of a unit takes the row passes z, z + gridDim.z, ... of its segment (the launcher
  // splits when there are fewer units than CTA slots); a CTA without a pass leaves at once.
  // (Only the register-cached kernel is launched with gridDim.z > 1.)
  const int row_first = unit.row_begin + (CACHE ? static_cast<int>(blockIdx.z) * (NT * 8) : 0);
  const int row_step = (CACHE ? static_cast<int>(gridDim.z) : 1) * (NT * 8);
  if (seg >= nseg || !unit_live(args, unit) || row_first >= unit.row_end) return;
  const int expert = unit.expert;

  const int r = warp >> 2, og = warp & 3;  // record and 16-output group of this warp
  const int tiles = tiles_per_expert(args.proj[0].out_features);
  const int tile0 = DUAL ? static_cast<int>(blockIdx.x) : 2 * static_cast<int>(blockIdx.x);
  const bool tile_valid = tile0 + (DUAL ? 0 : r) < tiles;
  const int rank = args.proj[0].rank;
  const int chunks = num_chunks(rank);
  const bool lane_order = args.hidden_lane_order != 0;

  StagedTile st;
  st.rec = rec_base + r * args.rec_slot_bytes;
  st.col = col_base + (DUAL ? r : 0) * args.col_slot_bytes;
  st.gmap = gmap_base + r * 512;
  const uint8_t* hrows_set = hrows + (DUAL ? r : 0) * NT * 8 * kHiddenRowBytes;
  const uint8_t* hsal_set = hsal + (DUAL ? r : 0) * args.sal_slots * NT * 8 * 64;
  auto col_of = [&](int set) { return static_cast<const uint8_t*>(col_base + set * args.col_slot_bytes); };

  int staged_chunk = -1;
  uint32_t par_w = 0u, par_h = 0u;
  bool dead = false;
  uint32_t a_cache[CACHE ? kChunkRows : 1][2][4];
  int cached_rows = -1;  // packed rows held in a_cache once the chunk has been unpacked
  for (int r0 = row_first; r0 < unit.row_end; r0 += row_step) {
    const int rows = min(NT * 8, unit.row_end - r0);
    const int nt_count = (rows + 7) >> 3;
    float acc[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[nt][c] = 0.f;
    auto row_src = [&](int n) { return args.row_gather ? args.row_gather[r0 + n] : (r0 + n); };

    for (int kc = 0; kc < chunks; ++kc) {
      const int p0 = kc * kChunkRows;
      // the first chunk of a unit starts right behind the set-up barrier (planes already zeroed there)
      const bool first_iter = staged_chunk < 0;
      if (!first_iter) __syncthreads();  // earlier consumers of the staging buffers are done
      if (dead) break;
      const bool need_w = staged_chunk != kc;
      if (need_w) {
        if (lane == 0 && warp < 2) {
          const int rr = warp;
          const TrisProjView& v = args.proj[DUAL ? rr : 0];
          const int tl = tile0 + (DUAL ? 0 : rr);
          const bool valid = tl < tiles;
          const uint2 d = valid ? load_desc(v, expert, tl, kc) : make_uint2(0u, 0u);
          issue_record(v, expert, kc, d, rec_base + rr * args.rec_slot_bytes,
                       (DUAL || rr == 0) ? col_base + rr * args.col_slot_bytes : nullptr, valid, &mbar[0]);
        }
        if (!first_iter) reinterpret_cast<uint4*>(gmap_base)[tid] = make_uint4(0u, 0u, 0u, 0u);  // 256 threads x 16 B = both planes
      }
      if (waited) issue_hidden<NT, NH>(hrows, args.hidden, rank, p0, rows, lane_order, args.hidden_stride, &mbar[1], row_src, args.col_scale);
      bool ok = true;
      if (need_w) {
        if (!first_iter) __syncthreads();  // planes zeroed
        ok = mbar_wait_bounded(&mbar[0], par_w);
        par_w ^= 1u;
        if (ok && tile_valid) gr_decode_block(st.rec, og, const_cast<uint32_t*>(st.gmap), lane);
        staged_chunk = kc;
      }
      if (!waited) {  // first pass of a CTA that staged its weights ahead of the predecessor's end
        pdl_wait();
        pdl_launch_dependents();
        waited = true;
        issue_hidden<NT, NH>(hrows, args.hidden, rank, p0, rows, lane_order, args.hidden_stride, &mbar[1], row_src, args.col_scale);
      }
      ok = mbar_wait_bounded(&mbar[1], par_h) && ok;
      par_h ^= 1u;
      if (__syncthreads_or(!ok)) {  // also publishes the decoded planes, re-ordered rows and column records
        mbar_wait_bounded(&mbar[0], par_w ^ 1u);  // copies that may still be in flight
        mbar_wait_bounded(&mbar[1], par_h ^ 1u);
        if (tid == 0 && args.status) atomicExch(args.status, TRIS_ERR_TIMEOUT);
        dead = true;
        break;
      }
      gather_salient<NT, NH>(hsal, hrows, rows, args.sal_slots, col_of);
      __syncthreads();
      if (tile_valid) {
        if constexpr (CACHE) {
          if (chunks == 1) {
            if (cached_rows < 0) cached_rows = unpack_chunk_ns(st, og * 16, lane, a_cache);
            main_chunk_cached<NT>(st, a_cache, cached_rows, hrows_set, hsal_set, og * 16, lane, nt_count, acc);
          } else {
            main_chunk<NT>(st, hrows_set, hsal_set, og * 16, lane, nt_count, acc);
          }
        } else {
          main_chunk<NT>(st, hrows_set, hsal_set, og * 16, lane, nt_count, acc);
        }
      }
    }
    if (dead) continue;
    finish_rows<NT, MODE>(args, hrows, r, og, tile_valid, expert, tile0, r0, rows, nt_count, acc);
  }
}

// ---- persistent CTAs, records of the next unit prefetched (projections of one chunk) -----------------
// grid (CTAs); unit u = segment * units_x + x, x = output tile (dual) or pair of tiles (single)
template <int NT, int MODE>
__global__ void __launch_bounds__(kThreads, 3) grouped_tiled_persistent_kernel(const __grid_constant__ TiledArgs args) {
  constexpr bool DUAL = MODE != MODE_SINGLE;
  constexpr int NH = DUAL ? 2 : 1;
  extern __shared__ uint4 smem_raw[];
  uint8_t* sm = reinterpret_cast<uint8_t*>(smem_raw);
  const SmemLayout L = smem_layout(args.rec_slot_bytes, args.col_slot_bytes, args.sal_slots, NH, NT, 2);
  uint64_t* mbar = reinterpret_cast<uint64_t*>(sm);  // [0], [1] records of the two stages, [2] activation rows
  uint32_t* gmap_base = reinterpret_cast<uint32_t*>(sm + L.gmap_off);
  uint8_t* hsal = sm + L.hsal_off;
  uint8_t* hrows = sm + L.hrows_off;
  auto stage_rec = [&](int stage, int rr) { return sm + 64 + stage * L.stage_bytes + rr * args.rec_slot_bytes; };
  auto stage_col = [&](int stage, int set) { return sm + 64 + stage * L.stage_bytes + 2 * args.rec_slot_bytes + set * args.col_slot_bytes; };

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    mbar_init(&mbar[0], 2);
    mbar_init(&mbar[1], 2);
    mbar_init(&mbar[2], kWarps);
    fence_mbar_init();
  }
  __syncthreads();
  bool waited = false;
  if (!args.weights_before_wait) {
    pdl_wait();
    pdl_launch_dependents();
    waited = true;
  }
  const int tiles = tiles_per_expert(args.proj[0].out_features);
  const int units_x = DUAL ? tiles : (tiles + 1) / 2;
  const int nseg = args.num_segments_dev ? min(*args.num_segments_dev, args.num_segments) : args.num_segments;
  const int total = nseg * units_x;
  const int G = gridDim.x;
  int u = blockIdx.x;
  if (u >= total) {
    if (!waited) {
      pdl_wait();
      pdl_launch_dependents();
    }
    return;
  }
  const int r = warp >> 2, og = warp & 3;
  const int rank = args.proj[0].rank;
  const bool lane_order = args.hidden_lane_order != 0;
  const bool issuer = lane == 0 && warp < 2;  // fetches record `warp` of every unit
  const TrisProjView& iv = args.proj[DUAL ? (warp & 1) : 0];

  auto tile_of = [&](int unit, int rr) { const int x = unit % units_x; return DUAL ? x : 2 * x + rr; };
  auto fetch = [&](int unit, int expert, uint2 d, int stage) {  // issuer only
    const int rr = warp;
    const bool valid = tile_of(unit, rr) < tiles && expert >= 0 && expert < args.proj[0].num_experts;
    issue_record(iv, expert, 0, d, stage_rec(stage, rr), (DUAL || rr == 0) ? stage_col(stage, rr) : nullptr, valid, &mbar[stage]);
  };
  auto desc_of = [&](int unit, int expert) {  // issuer only
    const int tl = tile_of(unit, warp);
    if (tl >= tiles || expert < 0 || expert >= args.proj[0].num_experts) return make_uint2(0u, 0u);
    return load_desc(iv, expert, tl, 0);
  };

  // pipeline fill: unit u in flight, descriptor of u + G and expert of u + 2G in registers
  UnitRoute cur = load_unit_route(args, u / units_x);
  int e1 = -1, e2 = -1;
  uint2 d1 = make_uint2(0u, 0u);
  if (issuer) {
    fetch(u, cur.expert, desc_of(u, cur.expert), 0);
    if (u + G < total) {
      e1 = args.expert_ids[(u + G) / units_x];
      d1 = desc_of(u + G, e1);
    }
    if (u + 2 * G < total) e2 = args.expert_ids[(u + 2 * G) / units_x];
  }
  UnitRoute nxt = cur;
  if (u + G < total) nxt = load_unit_route(args, (u + G) / units_x);

  uint32_t par_h = 0u;
  bool dead = false;
  for (int it = 0;; ++it) {
    const int stage = it & 1;
    __syncthreads();  // the previous unit is finished: its stage, the planes and the activation rows are free
    if (issuer) {
      if (u + G < total) fetch(u + G, e1, d1, stage ^ 1);
      e1 = e2;
      d1 = (u + 2 * G < total) ? desc_of(u + 2 * G, e1) : make_uint2(0u, 0u);
      e2 = (u + 3 * G < total) ? args.expert_ids[(u + 3 * G) / units_x] : -1;
    }
    const bool live = unit_live(args, cur);
    const int expert = cur.expert;
    const int tile0 = tile_of(u, 0);
    const bool tile_valid = tile0 + (DUAL ? 0 : r) < tiles;
    StagedTile st;
    st.rec = stage_rec(stage, r);
    st.col = stage_col(stage, DUAL ? r : 0);
    st.gmap = gmap_base + r * 512;
    const uint8_t* hrows_set = hrows + (DUAL ? r : 0) * NT * 8 * kHiddenRowBytes;
    const uint8_t* hsal_set = hsal + (DUAL ? r : 0) * args.sal_slots * NT * 8 * 64;
    auto col_of = [&](int set) { return static_cast<const uint8_t*>(stage_col(stage, set)); };

    reinterpret_cast<uint4*>(gmap_base)[tid] = make_uint4(0u, 0u, 0u, 0u);
    int r0 = cur.row_begin;
    int rows = live ? min(NT * 8, cur.row_end - r0) : 0;
    auto row_src = [&](int n) { return args.row_gather ? args.row_gather[r0 + n] : (r0 + n); };
    if (waited && live) issue_hidden<NT, NH>(hrows, args.hidden, rank, 0, rows, lane_order, args.hidden_stride, &mbar[2], row_src, args.col_scale);
    __syncthreads();  // planes zeroed
    bool ok = mbar_wait_bounded(&mbar[stage], (it >> 1) & 1);
    if (ok && live && tile_valid) gr_decode_block(st.rec, og, const_cast<uint32_t*>(st.gmap), lane);
    if (!waited) {
      pdl_wait();
      pdl_launch_dependents();
      waited = true;
      if (live) issue_hidden<NT, NH>(hrows, args.hidden, rank, 0, rows, lane_order, args.hidden_stride, &mbar[2], row_src, args.col_scale);
    }
    for (; live;) {
      const int nt_count = (rows + 7) >> 3;
      ok = mbar_wait_bounded(&mbar[2], par_h) && ok;
      par_h ^= 1u;
      if (__syncthreads_or(!ok)) {  // also publishes the decoded planes and re-ordered rows
        mbar_wait_bounded(&mbar[2], par_h ^ 1u);
        dead = true;
        break;
      }
      gather_salient<NT, NH>(hsal, hrows, rows, args.sal_slots, col_of);
      __syncthreads();
      float acc[NT][4];
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[nt][c] = 0.f;
      if (tile_valid) main_chunk<NT>(st, hrows_set, hsal_set, og * 16, lane, nt_count, acc);
      finish_rows<NT, MODE>(args, hrows, r, og, tile_valid, expert, tile0, r0, rows, nt_count, acc);
      r0 += NT * 8;
      if (r0 >= cur.row_end) break;
      rows = min(NT * 8, cur.row_end - r0);
      __syncthreads();  // the stores have read the scratch: the activation rows can be refilled
      issue_hidden<NT, NH>(hrows, args.hidden, rank, 0, rows, lane_order, args.hidden_stride, &mbar[2], row_src, args.col_scale);
    }
    if (__syncthreads_or(dead || !ok)) {
      if (u + G < total) mbar_wait_bounded(&mbar[stage ^ 1], ((it + 1) >> 1) & 1);  // the prefetch in flight
      if (tid == 0 && args.status) atomicExch(args.status, TRIS_ERR_TIMEOUT);
      return;
    }
    u += G;
    if (u >= total) return;
    cur = nxt;
    if (u + G < total) nxt = load_unit_route(args, (u + G) / units_x);
  }
}

// ---- dump kernel: decoded g_map words and dequantised weights from the records --------------------
// grid (tiles, chunks, E); dense_out [E, pr, O] and weights_out [E, O, rank] may each be null
__global__ void __launch_bounds__(kThreads) tiled_dump_kernel(TrisProjView v, int32_t* dense_out, __half* weights_out,
                                                              int rec_slot_bytes, int32_t* status) {
  extern __shared__ uint4 smem_raw[];
  uint8_t* sm = reinterpret_cast<uint8_t*>(smem_raw);
  uint64_t* mbar = reinterpret_cast<uint64_t*>(sm);
  uint8_t* rec = sm + 64;
  uint8_t* col = rec + rec_slot_bytes;
  uint32_t* gmap = reinterpret_cast<uint32_t*>(col + v.col_record_bytes);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int tile = blockIdx.x, chunk = blockIdx.y, e = blockIdx.z;
  const int o0 = tile * kTileOut, p0 = chunk * kChunkRows;
  const int pr = (v.rank + 31) >> 5;
  if (tid == 0) {
    mbar_init(&mbar[0], 1);
    fence_mbar_init();
  }
  __syncthreads();
  if (tid == 0) issue_record(v, e, chunk, load_desc(v, e, tile, chunk), rec, col, true, &mbar[0]);
  if (tid < 128) reinterpret_cast<uint4*>(gmap)[tid] = make_uint4(0u, 0u, 0u, 0u);
  __syncthreads();
  const bool ok = mbar_wait_bounded(&mbar[0], 0u);
  if (ok && warp < 4) gr_decode_block(rec, warp, gmap, lane);
  if (__syncthreads_or(!ok)) {
    mbar_wait_bounded(&mbar[0], 0u);
    if (tid == 0 && status) atomicExch(status, TRIS_ERR_TIMEOUT);
    return;
  }
  if (dense_out) {
    for (int i = tid; i < kChunkRows * kTileOut; i += kThreads) {
      const int p = i / kTileOut, o = i % kTileOut;
      if (p0 + p < pr && o0 + o < v.out_features)
        dense_out[(static_cast<size_t>(e) * pr + p0 + p) * v.out_features + o0 + o] = static_cast<int32_t>(gmap[i]);
    }
  }
  if (!weights_out) return;
  StagedTile st{rec, col, gmap};
  const int g = lane >> 2, t = lane & 3;
  const LaneShifts ls = lane_shifts(t);
  auto store_pair = [&](int o, int col_lo, uint32_t bits) {
    if (o >= v.out_features) return;
    __half* row = weights_out + (static_cast<size_t>(e) * v.out_features + o) * v.rank;
    const int ca = 32 * p0 + col_lo, cb = ca + 16;
    if (ca < v.rank) row[ca] = __ushort_as_half(static_cast<unsigned short>(bits & 0xFFFFu));
    if (cb < v.rank) row[cb] = __ushort_as_half(static_cast<unsigned short>(bits >> 16));
  };
  if (warp < 4) {
    const ColHeader* ch = reinterpret_cast<const ColHeader*>(col);
    int p = 0;
    for (int slot = 0; slot < ch->num_slots; ++slot) {
      const RowScalesNs rs = load_row_scales_ns(st, slot, warp * 16, lane);
      for (; p < ch->slot_end[slot]; ++p) {
        uint32_t a[2][4];
        unpack_fragments_ns(st, p, warp * 16, lane, rs, ls, a);
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
          for (int i = 0; i < 4; ++i) store_pair(o0 + warp * 16 + g + 8 * h, 32 * p + lane_pair_col(t, i), a[h][i]);
      }
    }
  }
  __syncthreads();  // the salient columns overwrite the +-0 the main unpack left there
  if (warp < 4) {
    const int sal_words = reinterpret_cast<const ColHeader*>(col)->sal_words;
    for (int q = 0; q < sal_words; ++q) {
      uint32_t a[2][4];
      unpack_fragments_sal(st, q, warp * 16, lane, ls, a);
      const uint16_t* salcol = reinterpret_cast<const uint16_t*>(col + kColHdrBytes + kColTabBytes + q * kSalEntryBytes + 192);
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int o = o0 + warp * 16 + g + 8 * h;
        if (o >= v.out_features) continue;
        __half* row = weights_out + (static_cast<size_t>(e) * v.out_features + o) * v.rank;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int slot = lane_pair_col(t, i);
          const unsigned c_lo = salcol[slot], c_hi = salcol[slot + 16];
          if (c_lo != 0xFFFFu) row[32 * p0 + c_lo] = __ushort_as_half(static_cast<unsigned short>(a[h][i] & 0xFFFFu));
          if (c_hi != 0xFFFFu) row[32 * p0 + c_hi] = __ushort_as_half(static_cast<unsigned short>(a[h][i] >> 16));
        }
      }
    }
  }
}

// ---- host side --------------------------------------------------------------------------------------
// typical rows per segment up to which the persistent decode kernels are used
constexpr int kTiledDecodeMaxRows = 64;

static inline int rec_slot_bytes_for(int max_record_bytes) { return ((max_record_bytes + 15) & ~15) + 16; }

static int sm_count() {
  static int cached[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

template <typename Kernel>
static int configure_smem(Kernel kernel, size_t smem, size_t (&configured)[64]) {
  int dev = 0;
  TRIS_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64 || configured[dev] < smem) {
    TRIS_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    if (dev >= 0 && dev < 64) configured[dev] = smem;
  }
  return TRIS_OK;
}

template <int NT, int MODE>
static int launch_tiled(const TiledArgs& args, cudaStream_t stream, bool pdl) {
  constexpr int NH = (MODE == MODE_SINGLE) ? 1 : 2;
  const int tiles = tiles_per_expert(args.proj[0].out_features);
  const int units_x = MODE == MODE_SINGLE ? (tiles + 1) / 2 : tiles;
  const size_t smem = smem_layout(args.rec_slot_bytes, args.col_slot_bytes, args.sal_slots, NH, NT, 1).total;
  const bool four_per_sm = 4 * (smem + 1024) <= 227 * 1024;
  if (num_chunks(args.proj[0].rank) == 1 && !four_per_sm) {
    // the one-CTA-per-unit kernel would not reach four CTAs per SM: persistent CTAs that prefetch the next record
    const size_t smem2 = smem_layout(args.rec_slot_bytes, args.col_slot_bytes, args.sal_slots, NH, NT, 2).total;
    if (smem2 <= 227 * 1024) {
      auto kernel = grouped_tiled_persistent_kernel<NT, MODE>;
      static size_t configured[64] = {};  // per instantiation, per device: largest size set so far
      int st = configure_smem(kernel, smem2, configured);
      if (st != TRIS_OK) return st;
      const int per_sm = std::max<int>(1, std::min<size_t>(3, (227 * 1024) / (smem2 + 1024)));
      const long long units = static_cast<long long>(units_x) * args.num_segments;
      const int grid = static_cast<int>(std::min<long long>(units, static_cast<long long>(sm_count()) * per_sm));
      return check_cuda(launch_kernel(kernel, dim3(grid), dim3(kThreads), smem2, stream, pdl, 1, args),
                        "grouped_tiled_persistent_kernel launch");
    }
  }
  TRIS_REQUIRE(smem <= 227 * 1024, TRIS_ERR_UNSUPPORTED, "grouped_tiled_kernel: %zu bytes of shared memory", smem);
  auto kernel = grouped_tiled_kernel<NT, MODE, false>;
  static size_t configured[64] = {};
  int st = configure_smem(kernel, smem, configured);
  if (st != TRIS_OK) return st;
  return check_cuda(launch_kernel(kernel, dim3(units_x, args.num_segments), dim3(kThreads), smem, stream, pdl, 1, args),
                    "grouped_tiled_kernel launch");
}

// Prefill-sized segments of a single-chunk projection: one CTA per unit, 32 rows per pass, weights
// unpacked once per unit and kept in registers.
// Row split of the cached kernel: with fewer units than CTA slots (two per SM) - few local experts with long
// segments, as on an expert-parallel rank - up to `g_row_split_max` CTAs share a unit's row passes, each
// decoding and unpacking the unit's weights for itself.
static std::atomic<int> g_row_split_max{4};
static int cached_row_split(int units, int max_rows) {
  const int limit = g_row_split_max.load(std::memory_order_relaxed);
  if (limit <= 1 || units <= 0) return 1;
  const int passes = (max_rows + 31) / 32;
  return std::max(1, std::min({limit, 2 * sm_count() / units, passes}));
}

template <int MODE>
static int launch_tiled_cached(const TiledArgs& args, int max_rows, cudaStream_t stream, bool pdl) {
  constexpr int NH = (MODE == MODE_SINGLE) ? 1 : 2;
  constexpr int NT = 4;
  const int tiles = tiles_per_expert(args.proj[0].out_features);
  const int units_x = MODE == MODE_SINGLE ? (tiles + 1) / 2 : tiles;
  const size_t smem = smem_layout(args.rec_slot_bytes, args.col_slot_bytes, args.sal_slots, NH, NT, 1).total;
  TRIS_REQUIRE(smem <= 227 * 1024, TRIS_ERR_UNSUPPORTED, "grouped_tiled_kernel: %zu bytes of shared memory", smem);
  auto kernel = grouped_tiled_kernel<NT, MODE, true>;
  static size_t configured[64] = {};
  int st = configure_smem(kernel, smem, configured);
  if (st != TRIS_OK) return st;
  const int split = cached_row_split(units_x * args.num_segments, max_rows);
  return check_cuda(launch_kernel(kernel, dim3(units_x, args.num_segments, split), dim3(kThreads), smem, stream, pdl, 1, args),
                    "grouped_tiled_kernel (cached weights) launch");
}

template <int MODE>
static int dispatch_tiled(const TiledArgs& args, int max_rows, cudaStream_t stream, bool pdl) {
  if (max_rows > kTiledDecodeMaxRows && num_chunks(args.proj[0].rank) == 1) return launch_tiled_cached<MODE>(args, max_rows, stream, pdl);
  if (max_rows <= 8) return launch_tiled<1, MODE>(args, stream, pdl);
  if (max_rows <= 16) return launch_tiled<2, MODE>(args, stream, pdl);
  // 24 rows per pass also for segments of up to 64 rows: with 32 rows per pass the tile no longer fits four
  // CTAs per SM, and four CTAs that re-unpack for a second or third pass beat three that do not (measured at
  // 32 / 40 / 48 rows per expert: 55.9 / 63.6 / 75.6 us against 63.3 / 69.2 / 83.0 for both grouped kernels)
  return launch_tiled<3, MODE>(args, stream, pdl);
}

}  // namespace tr

bool proj_has_tile_records(const TrisProjView& v) {
  return v.tile_records != nullptr && v.tile_desc != nullptr && v.col_records != nullptr && v.use_block_gr &&
         v.expert_slot == nullptr && v.gmap_slot == nullptr && v.col_record_bytes > 0 && v.max_record_bytes > 0;
}

// mode: 0 single projection, 1 gate/up pair, 2 gate/up pair with SiLU * mul
int launch_grouped_tiled(const TrisProjView* proj_a, const TrisProjView* proj_b, const TrisRouteView* route,
                         const void* hidden_a, const void* hidden_b, void* out_a, void* out_b, int mode, int max_rows,
                         cudaStream_t stream, LaunchOpts opts) {
  using namespace tr;
  // Rows per pass: a longer segment costs a second pass that only re-unpacks (the decoded planes
  // stay), so size the activation tile for mean + 2 sigma of a balanced router rather than for the
  // worst case; smaller tiles mean more resident CTAs.
  if (route->num_segments > 0 && max_rows <= kTiledDecodeMaxRows) {
    const double mean = static_cast<double>(route->num_rows) / route->num_segments;
    max_rows = std::max(1, std::min(max_rows, static_cast<int>(ceil(mean + 2.0 * sqrt(mean)))));
  }
  TiledArgs a{};
  a.proj[0] = *proj_a;
  a.proj[1] = proj_b ? *proj_b : *proj_a;
  a.hidden[0] = static_cast<const __half*>(hidden_a);
  a.hidden[1] = static_cast<const __half*>(hidden_b ? hidden_b : hidden_a);
  a.out[0] = static_cast<__half*>(out_a);
  a.out[1] = static_cast<__half*>(out_b ? out_b : out_a);
  a.expert_ids = route->expert_ids;
  a.segment_offsets = route->segment_offsets;
  a.num_segments_dev = route->num_segments_dev;
  a.row_gather = route->row_gather;
  a.out_scatter = route->out_row_scatter;
  a.status = route->status_dev;
  a.num_segments = route->num_segments;
  a.num_rows = route->num_rows;
  a.hidden_lane_order = (route->flags & TRIS_ROUTE_HIDDEN_LANE_ORDER) != 0;
  a.hidden_stride = route->hidden_row_stride > 0 ? route->hidden_row_stride : proj_a->rank;
  a.weights_before_wait = opts.pdl && opts.weights_before_wait;
  a.rec_slot_bytes = rec_slot_bytes_for(std::max(a.proj[0].max_record_bytes, a.proj[1].max_record_bytes));
  a.col_slot_bytes = std::max(a.proj[0].col_record_bytes, a.proj[1].col_record_bytes);
  a.sal_slots = std::max(1, std::max(a.proj[0].max_sal_words, a.proj[1].max_sal_words));
  a.col_scale = static_cast<const __half*>(route->hidden_col_scale);
  TRIS_REQUIRE(a.col_scale == nullptr || !a.hidden_lane_order, TRIS_ERR_INVALID_ARG,
               "grouped (tile records): hidden_col_scale needs row-major activation rows");
  TRIS_REQUIRE(!a.hidden_lane_order || proj_a->rank % 32 == 0, TRIS_ERR_INVALID_ARG,
               "grouped (tile records): lane-order activations need rank %% 32 == 0");
  TRIS_REQUIRE(a.hidden_stride >= proj_a->rank, TRIS_ERR_INVALID_ARG, "grouped (tile records): hidden_row_stride < rank");
  if (mode == MODE_SINGLE) return dispatch_tiled<MODE_SINGLE>(a, max_rows, stream, opts.pdl);
  if (mode == MODE_DUAL_SILU) return dispatch_tiled<MODE_DUAL_SILU>(a, max_rows, stream, opts.pdl);
  return dispatch_tiled<MODE_DUAL_STORE>(a, max_rows, stream, opts.pdl);
}

int launch_tiled_dump(const TrisProjView* proj, int32_t* dense_out, void* weights_out, cudaStream_t stream) {
  using namespace tr;
  const int rec_slot = rec_slot_bytes_for(proj->max_record_bytes);
  const size_t smem = 64 + static_cast<size_t>(rec_slot) + proj->col_record_bytes + 2048;
  TRIS_CUDA(cudaFuncSetAttribute(tiled_dump_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
  dim3 grid(tiles_per_expert(proj->out_features), num_chunks(proj->rank), proj->num_experts);
  tiled_dump_kernel<<<grid, kThreads, smem, stream>>>(*proj, dense_out, static_cast<__half*>(weights_out), rec_slot, nullptr);
  return check_cuda(cudaGetLastError(), "tiled_dump_kernel launch");
}

}  // namespace tris

extern "C" int tris_set_grouped_row_split_max(int32_t ctas) {
  return tris::tr::g_row_split_max.exchange(ctas < 1 ? 1 : (ctas > 16 ? 16 : ctas), std::memory_order_relaxed);
}
