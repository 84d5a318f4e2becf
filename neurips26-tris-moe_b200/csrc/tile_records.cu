// Load-time builder of the tile-major records described in tile_records.cuh: a plan pass that
// sizes every record and lays the records out back to back, and a fill pass that gathers the
// E-stacked payload tensors (QL:1512-1636 of the TriS-MoE tree) into them.  Runs once per
// projection when a payload is prepared; nothing here is on the per-token path.
#include <algorithm>

#include "tile_records.cuh"

namespace tris {
namespace tr {

struct BuildDims {
  int pr, nkb, nob, nblk, tiles, chunks;
};
__host__ __device__ inline BuildDims build_dims(const TrisProjView& v) {
  BuildDims d;
  d.pr = (v.rank + 31) / 32;
  d.nkb = (d.pr + 1) / 2;
  d.nob = (v.out_features + 63) / 64;
  d.nblk = d.nkb * d.nob;
  d.tiles = tiles_per_expert(v.out_features);
  d.chunks = num_chunks(v.rank);
  return d;
}

// desc[idx] = {offset in 16-byte units (filled by the scan), bytes}; idx = (e * tiles + tile) * chunks + chunk
__global__ void plan_records_kernel(TrisProjView v, uint2* desc) {
  const BuildDims d = build_dims(v);
  const int total = v.num_experts * d.tiles * d.chunks;
  for (int idx = blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += gridDim.x * blockDim.x) {
    const int chunk = idx % d.chunks, tile = (idx / d.chunks) % d.tiles, e = idx / (d.chunks * d.tiles);
    ChunkPlan plan;
    plan_chunk(v.c_map + static_cast<size_t>(e) * d.pr,
               v.packed_row_group ? v.packed_row_group + static_cast<size_t>(e) * d.pr : nullptr, d.pr,
               chunk * kChunkRows, v.rank, plan, nullptr);
    int gr_words = 0;
    const int32_t* off = v.q_gmap_gr_offsets + static_cast<size_t>(e) * (d.nblk + 1);
    for (int b = 0; b < 4; ++b) {
      const int kb = 4 * chunk + b;
      if (kb >= d.nkb) break;
      const int bi = kb * d.nob + tile;
      gr_words += max(0, min(off[bi + 1] - off[bi], TRIS_GR_BLOCK_WORDS));
    }
    desc[idx] = make_uint2(0u, static_cast<uint32_t>(record_bytes(plan.num_slots, (plan.num_steps + 1) >> 1, gr_words)));
    if (tile == 0) atomicMax(reinterpret_cast<int*>(&desc[total].x), (plan.num_steps + 1) >> 1);  // scratch entry behind the table
  }
}

// Single CTA: exclusive scan of the record sizes; info = {total bytes, max record bytes, max salient words, 0}.
__global__ void scan_records_kernel(uint2* desc, int total, int64_t* info) {
  __shared__ unsigned long long carry;
  __shared__ unsigned long long partial[1024];
  __shared__ unsigned int max_bytes;
  if (threadIdx.x == 0) {
    carry = 0ull;
    max_bytes = 0u;
  }
  __syncthreads();
  for (int base = 0; base < total; base += blockDim.x) {
    const int i = base + threadIdx.x;
    const unsigned int bytes = (i < total) ? desc[i].y : 0u;
    partial[threadIdx.x] = bytes;
    atomicMax(&max_bytes, bytes);
    __syncthreads();
    for (int s = 1; s < blockDim.x; s <<= 1) {  // Hillis-Steele inclusive scan
      const unsigned long long add = (threadIdx.x >= s) ? partial[threadIdx.x - s] : 0ull;
      __syncthreads();
      partial[threadIdx.x] += add;
      __syncthreads();
    }
    if (i < total) desc[i].x = static_cast<uint32_t>((carry + partial[threadIdx.x] - bytes) >> 4);
    __syncthreads();
    if (threadIdx.x == blockDim.x - 1) carry += partial[threadIdx.x];
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    info[0] = static_cast<int64_t>(carry);
    info[1] = max_bytes;
    info[2] = static_cast<int>(desc[total].x);
    info[3] = 0;
  }
}

__device__ __forceinline__ uint32_t half_of_pack(unsigned long long pack, int which) {
  return static_cast<uint32_t>(pack >> (16 * which)) & 0xFFFFu;
}

// grid (chunks, E), 128 threads
__global__ void build_col_records_kernel(TrisProjView v, uint8_t* col_records, int max_sal_words) {
  __shared__ ChunkPlan plan;
  __shared__ uint16_t col_of_slot[kMaxSalWords * 32];
  const BuildDims d = build_dims(v);
  const int chunk = blockIdx.x, e = blockIdx.y, p0 = chunk * kChunkRows;
  const int stride = col_record_bytes(max_sal_words);
  uint8_t* rec = col_records + (static_cast<size_t>(e) * d.chunks + chunk) * stride;
  const int32_t* cmap = v.c_map + static_cast<size_t>(e) * d.pr;
  if (threadIdx.x == 0)
    plan_chunk(cmap, v.packed_row_group ? v.packed_row_group + static_cast<size_t>(e) * d.pr : nullptr, d.pr, p0, v.rank,
               plan, col_of_slot);
  __syncthreads();
  const unsigned long long* cp = reinterpret_cast<const unsigned long long*>(v.col_pack3) + static_cast<size_t>(e) * v.rank;
  if (threadIdx.x == 0) {
    ColHeader h = {};
    for (int p = 0; p < kChunkRows; ++p) h.slot_of_row[p] = plan.slot_of_row[p];
    for (int s = 0; s < 2 * kMaxSalWords; ++s) h.sal_slot[s >> 1][s & 1] = (s < plan.num_steps) ? plan.step_slot[s] : 0;
    h.num_salient = static_cast<uint16_t>(plan.num_salient);
    h.sal_words = static_cast<uint8_t>((plan.num_steps + 1) >> 1);
    h.num_slots = static_cast<uint8_t>(plan.num_slots);
    for (int sl = 0; sl < kChunkRows; ++sl) h.slot_end[sl] = 0;
    for (int p = 0; p < kChunkRows && p0 + p < d.pr; ++p) h.slot_end[plan.slot_of_row[p]] = static_cast<uint8_t>(p + 1);
    *reinterpret_cast<ColHeader*>(rec) = h;
  }
  // column scale table of the main loop: [packed row][t][pair i]{d, nd}, zero at salient columns
  uint32_t* coltab = reinterpret_cast<uint32_t*>(rec + kColHdrBytes);
  for (int i = threadIdx.x; i < kChunkRows * 16; i += blockDim.x) {
    const int p = i >> 4, t = (i >> 2) & 3, pi = i & 3;
    const int pg = p0 + p;
    uint32_t cd2 = 0u, cn2 = 0u;
    if (pg < d.pr) {
      const uint32_t cw = static_cast<uint32_t>(cmap[pg]);
      for (int h = 0; h < 2; ++h) {
        const int j = lane_pair_col(t, pi) + 16 * h;
        const int c = 32 * pg + j;
        if (c < v.rank && !((cw >> j) & 1u)) {
          cd2 |= half_of_pack(cp[c], 2) << (16 * h);
          cn2 |= half_of_pack(cp[c], 3) << (16 * h);
        }
      }
    }
    coltab[(p * 4 + t) * 8 + 2 * pi] = cd2;
    coltab[(p * 4 + t) * 8 + 2 * pi + 1] = cn2;
  }
  // salient words
  for (int i = threadIdx.x; i < max_sal_words * 16; i += blockDim.x) {
    const int q = i >> 4, t = (i >> 2) & 3, pi = i & 3;
    uint8_t* ent = rec + kColHdrBytes + kColTabBytes + q * kSalEntryBytes;
    uint16_t* salpos = reinterpret_cast<uint16_t*>(ent);
    uint32_t* salc = reinterpret_cast<uint32_t*>(ent + 64);
    uint32_t c1 = 0u, c2 = 0u;
    for (int h = 0; h < 2; ++h) {
      const int slot = lane_pair_col(t, pi) + 16 * h;
      const unsigned col = col_of_slot[q * 32 + slot];
      unsigned pos = 0u;
      if (col != 0xFFFFu) {
        pos = 2u * ((col & ~31u) + lane_order_pos(col & 31u));
        const unsigned long long pack = cp[32 * p0 + col];
        c1 |= half_of_pack(pack, 0) << (16 * h);
        c2 |= half_of_pack(pack, 1) << (16 * h);
      }
      salpos[t * 8 + 2 * pi + h] = static_cast<uint16_t>(pos);
    }
    salc[t * 8 + 2 * pi] = c1;
    salc[t * 8 + 2 * pi + 1] = c2;
  }
  for (int i = threadIdx.x; i < max_sal_words * 32; i += blockDim.x) {
    uint16_t* salcol = reinterpret_cast<uint16_t*>(rec + kColHdrBytes + kColTabBytes + (i >> 5) * kSalEntryBytes + 192);
    salcol[i & 31] = col_of_slot[i];
  }
}

// grid (tiles * chunks, E), 256 threads
__global__ void build_tile_records_kernel(TrisProjView v, const uint2* desc, uint8_t* records) {
  __shared__ ChunkPlan plan;
  __shared__ uint16_t col_of_slot[kMaxSalWords * 32];
  __shared__ RecHeader hdr;
  __shared__ int blk_src[4];    // word offset of each block inside the expert's stream
  __shared__ int slot_group[kChunkRows];
  if (threadIdx.x < kChunkRows) slot_group[threadIdx.x] = -1;
  __syncthreads();
  const BuildDims d = build_dims(v);
  const int chunk = blockIdx.x % d.chunks, tile = blockIdx.x / d.chunks, e = blockIdx.y;
  const int p0 = chunk * kChunkRows, o0 = tile * kTileOut;
  const int idx = (e * d.tiles + tile) * d.chunks + chunk;
  uint8_t* rec = records + static_cast<size_t>(desc[idx].x) * 16;
  const int32_t* cmap = v.c_map + static_cast<size_t>(e) * d.pr;
  const int32_t* groups = v.packed_row_group ? v.packed_row_group + static_cast<size_t>(e) * d.pr : nullptr;
  if (threadIdx.x == 0) {
    plan_chunk(cmap, groups, d.pr, p0, v.rank, plan, col_of_slot);
    for (int p = 0; p < kChunkRows; ++p)
      if (p0 + p < d.pr) slot_group[plan.slot_of_row[p]] = groups ? groups[p0 + p] : 0;
    RecHeader h = {};
    const int sal_words = (plan.num_steps + 1) >> 1;
    const int32_t* off = v.q_gmap_gr_offsets + static_cast<size_t>(e) * (d.nblk + 1);
    const int32_t* meta = v.q_gmap_gr_meta + static_cast<size_t>(e) * d.nblk;
    int words = 0;
    for (int b = 0; b < 4; ++b) {
      const int kb = 4 * chunk + b;
      int count = 0, m = 0, src = 0;
      if (kb < d.nkb) {
        const int bi = kb * d.nob + tile;
        src = off[bi];
        count = max(0, min(off[bi + 1] - off[bi], TRIS_GR_BLOCK_WORDS));
        m = meta[bi];
      }
      h.blk[b][0] = static_cast<uint32_t>(words) | (static_cast<uint32_t>(count) << 16);
      h.blk[b][1] = static_cast<uint32_t>(m);
      blk_src[b] = src;
      words += count;
    }
    h.off_rowtab = kHdrBytes + kS1Bytes;
    h.off_gridx = h.off_rowtab + plan.num_slots * kSlotBytes;
    h.off_ss1 = h.off_gridx + kGridxBytes;
    h.off_ss2 = h.off_ss1 + sal_words * kSalPlaneBytes;
    h.off_gr = h.off_ss2 + sal_words * kSalPlaneBytes;
    h.num_slots = static_cast<uint8_t>(plan.num_slots);
    h.sal_words = static_cast<uint8_t>(sal_words);
    h.gr_words = static_cast<uint32_t>(words);
    hdr = h;
    *reinterpret_cast<RecHeader*>(rec) = h;
  }
  __syncthreads();
  const uint32_t* stream = reinterpret_cast<const uint32_t*>(v.q_gmap_gr_words) + static_cast<size_t>(e) * v.gr_max_words;
  if (threadIdx.x < 4) {
    // Parse the block once: may the kernels decode it with the 32-bit-view loop?
    const int b = threadIdx.x;
    const int count = static_cast<int>(hdr.blk[b][0] >> 16), meta = static_cast<int>(hdr.blk[b][1]);
    if (count > 0 && !(meta & TRIS_GR_META_RAW_FLAG)) {
      const int k = meta & TRIS_GR_META_K_MASK, one_count = meta >> TRIS_GR_META_ONE_COUNT_SHIFT;
      const int total_bits = count << 5;
      auto bit = [&](int bp) { return (stream[blk_src[b] + (bp >> 5)] >> (bp & 31)) & 1u; };
      int bp = 0, flat = 0;
      bool slow = blk_src[b] < 0 || blk_src[b] + count > v.gr_max_words;
      for (int n = 0; n < one_count && !slow; ++n) {
        int t = 0;
        while (bp < total_bits && !bit(bp)) { ++t; ++bp; }
        if (bp >= total_bits || t + 1 + k > 32 || bp + 1 + k > total_bits) { slow = true; break; }
        ++bp;
        int rem = 0;
        for (int j = 0; j < k; ++j, ++bp) rem |= static_cast<int>(bit(bp)) << j;
        flat += (t << k) + rem;
        if (flat >= TRIS_GR_BLOCK_WORDS * 32) { slow = true; break; }
        ++flat;
      }
      if (slow) {
        hdr.blk[b][1] |= kBlockSlowFlag;
        reinterpret_cast<RecHeader*>(rec)->blk[b][1] |= kBlockSlowFlag;
      }
    }
  }
  __syncthreads();
  const uint32_t* qw1 = reinterpret_cast<const uint32_t*>(v.qweight1) + static_cast<size_t>(e) * d.pr * v.out_features;
  // sign plane
  uint32_t* s1 = reinterpret_cast<uint32_t*>(rec + kHdrBytes);
  for (int i = threadIdx.x; i < kChunkRows * kTileOut; i += blockDim.x) {
    const int p = i / kTileOut, o = i % kTileOut;
    s1[i] = (p0 + p < d.pr && o0 + o < v.out_features) ? qw1[static_cast<size_t>(p0 + p) * v.out_features + o0 + o] : 0u;
  }
  // row scale slots
  uint2* rowtab = reinterpret_cast<uint2*>(rec + hdr.off_rowtab);
  for (int i = threadIdx.x; i < hdr.num_slots * kTileOut; i += blockDim.x) {
    const int slot = i / kTileOut, o = i % kTileOut;
    uint2 rp = make_uint2(0u, 0u);
    const int grp = slot_group[slot];
    if (o0 + o < v.out_features && grp >= 0 && grp < v.num_groups) {
      const unsigned long long w = static_cast<unsigned long long>(
          v.row_pack3[(static_cast<size_t>(e) * v.out_features + o0 + o) * v.num_groups + grp]);
      rp = make_uint2(static_cast<uint32_t>(w), static_cast<uint32_t>(w >> 32));
    }
    rowtab[i] = rp;
  }
  // block-GR sub-stream index and words
  uint32_t* gridx = reinterpret_cast<uint32_t*>(rec + hdr.off_gridx);
  for (int i = threadIdx.x; i < 4 * 32; i += blockDim.x) {
    const int b = i >> 5, kb = 4 * chunk + b;
    uint32_t val = 0u;
    if (kb < d.nkb && v.gr_index) val = v.gr_index[(static_cast<size_t>(e) * d.nblk + kb * d.nob + tile) * 32 + (i & 31)];
    gridx[i] = val;
  }
  uint32_t* gr = reinterpret_cast<uint32_t*>(rec + hdr.off_gr);
  for (int b = 0; b < 4; ++b) {
    const int dst = static_cast<int>(hdr.blk[b][0] & 0xFFFFu), count = static_cast<int>(hdr.blk[b][0] >> 16);
    for (int i = threadIdx.x; i < count; i += blockDim.x) {
      const int s = blk_src[b] + i;
      gr[dst + i] = (s >= 0 && s < v.gr_max_words) ? stream[s] : 0u;
    }
  }
  for (int i = static_cast<int>(hdr.gr_words) + threadIdx.x; i < ((static_cast<int>(hdr.gr_words) + 3) & ~3); i += blockDim.x)
    gr[i] = 0u;
  // sign bits of the salient columns, slot order
  uint32_t* ss1 = reinterpret_cast<uint32_t*>(rec + hdr.off_ss1);
  uint32_t* ss2 = reinterpret_cast<uint32_t*>(rec + hdr.off_ss2);
  const int32_t* pre2 = v.qweight2_sparse_prefix ? v.qweight2_sparse_prefix + static_cast<size_t>(e) * (d.pr + 1) : nullptr;
  const uint32_t* qw2 = reinterpret_cast<const uint32_t*>(v.qweight2_sparse) + static_cast<size_t>(e) * v.sign2_rows * v.out_features;
  for (int i = threadIdx.x; i < hdr.sal_words * kTileOut; i += blockDim.x) {
    const int q = i / kTileOut, o = i % kTileOut;
    uint32_t w1 = 0u, w2 = 0u;
    if (o0 + o < v.out_features) {
      for (int j = 0; j < 32; ++j) {
        const unsigned col = col_of_slot[q * 32 + j];
        if (col == 0xFFFFu) continue;
        const int pg = p0 + static_cast<int>(col >> 5), bit = col & 31;
        w1 |= ((qw1[static_cast<size_t>(pg) * v.out_features + o0 + o] >> bit) & 1u) << j;
        if (pre2 && v.qweight2_sparse && v.sign2_rows > 0) {
          const int rank2 = pre2[pg] + __popc(static_cast<uint32_t>(cmap[pg]) & ((1u << bit) - 1u));
          if (rank2 >= 0 && (rank2 >> 5) < v.sign2_rows)
            w2 |= ((qw2[static_cast<size_t>(rank2 >> 5) * v.out_features + o0 + o] >> (rank2 & 31)) & 1u) << j;
        }
      }
    }
    ss1[i] = w1;
    ss2[i] = w2;
  }
}

static int validate_for_records(const TrisProjView* v, const char* name) {
  TRIS_REQUIRE(v != nullptr, TRIS_ERR_INVALID_ARG, "%s: null projection view", name);
  TRIS_REQUIRE(v->num_experts > 0 && v->out_features > 0 && v->rank > 0 && v->num_groups > 0, TRIS_ERR_INVALID_ARG,
               "%s: non-positive dims", name);
  TRIS_REQUIRE(v->use_block_gr && v->q_gmap_gr_words && v->q_gmap_gr_offsets && v->q_gmap_gr_meta, TRIS_ERR_UNSUPPORTED,
               "%s: tile records need a block-GR payload", name);
  TRIS_REQUIRE(v->gr_index != nullptr && v->gr_substreams == 32, TRIS_ERR_INVALID_ARG,
               "%s: needs the 32-way sub-stream index (tris_block_gr_build_index)", name);
  TRIS_REQUIRE(v->qweight1 && v->c_map && v->col_pack3 && v->row_pack3, TRIS_ERR_INVALID_ARG,
               "%s: qweight1/c_map/col_pack3/row_pack3 must be set", name);
  TRIS_REQUIRE(v->packed_row_group != nullptr || v->num_groups == 1, TRIS_ERR_INVALID_ARG,
               "%s: packed_row_group missing (call tris_build_row_groups)", name);
  TRIS_REQUIRE(!v->expert_slot && !v->gmap_slot, TRIS_ERR_UNSUPPORTED, "%s: paged payloads have no tile records", name);
  return TRIS_OK;
}

}  // namespace tr
}  // namespace tris

using namespace tris;
using namespace tris::tr;

extern "C" int64_t tris_tile_record_count(const TrisProjView* proj) {
  if (proj == nullptr || proj->num_experts <= 0 || proj->out_features <= 0 || proj->rank <= 0) return 0;
  const BuildDims d = build_dims(*proj);
  return static_cast<int64_t>(proj->num_experts) * d.tiles * d.chunks;
}

extern "C" int64_t tris_col_record_bytes(const TrisProjView* proj, int32_t max_sal_words) {
  if (proj == nullptr || max_sal_words < 0 || max_sal_words > kMaxSalWords) return 0;
  const BuildDims d = build_dims(*proj);
  return static_cast<int64_t>(proj->num_experts) * d.chunks * col_record_bytes(max_sal_words);
}

extern "C" int tris_tile_records_plan(const TrisProjView* proj, uint32_t* desc_out, int64_t* info_out, void* stream) {
  int st = validate_for_records(proj, "tris_tile_records_plan");
  if (st != TRIS_OK) return st;
  TRIS_REQUIRE(desc_out && info_out, TRIS_ERR_INVALID_ARG, "tris_tile_records_plan: null output");
  const int64_t total = tris_tile_record_count(proj);
  TRIS_REQUIRE(total > 0 && total < (1ll << 30), TRIS_ERR_UNSUPPORTED, "tris_tile_records_plan: %lld records", static_cast<long long>(total));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  uint2* desc = reinterpret_cast<uint2*>(desc_out);
  TRIS_CUDA(cudaMemsetAsync(desc + total, 0, sizeof(uint2), s));
  const int threads = 128;
  plan_records_kernel<<<static_cast<int>(std::min<int64_t>((total + threads - 1) / threads, 4096)), threads, 0, s>>>(*proj, desc);
  TRIS_CUDA(cudaGetLastError());
  scan_records_kernel<<<1, 1024, 0, s>>>(desc, static_cast<int>(total), info_out);
  return check_cuda(cudaGetLastError(), "tile record plan kernels");
}

extern "C" int tris_tile_records_build(const TrisProjView* proj, const uint32_t* desc, void* records_out,
                                       void* col_records_out, int32_t max_sal_words, void* stream) {
  int st = validate_for_records(proj, "tris_tile_records_build");
  if (st != TRIS_OK) return st;
  TRIS_REQUIRE(desc && records_out && col_records_out, TRIS_ERR_INVALID_ARG, "tris_tile_records_build: null pointer");
  TRIS_REQUIRE(max_sal_words >= 0 && max_sal_words <= kMaxSalWords, TRIS_ERR_INVALID_ARG,
               "tris_tile_records_build: max_sal_words=%d", max_sal_words);
  TRIS_REQUIRE((reinterpret_cast<uintptr_t>(records_out) & 15u) == 0 && (reinterpret_cast<uintptr_t>(col_records_out) & 15u) == 0,
               TRIS_ERR_INVALID_ARG, "tris_tile_records_build: record buffers must be 16-byte aligned");
  const BuildDims d = build_dims(*proj);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  build_col_records_kernel<<<dim3(d.chunks, proj->num_experts), 128, 0, s>>>(*proj, static_cast<uint8_t*>(col_records_out), max_sal_words);
  TRIS_CUDA(cudaGetLastError());
  build_tile_records_kernel<<<dim3(d.tiles * d.chunks, proj->num_experts), 256, 0, s>>>(*proj, reinterpret_cast<const uint2*>(desc),
                                                                                        static_cast<uint8_t*>(records_out));
  return check_cuda(cudaGetLastError(), "tile record build kernels");
}
